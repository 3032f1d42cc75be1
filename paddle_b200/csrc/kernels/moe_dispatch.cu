// Expert-parallel token exchange fused with the fp8 quantisation of the expert GEMM operand, over NVLink peer memory
// (one process per GPU, symmetric buffers, no host synchronisation, no library collective):
//
//   pd_moe_dispatch_fp8 : every routed copy (token t, choice j) is quantised to e4m3 with one scale per 128 columns
//                         and written - payload and scales - with plain peer stores straight into the buffer of the
//                         rank that owns its expert, at slot [local expert][source rank][position].  Every (expert,
//                         source) pair has a fixed capacity, so no counts have to be exchanged before data moves;
//                         the actual row counts travel with the data.  The last CTA of the launch publishes an arrival
//                         flag on every peer, waits (bounded) for the flags of all sources and writes the segment
//                         table (start, end, expert) that the grouped block-scaled GEMM consumes: when the kernel has
//                         ended, this rank's expert input is complete.
//   pd_moe_combine      : after the experts ran, every rank announces its outputs and each token gathers its k
//                         expert rows from the owners' buffers with peer loads, scales them by the gate values and sums
//                         them (fp32) - the weighted combine is the epilogue of the gather.
//
// The reference moves tokens with grouped ncclSend / ncclRecv driven by counts that were first copied to the host
// (paddle/phi/kernels/gpu/global_scatter_kernel.cu:57-75,109-133, global_gather_kernel.cu; Python side
// python/paddle/incubate/distributed/models/moe/moe_layer.py:95-258) and quantises nothing on the way.
// Protocol: device-resident epochs (CUDA-graph replayable), every wait bounded with a status report, flags never
// reset.  A dispatch and the combine that follows it form a barrier pair: a rank can start dispatch e + 1 only after its
// combine e, which needs every peer's experts of epoch e to have finished - so the receive buffers need no second slot.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "host_utils.h"
#include "sm100_prims.cuh"

namespace pd {
namespace moex {

typedef __nv_bfloat16 bf16;
constexpr int MAX_RANKS = 8;
constexpr int THREADS = 256;
constexpr float E4M3_MAX = 448.f;

struct DispatchArgs {
  const bf16* x;             // [T, H]
  const int* expert;         // [T * k] global expert id (rank-major: expert g lives on rank g / E_local), < 0 = pruned
  const int* slot;           // [T * k] position of the copy among this rank's copies for that expert; >= cap: dropped
  const float* row_scale;    // optional [T * k]: multiplier applied before quantisation (backward: the gate values)
  const int* send_counts;    // [nranks * E_local] copies this rank routes to every global expert (not clamped)
  int T, k, H, cap, E_local, rank, nranks;
  uint8_t* xq[MAX_RANKS];    // every rank's payload buffer  [E_local][nranks][cap][H] e4m3
  float* xs[MAX_RANKS];      // every rank's scale buffer    [E_local][nranks][cap][H / 128]
  int* counts[MAX_RANKS];    // every rank's row counts      [E_local][nranks]
  int* ready[MAX_RANKS];     // every rank's arrival flags   [nranks]
  int* state;                // local: [0] epoch, [1] finished CTAs
  int* seg_start;            // local out [E_local * nranks]
  int* seg_end;              // local out [E_local * nranks]
  int* expert_map;           // local out [E_local * nranks]
  unsigned long long wait_ns;
  int* status;
};

// one warp per routed copy; a lane owns 4 consecutive columns of every 128-column block
__global__ void __launch_bounds__(THREADS) moe_dispatch_fp8_kernel(DispatchArgs a) {
  const int epoch = a.state[0] + 1;
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = THREADS / 32;
  const int nb = a.H / 128;
  const int copies = a.T * a.k;
  for (int c = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); c < copies; c += gridDim.x * warps_per_cta) {
    const int g = a.expert[c];
    const int pos = a.slot[c];
    if (g < 0 || pos >= a.cap) continue;                         // pruned by the gate / over capacity: dropped
    const int dst = g / a.E_local, e = g - dst * a.E_local;
    const size_t row = (static_cast<size_t>(e) * a.nranks + a.rank) * a.cap + pos;
    const bf16* src = a.x + static_cast<size_t>(c / a.k) * a.H;
    uint8_t* q = a.xq[dst] + row * a.H;
    float* sc = a.xs[dst] + row * nb;
    const float mul = a.row_scale != nullptr ? a.row_scale[c] : 1.f;
    for (int kb = 0; kb < nb; ++kb) {
      const uint2 raw = *reinterpret_cast<const uint2*>(src + kb * 128 + lane * 4);
      float2 v0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
      float2 v1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      v0.x *= mul; v0.y *= mul; v1.x *= mul; v1.y *= mul;
      float amax = fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v1.x), fabsf(v1.y)));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float scale = fmaxf(amax, 1e-12f) / E4M3_MAX;
      const float inv = 1.f / scale;
      __nv_fp8_e4m3 o4[4] = {__nv_fp8_e4m3(v0.x * inv), __nv_fp8_e4m3(v0.y * inv), __nv_fp8_e4m3(v1.x * inv),
                             __nv_fp8_e4m3(v1.y * inv)};
      *reinterpret_cast<uint32_t*>(q + kb * 128 + lane * 4) = *reinterpret_cast<uint32_t*>(o4);   // 128 B per warp
      if (lane == 0) sc[kb] = scale;
    }
  }
  // ---- completion: every CTA makes its stores visible system-wide, the last one to finish does the signalling
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x != 0) return;
  if (atomicAdd(a.state + 1, 1) != static_cast<int>(gridDim.x) - 1) return;
  __threadfence();
  const int n_seg = a.E_local * a.nranks;
  // row counts first, then the flag (release): the receiver reads the counts after it has seen the flag
  for (int g = 0; g < n_seg; ++g) {
    const int dst = g / a.E_local, e = g - dst * a.E_local;
    a.counts[dst][e * a.nranks + a.rank] = min(a.send_counts[g], a.cap);
  }
  asm volatile("fence.acq_rel.sys;" ::: "memory");
  for (int r = 0; r < a.nranks; ++r) st_release_sys(a.ready[r] + a.rank, epoch);
  bool ok = true;
  for (int r = 0; r < a.nranks && ok; ++r)
    ok = flag_wait_ge(a.ready[a.rank] + r, epoch, a.wait_ns, a.status, 900 + r);
  if (ok) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    const volatile int* cnt = a.counts[a.rank];
    for (int s = 0; s < n_seg; ++s) {            // segment s = (local expert e, source rank r), e-major
      a.seg_start[s] = s * a.cap;
      a.seg_end[s] = s * a.cap + cnt[s];
      a.expert_map[s] = s / a.nranks;
    }
  }
  a.state[1] = 0;
  __threadfence();
  a.state[0] = epoch;
}

// 16-byte load that bypasses L1 (the rows were written by another GPU's kernels during this epoch)
__device__ __forceinline__ uint4 ld_peer_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)
               : "memory");
  return v;
}

struct CombineArgs {
  const bf16* y[MAX_RANKS];  // every rank's expert output buffer [E_local][nranks][cap][H] bf16
  const int* expert;         // [T * k]
  const int* slot;           // [T * k]
  const float* weight;       // optional [T * k] gate values (null: plain sum over the k copies)
  bf16* out;                 // [T, H]
  bf16* rows_out;            // optional [T * k, H]: the gathered, unweighted expert rows (kept for backward)
  int T, k, H, cap, E_local, rank, nranks;
  int* oready[MAX_RANKS];    // every rank's "expert outputs of epoch e are complete" flags [nranks]
  int* state;                // local: [0] epoch, [1] finished CTAs
  unsigned long long wait_ns;
  int* status;
};

// one warp per token; a lane owns 8 consecutive columns (16 bytes) of every 256-column stripe
__global__ void __launch_bounds__(THREADS) moe_combine_kernel(CombineArgs a) {
  __shared__ int verdict;
  const int epoch = a.state[0] + 1;
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) {
      // this launch is ordered after this rank's expert GEMMs on the stream: their output is complete
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      for (int r = 0; r < a.nranks; ++r) st_release_sys(a.oready[r] + a.rank, epoch);
    }
    bool ok = true;
    for (int r = 0; r < a.nranks && ok; ++r)
      ok = flag_wait_ge(a.oready[a.rank] + r, epoch, a.wait_ns, a.status, 950 + r);
    verdict = ok ? 1 : 0;
  }
  __syncthreads();
  if (verdict) {
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = THREADS / 32;
    const int nvec = a.H / 8;
    for (int t = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); t < a.T; t += gridDim.x * warps_per_cta) {
      for (int v0 = lane; v0 < nvec; v0 += 32 * 4) {
        // up to 4 stripes x k copies of 16-byte peer loads are in flight before any is consumed
        float acc[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[u][i] = 0.f;
        for (int j = 0; j < a.k; ++j) {
          const int c = t * a.k + j;
          const int g = a.expert[c];
          const int pos = a.slot[c];
          const bool live = g >= 0 && pos < a.cap;
          const int dst = live ? g / a.E_local : 0, e = live ? g - dst * a.E_local : 0;
          const bf16* row = a.y[dst] + ((static_cast<size_t>(e) * a.nranks + a.rank) * a.cap + (live ? pos : 0)) * a.H;
          const float w = a.weight != nullptr ? a.weight[c] : 1.f;
          uint4 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int vi = v0 + u * 32;
            v[u] = make_uint4(0u, 0u, 0u, 0u);
            if (live && vi < nvec) v[u] = ld_peer_v4(reinterpret_cast<const uint4*>(row) + vi);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int vi = v0 + u * 32;
            if (vi >= nvec) continue;
            if (a.rows_out != nullptr)
              *(reinterpret_cast<uint4*>(a.rows_out + static_cast<size_t>(c) * a.H) + vi) = v[u];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = __bfloat1622float2(h[i]);
              acc[u][2 * i] = fmaf(w, f.x, acc[u][2 * i]);
              acc[u][2 * i + 1] = fmaf(w, f.y, acc[u][2 * i + 1]);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int vi = v0 + u * 32;
          if (vi >= nvec) continue;
          uint4 o;
          o.x = pack_bf16x2(acc[u][0], acc[u][1]);
          o.y = pack_bf16x2(acc[u][2], acc[u][3]);
          o.z = pack_bf16x2(acc[u][4], acc[u][5]);
          o.w = pack_bf16x2(acc[u][6], acc[u][7]);
          *(reinterpret_cast<uint4*>(a.out + static_cast<size_t>(t) * a.H) + vi) = o;
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.state + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      a.state[1] = 0;
      __threadfence();
      a.state[0] = epoch;
    }
  }
}

}  // namespace moex
}  // namespace pd

using namespace pd;
using namespace pd::moex;

// Buffers of rank r (peer_* arrays hold the address of every rank's buffer as mapped into this process):
//   xq [E_local][nranks][cap][H] e4m3, xs [E_local][nranks][cap][H/128] f32, counts [E_local][nranks] i32,
//   ready [nranks] i32 (zeroed once).  state: 2 local i32 zeroed once.  seg_* / expert_map: local i32 [E_local*nranks].
PD_EXPORT int pd_moe_dispatch_fp8(const void* x, const int* expert, const int* slot, const float* row_scale,
                                  const int* send_counts, int T, int k, int H, int cap, int E_local, int rank, int nranks,
                                  const unsigned long long* peer_xq, const unsigned long long* peer_xs,
                                  const unsigned long long* peer_counts, const unsigned long long* peer_ready, int* state,
                                  int* seg_start, int* seg_end, int* expert_map, int wait_ms, int* status,
                                  cudaStream_t stream) {
  if (T <= 0 || k <= 0 || H <= 0 || (H % 128) || cap <= 0 || E_local <= 0 || nranks < 1 || nranks > MAX_RANKS ||
      E_local * nranks > 64)
    return kErrBadShape;
  if (!aligned16(x)) return kErrAlignment;
  DispatchArgs a;
  a.x = static_cast<const bf16*>(x); a.expert = expert; a.slot = slot; a.row_scale = row_scale; a.send_counts = send_counts;
  a.T = T; a.k = k; a.H = H; a.cap = cap; a.E_local = E_local; a.rank = rank; a.nranks = nranks;
  for (int i = 0; i < MAX_RANKS; ++i) {
    const int j = i < nranks ? i : 0;
    a.xq[i] = reinterpret_cast<uint8_t*>(peer_xq[j]);
    a.xs[i] = reinterpret_cast<float*>(peer_xs[j]);
    a.counts[i] = reinterpret_cast<int*>(peer_counts[j]);
    a.ready[i] = reinterpret_cast<int*>(peer_ready[j]);
  }
  a.state = state; a.seg_start = seg_start; a.seg_end = seg_end; a.expert_map = expert_map;
  a.wait_ns = static_cast<unsigned long long>(wait_ms) * 1000000ull;
  a.status = status;
  const long long copies = static_cast<long long>(T) * k;
  long long grid = (copies + THREADS / 32 - 1) / (THREADS / 32);
  const int cap_grid = sm_count() * 4;
  if (grid > cap_grid) grid = cap_grid;
  moe_dispatch_fp8_kernel<<<static_cast<int>(grid), THREADS, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

// y buffers: [E_local][nranks][cap][H] bf16 on every rank; oready: [nranks] i32 zeroed once; state: 2 local i32.
PD_EXPORT int pd_moe_combine(const int* expert, const int* slot, const float* weight, void* out, void* rows_out, int T,
                             int k, int H, int cap, int E_local, int rank, int nranks, const unsigned long long* peer_y,
                             const unsigned long long* peer_oready, int* state, int wait_ms, int* status,
                             cudaStream_t stream) {
  if (T <= 0 || k <= 0 || H <= 0 || (H % 8) || cap <= 0 || E_local <= 0 || nranks < 1 || nranks > MAX_RANKS)
    return kErrBadShape;
  if (!aligned16(out) || (rows_out != nullptr && !aligned16(rows_out))) return kErrAlignment;
  CombineArgs a;
  for (int i = 0; i < MAX_RANKS; ++i) {
    const int j = i < nranks ? i : 0;
    a.y[i] = reinterpret_cast<const bf16*>(peer_y[j]);
    a.oready[i] = reinterpret_cast<int*>(peer_oready[j]);
  }
  a.expert = expert; a.slot = slot; a.weight = weight; a.out = static_cast<bf16*>(out);
  a.rows_out = static_cast<bf16*>(rows_out);
  a.T = T; a.k = k; a.H = H; a.cap = cap; a.E_local = E_local; a.rank = rank; a.nranks = nranks;
  a.state = state;
  a.wait_ns = static_cast<unsigned long long>(wait_ms) * 1000000ull;
  a.status = status;
  int grid = (T + THREADS / 32 - 1) / (THREADS / 32);
  const int cap_grid = sm_count() * 4;
  if (grid > cap_grid) grid = cap_grid;
  moe_combine_kernel<<<grid, THREADS, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}
