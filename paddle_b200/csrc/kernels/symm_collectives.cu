// Standalone collectives over symmetric (peer-mapped) memory for small and medium messages, where a library
// collective is dominated by launch and protocol latency:
//   pd_symm_all_reduce     : one-shot - every rank pushes its whole vector into row [rank] of every peer's receive
//                            buffer, then sums the n rows it received (fp32 accumulation, rank order: deterministic)
//   pd_symm_all_gather     : every rank pushes its shard into slot [rank] of every peer's output buffer
//   pd_symm_reduce_scatter : every rank pushes slice d of its vector to rank d, which sums the n rows
// (reference: ProcessGroupNCCL::AllReduce / AllGather / ReduceScatter, paddle/fluid/distributed/collective/
// process_group_nccl.cc:241,197,408 - the NCCL calls remain the path for large messages).
// Same protocol as the fused kernels: plain peer stores, one release-add per chunk on the destination's counter,
// bounded acquire-wait on the own counters, device-resident epoch (CUDA-graph replayable), two alternating slots.
#include <cuda_bf16.h>

#include "host_utils.h"
#include "sm100_prims.cuh"

namespace pd {
namespace sc {

typedef __nv_bfloat16 bf16;
constexpr int CHUNK_BYTES = 16384;
constexpr int THREADS = 256;
constexpr int MAX_RANKS = 8;

struct Args {
  const uint8_t* in;             // local input
  uint8_t* out;                  // local output
  uint8_t* recv[MAX_RANKS];      // receive buffers: [2][nranks][row_bytes_padded]
  int* cnt[MAX_RANKS];           // per-chunk counters
  int64_t in_row_bytes;          // bytes this rank contributes per destination row
  int64_t row_pad;               // padded row size in the receive buffer
  int rank, nranks, chunks, kind, is_bf16;   // kind 0 all_reduce, 1 all_gather, 2 reduce_scatter
  int chunk_bytes;               // multiple of CHUNK_BYTES, the same on every rank for a given call
  int* state;
  int* seen;                     // local, per chunk: arrivals consumed so far (calls of different sizes touch different chunks)
  unsigned long long wait_ns;
  int* status;
};

// 16-byte copies with four loads in flight per thread before the first store: over NVLink the copy is bound by the
// number of outstanding requests, not by issue rate.
__device__ __forceinline__ void copy_bytes(uint8_t* dst, const uint8_t* src, int64_t n, bool src_is_peer_written) {
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | n) & 15u) == 0) {
    const int64_t step = static_cast<int64_t>(THREADS) * 16;
    int64_t i = threadIdx.x * 16;
    for (; i + 3 * step < n; i += 4 * step) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint4* p = reinterpret_cast<const uint4*>(src + i + u * step);
        v[u] = src_is_peer_written ? __ldcg(p) : *p;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) *reinterpret_cast<uint4*>(dst + i + u * step) = v[u];
    }
    for (; i < n; i += step) {
      const uint4* p = reinterpret_cast<const uint4*>(src + i);
      *reinterpret_cast<uint4*>(dst + i) = src_is_peer_written ? __ldcg(p) : *p;
    }
  } else {
    for (int64_t i = threadIdx.x; i < n; i += THREADS) dst[i] = src_is_peer_written ? __ldcg(src + i) : src[i];
  }
}

__device__ __forceinline__ void add_bf16x8(float* acc, const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    acc[2 * e] += __uint_as_float(w[e] << 16);
    acc[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
  }
}

__global__ void __launch_bounds__(THREADS) symm_collective_kernel(Args a) {
  __shared__ int verdict;
  const int epoch = a.state[0] + 1;
  const int64_t slot_off = static_cast<int64_t>(epoch & 1) * a.nranks * a.row_pad;
  // ---- push: item = (destination, chunk)
  const int items = a.nranks * a.chunks;
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    const int dst = (a.rank + 1 + it / a.chunks) % a.nranks;
    const int c = it % a.chunks;
    const int64_t b0 = static_cast<int64_t>(c) * a.chunk_bytes;
    const int64_t n = min(static_cast<int64_t>(a.chunk_bytes), a.in_row_bytes - b0);
    // all_reduce / all_gather send the same bytes to everybody; reduce_scatter sends slice `dst`
    const uint8_t* src = a.in + (a.kind == 2 ? static_cast<int64_t>(dst) * a.in_row_bytes : 0) + b0;
    copy_bytes(a.recv[dst] + slot_off + static_cast<int64_t>(a.rank) * a.row_pad + b0, src, n, false);
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) red_release_sys_add(a.cnt[dst] + c, 1);
  }
  // ---- consume the n rows that arrived here
  const uint8_t* base = a.recv[a.rank] + slot_off;
  for (int c = blockIdx.x; c < a.chunks; c += gridDim.x) {
    if (threadIdx.x == 0) {
      // expected arrivals are tracked per chunk, not derived from the epoch: a short message leaves the counters of
      // the higher chunks untouched while the epoch still advances
      const int target = a.seen[c] + a.nranks;
      verdict = flag_wait_ge(a.cnt[a.rank] + c, target, a.wait_ns, a.status, 800) ? 1 : 0;
      a.seen[c] = target;
    }
    __syncthreads();
    const bool ok = verdict != 0;
    __syncthreads();
    if (!ok) continue;
    const int64_t b0 = static_cast<int64_t>(c) * a.chunk_bytes;
    const int64_t n = min(static_cast<int64_t>(a.chunk_bytes), a.in_row_bytes - b0);
    if (a.kind == 1) {
      for (int r = 0; r < a.nranks; ++r)
        copy_bytes(a.out + static_cast<int64_t>(r) * a.in_row_bytes + b0, base + static_cast<int64_t>(r) * a.row_pad + b0, n,
                   true);
    } else {
      uint8_t* o = a.out + b0;
      const bool vec = ((reinterpret_cast<uintptr_t>(o) | n) & 15u) == 0;      // rows start 256-byte aligned
      int64_t done = 0;
      if (vec) {
        for (int64_t i = threadIdx.x * 16; i < n; i += THREADS * 16) {
          if (a.is_bf16) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < a.nranks; ++r)
              add_bf16x8(acc, __ldcg(reinterpret_cast<const uint4*>(base + static_cast<int64_t>(r) * a.row_pad + b0 + i)));
            uint4 ov;
            ov.x = pack_bf16x2(acc[0], acc[1]);
            ov.y = pack_bf16x2(acc[2], acc[3]);
            ov.z = pack_bf16x2(acc[4], acc[5]);
            ov.w = pack_bf16x2(acc[6], acc[7]);
            *reinterpret_cast<uint4*>(o + i) = ov;
          } else {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < a.nranks; ++r) {
              const float4 t = __ldcg(reinterpret_cast<const float4*>(base + static_cast<int64_t>(r) * a.row_pad + b0 + i));
              acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
            }
            *reinterpret_cast<float4*>(o + i) = acc;
          }
        }
        done = n;
      }
      if (a.is_bf16) {
        bf16* ob = reinterpret_cast<bf16*>(o);
        for (int64_t i = done / 2 + threadIdx.x; i < n / 2; i += THREADS) {
          float s = 0.f;
          for (int r = 0; r < a.nranks; ++r)
            s += __bfloat162float(__ldcg(reinterpret_cast<const bf16*>(base + static_cast<int64_t>(r) * a.row_pad + b0) + i));
          ob[i] = __float2bfloat16(s);
        }
      } else {
        float* of = reinterpret_cast<float*>(o);
        for (int64_t i = done / 4 + threadIdx.x; i < n / 4; i += THREADS) {
          float s = 0.f;
          for (int r = 0; r < a.nranks; ++r)
            s += __ldcg(reinterpret_cast<const float*>(base + static_cast<int64_t>(r) * a.row_pad + b0) + i);
          of[i] = s;
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

}  // namespace sc
}  // namespace pd

PD_EXPORT int pd_symm_chunk_bytes() { return pd::sc::CHUNK_BYTES; }

// kind 0 all_reduce (in: row_bytes, out: row_bytes), 1 all_gather (in: row_bytes, out: nranks * row_bytes),
// 2 reduce_scatter (in: nranks * row_bytes, out: row_bytes).  peer_recv[r]: [2][nranks][row_pad] bytes on rank r,
// peer_cnt[r]: int32 [ceil(row_pad / 16384)] zeroed once; state: 2 local int32 zeroed once; seen: local int32
// [ceil(row_pad / 16384)] zeroed once.
PD_EXPORT int pd_symm_collective(int kind, const void* in, void* out, int64_t row_bytes, int64_t row_pad, int is_bf16,
                                 int rank, int nranks, const unsigned long long* peer_recv,
                                 const unsigned long long* peer_cnt, int* state, int* seen, int wait_ms, int* status,
                                 cudaStream_t stream) {
  using namespace pd;
  using namespace pd::sc;
  if (kind < 0 || kind > 2 || row_bytes <= 0 || row_pad < row_bytes || nranks < 1 || nranks > MAX_RANKS) return kErrBadShape;
  if (kind != 1 && (row_bytes % (is_bf16 ? 2 : 4))) return kErrBadShape;
  Args a;
  a.in = static_cast<const uint8_t*>(in);
  a.out = static_cast<uint8_t*>(out);
  for (int i = 0; i < MAX_RANKS; ++i) {
    a.recv[i] = reinterpret_cast<uint8_t*>(peer_recv[i < nranks ? i : 0]);
    a.cnt[i] = reinterpret_cast<int*>(peer_cnt[i < nranks ? i : 0]);
  }
  a.in_row_bytes = row_bytes; a.row_pad = row_pad; a.rank = rank; a.nranks = nranks;
  // about four chunks per CTA and destination for large messages (fewer system-scope fences per byte), never
  // smaller than CHUNK_BYTES; every rank derives the same value from the same row_bytes
  {
    const int64_t want = row_bytes / (static_cast<int64_t>(sm_count()) * 2 * 4 / nranks + 1);
    int64_t cb = (want + CHUNK_BYTES - 1) / CHUNK_BYTES * CHUNK_BYTES;
    if (cb < CHUNK_BYTES) cb = CHUNK_BYTES;
    if (cb > 16 * CHUNK_BYTES) cb = 16 * CHUNK_BYTES;
    a.chunk_bytes = static_cast<int>(cb);
  }
  a.chunks = static_cast<int>((row_bytes + a.chunk_bytes - 1) / a.chunk_bytes);
  a.kind = kind; a.is_bf16 = is_bf16; a.state = state; a.seen = seen;
  a.wait_ns = static_cast<unsigned long long>(wait_ms) * 1000000ull;
  a.status = status;
  const int64_t items = static_cast<int64_t>(a.chunks) * nranks;
  const int cap = sm_count() * 2;
  symm_collective_kernel<<<static_cast<int>(items < cap ? items : cap), THREADS, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}
