// Gradient reduce-scatter fused with scaling and the partitioned AdamW update, in ONE kernel over peer memory
// (sharding stage 1/2: every rank owns 1/n of a flat gradient bucket and the optimizer state for it).
// Reference sequence: NCCL reduce_scatter of the fused buffer (tensor_fusion_helper.py FusedCommBuffer), a scale
// kernel, then adamw per parameter (dygraph_sharding_optimizer.py + adamw_kernel.cu).
//
// Phase 1 (push): the bucket is cut into 8192-element chunks; chunk c of the slice owned by rank d is copied with
// 128-bit peer stores into row [this rank] of d's receive buffer and one release-add is published on d's counter for
// chunk c.  Every CTA finishes all its pushes before it waits for anything, so ranks cannot block each other.
// Phase 2 (reduce + update): for each chunk of the OWN slice wait (bounded) until all n rows have arrived, sum them
// in fp32 in rank order (deterministic), multiply by grad_scale (1/n averaging x inverse loss scale x clip
// coefficient), apply AdamW to master / moment1 / moment2 and refresh the bf16 parameter slice.
// The epoch is device-resident (state[0]), counters are monotonic, and the receive buffer alternates between two
// slots, exactly as in gemm_ar.cu, so the launch is CUDA-graph replayable.
#include <cuda_bf16.h>

#include "host_utils.h"
#include "sm100_prims.cuh"

namespace pd {
namespace rsa {

typedef __nv_bfloat16 bf16;
constexpr int CHUNK = 8192;
constexpr int THREADS = 256;
constexpr int MAX_RANKS = 8;

struct Args {
  const float* grad;             // [nranks * shard] this rank's local gradients (fp32)
  float* recv[MAX_RANKS];        // each rank's receive buffer: [2][nranks][shard_padded] fp32
  int* cnt[MAX_RANKS];           // each rank's per-chunk counters [chunks]
  float *master, *m, *v;         // [shard] optimizer state of the owned slice
  bf16* param;                   // [shard] bf16 parameters of the owned slice (may be null)
  int64_t shard, shard_padded;
  int rank, nranks, chunks;
  float lr, beta1, beta2, eps, coeff, beta1_pow, beta2_pow;
  const float* grad_scale;       // optional device scalar
  const int* skip;               // optional device flag: nonzero -> reduce only, no update
  float* gout;                   // optional [shard]: store the reduced, scaled gradient here and do NOT update (the
                                 // two-phase form: global-norm clipping needs the norm of the reduced gradient first)
  int* state;                    // [0] epoch, [1] finished CTAs
  unsigned long long wait_ns;
  int* status;
};

__global__ void __launch_bounds__(THREADS) rs_adamw_kernel(Args a) {
  __shared__ int verdict;
  const int epoch = a.state[0] + 1;
  const int slot = epoch & 1;
  const int64_t slot_off = static_cast<int64_t>(slot) * a.nranks * a.shard_padded;
  // ---------------------------------------------------------------- phase 1: push my contributions to the owners
  const int items = a.nranks * a.chunks;
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    const int dst = (a.rank + 1 + it / a.chunks) % a.nranks;       // start with the neighbour: spreads link load
    const int c = it % a.chunks;
    const int64_t e0 = static_cast<int64_t>(c) * CHUNK;
    const int64_t n = min(static_cast<int64_t>(CHUNK), a.shard - e0);
    const float* src = a.grad + static_cast<int64_t>(dst) * a.shard + e0;
    float* dstp = a.recv[dst] + slot_off + static_cast<int64_t>(a.rank) * a.shard_padded + e0;
    const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dstp)) & 15u) == 0;
    if (vec) {
      for (int64_t i = threadIdx.x * 4; i + 3 < n; i += THREADS * 4)
        *reinterpret_cast<float4*>(dstp + i) = __ldg(reinterpret_cast<const float4*>(src + i));
      for (int64_t i = (n & ~int64_t(3)) + threadIdx.x; i < n; i += THREADS) dstp[i] = src[i];
    } else {
      for (int64_t i = threadIdx.x; i < n; i += THREADS) dstp[i] = src[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) red_release_sys_add(a.cnt[dst] + c, 1);
  }
  // ---------------------------------------------------------------- phase 2: reduce my slice, AdamW
  const float gscale = a.grad_scale ? *a.grad_scale : 1.f;
  const bool skip = a.skip != nullptr && *a.skip != 0;
  const float bc1 = 1.f - a.beta1_pow;
  const float inv_sqrt_bc2 = rsqrtf(1.f - a.beta2_pow);
  const float step_size = -(a.lr / bc1);
  const float decay = 1.f - a.lr * a.coeff;
  const float* base = a.recv[a.rank] + slot_off;
  for (int c = blockIdx.x; c < a.chunks; c += gridDim.x) {
    if (threadIdx.x == 0)
      verdict = flag_wait_ge(a.cnt[a.rank] + c, epoch * a.nranks, a.wait_ns, a.status, 700) ? 1 : 0;
    __syncthreads();
    const bool ok = verdict != 0;
    __syncthreads();
    if (!ok || (skip && a.gout == nullptr)) continue;
    const int64_t e0 = static_cast<int64_t>(c) * CHUNK;
    const int64_t n = min(static_cast<int64_t>(CHUNK), a.shard - e0);
    for (int64_t i = threadIdx.x * 4; i < n; i += THREADS * 4) {
      float g[4] = {0.f, 0.f, 0.f, 0.f};
      const int w = (n - i) < 4 ? static_cast<int>(n - i) : 4;
      for (int r = 0; r < a.nranks; ++r) {
        const float* row = base + static_cast<int64_t>(r) * a.shard_padded + e0 + i;
        if (w == 4) {
          const float4 t = __ldcg(reinterpret_cast<const float4*>(row));
          g[0] += t.x; g[1] += t.y; g[2] += t.z; g[3] += t.w;
        } else {
          for (int j = 0; j < w; ++j) g[j] += __ldcg(row + j);
        }
      }
      if (a.gout != nullptr) {                 // phase A of the two-phase form: reduced gradient out, no update
        for (int j = 0; j < w; ++j) a.gout[e0 + i + j] = g[j] * gscale;
        continue;
      }
      for (int j = 0; j < w; ++j) {
        const int64_t e = e0 + i + j;
        const float gj = g[j] * gscale;
        float p = a.master[e] * decay;
        const float mj = a.beta1 * a.m[e] + (1.f - a.beta1) * gj;
        const float vj = a.beta2 * a.v[e] + (1.f - a.beta2) * gj * gj;
        p += (mj / (sqrtf(vj) * inv_sqrt_bc2 + a.eps)) * step_size;
        a.master[e] = p;
        a.m[e] = mj;
        a.v[e] = vj;
        if (a.param != nullptr) a.param[e] = __float2bfloat16(p);
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

}  // namespace rsa
}  // namespace pd

PD_EXPORT int pd_rs_adamw_chunk() { return pd::rsa::CHUNK; }

// grad: fp32 [nranks * shard]; peer_recv[r] -> rank r's buffer [2][nranks][shard_padded] fp32; peer_cnt[r] -> rank r's
// int32 [ceil(shard / 8192)] counters (zeroed once); state: 2 local int32 (zeroed once).  shard_padded >= shard and a
// multiple of 4.  The grid is capped at 2 CTAs per SM; every rank must call with the same shapes.
// grad_out (last argument, may be null): when given, the reduced gradient (x grad_scale) of the owned slice is written
// there and nothing is updated - master / m / v / param_bf16 are not touched and may be null.
PD_EXPORT int pd_rs_adamw(const float* grad, int64_t shard, int64_t shard_padded, int rank, int nranks,
                          const unsigned long long* peer_recv, const unsigned long long* peer_cnt, float* master, float* m,
                          float* v, void* param_bf16, float lr, float beta1, float beta2, float eps, float coeff,
                          float beta1_pow, float beta2_pow, const float* grad_scale, const int* skip, int* state,
                          int wait_ms, int* status, cudaStream_t stream, float* grad_out) {
  using namespace pd;
  using namespace pd::rsa;
  if (shard <= 0 || shard_padded < shard || (shard_padded % 4) || nranks < 1 || nranks > MAX_RANKS) return kErrBadShape;
  Args a;
  a.grad = grad;
  for (int i = 0; i < MAX_RANKS; ++i) {
    a.recv[i] = reinterpret_cast<float*>(peer_recv[i < nranks ? i : 0]);
    a.cnt[i] = reinterpret_cast<int*>(peer_cnt[i < nranks ? i : 0]);
  }
  a.master = master; a.m = m; a.v = v; a.param = (bf16*)param_bf16;
  a.shard = shard; a.shard_padded = shard_padded; a.rank = rank; a.nranks = nranks;
  a.chunks = static_cast<int>((shard + CHUNK - 1) / CHUNK);
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.coeff = coeff; a.beta1_pow = beta1_pow; a.beta2_pow = beta2_pow;
  a.grad_scale = grad_scale; a.skip = skip; a.state = state; a.gout = grad_out;
  a.wait_ns = static_cast<unsigned long long>(wait_ms) * 1000000ull;
  a.status = status;
  const int64_t items = static_cast<int64_t>(a.chunks) * nranks;
  const int cap = sm_count() * 2;
  const int grid = static_cast<int>(items < cap ? items : cap);
  rs_adamw_kernel<<<grid, THREADS, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}
