// Token sampling for the decode loop, one CTA per sequence, no sort:
//   pd_sample_top_p_top_k : softmax(logits / temperature) restricted to the k most likely tokens and to the smallest set
//                           whose probability mass reaches p (nucleus), renormalised, one token drawn from it.
// The reference sorts the whole vocabulary per row (top_p_sampling: python/paddle/tensor/search.py, kernel
// paddle/phi/kernels/gpu/top_p_sampling_kernel.cu).  Here the row lives in shared memory as fp32 and the cut is found by
// bisection on the probability VALUE: for a threshold t, count(prob >= t) and mass(prob >= t) are one pass each, both are
// monotone in t, so ~30 passes over shared memory find the largest t whose kept set still satisfies both limits - the
// same set a sort would give (ties at the cut are all kept).  The draw walks the kept tokens in index order with a
// block-wide prefix sum.  Randomness: Philox4x32-10 at (seed, subsequence = row, offset).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <curand_kernel.h>
#include <float.h>
#include <stdint.h>

#include "host_utils.h"

namespace pd {
namespace smp {

constexpr int THREADS = 512;
constexpr int WARPS = THREADS / 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// block-wide reductions through `red` (WARPS floats + 1); every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x < WARPS) ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
    t = warp_sum(t);
    if (threadIdx.x == 0) red[WARPS] = t;
  }
  __syncthreads();
  return red[WARPS];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x < WARPS) ? red[threadIdx.x] : -FLT_MAX;
  if (threadIdx.x < 32) {
    t = warp_max(t);
    if (threadIdx.x == 0) red[WARPS] = t;
  }
  __syncthreads();
  return red[WARPS];
}

template <typename T>
__global__ void __launch_bounds__(THREADS) sample_kernel(const T* __restrict__ logits, int64_t ld, int V,
                                                         const float* __restrict__ top_p, int top_k, float inv_temp,
                                                         int input_is_prob, unsigned long long seed,
                                                         unsigned long long offset,
                                                         const long long* __restrict__ draw_counter,
                                                         long long* __restrict__ out_id, float* __restrict__ out_prob) {
  extern __shared__ float prob[];           // V probabilities
  __shared__ float red[WARPS + 2];
  __shared__ float warp_tot[WARPS];
  __shared__ int pick;
  const int row = blockIdx.x;
  const T* x = logits + static_cast<int64_t>(row) * ld;
  // ---- probabilities
  float mx = -FLT_MAX;
  for (int i = threadIdx.x; i < V; i += THREADS) {
    const float v = static_cast<float>(x[i]) * (input_is_prob ? 1.f : inv_temp);
    prob[i] = v;
    mx = fmaxf(mx, v);
  }
  mx = block_max(mx, red);
  float sum = 0.f;
  if (!input_is_prob) {
    for (int i = threadIdx.x; i < V; i += THREADS) {
      const float e = __expf(prob[i] - mx);
      prob[i] = e;
      sum += e;
    }
    sum = block_sum(sum, red);
    const float inv = 1.f / sum;
    for (int i = threadIdx.x; i < V; i += THREADS) prob[i] *= inv;
    mx = inv;                                 // the largest probability: exp(0) / sum
    __syncthreads();
  }
  // ---- the cut: largest t with count(prob >= t) <= k' and the set still reaching mass p ... found as the largest t
  // such that mass(prob >= t) >= p_eff and count(prob >= t) >= 1, then tightened by the top-k count
  const float p_lim = fminf(fmaxf(top_p != nullptr ? top_p[row] : 1.f, 0.f), 1.f);
  float lo = 0.f, hi = mx;                    // invariant: set(lo) satisfies "mass >= p_lim"; set(hi) is the arg-max only
  // nucleus: smallest set (= largest threshold) whose mass reaches p_lim
  for (int it = 0; it < 30; ++it) {
    const float mid = 0.5f * (lo + hi);
    float m = 0.f;
    for (int i = threadIdx.x; i < V; i += THREADS) m += prob[i] >= mid ? prob[i] : 0.f;
    m = block_sum(m, red);
    if (m >= p_lim) lo = mid; else hi = mid;
  }
  float thr = lo;
  if (top_k > 0 && top_k < V) {
    // top-k: smallest threshold whose set has at most k members; the final cut is the tighter of the two
    float klo = 0.f, khi = mx;                // count(klo) may exceed k, count(khi) >= 1
    for (int it = 0; it < 30; ++it) {
      const float mid = 0.5f * (klo + khi);
      float c = 0.f;
      for (int i = threadIdx.x; i < V; i += THREADS) c += prob[i] >= mid ? 1.f : 0.f;
      c = block_sum(c, red);
      if (c > static_cast<float>(top_k)) klo = mid; else khi = mid;
    }
    thr = fmaxf(thr, khi);
  }
  thr = fminf(thr, mx);                       // the most likely token always stays
  // ---- draw: u * mass(kept), then the first index whose running kept mass passes it
  float kept = 0.f;
  for (int i = threadIdx.x; i < V; i += THREADS) kept += prob[i] >= thr ? prob[i] : 0.f;
  kept = block_sum(kept, red);
  curandStatePhilox4_32_10_t st;
  // a device-resident draw counter lets a captured launch (CUDA graph) draw fresh numbers at every replay
  if (draw_counter != nullptr) offset += static_cast<unsigned long long>(*draw_counter) * 4ull;
  curand_init(seed, static_cast<unsigned long long>(row), offset, &st);
  const float target = curand_uniform(&st) * kept;      // (0, kept]
  if (threadIdx.x == 0) pick = -1;
  // contiguous chunks per thread so that "first index" is well defined: thread t owns [t * per, (t + 1) * per)
  const int per = (V + THREADS - 1) / THREADS;
  const int b0 = threadIdx.x * per, b1 = min(V, b0 + per);
  float mine = 0.f;
  for (int i = b0; i < b1; ++i) mine += prob[i] >= thr ? prob[i] : 0.f;
  // exclusive prefix over threads: warp scan + scan of the warp totals
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, incl, o);
    if ((threadIdx.x & 31) >= o) incl += n;
  }
  if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = incl;
  __syncthreads();
  float before = 0.f;
  for (int w = 0; w < (threadIdx.x >> 5); ++w) before += warp_tot[w];
  const float excl = before + incl - mine;
  if (target > excl && target <= excl + mine) {
    float run = excl;
    int chosen = -1;
    for (int i = b0; i < b1; ++i) {
      if (prob[i] >= thr) {
        run += prob[i];
        chosen = i;
        if (run >= target) break;
      }
    }
    if (chosen >= 0) atomicMax(&pick, chosen);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int id = pick;
    if (id < 0) {                              // rounding left the target past the last kept token: take that token
      for (int i = V - 1; i >= 0 && id < 0; --i)
        if (prob[i] >= thr) id = i;
      if (id < 0) id = 0;
    }
    out_id[row] = id;
    if (out_prob != nullptr) out_prob[row] = prob[id];
  }
}

}  // namespace smp
}  // namespace pd

// logits: [rows, V] (row stride ld elements) bf16 (is_f32 = 0) or fp32; input_is_prob = 1 when they already are
// probabilities.  top_p: fp32 [rows] or null (= 1); top_k <= 0: no count limit.  out_id: int64 [rows]; out_prob: fp32
// [rows] or null (probability of the drawn token before renormalisation).  V * 4 bytes must fit in shared memory.
// draw_counter: optional device int64; the Philox offset used is offset + 4 * (*draw_counter).
PD_EXPORT int pd_sample_top_p_top_k(const void* logits, int is_f32, int64_t rows, int64_t ld, int V, const float* top_p,
                                    int top_k, float temperature, int input_is_prob, unsigned long long seed,
                                    unsigned long long offset, long long* out_id, float* out_prob, cudaStream_t stream,
                                    const long long* draw_counter) {
  using namespace pd;
  using namespace pd::smp;
  if (rows <= 0 || V <= 0 || temperature <= 0.f) return kErrBadShape;
  const size_t smem = static_cast<size_t>(V) * sizeof(float);
  if (smem > 200 * 1024) return kErrTooLarge;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(sample_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(sample_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=
            cudaSuccess)
      return kErrCuda;
    configured = true;
  }
  if (is_f32)
    sample_kernel<float><<<static_cast<unsigned>(rows), THREADS, smem, stream>>>(
        static_cast<const float*>(logits), ld, V, top_p, top_k, 1.f / temperature, input_is_prob, seed, offset, draw_counter, out_id,
        out_prob);
  else
    sample_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), THREADS, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(logits), ld, V, top_p, top_k, 1.f / temperature, input_is_prob, seed, offset, draw_counter,
        out_id, out_prob);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}
