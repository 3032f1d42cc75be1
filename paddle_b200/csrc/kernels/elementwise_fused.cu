// Fused element-wise kernels of the transformer blocks that are bandwidth-bound: one read of every input, one write of
// the output, 16-byte accesses.
//   pd_dropout_add : out = dropout(x) [+ y] with a Philox4x32-10 stream addressed by (seed, offset), so the backward
//                    pass (and a recomputation) regenerates the same keep decisions instead of storing a mask
//                    (reference: paddle/phi/kernels/fusion/gpu/fused_dropout_add_kernel.cu:86-120 - curand_init(seed,
//                    thread index, increment) and four uniforms per draw; the stream here uses the same generator and
//                    the same addressing, with this file's launch geometry).
//   pd_bias_act    : out = act(x + bias), act in {identity, relu, gelu, gelu_tanh, silu, swiglu, geglu}; the gated forms
//                    read 2F columns and write F (reference: paddle/phi/kernels/fusion/gpu/fused_bias_act_kernel.cu).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <curand_kernel.h>
#include <stdint.h>

#include "host_utils.h"

namespace pd {
namespace ew {

typedef __nv_bfloat16 bf16;
constexpr int THREADS = 256;
constexpr int MAX_BLOCKS_PER_SM = 8;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    f[2 * e] = __uint_as_float(w[e] << 16);
    f[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
}

// Thread t owns Philox subsequence t; per step it draws 8 uniforms (two draws of four) for elements
// [8 * (t + step * threads_total), +8).  keep <=> uniform >= p  (curand_uniform is in (0, 1]).
template <typename T>
__global__ void __launch_bounds__(THREADS) dropout_add_kernel(const T* __restrict__ x, const T* __restrict__ y,
                                                              T* __restrict__ out, int64_t n, float p, float keep_scale,
                                                              unsigned long long seed, unsigned long long offset) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x;
  const int64_t total = static_cast<int64_t>(gridDim.x) * THREADS;
  curandStatePhilox4_32_10_t st;
  curand_init(seed, static_cast<unsigned long long>(tid), offset, &st);
  for (int64_t i = tid * 8; i < n; i += total * 8) {
    const float4 r0 = curand_uniform4(&st), r1 = curand_uniform4(&st);
    const float r[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
    if (sizeof(T) == 2 && i + 8 <= n) {
      float xv[8], yv[8], o[8];
      unpack8(*reinterpret_cast<const uint4*>(x + i), xv);
      if (y != nullptr) unpack8(*reinterpret_cast<const uint4*>(y + i), yv);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (r[e] >= p ? xv[e] * keep_scale : 0.f) + (y != nullptr ? yv[e] : 0.f);
      *reinterpret_cast<uint4*>(out + i) = pack8(o);
    } else {
      for (int e = 0; e < 8 && i + e < n; ++e) {
        const float xv = static_cast<float>(x[i + e]);
        const float yv = y != nullptr ? static_cast<float>(y[i + e]) : 0.f;
        out[i + e] = static_cast<T>((r[e] >= p ? xv * keep_scale : 0.f) + yv);
      }
    }
  }
}

__device__ __forceinline__ float act_apply(float x, int act) {
  switch (act) {
    case 1: return fmaxf(x, 0.f);
    case 2: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case 3: return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    case 4: return x / (1.f + __expf(-x));
    default: return x;
  }
}

// act 0-4: out[r, c] = act(x[r, c] + bias[c]), cols = F.  act 5 (swiglu) / 6 (geglu): x is [rows, 2F] (gate | up halves),
// out[r, c] = silu|gelu(x[r, c] + bias[c]) * (x[r, F + c] + bias[F + c]).
__global__ void __launch_bounds__(THREADS) bias_act_kernel(const bf16* __restrict__ x, const bf16* __restrict__ bias,
                                                           bf16* __restrict__ out, int64_t rows, int F, int act) {
  const int vec_per_row = F >> 3;
  const int64_t work = rows * vec_per_row;
  const bool gated = act >= 5;
  const int in_cols = gated ? 2 * F : F;
  for (int64_t w = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x; w < work;
       w += static_cast<int64_t>(gridDim.x) * THREADS) {
    const int64_t r = w / vec_per_row;
    const int c = static_cast<int>(w - r * vec_per_row) << 3;
    float a[8], b[8], g[8], bg[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(x + r * in_cols + c), a);
    if (bias != nullptr) {
      unpack8(__ldg(reinterpret_cast<const uint4*>(bias + c)), b);
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] += b[e];
    }
    if (gated) {
      unpack8(*reinterpret_cast<const uint4*>(x + r * in_cols + F + c), g);
      if (bias != nullptr) {
        unpack8(__ldg(reinterpret_cast<const uint4*>(bias + F + c)), bg);
#pragma unroll
        for (int e = 0; e < 8; ++e) g[e] += bg[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = act_apply(a[e], act == 5 ? 4 : 2) * g[e];
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = act_apply(a[e], act);
    }
    *reinterpret_cast<uint4*>(out + r * F + c) = pack8(o);
  }
}

inline int blocks_for(int64_t work_items) {
  int64_t b = (work_items + THREADS - 1) / THREADS;
  const int64_t cap = static_cast<int64_t>(sm_count()) * MAX_BLOCKS_PER_SM;
  if (b > cap) b = cap;
  return static_cast<int>(b < 1 ? 1 : b);
}

}  // namespace ew
}  // namespace pd

// out = dropout(x) + y (y may be null).  is_f32: element type (0 = bf16).  p in [0, 1); upscale = 1 scales kept
// elements by 1 / (1 - p) ("upscale_in_train").  The launch geometry is a function of n alone, so the same
// (seed, offset, n) always reproduces the same keep decisions; one call consumes `pd_dropout_offset_step(n)` offsets.
PD_EXPORT int pd_dropout_add(const void* x, const void* y, void* out, int64_t n, int is_f32, float p, int upscale,
                             unsigned long long seed, unsigned long long offset, cudaStream_t stream) {
  using namespace pd;
  using namespace pd::ew;
  if (n <= 0 || p < 0.f || p >= 1.f) return kErrBadShape;
  if (!is_f32 && (!aligned16(x) || !aligned16(out) || (y != nullptr && !aligned16(y)))) return kErrAlignment;
  const float ks = upscale ? 1.f / (1.f - p) : 1.f;
  const int blocks = blocks_for((n + 7) / 8);
  if (is_f32)
    dropout_add_kernel<float><<<blocks, THREADS, 0, stream>>>((const float*)x, (const float*)y, (float*)out, n, p, ks, seed,
                                                             offset);
  else
    dropout_add_kernel<bf16><<<blocks, THREADS, 0, stream>>>((const bf16*)x, (const bf16*)y, (bf16*)out, n, p, ks, seed,
                                                           offset);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

// Philox offsets one pd_dropout_add call over n elements advances a thread's subsequence by (a multiple of four, as the
// reference's generator bookkeeping expects).
PD_EXPORT long long pd_dropout_offset_step(int64_t n) {
  using namespace pd::ew;
  const int64_t threads = static_cast<int64_t>(blocks_for((n + 7) / 8)) * THREADS;
  const int64_t steps = (n + threads * 8 - 1) / (threads * 8);
  return steps * 8;
}

// x: bf16 [rows, F] (act 0-4) or [rows, 2F] (act 5 swiglu, 6 geglu); bias: bf16 [F] / [2F] or null; out: bf16 [rows, F].
PD_EXPORT int pd_bias_act(const void* x, const void* bias, void* out, int64_t rows, int F, int act, cudaStream_t stream) {
  using namespace pd;
  using namespace pd::ew;
  if (rows <= 0 || F <= 0 || (F % 8) || act < 0 || act > 6) return kErrBadShape;
  if (!aligned16(x) || !aligned16(out) || (bias != nullptr && !aligned16(bias))) return kErrAlignment;
  bias_act_kernel<<<blocks_for(rows * (F >> 3)), THREADS, 0, stream>>>((const bf16*)x, (const bf16*)bias, (bf16*)out, rows,
                                                                       F, act);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}
