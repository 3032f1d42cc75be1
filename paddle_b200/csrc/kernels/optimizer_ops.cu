// Multi-tensor optimizer kernels: one launch updates every tensor of a parameter group.
// The tensor list lives in a device-resident table that the Python side builds once (parameter
// sets are static), so there is no per-step host marshalling and no kernel-argument size limit.
//
//   adamw          : Paddle's AdamW update (paddle/phi/kernels/gpu/adamw_kernel.cu:62-93) on fp32
//                    master weights, with gradient unscale / clip coefficient read from a device
//                    scalar, a device-side skip flag (found_inf), and the bf16 parameter refreshed
//                    in the same pass.
//   sq_l2_norm     : sum of squares over the whole list (squared_l2_norm per tensor in the
//                    reference, paddle/phi/kernels/gpu/squared_l2_norm_kernel.cu), two-stage and
//                    deterministic.
//   check_finite_and_unscale : paddle/phi/kernels/gpu/amp_kernel.cu:28
//   sgd / momentum : simple variants for the remaining optimizers.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_utils.h"

namespace pd {
namespace opt {

typedef __nv_bfloat16 bf16;
constexpr int CHUNK = 4096;     // elements per CTA-iteration
constexpr int THREADS = 256;

// Device table layout (int64 words):
//   [0] num_tensors  [1] total_chunks
//   then per tensor t (stride 8): numel, chunk_prefix, ptr_param, ptr_grad, ptr_master, ptr_m, ptr_v, flags
//   flags bit0: param is bf16 (else fp32), bit1: grad is bf16 (else fp32), bit2: has master
struct TensorRec {
  int64_t numel, chunk_prefix;
  void *param, *grad;
  float *master, *m, *v;
  int64_t flags;
};

__device__ __forceinline__ int find_tensor(const TensorRec* recs, int n, int64_t chunk) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (recs[mid].chunk_prefix <= chunk) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// 4-element accessors: fp32 as one 128-bit access, bf16 as one 64-bit access.
__device__ __forceinline__ float4 load4(const void* base, bool is_bf16, int64_t e) {
  if (is_bf16) {
    const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const bf16*>(base) + e);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
  }
  return *reinterpret_cast<const float4*>(static_cast<const float*>(base) + e);
}
__device__ __forceinline__ void store4(void* base, bool is_bf16, int64_t e, float4 x) {
  if (is_bf16) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo);
    raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(static_cast<bf16*>(base) + e) = raw;
  } else {
    *reinterpret_cast<float4*>(static_cast<float*>(base) + e) = x;
  }
}
// A chunk may take the vector path when it lies wholly inside its tensor and every pointer the kernel
// touches is 16-byte aligned (chunk offsets are multiples of 4096 elements, so only the bases matter).
__device__ __forceinline__ bool vec_ok(const TensorRec& r, int64_t base, bool need_state) {
  uintptr_t bits = reinterpret_cast<uintptr_t>(r.param) | reinterpret_cast<uintptr_t>(r.grad);
  if (need_state)
    bits |= reinterpret_cast<uintptr_t>(r.master) | reinterpret_cast<uintptr_t>(r.m) |
            reinterpret_cast<uintptr_t>(r.v);
  return (bits & 15u) == 0 && base + CHUNK <= r.numel;
}

struct AdamWArgs {
  float lr, beta1, beta2, eps, coeff, beta1_pow, beta2_pow;
  const float* grad_scale;  // optional device scalar multiplied into every gradient
  const int* skip;          // optional device flag: nonzero => leave everything untouched
  const float* lr_ratio;    // unused slot kept for layer-wise lr decay tables (may be null)
};

__global__ void __launch_bounds__(THREADS) adamw_multi_kernel(const int64_t* __restrict__ table,
                                                              AdamWArgs a) {
  if (a.skip != nullptr && *a.skip != 0) return;
  const int n = static_cast<int>(table[0]);
  const int64_t total_chunks = table[1];
  const TensorRec* recs = reinterpret_cast<const TensorRec*>(table + 2);
  const float gscale = a.grad_scale ? *a.grad_scale : 1.f;
  const float bc1 = 1.f - a.beta1_pow;
  const float inv_sqrt_bc2 = rsqrtf(1.f - a.beta2_pow);
  const float step_size = -(a.lr / bc1);
  const float decay = 1.f - a.lr * a.coeff;
  for (int64_t chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    const TensorRec r = recs[find_tensor(recs, n, chunk)];
    const int64_t base = (chunk - r.chunk_prefix) * CHUNK;
    const bool p_bf16 = r.flags & 1, g_bf16 = r.flags & 2, has_master = r.flags & 4;
    if (vec_ok(r, base, true)) {
      constexpr int IT = CHUNK / (THREADS * 4);
      float4 g4[IT], p4[IT], m4[IT], v4[IT];
#pragma unroll
      for (int it = 0; it < IT; ++it) {   // all loads first: 4 independent 128-bit streams per thread
        const int64_t e = base + (it * THREADS + threadIdx.x) * 4;
        g4[it] = load4(r.grad, g_bf16, e);
        p4[it] = has_master ? *reinterpret_cast<const float4*>(r.master + e) : load4(r.param, p_bf16, e);
        m4[it] = *reinterpret_cast<const float4*>(r.m + e);
        v4[it] = *reinterpret_cast<const float4*>(r.v + e);
      }
#pragma unroll
      for (int it = 0; it < IT; ++it) {
        const int64_t e = base + (it * THREADS + threadIdx.x) * 4;
        float* g = reinterpret_cast<float*>(&g4[it]);
        float* p = reinterpret_cast<float*>(&p4[it]);
        float* m = reinterpret_cast<float*>(&m4[it]);
        float* v = reinterpret_cast<float*>(&v4[it]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float gj = g[j] * gscale;
          p[j] *= decay;
          m[j] = a.beta1 * m[j] + (1.f - a.beta1) * gj;
          v[j] = a.beta2 * v[j] + (1.f - a.beta2) * gj * gj;
          p[j] += (m[j] / (sqrtf(v[j]) * inv_sqrt_bc2 + a.eps)) * step_size;
        }
        *reinterpret_cast<float4*>(r.m + e) = m4[it];
        *reinterpret_cast<float4*>(r.v + e) = v4[it];
        if (has_master) *reinterpret_cast<float4*>(r.master + e) = p4[it];
        store4(r.param, p_bf16, e, p4[it]);
      }
      continue;
    }
#pragma unroll 4
    for (int i = threadIdx.x; i < CHUNK; i += THREADS) {
      const int64_t e = base + i;
      if (e >= r.numel) break;
      float g = g_bf16 ? __bfloat162float(static_cast<const bf16*>(r.grad)[e])
                       : static_cast<const float*>(r.grad)[e];
      g *= gscale;
      float p = has_master ? r.master[e]
                           : (p_bf16 ? __bfloat162float(static_cast<const bf16*>(r.param)[e])
                                     : static_cast<const float*>(r.param)[e]);
      float m = r.m[e], v = r.v[e];
      p *= decay;
      m = a.beta1 * m + (1.f - a.beta1) * g;
      v = a.beta2 * v + (1.f - a.beta2) * g * g;
      const float denom = sqrtf(v) * inv_sqrt_bc2 + a.eps;
      p += (m / denom) * step_size;
      r.m[e] = m;
      r.v[e] = v;
      if (has_master) r.master[e] = p;
      if (p_bf16) static_cast<bf16*>(r.param)[e] = __float2bfloat16(p);
      else static_cast<float*>(r.param)[e] = p;
    }
  }
}

// Flat-buffer AdamW (one contiguous slice: sharded optimizers, fused comm buffers). 128-bit accesses.
__global__ void __launch_bounds__(THREADS) adamw_flat_kernel(bf16* __restrict__ param_bf16,
                                                             float* __restrict__ master,
                                                             const float* __restrict__ grad,
                                                             float* __restrict__ m,
                                                             float* __restrict__ v, int64_t n,
                                                             AdamWArgs a) {
  if (a.skip != nullptr && *a.skip != 0) return;
  const float gscale = a.grad_scale ? *a.grad_scale : 1.f;
  const float bc1 = 1.f - a.beta1_pow;
  const float inv_sqrt_bc2 = rsqrtf(1.f - a.beta2_pow);
  const float step_size = -(a.lr / bc1);
  const float decay = 1.f - a.lr * a.coeff;
  const int64_t nvec = n >> 2;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(THREADS) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * THREADS) {
    float4 g4 = reinterpret_cast<const float4*>(grad)[i];
    float4 p4 = reinterpret_cast<float4*>(master)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float* g = reinterpret_cast<float*>(&g4);
    float* p = reinterpret_cast<float*>(&p4);
    float* mm = reinterpret_cast<float*>(&m4);
    float* vv = reinterpret_cast<float*>(&v4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = g[j] * gscale;
      p[j] *= decay;
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gj;
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gj * gj;
      p[j] += (mm[j] / (sqrtf(vv[j]) * inv_sqrt_bc2 + a.eps)) * step_size;
    }
    reinterpret_cast<float4*>(master)[i] = p4;
    reinterpret_cast<float4*>(m)[i] = m4;
    reinterpret_cast<float4*>(v)[i] = v4;
    if (param_bf16 != nullptr) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(p[0], p[1]);
      __nv_bfloat162 hi = __floats2bfloat162_rn(p[2], p[3]);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(param_bf16)[i] = o;
    }
  }
  for (int64_t e = (nvec << 2) + blockIdx.x * static_cast<int64_t>(THREADS) + threadIdx.x; e < n;
       e += static_cast<int64_t>(gridDim.x) * THREADS) {
    const float gj = grad[e] * gscale;
    float p = master[e] * decay;
    const float mj = a.beta1 * m[e] + (1.f - a.beta1) * gj;
    const float vj = a.beta2 * v[e] + (1.f - a.beta2) * gj * gj;
    p += (mj / (sqrtf(vj) * inv_sqrt_bc2 + a.eps)) * step_size;
    master[e] = p; m[e] = mj; v[e] = vj;
    if (param_bf16 != nullptr) param_bf16[e] = __float2bfloat16(p);
  }
}

// partial[blockIdx] = sum over this CTA's chunks of grad^2 (the list's grads; fp32 accumulate)
__global__ void __launch_bounds__(THREADS) sq_l2_norm_kernel(const int64_t* __restrict__ table,
                                                             float* __restrict__ partial) {
  __shared__ float red[THREADS / 32];
  const int n = static_cast<int>(table[0]);
  const int64_t total_chunks = table[1];
  const TensorRec* recs = reinterpret_cast<const TensorRec*>(table + 2);
  float acc = 0.f;
  for (int64_t chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    const TensorRec r = recs[find_tensor(recs, n, chunk)];
    const int64_t base = (chunk - r.chunk_prefix) * CHUNK;
    const bool g_bf16 = r.flags & 2;
    if ((reinterpret_cast<uintptr_t>(r.grad) & 15u) == 0 && base + CHUNK <= r.numel) {
      constexpr int IT = CHUNK / (THREADS * 4);
      float4 g4[IT];
#pragma unroll
      for (int it = 0; it < IT; ++it) g4[it] = load4(r.grad, g_bf16, base + (it * THREADS + threadIdx.x) * 4);
#pragma unroll
      for (int it = 0; it < IT; ++it)
        acc += g4[it].x * g4[it].x + g4[it].y * g4[it].y + g4[it].z * g4[it].z + g4[it].w * g4[it].w;
      continue;
    }
    for (int i = threadIdx.x; i < CHUNK; i += THREADS) {
      const int64_t e = base + i;
      if (e >= r.numel) break;
      const float g = g_bf16 ? __bfloat162float(static_cast<const bf16*>(r.grad)[e])
                             : static_cast<const float*>(r.grad)[e];
      acc += g * g;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < THREADS / 32; ++w) s += red[w];
    partial[blockIdx.x] = s;
  }
}
// out[0] (+)= sum(partial[0..n))  in a fixed order
__global__ void final_sum_kernel(const float* __restrict__ partial, int n, float* __restrict__ out,
                                 int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) t += red[w];
    out[0] = accumulate ? out[0] + t : t;
  }
}

// grads *= inv_scale ; found_inf |= any(!isfinite)
__global__ void __launch_bounds__(THREADS) unscale_check_kernel(const int64_t* __restrict__ table,
                                                                const float* __restrict__ inv_scale,
                                                                int* __restrict__ found_inf) {
  const int n = static_cast<int>(table[0]);
  const int64_t total_chunks = table[1];
  const TensorRec* recs = reinterpret_cast<const TensorRec*>(table + 2);
  const float s = *inv_scale;
  bool bad = false;
  for (int64_t chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    const TensorRec r = recs[find_tensor(recs, n, chunk)];
    const int64_t base = (chunk - r.chunk_prefix) * CHUNK;
    const bool g_bf16 = r.flags & 2;
    for (int i = threadIdx.x; i < CHUNK; i += THREADS) {
      const int64_t e = base + i;
      if (e >= r.numel) break;
      if (g_bf16) {
        bf16* gp = static_cast<bf16*>(r.grad);
        const float g = __bfloat162float(gp[e]) * s;
        bad |= !isfinite(g);
        gp[e] = __float2bfloat16(g);
      } else {
        float* gp = static_cast<float*>(r.grad);
        const float g = gp[e] * s;
        bad |= !isfinite(g);
        gp[e] = g;
      }
    }
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(found_inf, 1);
}

// momentum / sgd on the same table: v = mu*v + g (+wd*p); p -= lr*v (nesterov: p -= lr*(g + mu*v))
__global__ void __launch_bounds__(THREADS) momentum_multi_kernel(const int64_t* __restrict__ table,
                                                                 float lr, float mu, float wd,
                                                                 int nesterov, int use_momentum,
                                                                 const float* grad_scale) {
  const int n = static_cast<int>(table[0]);
  const int64_t total_chunks = table[1];
  const TensorRec* recs = reinterpret_cast<const TensorRec*>(table + 2);
  const float gscale = grad_scale ? *grad_scale : 1.f;
  for (int64_t chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    const TensorRec r = recs[find_tensor(recs, n, chunk)];
    const int64_t base = (chunk - r.chunk_prefix) * CHUNK;
    const bool p_bf16 = r.flags & 1, g_bf16 = r.flags & 2, has_master = r.flags & 4;
    for (int i = threadIdx.x; i < CHUNK; i += THREADS) {
      const int64_t e = base + i;
      if (e >= r.numel) break;
      float g = (g_bf16 ? __bfloat162float(static_cast<const bf16*>(r.grad)[e])
                        : static_cast<const float*>(r.grad)[e]) * gscale;
      float p = has_master ? r.master[e]
                           : (p_bf16 ? __bfloat162float(static_cast<const bf16*>(r.param)[e])
                                     : static_cast<const float*>(r.param)[e]);
      g += wd * p;
      if (use_momentum) {
        const float v = mu * r.m[e] + g;
        r.m[e] = v;
        p -= lr * (nesterov ? (g + mu * v) : v);
      } else {
        p -= lr * g;
      }
      if (has_master) r.master[e] = p;
      if (p_bf16) static_cast<bf16*>(r.param)[e] = __float2bfloat16(p);
      else static_cast<float*>(r.param)[e] = p;
    }
  }
}

inline int grid_for_chunks(int64_t chunks) {
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  int64_t g = chunks < cap ? chunks : cap;
  return static_cast<int>(g < 1 ? 1 : g);
}

}  // namespace opt
}  // namespace pd

using namespace pd;
using namespace pd::opt;

PD_EXPORT int pd_opt_chunk_size() { return CHUNK; }

PD_EXPORT int pd_adamw_multi(const int64_t* table, int64_t total_chunks, float lr, float beta1, float beta2,
                             float eps, float coeff, float beta1_pow, float beta2_pow,
                             const float* grad_scale, const int* skip, cudaStream_t stream) {
  if (total_chunks <= 0) return kLaunchOk;
  AdamWArgs a{lr, beta1, beta2, eps, coeff, beta1_pow, beta2_pow, grad_scale, skip, nullptr};
  adamw_multi_kernel<<<grid_for_chunks(total_chunks), THREADS, 0, stream>>>(table, a);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

// param_bf16 may be null (fp32-only parameters).  All fp32 buffers must be 16-byte aligned.
PD_EXPORT int pd_adamw_flat(void* param_bf16, float* master, const float* grad, float* m, float* v,
                            int64_t n, float lr, float beta1, float beta2, float eps, float coeff,
                            float beta1_pow, float beta2_pow, const float* grad_scale, const int* skip,
                            cudaStream_t stream) {
  if (n <= 0) return kLaunchOk;
  if (!aligned16(master) || !aligned16(grad) || !aligned16(m) || !aligned16(v) ||
      (param_bf16 && (reinterpret_cast<uintptr_t>(param_bf16) & 7u)))
    return kErrAlignment;
  AdamWArgs a{lr, beta1, beta2, eps, coeff, beta1_pow, beta2_pow, grad_scale, skip, nullptr};
  const int64_t blocks = ((n >> 2) + THREADS - 1) / THREADS;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  adamw_flat_kernel<<<static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks)), THREADS, 0, stream>>>(
      (bf16*)param_bf16, master, grad, m, v, n, a);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

// partial must hold pd_l2norm_parts(total_chunks) floats; out[0] (+)= sum of squares.
PD_EXPORT int pd_l2norm_parts(int64_t total_chunks) { return grid_for_chunks(total_chunks); }
PD_EXPORT int pd_sq_l2_norm_multi(const int64_t* table, int64_t total_chunks, float* partial, float* out,
                                  int accumulate, cudaStream_t stream) {
  if (total_chunks <= 0) return kLaunchOk;
  const int g = grid_for_chunks(total_chunks);
  sq_l2_norm_kernel<<<g, THREADS, 0, stream>>>(table, partial);
  final_sum_kernel<<<1, 256, 0, stream>>>(partial, g, out, accumulate);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

PD_EXPORT int pd_unscale_check_multi(const int64_t* table, int64_t total_chunks, const float* inv_scale,
                                     int* found_inf, cudaStream_t stream) {
  if (total_chunks <= 0) return kLaunchOk;
  unscale_check_kernel<<<grid_for_chunks(total_chunks), THREADS, 0, stream>>>(table, inv_scale, found_inf);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

PD_EXPORT int pd_momentum_multi(const int64_t* table, int64_t total_chunks, float lr, float mu, float wd,
                                int nesterov, int use_momentum, const float* grad_scale,
                                cudaStream_t stream) {
  if (total_chunks <= 0) return kLaunchOk;
  momentum_multi_kernel<<<grid_for_chunks(total_chunks), THREADS, 0, stream>>>(table, lr, mu, wd, nesterov,
                                                                              use_momentum, grad_scale);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}
