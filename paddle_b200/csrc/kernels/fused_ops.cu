// Bandwidth-bound fused operators (one pass over HBM, 128-bit accesses, fp32 math):
//   rms_norm fwd/bwd (+residual add), layer_norm fwd/bwd, rotary embedding fwd/bwd, swiglu fwd/bwd,
//   softmax-cross-entropy fwd/bwd (hard labels, ignore_index, vocab-parallel partials),
//   embedding gather / scatter-add grad, add+cast helpers.
// Paddle counterparts: rms_norm (paddle/phi/kernels/gpu/rms_norm_kernel.cu:427),
// fused_rotary_position_embedding (paddle/phi/kernels/fusion/gpu/fused_rope_utils.h:236,346),
// swiglu (paddle/phi/kernels/gpu/swiglu_kernel.cu:26), cross_entropy_with_softmax
// (paddle/phi/kernels/gpu/cross_entropy_kernel.cu:833), c_softmax_with_cross_entropy
// (paddle/phi/kernels/gpu/c_softmax_with_cross_entropy_kernel.cu:55-132), embedding
// (paddle/phi/kernels/gpu/embedding_kernel.cu:25, embedding_grad_kernel.cu:44).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include <atomic>

#include "host_utils.h"
#include "pd_no_alloc.h"

namespace pd {
namespace ew {

typedef __nv_bfloat16 bf16;

struct __align__(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const bf16* p, float (&f)[8]) {
  bf16x8 r = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(r.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(bf16* p, const float (&f)[8]) {
  bf16x8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = r;
}
__device__ __forceinline__ void load8(const float* p, float (&f)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p);
  float4 b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void store8(float* p, const float (&f)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

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
// Block-wide sum; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : -FLT_MAX;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// ------------------------------------------------------------------------------------------ RMSNorm
// y = (x [+ residual]) * rsqrt(mean(.^2) + eps) * w ; optionally writes the pre-norm sum
// (residual_out) and inv_rms.  H % 8 == 0.  One CTA per row, row cached in registers (H <= 8192)
// or re-read from L2 beyond that.
constexpr int RN_THREADS = 256;
constexpr int RN_MAXIT = 4;

constexpr int RNW_THREADS = 128;   // small CTAs: four rows each, so CTA turnover does not idle half an SM
// Warp-per-row variant for H = 256 * NV: the row stays in registers as packed bf16 (NV 128-bit words per
// lane, all loads issued before the first use), the reduction is shuffle-only, no CTA barrier.  With a
// residual the bf16-rounded sum is what gets normalised (and stored when residual_out is given).
template <typename WT, int NV>
__global__ void __launch_bounds__(RNW_THREADS, (NV <= 16 ? 4 : 2)) rms_norm_fwd_warp_kernel(
    const bf16* __restrict__ x, const bf16* __restrict__ residual, const WT* __restrict__ w,
    bf16* __restrict__ y, bf16* __restrict__ residual_out, float* __restrict__ inv_rms, int64_t rows,
    float eps) {
  constexpr int H = NV * 256;
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (RNW_THREADS / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  uint4 cache[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) cache[k] = __ldg(xr + lane + 32 * k);
  if (residual != nullptr) {
    const uint4* rr = reinterpret_cast<const uint4*>(residual + row * H);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const uint4 rc = __ldg(rr + lane + 32 * k);
      __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&cache[k]);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&rc);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fa = __bfloat1622float2(a[j]), fb = __bfloat1622float2(b[j]);
        a[j] = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
      }
      if (residual_out != nullptr)
        reinterpret_cast<uint4*>(residual_out + row * H)[lane + 32 * k] = cache[k];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&cache[k]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(a[j]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / static_cast<float>(H) + eps);
  if (lane == 0 && inv_rms != nullptr) inv_rms[row] = r;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    float xv[8], wv[8], o[8];
    const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&cache[k]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(a[j]);
      xv[2 * j] = f.x;
      xv[2 * j + 1] = f.y;
    }
    load8(w + (lane + 32 * k) * 8, wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = xv[j] * r * wv[j];
    store8(y + row * H + (lane + 32 * k) * 8, o);
  }
}

template <typename WT>
__global__ void __launch_bounds__(RN_THREADS) rms_norm_fwd_kernel(
    const bf16* __restrict__ x, const bf16* __restrict__ residual, const WT* __restrict__ w,
    bf16* __restrict__ y, bf16* __restrict__ residual_out, float* __restrict__ inv_rms, int H,
    float eps) {
  __shared__ float red[33];
  const size_t row = blockIdx.x;
  const bf16* xr = x + row * H;
  const int nvec = H >> 3;
  float cache[RN_MAXIT][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < RN_MAXIT; ++it) {
    const int i = threadIdx.x + it * RN_THREADS;
    if (i < nvec) {
      load8(xr + i * 8, cache[it]);
      if (residual != nullptr) {
        float r[8];
        load8(residual + row * H + i * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) cache[it][j] += r[j];
        if (residual_out != nullptr) {
          // round the sum to bf16 first so that y is computed from exactly what is saved
          store8(residual_out + row * H + i * 8, cache[it]);
          load8(residual_out + row * H + i * 8, cache[it]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += cache[it][j] * cache[it][j];
    }
  }
  for (int i = threadIdx.x + RN_MAXIT * RN_THREADS; i < nvec; i += RN_THREADS) {
    float t[8];
    load8(xr + i * 8, t);
    if (residual != nullptr) {
      float r[8];
      load8(residual + row * H + i * 8, r);
#pragma unroll
      for (int j = 0; j < 8; ++j) t[j] += r[j];
      if (residual_out != nullptr) {
        store8(residual_out + row * H + i * 8, t);
        load8(residual_out + row * H + i * 8, t);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += t[j] * t[j];
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / static_cast<float>(H) + eps);
  if (threadIdx.x == 0 && inv_rms != nullptr) inv_rms[row] = r;
#pragma unroll
  for (int it = 0; it < RN_MAXIT; ++it) {
    const int i = threadIdx.x + it * RN_THREADS;
    if (i < nvec) {
      float wv[8], o[8];
      load8(w + i * 8, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = cache[it][j] * r * wv[j];
      store8(y + row * H + i * 8, o);
    }
  }
  for (int i = threadIdx.x + RN_MAXIT * RN_THREADS; i < nvec; i += RN_THREADS) {
    float t[8], wv[8], o[8];
    const bf16* src = (residual != nullptr && residual_out != nullptr) ? residual_out + row * H : xr;
    load8(src + i * 8, t);
    if (residual != nullptr && residual_out == nullptr) {
      float rr[8];
      load8(residual + row * H + i * 8, rr);
#pragma unroll
      for (int j = 0; j < 8; ++j) t[j] += rr[j];
    }
    load8(w + i * 8, wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = t[j] * r * wv[j];
    store8(y + row * H + i * 8, o);
  }
}

// dx = r * (g - x * r^2 * mean(g * x)),  g = dy * w ;  dw partial[blockIdx] += dy * x * r.
// Persistent over rows so that the dw partials stay in registers; H <= 8 * 256 * RN_MAXIT for the
// register path (larger H falls back to shared-memory-free re-reads with atomics on partials).
template <typename WT>
__global__ void __launch_bounds__(RN_THREADS) rms_norm_bwd_kernel(
    const bf16* __restrict__ dy, const bf16* __restrict__ x, const WT* __restrict__ w,
    const float* __restrict__ inv_rms, bf16* __restrict__ dx, const bf16* __restrict__ dx_add,
    float* __restrict__ dw_partial, int rows, int H) {
  __shared__ float red[33];
  const int nvec = H >> 3;
  float dwacc[RN_MAXIT][8];
#pragma unroll
  for (int it = 0; it < RN_MAXIT; ++it)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[it][j] = 0.f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t off = static_cast<size_t>(row) * H;
    const float r = inv_rms[row];
    float xs[RN_MAXIT][8], gs[RN_MAXIT][8];
    float dot = 0.f;
#pragma unroll
    for (int it = 0; it < RN_MAXIT; ++it) {
      const int i = threadIdx.x + it * RN_THREADS;
      if (i < nvec) {
        float wv[8];
        load8(x + off + i * 8, xs[it]);
        load8(dy + off + i * 8, gs[it]);
        load8(w + i * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dwacc[it][j] += gs[it][j] * xs[it][j] * r;
          gs[it][j] *= wv[j];
          dot += gs[it][j] * xs[it][j];
        }
      }
    }
    dot = block_sum(dot, red);
    const float c = dot * r * r / static_cast<float>(H);
#pragma unroll
    for (int it = 0; it < RN_MAXIT; ++it) {
      const int i = threadIdx.x + it * RN_THREADS;
      if (i < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r * (gs[it][j] - xs[it][j] * c);
        if (dx_add != nullptr) {
          float a[8];
          load8(dx_add + off + i * 8, a);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += a[j];
        }
        store8(dx + off + i * 8, o);
      }
    }
  }
#pragma unroll
  for (int it = 0; it < RN_MAXIT; ++it) {
    const int i = threadIdx.x + it * RN_THREADS;
    if (i < nvec) store8(dw_partial + static_cast<size_t>(blockIdx.x) * H + i * 8, dwacc[it]);
  }
}

// out[c] = sum_p partial[p, c]   (fp32), optionally accumulating into an existing fp32 buffer
__global__ void column_sum_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                  int parts, int H, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[static_cast<size_t>(p) * H + c];
  out[c] = accumulate ? out[c] + s : s;
}

// ------------------------------------------------------------------------------------------ LayerNorm
template <typename WT>
__global__ void __launch_bounds__(RN_THREADS) layer_norm_fwd_kernel(
    const bf16* __restrict__ x, const WT* __restrict__ w, const WT* __restrict__ b,
    bf16* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, int H,
    float eps) {
  __shared__ float red[33];
  const size_t row = blockIdx.x;
  const int nvec = H >> 3;
  float cache[RN_MAXIT][8];
  float s = 0.f;
#pragma unroll
  for (int it = 0; it < RN_MAXIT; ++it) {
    const int i = threadIdx.x + it * RN_THREADS;
    if (i < nvec) {
      load8(x + row * H + i * 8, cache[it]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += cache[it][j];
    }
  }
  const float mean = block_sum(s, red) / static_cast<float>(H);
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < RN_MAXIT; ++it) {
    const int i = threadIdx.x + it * RN_THREADS;
    if (i < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = cache[it][j] - mean;
        ss += d * d;
      }
    }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / static_cast<float>(H) + eps);
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
#pragma unroll
  for (int it = 0; it < RN_MAXIT; ++it) {
    const int i = threadIdx.x + it * RN_THREADS;
    if (i < nvec) {
      float wv[8], bv[8], o[8];
      load8(w + i * 8, wv);
      if (b != nullptr) load8(b + i * 8, bv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (cache[it][j] - mean) * rstd * wv[j] + (b ? bv[j] : 0.f);
      store8(y + row * H + i * 8, o);
    }
  }
}

template <typename WT>
__global__ void __launch_bounds__(RN_THREADS) layer_norm_bwd_kernel(
    const bf16* __restrict__ dy, const bf16* __restrict__ x, const WT* __restrict__ w,
    const float* __restrict__ mean, const float* __restrict__ rstd, bf16* __restrict__ dx,
    float* __restrict__ dw_partial, float* __restrict__ db_partial, int rows, int H) {
  __shared__ float red[33];
  const int nvec = H >> 3;
  float dwacc[RN_MAXIT][8], dbacc[RN_MAXIT][8];
#pragma unroll
  for (int it = 0; it < RN_MAXIT; ++it)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[it][j] = dbacc[it][j] = 0.f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t off = static_cast<size_t>(row) * H;
    const float mu = mean[row], r = rstd[row];
    float xh[RN_MAXIT][8], gs[RN_MAXIT][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int it = 0; it < RN_MAXIT; ++it) {
      const int i = threadIdx.x + it * RN_THREADS;
      if (i < nvec) {
        float wv[8];
        load8(x + off + i * 8, xh[it]);
        load8(dy + off + i * 8, gs[it]);
        load8(w + i * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[it][j] = (xh[it][j] - mu) * r;
          dwacc[it][j] += gs[it][j] * xh[it][j];
          dbacc[it][j] += gs[it][j];
          gs[it][j] *= wv[j];
          s1 += gs[it][j];
          s2 += gs[it][j] * xh[it][j];
        }
      }
    }
    s1 = block_sum(s1, red) / static_cast<float>(H);
    s2 = block_sum(s2, red) / static_cast<float>(H);
#pragma unroll
    for (int it = 0; it < RN_MAXIT; ++it) {
      const int i = threadIdx.x + it * RN_THREADS;
      if (i < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r * (gs[it][j] - s1 - xh[it][j] * s2);
        store8(dx + off + i * 8, o);
      }
    }
  }
#pragma unroll
  for (int it = 0; it < RN_MAXIT; ++it) {
    const int i = threadIdx.x + it * RN_THREADS;
    if (i < nvec) {
      store8(dw_partial + static_cast<size_t>(blockIdx.x) * H + i * 8, dwacc[it]);
      store8(db_partial + static_cast<size_t>(blockIdx.x) * H + i * 8, dbacc[it]);
    }
  }
}

// ------------------------------------------------------------------------------------------ RoPE
// x: [tokens, heads, D] bf16 (row stride given in elements so q/k may live inside a packed qkv
// buffer), cos/sin: [max_pos, D] fp32 with the pairing convention baked into the table.
// half_style = 1: pairs are (i, i + D/2) ("rotate half"); 0: pairs are (2i, 2i+1) ("every two").
// sin_sign = +1 forward, -1 backward.  pos = position_ids[token] if given else token % seq_len.
__global__ void rope_kernel(const bf16* __restrict__ x, bf16* __restrict__ out,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            const int64_t* __restrict__ position_ids, int tokens, int heads, int D,
                            int64_t token_stride, int64_t out_token_stride, int seq_len,
                            int half_style, float sin_sign) {
  const int vec_per_head = D >> 4;  // each thread handles 8 pairs = 16 elements
  const int64_t total = static_cast<int64_t>(tokens) * heads * vec_per_head;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(idx % vec_per_head);
    const int64_t th = idx / vec_per_head;
    const int h = static_cast<int>(th % heads);
    const int64_t tok = th / heads;
    const int64_t pos = position_ids ? position_ids[tok] : (tok % seq_len);
    const bf16* src = x + tok * token_stride + static_cast<int64_t>(h) * D;
    bf16* dst = out + tok * out_token_stride + static_cast<int64_t>(h) * D;
    const float* c = cos_t + pos * D;
    const float* s = sin_t + pos * D;
    if (half_style) {
      const int i0 = v * 8, i1 = i0 + (D >> 1);
      float a[8], b[8], ca[8], sa[8], cb[8], sb[8], oa[8], ob[8];
      load8(src + i0, a);
      load8(src + i1, b);
      load8(c + i0, ca); load8(s + i0, sa);
      load8(c + i1, cb); load8(s + i1, sb);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        oa[j] = a[j] * ca[j] - b[j] * sa[j] * sin_sign;
        ob[j] = b[j] * cb[j] + a[j] * sb[j] * sin_sign;
      }
      store8(dst + i0, oa);
      store8(dst + i1, ob);
    } else {
      const int i0 = v * 16;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float a[8], cc[8], sn[8], o[8];
        load8(src + i0 + hh * 8, a);
        load8(c + i0 + hh * 8, cc);
        load8(s + i0 + hh * 8, sn);
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          o[j] = a[j] * cc[j] - a[j + 1] * sn[j] * sin_sign;
          o[j + 1] = a[j + 1] * cc[j + 1] + a[j] * sn[j + 1] * sin_sign;
        }
        store8(dst + i0 + hh * 8, o);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ SwiGLU
// out[r, c] = silu(x[r, c]) * y[r, c];  x and y may be the two halves of one [rows, 2F] buffer
// (ld_in = 2F) or separate buffers (ld_in = F).
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ y,
                                  bf16* __restrict__ out, int64_t rows, int F, int64_t ld_in) {
  const int vpr = F >> 3;
  const int64_t total = rows * vpr;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = idx / vpr;
    const int c = static_cast<int>(idx % vpr) * 8;
    float a[8], b[8], o[8];
    load8(x + r * ld_in + c, a);
    load8(y + r * ld_in + c, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = a[j] / (1.f + __expf(-a[j])) * b[j];
    store8(out + r * F + c, o);
  }
}
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ y,
                                  const bf16* __restrict__ dout, bf16* __restrict__ dx,
                                  bf16* __restrict__ dy, int64_t rows, int F, int64_t ld_in) {
  const int vpr = F >> 3;
  const int64_t total = rows * vpr;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = idx / vpr;
    const int c = static_cast<int>(idx % vpr) * 8;
    float a[8], b[8], g[8], da[8], db[8];
    load8(x + r * ld_in + c, a);
    load8(y + r * ld_in + c, b);
    load8(dout + r * F + c, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-a[j]));
      const float silu = a[j] * sg;
      da[j] = g[j] * b[j] * (sg + silu * (1.f - sg));
      db[j] = g[j] * silu;
    }
    store8(dx + r * ld_in + c, da);
    store8(dy + r * ld_in + c, db);
  }
}

// ------------------------------------------------------------------------------------------ softmax CE
// Row-wise statistics over a (possibly vocab-sharded) logits row: max, sum exp(x - max), and the
// logit of the label if it falls in [vocab_start, vocab_start + V).  For the unsharded case the
// loss is written directly.  logits: [T, V] bf16 or fp32.
constexpr int CE_THREADS = 512;
template <typename T>
__global__ void __launch_bounds__(CE_THREADS) ce_stats_kernel(
    const T* __restrict__ logits, const int64_t* __restrict__ labels, float* __restrict__ row_max,
    float* __restrict__ row_sum, float* __restrict__ row_tgt, float* __restrict__ loss, int V,
    int64_t vocab_start, int64_t ignore_index) {
  __shared__ float red[33];
  const size_t row = blockIdx.x;
  const T* xr = logits + row * V;
  const int nvec = V >> 3;
  float m = -FLT_MAX, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float t[8];
    load8(xr + i * 8, t);
    float lm = t[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, t[j]);
    if (lm > m) {
      s *= __expf(m - lm);
      m = lm;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(t[j] - m);
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += CE_THREADS) {  // tail (V % 8)
    const float t = static_cast<float>(xr[i]);
    if (t > m) {
      s *= __expf(m - t);
      m = t;
    }
    s += __expf(t - m);
  }
  const float gm = block_max(m, red);
  s *= __expf(m - gm);
  const float gs = block_sum(s, red);
  if (threadIdx.x == 0) {
    const int64_t lab = labels[row];
    const int64_t local = lab - vocab_start;
    const bool in_range = (lab != ignore_index) && local >= 0 && local < V;
    const float tgt = in_range ? static_cast<float>(xr[local]) : 0.f;
    if (row_max) row_max[row] = gm;
    if (row_sum) row_sum[row] = gs;
    if (row_tgt) row_tgt[row] = tgt;
    if (loss) loss[row] = (lab == ignore_index) ? 0.f : (logf(gs) + gm - tgt);
  }
}
// dlogits[r, c] = (exp(x - lse[r]) - [c == label]) * dloss[r] * scale   (0 for ignored rows)
template <typename T>
__global__ void __launch_bounds__(CE_THREADS) ce_bwd_kernel(
    const T* __restrict__ logits, const int64_t* __restrict__ labels, const float* __restrict__ lse,
    const float* __restrict__ dloss, int dloss_is_scalar, T* __restrict__ dlogits, int V,
    int64_t vocab_start, int64_t ignore_index, float scale) {
  const size_t row = blockIdx.x;
  const T* xr = logits + row * V;
  T* dr = dlogits + row * V;
  const int64_t lab = labels[row];
  const float g = (lab == ignore_index) ? 0.f : dloss[dloss_is_scalar ? 0 : row] * scale;
  const float l = lse[row];
  const int64_t local = lab - vocab_start;
  const int nvec = V >> 3;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float t[8], o[8];
    load8(xr + i * 8, t);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p = __expf(t[j] - l);
      o[j] = (p - ((i * 8 + j) == local ? 1.f : 0.f)) * g;
    }
    store8(dr + i * 8, o);
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += CE_THREADS) {
    const float p = __expf(static_cast<float>(xr[i]) - l);
    dr[i] = static_cast<T>((p - (i == local ? 1.f : 0.f)) * g);
  }
}

// ------------------------------------------------------------------------------------------ embedding
// out[t, :] = table[ids[t] - vocab_start, :] (zero if outside [vocab_start, vocab_start + rows))
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ ids, const bf16* __restrict__ table,
                                     bf16* __restrict__ out, int64_t tokens, int H, int64_t rows,
                                     int64_t vocab_start) {
  const int vpr = H >> 3;
  const int64_t total = tokens * vpr;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = idx / vpr;
    const int c = static_cast<int>(idx % vpr) * 8;
    const int64_t id = ids[t] - vocab_start;
    bf16x8 v;
    if (id >= 0 && id < rows) {
      v = *reinterpret_cast<const bf16x8*>(table + id * H + c);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v.v[j] = __floats2bfloat162_rn(0.f, 0.f);
    }
    *reinterpret_cast<bf16x8*>(out + t * H + c) = v;
  }
}
// dtable[ids[t] - vocab_start, :] += dout[t, :]   (fp32 accumulation buffer, atomics)
__global__ void embedding_bwd_kernel(const int64_t* __restrict__ ids, const bf16* __restrict__ dout,
                                     float* __restrict__ dtable, int64_t tokens, int H, int64_t rows,
                                     int64_t vocab_start, int64_t padding_idx) {
  const int vpr = H >> 3;
  const int64_t total = tokens * vpr;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = idx / vpr;
    const int c = static_cast<int>(idx % vpr) * 8;
    const int64_t raw = ids[t];
    const int64_t id = raw - vocab_start;
    if (id < 0 || id >= rows || raw == padding_idx) continue;
    float g[8];
    load8(dout + t * H + c, g);
    float* dst = dtable + id * H + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, g[j]);
  }
}

// ------------------------------------------------------------------------------------------ misc
// acc(fp32) += src(bf16)   — main_grad accumulation (paddle/distributed/fleet/utils/mix_precision_utils.py:54-70)
__global__ void accumulate_bf16_into_f32_kernel(const bf16* __restrict__ src, float* __restrict__ acc,
                                                int64_t n) {
  const int64_t nvec = n >> 3;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float s[8], a[8];
    load8(src + i * 8, s);
    load8(acc + i * 8, a);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] += s[j];
    store8(acc + i * 8, a);
  }
  for (int64_t i = (nvec << 3) + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    acc[i] += __bfloat162float(src[i]);
}
// out(bf16) = a(bf16) + b(bf16)
__global__ void add_bf16_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b,
                                bf16* __restrict__ out, int64_t n) {
  const int64_t nvec = n >> 3;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float x[8], y[8];
    load8(a + i * 8, x);
    load8(b + i * 8, y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += y[j];
    store8(out + i * 8, x);
  }
  for (int64_t i = (nvec << 3) + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    out[i] = __float2bfloat16(__bfloat162float(a[i]) + __bfloat162float(b[i]));
}

inline int grid_for(int64_t work_items, int threads) {
  int64_t b = (work_items + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace ew
}  // namespace pd

using namespace pd;
using namespace pd::ew;

#define PD_CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda)

#ifdef PD_DEBUG_BOUNDS
#include "sm100_prims.cuh"
// First recorded violation of the debug-bounds build over all kernel files: {kind, x, y, block, thread, 0, 0, 0};
// kind 0 = none.  Reading clears the records.
PD_EXPORT int pd_debug_bounds_read(int* out8) {
  int first[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  pd::PdBoundsReaders& readers = pd::pd_bounds_readers();
  for (int k = 0; k < readers.n; ++k) {
    int rec[8];
    if (readers.fn[k](rec) != 0) return kErrCuda;
    if (first[0] == 0 && rec[0] != 0)
      for (int i = 0; i < 8; ++i) first[i] = rec[i];
  }
  for (int i = 0; i < 8; ++i) out8[i] = first[i];
  return kLaunchOk;
}
#endif

// w_is_f32: weight dtype (0 = bf16, 1 = fp32).  residual / residual_out / inv_rms may be null.
PD_EXPORT int pd_rms_norm_fwd(const void* x, const void* residual, const void* w, int w_is_f32, void* y,
                              void* residual_out, float* inv_rms, int64_t rows, int H, float eps,
                              cudaStream_t stream) {
  if (H % 8 != 0 || rows <= 0) return kErrBadShape;
  const bool al = aligned16(x) && aligned16(y) && aligned16(w) && (residual == nullptr || aligned16(residual)) &&
                  (residual_out == nullptr || aligned16(residual_out));
#define PD_RMS_WARP(NV)                                                                                  \
  if (al && H == (NV) * 256) {                                                                           \
    const unsigned blocks = static_cast<unsigned>((rows + RNW_THREADS / 32 - 1) / (RNW_THREADS / 32));   \
    if (w_is_f32)                                                                                        \
      rms_norm_fwd_warp_kernel<float, NV><<<blocks, RNW_THREADS, 0, stream>>>(                           \
          (const bf16*)x, (const bf16*)residual, (const float*)w, (bf16*)y, (bf16*)residual_out, inv_rms, \
          rows, eps);                                                                                    \
    else                                                                                                 \
      rms_norm_fwd_warp_kernel<bf16, NV><<<blocks, RNW_THREADS, 0, stream>>>(                            \
          (const bf16*)x, (const bf16*)residual, (const bf16*)w, (bf16*)y, (bf16*)residual_out, inv_rms,  \
          rows, eps);                                                                                    \
    return PD_CHECK_LAUNCH();                                                                            \
  }
  PD_RMS_WARP(8)
  PD_RMS_WARP(16)
  PD_RMS_WARP(20)
#undef PD_RMS_WARP
  if (w_is_f32)
    rms_norm_fwd_kernel<float><<<static_cast<unsigned>(rows), RN_THREADS, 0, stream>>>(
        (const bf16*)x, (const bf16*)residual, (const float*)w, (bf16*)y, (bf16*)residual_out, inv_rms, H, eps);
  else
    rms_norm_fwd_kernel<bf16><<<static_cast<unsigned>(rows), RN_THREADS, 0, stream>>>(
        (const bf16*)x, (const bf16*)residual, (const bf16*)w, (bf16*)y, (bf16*)residual_out, inv_rms, H, eps);
  return PD_CHECK_LAUNCH();
}

// Returns the number of partial rows the caller must provide in dw_partial ([parts, H] fp32).
PD_EXPORT int pd_rms_norm_bwd_parts(int64_t rows) {
  const int cap = sm_count() * 2;
  return rows < cap ? static_cast<int>(rows) : cap;
}
// dx_add (optional): extra gradient added into dx (the residual branch), dw: [H] fp32
PD_EXPORT int pd_rms_norm_bwd(const void* dy, const void* x, const void* w, int w_is_f32,
                              const float* inv_rms, void* dx, const void* dx_add, float* dw_partial,
                              float* dw, int dw_accumulate, int64_t rows, int H, cudaStream_t stream) {
  if (H % 8 != 0 || H > 8 * RN_THREADS * RN_MAXIT || rows <= 0) return kErrBadShape;
  const int parts = pd_rms_norm_bwd_parts(rows);
  if (w_is_f32)
    rms_norm_bwd_kernel<float><<<parts, RN_THREADS, 0, stream>>>(
        (const bf16*)dy, (const bf16*)x, (const float*)w, inv_rms, (bf16*)dx, (const bf16*)dx_add, dw_partial,
        static_cast<int>(rows), H);
  else
    rms_norm_bwd_kernel<bf16><<<parts, RN_THREADS, 0, stream>>>(
        (const bf16*)dy, (const bf16*)x, (const bf16*)w, inv_rms, (bf16*)dx, (const bf16*)dx_add, dw_partial,
        static_cast<int>(rows), H);
  column_sum_kernel<<<(H + 255) / 256, 256, 0, stream>>>(dw_partial, dw, parts, H, dw_accumulate);
  return PD_CHECK_LAUNCH();
}

PD_EXPORT int pd_layer_norm_fwd(const void* x, const void* w, const void* b, int w_is_f32, void* y,
                                float* mean, float* rstd, int64_t rows, int H, float eps,
                                cudaStream_t stream) {
  if (H % 8 != 0 || H > 8 * RN_THREADS * RN_MAXIT || rows <= 0) return kErrBadShape;
  if (w_is_f32)
    layer_norm_fwd_kernel<float><<<static_cast<unsigned>(rows), RN_THREADS, 0, stream>>>(
        (const bf16*)x, (const float*)w, (const float*)b, (bf16*)y, mean, rstd, H, eps);
  else
    layer_norm_fwd_kernel<bf16><<<static_cast<unsigned>(rows), RN_THREADS, 0, stream>>>(
        (const bf16*)x, (const bf16*)w, (const bf16*)b, (bf16*)y, mean, rstd, H, eps);
  return PD_CHECK_LAUNCH();
}
PD_EXPORT int pd_layer_norm_bwd(const void* dy, const void* x, const void* w, int w_is_f32,
                                const float* mean, const float* rstd, void* dx, float* dw_partial,
                                float* db_partial, float* dw, float* db, int64_t rows, int H,
                                cudaStream_t stream) {
  if (H % 8 != 0 || H > 8 * RN_THREADS * RN_MAXIT || rows <= 0) return kErrBadShape;
  const int parts = pd_rms_norm_bwd_parts(rows);
  if (w_is_f32)
    layer_norm_bwd_kernel<float><<<parts, RN_THREADS, 0, stream>>>(
        (const bf16*)dy, (const bf16*)x, (const float*)w, mean, rstd, (bf16*)dx, dw_partial, db_partial,
        static_cast<int>(rows), H);
  else
    layer_norm_bwd_kernel<bf16><<<parts, RN_THREADS, 0, stream>>>(
        (const bf16*)dy, (const bf16*)x, (const bf16*)w, mean, rstd, (bf16*)dx, dw_partial, db_partial,
        static_cast<int>(rows), H);
  column_sum_kernel<<<(H + 255) / 256, 256, 0, stream>>>(dw_partial, dw, parts, H, 0);
  column_sum_kernel<<<(H + 255) / 256, 256, 0, stream>>>(db_partial, db, parts, H, 0);
  return PD_CHECK_LAUNCH();
}

PD_EXPORT int pd_rope(const void* x, void* out, const float* cos_t, const float* sin_t,
                      const int64_t* position_ids, int64_t tokens, int heads, int D,
                      int64_t token_stride, int64_t out_token_stride, int seq_len, int half_style,
                      int backward, cudaStream_t stream) {
  if (D % 16 != 0 || tokens <= 0 || (token_stride % 8) || (out_token_stride % 8)) return kErrBadShape;
  const int64_t work = tokens * heads * (D >> 4);
  rope_kernel<<<grid_for(work, 256), 256, 0, stream>>>((const bf16*)x, (bf16*)out, cos_t, sin_t, position_ids,
                                                      static_cast<int>(tokens), heads, D, token_stride,
                                                      out_token_stride, seq_len, half_style,
                                                      backward ? -1.f : 1.f);
  return PD_CHECK_LAUNCH();
}

PD_EXPORT int pd_swiglu_fwd(const void* x, const void* y, void* out, int64_t rows, int F, int64_t ld_in,
                            cudaStream_t stream) {
  if (F % 8 != 0 || ld_in % 8 != 0 || rows <= 0) return kErrBadShape;
  swiglu_fwd_kernel<<<grid_for(rows * (F >> 3), 256), 256, 0, stream>>>((const bf16*)x, (const bf16*)y,
                                                                       (bf16*)out, rows, F, ld_in);
  return PD_CHECK_LAUNCH();
}
PD_EXPORT int pd_swiglu_bwd(const void* x, const void* y, const void* dout, void* dx, void* dy,
                            int64_t rows, int F, int64_t ld_in, cudaStream_t stream) {
  if (F % 8 != 0 || ld_in % 8 != 0 || rows <= 0) return kErrBadShape;
  swiglu_bwd_kernel<<<grid_for(rows * (F >> 3), 256), 256, 0, stream>>>(
      (const bf16*)x, (const bf16*)y, (const bf16*)dout, (bf16*)dx, (bf16*)dy, rows, F, ld_in);
  return PD_CHECK_LAUNCH();
}

// is_f32: logits dtype (0 = bf16, 1 = fp32).  Any of row_max/row_sum/row_tgt/loss may be null.
PD_EXPORT int pd_ce_stats(const void* logits, int is_f32, const int64_t* labels, float* row_max,
                          float* row_sum, float* row_tgt, float* loss, int64_t rows, int V,
                          int64_t vocab_start, int64_t ignore_index, cudaStream_t stream) {
  if (rows <= 0 || V <= 0) return kErrBadShape;
  if ((is_f32 ? (V % 4) : (V % 8)) != 0) return kErrAlignment;  // rows must stay 16-byte aligned
  if (is_f32)
    ce_stats_kernel<float><<<static_cast<unsigned>(rows), CE_THREADS, 0, stream>>>(
        (const float*)logits, labels, row_max, row_sum, row_tgt, loss, V, vocab_start, ignore_index);
  else
    ce_stats_kernel<bf16><<<static_cast<unsigned>(rows), CE_THREADS, 0, stream>>>(
        (const bf16*)logits, labels, row_max, row_sum, row_tgt, loss, V, vocab_start, ignore_index);
  return PD_CHECK_LAUNCH();
}
PD_EXPORT int pd_ce_bwd(const void* logits, int is_f32, const int64_t* labels, const float* lse,
                        const float* dloss, int dloss_is_scalar, void* dlogits, int64_t rows, int V,
                        int64_t vocab_start, int64_t ignore_index, float scale, cudaStream_t stream) {
  if (rows <= 0 || V <= 0) return kErrBadShape;
  if ((is_f32 ? (V % 4) : (V % 8)) != 0) return kErrAlignment;
  if (is_f32)
    ce_bwd_kernel<float><<<static_cast<unsigned>(rows), CE_THREADS, 0, stream>>>(
        (const float*)logits, labels, lse, dloss, dloss_is_scalar, (float*)dlogits, V, vocab_start,
        ignore_index, scale);
  else
    ce_bwd_kernel<bf16><<<static_cast<unsigned>(rows), CE_THREADS, 0, stream>>>(
        (const bf16*)logits, labels, lse, dloss, dloss_is_scalar, (bf16*)dlogits, V, vocab_start,
        ignore_index, scale);
  return PD_CHECK_LAUNCH();
}

PD_EXPORT int pd_embedding_fwd(const int64_t* ids, const void* table, void* out, int64_t tokens, int H,
                               int64_t rows, int64_t vocab_start, cudaStream_t stream) {
  if (H % 8 != 0 || tokens <= 0) return kErrBadShape;
  embedding_fwd_kernel<<<grid_for(tokens * (H >> 3), 256), 256, 0, stream>>>(
      ids, (const bf16*)table, (bf16*)out, tokens, H, rows, vocab_start);
  return PD_CHECK_LAUNCH();
}
PD_EXPORT int pd_embedding_bwd(const int64_t* ids, const void* dout, float* dtable, int64_t tokens, int H,
                               int64_t rows, int64_t vocab_start, int64_t padding_idx,
                               cudaStream_t stream) {
  if (H % 8 != 0 || tokens <= 0) return kErrBadShape;
  embedding_bwd_kernel<<<grid_for(tokens * (H >> 3), 256), 256, 0, stream>>>(
      ids, (const bf16*)dout, dtable, tokens, H, rows, vocab_start, padding_idx);
  return PD_CHECK_LAUNCH();
}

PD_EXPORT int pd_accumulate_bf16_into_f32(const void* src, float* acc, int64_t n, cudaStream_t stream) {
  if (n <= 0) return kErrBadShape;
  if (!aligned16(src) || !aligned16(acc)) return kErrAlignment;
  accumulate_bf16_into_f32_kernel<<<grid_for((n + 7) >> 3, 256), 256, 0, stream>>>((const bf16*)src, acc, n);
  return PD_CHECK_LAUNCH();
}
PD_EXPORT int pd_add_bf16(const void* a, const void* b, void* out, int64_t n, cudaStream_t stream) {
  if (n <= 0) return kErrBadShape;
  if (!aligned16(a) || !aligned16(b) || !aligned16(out)) return kErrAlignment;
  add_bf16_kernel<<<grid_for((n + 7) >> 3, 256), 256, 0, stream>>>((const bf16*)a, (const bf16*)b, (bf16*)out, n);
  return PD_CHECK_LAUNCH();
}

// ------------------------------------------------------------------------------------------ allocation-free entry
// RMSNorm backward for callers that must not allocate device memory (see pd_no_alloc.h).  The per-CTA
// partial sums of the weight gradient, which pd_rms_norm_bwd takes from the caller, live in a fixed array
// inside this library instead.
namespace pd {
namespace ew {
constexpr int NA_MAX_PARTS = 128;
constexpr int NA_MAX_H = 8192;
static __device__ __align__(256) float g_rms_bwd_scratch[NA_MAX_PARTS * NA_MAX_H];   // 4 MiB per GPU
}  // namespace ew
}  // namespace pd

PD_EXPORT int pd_rms_norm_bwd_static(const void* dy, const void* x, const void* w, int w_is_f32,
                                     const float* inv_rms, void* dx, const void* dx_add, float* dw,
                                     int dw_accumulate, int64_t rows, int H, cudaStream_t stream) {
  if (H % 8 != 0 || rows <= 0) return kErrBadShape;
  if (H > NA_MAX_H || H > 8 * RN_THREADS * RN_MAXIT) return kErrTooLarge;
  if (rows > 2147483647ll) return kErrTooLarge;      // the kernels index rows with 32-bit integers
  // The array's name is only a host-side handle: the device address is looked up once per device, with that
  // device current, and passed to the kernels.  The per-device cache is atomic: host threads that make their first
  // call on a device at the same time each look the address up and store the same value.
  static std::atomic<float*> scratch_of_device[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kErrCuda;
  float* partial = scratch_of_device[dev].load(std::memory_order_acquire);
  if (partial == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rms_bwd_scratch) != cudaSuccess || p == nullptr)
      return kErrCuda;
    scratch_of_device[dev].store(p, std::memory_order_release);
    partial = p;
  }
  const int parts = rows < NA_MAX_PARTS ? static_cast<int>(rows) : NA_MAX_PARTS;
  if (w_is_f32)
    rms_norm_bwd_kernel<float><<<parts, RN_THREADS, 0, stream>>>(
        (const bf16*)dy, (const bf16*)x, (const float*)w, inv_rms, (bf16*)dx, (const bf16*)dx_add, partial,
        static_cast<int>(rows), H);
  else
    rms_norm_bwd_kernel<bf16><<<parts, RN_THREADS, 0, stream>>>(
        (const bf16*)dy, (const bf16*)x, (const bf16*)w, inv_rms, (bf16*)dx, (const bf16*)dx_add, partial,
        static_cast<int>(rows), H);
  column_sum_kernel<<<(H + 255) / 256, 256, 0, stream>>>(partial, dw, parts, H, dw_accumulate);
  return PD_CHECK_LAUNCH();
}
