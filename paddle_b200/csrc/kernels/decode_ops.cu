// Inference (decode) kernels for sm_100a, head_dim 128, bf16, paged KV cache with 64-token pages:
//   pd_decode_qkv_prep     : bias + rotary embedding of q/k at each sequence's current position, append of the
//                            new k/v row into the cache page named by the block table, q written densely
//   pd_write_kv_cache      : prefill - copy [B, S, Hkv, 128] keys/values (strided views) into cache pages
//   pd_paged_decode_attn   : one query token per sequence against the paged cache (flash-decoding: optional
//                            split of the context over several CTAs + a merge pass)
//   pd_splitk_finalize     : fp32 split-K accumulator -> bf16 (+bias, +residual), accumulator re-zeroed
// Reference counterparts: masked_multihead_attention_kernel (bias + rope + cache append + attention,
// paddle/phi/kernels/fusion/gpu/masked_multihead_attention_kernel.cu), block_multihead_attention
// (paddle/phi/kernels/fusion/gpu/block_multi_head_attention_kernel.cu, block_attn.h), write_cache_kv in
// fused_multi_transformer_op.cu.h.
//
// The attention kernel is bandwidth-bound (each cached byte is used once per query head of its group), so it is
// built around the copy engine instead of tensor cores: a producer warp streams whole 16 KB K and V pages
// (contiguous per (block, kv head)) into a shared-memory ring with cp.async.bulk + mbarrier transaction counts;
// four consumer warps compute from shared memory, 8 lanes per token row (conflict-free 128-bit reads), online
// softmax per warp, merged across warps once per CTA.
#include <cuda_bf16.h>
#include <math.h>

#include "host_utils.h"
#include "sm100_prims.cuh"

namespace pd {
namespace dec {

typedef __nv_bfloat16 bf16;
constexpr int PAGE = 64, D = 128;
constexpr int PAGE_BYTES = PAGE * D * 2;   // 16 KB
constexpr int STAGES = 3;
constexpr int CWARPS = 4;
constexpr int THREADS = (CWARPS + 1) * 32;

struct AttnParams {
  const bf16* q;            // [B, Hq, 128]
  const bf16* k_cache;      // [num_blocks, Hkv, 64, 128]
  const bf16* v_cache;
  const int* block_table;   // [B, max_blocks]
  const int* seq_lens;      // [B]
  bf16* out;                // [B, Hq, 128]
  float* part_acc;          // [B, Hq, nsplit, 128]
  float* part_ml;           // [B, Hq, nsplit, 2]
  int B, Hq, Hkv, max_blocks, nsplit, len_offset;
  float scale_log2;
  int* status;
};

struct Bars {
  uint64_t full[STAGES], empty[STAGES];
  int abort_flag;
};

__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int site) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag, status, site) ? 1 : 0;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  if (ok) {
#pragma unroll 1
    for (int i = 0; i < 1024 && !mbar_try_wait(bar, parity); ++i) {
    }
  }
  return ok != 0;
}

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int G>
__global__ void __launch_bounds__(THREADS) paged_decode_attn_kernel(AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint8_t* sK = smem;
  uint8_t* sV = smem + STAGES * PAGE_BYTES;
  float* sMerge = reinterpret_cast<float*>(sV + STAGES * PAGE_BYTES);     // [CWARPS][G][130]
  Bars* bars = reinterpret_cast<Bars*>(sMerge + CWARPS * G * 130);
  volatile int* abort_flag = &bars->abort_flag;

  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq_len = p.seq_lens[b] + p.len_offset;
  const int pages = (seq_len + PAGE - 1) / PAGE;
  const int per = (pages + p.nsplit - 1) / p.nsplit;
  const int p0 = split * per, p1 = min(pages, p0 + per);
  const int npages = max(0, p1 - p0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], CWARPS);
    }
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();

  if (warp == CWARPS) {
    // ------------------------------------------------------------ producer: whole pages through the copy engine
    if (lane == 0) {
      const int* bt = p.block_table + static_cast<size_t>(b) * p.max_blocks;
      int armed = 0;
      bool ok = true;
      for (int i = 0; i < npages && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_flag, p.status, 100 + s)) { ok = false; break; }
        const size_t page = (static_cast<size_t>(bt[p0 + i]) * p.Hkv + h) * (PAGE * D);
        mbar_expect_tx(&bars->full[s], 2 * PAGE_BYTES);
        bulk_load(sK + s * PAGE_BYTES, p.k_cache + page, PAGE_BYTES, &bars->full[s]);
        bulk_load(sV + s * PAGE_BYTES, p.v_cache + page, PAGE_BYTES, &bars->full[s]);
        armed = i + 1;
      }
      if (!ok || *abort_flag) {     // copies in flight must land before the CTA may exit
        for (int i = max(0, armed - STAGES); i < armed; ++i) mbar_drain(&bars->full[i % STAGES], (i / STAGES) & 1);
      }
    }
    __syncwarp();
    return;
  }

  // -------------------------------------------------------------- consumers
  const int quarter = lane >> 3, sub = lane & 7;
  float qf[G][16];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const bf16* qp = p.q + (static_cast<size_t>(b) * p.Hq + h * G + g) * D;
    float t[8];
    unpack8(*reinterpret_cast<const uint4*>(qp + sub * 8), t);
#pragma unroll
    for (int i = 0; i < 8; ++i) qf[g][i] = t[i] * p.scale_log2;
    unpack8(*reinterpret_cast<const uint4*>(qp + 64 + sub * 8), t);
#pragma unroll
    for (int i = 0; i < 8; ++i) qf[g][8 + i] = t[i] * p.scale_log2;
  }
  float m[G], l[G], acc[G][16];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[g][i] = 0.f;
  }
  bool ok = true;
  for (int i = 0; i < npages; ++i) {
    const int s = i % STAGES;
    if (!warp_wait(&bars->full[s], (i / STAGES) & 1, abort_flag, p.status, 200 + s)) { ok = false; break; }
    const uint8_t* Kp = sK + s * PAGE_BYTES;
    const uint8_t* Vp = sV + s * PAGE_BYTES;
    const int n_valid = min(PAGE, seq_len - (p0 + i) * PAGE);
    float sc[G][4];
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int tok = warp * 16 + it * 4 + quarter;
      float kf[16];
      unpack8(*reinterpret_cast<const uint4*>(Kp + tok * 256 + sub * 16), kf);
      unpack8(*reinterpret_cast<const uint4*>(Kp + tok * 256 + 128 + sub * 16), kf + 8);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) d = fmaf(qf[g][e], kf[e], d);
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        d += __shfl_xor_sync(0xffffffffu, d, 4);
        sc[g][it] = tok < n_valid ? d : -INFINITY;
      }
    }
    float pr[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mx = fmaxf(fmaxf(sc[g][0], sc[g][1]), fmaxf(sc[g][2], sc[g][3]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_new = fmaxf(m[g], mx);
      if (m_new == -INFINITY) {
#pragma unroll
        for (int it = 0; it < 4; ++it) pr[g][it] = 0.f;
        continue;
      }
      const float factor = (m[g] == -INFINITY) ? 0.f : ex2(m[g] - m_new);
      m[g] = m_new;
      l[g] *= factor;
#pragma unroll
      for (int e = 0; e < 16; ++e) acc[g][e] *= factor;
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        pr[g][it] = ex2(sc[g][it] - m_new);
        l[g] += pr[g][it];
      }
    }
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int tok = warp * 16 + it * 4 + quarter;
      float vf[16];
      unpack8(*reinterpret_cast<const uint4*>(Vp + tok * 256 + sub * 16), vf);
      unpack8(*reinterpret_cast<const uint4*>(Vp + tok * 256 + 128 + sub * 16), vf + 8);
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < 16; ++e) acc[g][e] = fmaf(pr[g][it], vf[e], acc[g][e]);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&bars->empty[s]);
  }
  // ---- reduce over the four token quarters of the warp, then over warps through shared memory
#pragma unroll
  for (int g = 0; g < G; ++g) {
    l[g] += __shfl_xor_sync(0xffffffffu, l[g], 8);
    l[g] += __shfl_xor_sync(0xffffffffu, l[g], 16);
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], 8);
      acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], 16);
    }
    if (quarter == 0) {
      float* dst = sMerge + (warp * G + g) * 130;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        dst[sub * 8 + e] = acc[g][e];
        dst[64 + sub * 8 + e] = acc[g][8 + e];
      }
      if (sub == 0) {
        dst[128] = m[g];
        dst[129] = l[g];
      }
    }
  }
  named_bar_sync(1, CWARPS * 32);
  if (!ok) return;
  const int t = threadIdx.x;   // 0..127 = output dim
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < CWARPS; ++w) M = fmaxf(M, sMerge[(w * G + g) * 130 + 128]);
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < CWARPS; ++w) {
      const float* src = sMerge + (w * G + g) * 130;
      const float f = (src[128] == -INFINITY) ? 0.f : ex2(src[128] - M);
      L += src[129] * f;
      A += src[t] * f;
    }
    const size_t hq = static_cast<size_t>(b) * p.Hq + h * G + g;
    if (p.nsplit == 1) {
      p.out[hq * D + t] = __float2bfloat16(L > 0.f ? A / L : 0.f);
    } else {
      p.part_acc[(hq * p.nsplit + split) * D + t] = A;
      if (t == 0) {
        p.part_ml[(hq * p.nsplit + split) * 2] = M;
        p.part_ml[(hq * p.nsplit + split) * 2 + 1] = L;
      }
    }
  }
}

__global__ void __launch_bounds__(D) decode_merge_kernel(const float* __restrict__ part_acc,
                                                         const float* __restrict__ part_ml, bf16* __restrict__ out,
                                                         int nsplit) {
  const size_t hq = blockIdx.x;
  const int t = threadIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_ml[(hq * nsplit + s) * 2]);
  float L = 0.f, A = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = part_ml[(hq * nsplit + s) * 2];
    const float f = (ms == -INFINITY) ? 0.f : ex2(ms - M);
    L += part_ml[(hq * nsplit + s) * 2 + 1] * f;
    A += part_acc[(hq * nsplit + s) * D + t] * f;
  }
  out[hq * D + t] = __float2bfloat16(L > 0.f ? A / L : 0.f);
}

// One CTA per sequence; thread = (head, rotary pair).  qkv row layout: [Hq q heads | Hkv k heads | Hkv v heads] x 128.
__global__ void __launch_bounds__(256) decode_qkv_prep_kernel(
    const bf16* __restrict__ qkv, const bf16* __restrict__ bias, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, const int* __restrict__ seq_lens, const int* __restrict__ block_table,
    bf16* __restrict__ q_out, bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int Hq, int Hkv,
    int max_blocks, int64_t qkv_stride, int max_pos) {
  const int b = blockIdx.x;
  const int pos = seq_lens[b];
  if (pos >= max_pos || pos < 0) return;
  const int blk = block_table[static_cast<size_t>(b) * max_blocks + pos / PAGE];
  const int slot = pos % PAGE;
  const bf16* row = qkv + static_cast<size_t>(b) * qkv_stride;
  const int heads = Hq + 2 * Hkv;
  for (int idx = threadIdx.x; idx < heads * 64; idx += blockDim.x) {
    const int head = idx >> 6, i = idx & 63;
    float x1 = __bfloat162float(row[head * D + i]), x2 = __bfloat162float(row[head * D + 64 + i]);
    if (bias != nullptr) {
      x1 += __bfloat162float(bias[head * D + i]);
      x2 += __bfloat162float(bias[head * D + 64 + i]);
    }
    if (head < Hq + Hkv) {
      const float c = cos_t[static_cast<size_t>(pos) * 64 + i], s = sin_t[static_cast<size_t>(pos) * 64 + i];
      const float r1 = x1 * c - x2 * s, r2 = x2 * c + x1 * s;
      x1 = r1;
      x2 = r2;
    }
    bf16* dst;
    if (head < Hq) {
      dst = q_out + (static_cast<size_t>(b) * Hq + head) * D;
    } else {
      const int kvh = (head - Hq) % Hkv;
      bf16* cache = head < Hq + Hkv ? k_cache : v_cache;
      dst = cache + ((static_cast<size_t>(blk) * Hkv + kvh) * PAGE + slot) * D;
    }
    dst[i] = __float2bfloat16(x1);
    dst[64 + i] = __float2bfloat16(x2);
  }
}

// k, v: [B, S, Hkv, 128] with token/batch strides (elements).  One 16-byte chunk per thread.
__global__ void __launch_bounds__(256) write_kv_cache_kernel(
    const bf16* __restrict__ k, const bf16* __restrict__ v, const int* __restrict__ block_table,
    bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int S, int Hkv, int max_blocks, int64_t tok_stride,
    int64_t batch_stride, int start_pos, int64_t total) {
  const int chunks = Hkv * 16;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx % chunks);
    const int64_t ts = idx / chunks;
    const int s = static_cast<int>(ts % S), b = static_cast<int>(ts / S);
    const int pos = start_pos + s;
    const int blk = block_table[static_cast<size_t>(b) * max_blocks + pos / PAGE];
    const int hd = c >> 4, part = c & 15;
    const size_t src = static_cast<size_t>(b) * batch_stride + static_cast<size_t>(s) * tok_stride + hd * D + part * 8;
    const size_t dst = ((static_cast<size_t>(blk) * Hkv + hd) * PAGE + pos % PAGE) * D + part * 8;
    *reinterpret_cast<uint4*>(k_cache + dst) = *reinterpret_cast<const uint4*>(k + src);
    *reinterpret_cast<uint4*>(v_cache + dst) = *reinterpret_cast<const uint4*>(v + src);
  }
}

__global__ void __launch_bounds__(256) splitk_finalize_kernel(float* __restrict__ acc, const bf16* __restrict__ bias,
                                                              const bf16* __restrict__ residual,
                                                              bf16* __restrict__ out, int64_t M, int N) {
  const int64_t nvec = M * N / 4;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float4 a = reinterpret_cast<float4*>(acc)[i];
    reinterpret_cast<float4*>(acc)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int col = static_cast<int>((i * 4) % N);
    if (bias != nullptr) {
      a.x += __bfloat162float(bias[col]); a.y += __bfloat162float(bias[col + 1]);
      a.z += __bfloat162float(bias[col + 2]); a.w += __bfloat162float(bias[col + 3]);
    }
    if (residual != nullptr) {
      const uint2 r = reinterpret_cast<const uint2*>(residual)[i];
      a.x += __uint_as_float(r.x << 16); a.y += __uint_as_float(r.x & 0xffff0000u);
      a.z += __uint_as_float(r.y << 16); a.w += __uint_as_float(r.y & 0xffff0000u);
    }
    uint2 o;
    o.x = pack_bf16x2(a.x, a.y);
    o.y = pack_bf16x2(a.z, a.w);
    reinterpret_cast<uint2*>(out)[i] = o;
  }
}

constexpr int attn_smem(int G) { return 2 * STAGES * PAGE_BYTES + CWARPS * G * 130 * 4 + 256 + 128; }

template <int G>
static int launch_attn(const AttnParams& p, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(paged_decode_attn_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             attn_smem(G)) != cudaSuccess)
      return kErrCuda;
    configured = true;
  }
  dim3 grid(p.nsplit, p.Hkv, p.B);
  paged_decode_attn_kernel<G><<<grid, THREADS, attn_smem(G), stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

}  // namespace dec
}  // namespace pd

using namespace pd;
using namespace pd::dec;

// Suggested number of context splits so that the grid fills the GPU about twice.
PD_EXPORT int pd_decode_attn_splits(int B, int Hkv, int max_pages) {
  const int target = 2 * sm_count();
  int n = (target + B * Hkv - 1) / (B * Hkv);
  if (n > max_pages) n = max_pages;
  if (n > 32) n = 32;
  return n < 1 ? 1 : n;
}

// q [B,Hq,128], caches [num_blocks,Hkv,64,128], block_table [B,max_blocks] int32, seq_lens [B] int32 (attended
// length = seq_lens[b] + len_offset), out [B,Hq,128]; part_acc [B,Hq,nsplit,128] / part_ml [B,Hq,nsplit,2] fp32
// are needed only when nsplit > 1.
PD_EXPORT int pd_paged_decode_attn(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                   const int* seq_lens, void* out, float* part_acc, float* part_ml, int B, int Hq,
                                   int Hkv, int max_blocks, int nsplit, int len_offset, float scale, int* status,
                                   cudaStream_t stream) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || nsplit < 1 || max_blocks < 1) return kErrBadShape;
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache)) return kErrAlignment;
  if (nsplit > 1 && (part_acc == nullptr || part_ml == nullptr)) return kErrBadShape;
  AttnParams p{(const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, block_table, seq_lens, (bf16*)out,
               part_acc, part_ml, B, Hq, Hkv, max_blocks, nsplit, len_offset, scale * 1.4426950408889634f, status};
  int rc;
  switch (Hq / Hkv) {
    case 1: rc = launch_attn<1>(p, stream); break;
    case 2: rc = launch_attn<2>(p, stream); break;
    case 4: rc = launch_attn<4>(p, stream); break;
    case 8: rc = launch_attn<8>(p, stream); break;
    default: return kErrBadShape;
  }
  if (rc != kLaunchOk) return rc;
  if (nsplit > 1) {
    decode_merge_kernel<<<B * Hq, D, 0, stream>>>(part_acc, part_ml, (bf16*)out, nsplit);
    if (cudaGetLastError() != cudaSuccess) return kErrCuda;
  }
  return kLaunchOk;
}

// qkv [B, qkv_stride] rows of (Hq + 2 Hkv) x 128; cos/sin [max_pos, 64] fp32; position = seq_lens[b].
PD_EXPORT int pd_decode_qkv_prep(const void* qkv, const void* bias, const float* cos_t, const float* sin_t,
                                 const int* seq_lens, const int* block_table, void* q_out, void* k_cache,
                                 void* v_cache, int B, int Hq, int Hkv, int max_blocks, int64_t qkv_stride,
                                 int max_pos, cudaStream_t stream) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0) return kErrBadShape;
  decode_qkv_prep_kernel<<<B, 256, 0, stream>>>((const bf16*)qkv, (const bf16*)bias, cos_t, sin_t, seq_lens,
                                                block_table, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, Hq, Hkv,
                                                max_blocks, qkv_stride, max_pos);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

PD_EXPORT int pd_write_kv_cache(const void* k, const void* v, const int* block_table, void* k_cache, void* v_cache,
                                int B, int S, int Hkv, int max_blocks, int64_t tok_stride, int64_t batch_stride,
                                int start_pos, cudaStream_t stream) {
  if (B <= 0 || S <= 0 || Hkv <= 0) return kErrBadShape;
  if (!aligned16(k) || !aligned16(v) || !aligned16(k_cache) || !aligned16(v_cache) || (tok_stride % 8) ||
      (batch_stride % 8))
    return kErrAlignment;
  const int64_t total = static_cast<int64_t>(B) * S * Hkv * 16;
  const int64_t blocks = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  write_kv_cache_kernel<<<static_cast<int>(blocks < cap ? blocks : cap), 256, 0, stream>>>(
      (const bf16*)k, (const bf16*)v, block_table, (bf16*)k_cache, (bf16*)v_cache, S, Hkv, max_blocks, tok_stride,
      batch_stride, start_pos, total);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

// out[M,N] (bf16) = acc (+ bias[N]) (+ residual[M,N]); acc is zeroed for its next use.  N % 4 == 0.
PD_EXPORT int pd_splitk_finalize(float* acc, const void* bias, const void* residual, void* out, int64_t M, int N,
                                 cudaStream_t stream) {
  if (M <= 0 || N <= 0 || (N % 4)) return kErrBadShape;
  const int64_t nvec = M * N / 4;
  const int64_t blocks = (nvec + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  splitk_finalize_kernel<<<static_cast<int>(blocks < cap ? blocks : cap), 256, 0, stream>>>(
      acc, (const bf16*)bias, (const bf16*)residual, (bf16*)out, M, N);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}
