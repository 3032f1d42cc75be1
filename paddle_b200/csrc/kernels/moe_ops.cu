// Mixture-of-experts kernels for sm_100a:
//   pd_moe_topk_softmax        : router - softmax over experts, top-k (k <= 8), re-normalised weights, per-expert
//                                token counts (reference: top-k gating in python + number_count_kernel.cu)
//   pd_fp8_quant_1x128         : bf16 [T, H] -> e4m3 [T, H] + fp32 scales [T, H/128]      (activation blocks 1 x 128)
//   pd_fp8_quant_128x128_t     : bf16 W [K, N] -> e4m3 W^T [N, K] + fp32 scales [K/128, N/128] (weight blocks 128 x 128)
//   pd_grouped_gemm_fp8        : C[rows of expert e, :] = dequant(A_e) * dequant(W_e), all experts in ONE persistent
//                                launch; tokens are sorted by expert and `offsets[e]..offsets[e+1]` delimits expert e.
// Reference counterparts: the per-expert cuBLAS loop of moe_layer.py:_experts_forward and the fused_moe kernels
// (paddle/phi/kernels/fusion/cutlass/moe/*, fp8 paths in paddle/phi/kernels/fusion/fp8_gemm/).
//
// Block-scaled fp8 GEMM on tcgen05: the K loop advances in blocks of 128 (= the scale granularity = one 128-byte
// swizzled row of e4m3).  Each K block is ONE fresh accumulation (kind::f8f6f4, four K=32 MMAs) into one of two
// TMEM buffers; the epilogue warps read the finished buffer, multiply by a_scale[row, kb] * w_scale[kb, n-block] and
// add into fp32 registers while the tensor cores already work on the next K block in the other buffer.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <math.h>

#include "host_utils.h"
#include "sm100_prims.cuh"

namespace pd {
namespace moe {

typedef __nv_bfloat16 bf16;

// ------------------------------------------------------------------------------------------------ router
// One warp per token.  E <= 256 (8 values per lane).
__global__ void __launch_bounds__(256) topk_softmax_kernel(const float* __restrict__ logits, int T, int E, int k,
                                                           int normalize, float* __restrict__ weights,
                                                           int* __restrict__ indices, int* __restrict__ counts) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  float v[8];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? logits[static_cast<size_t>(t) * E + e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[i] = (lane + 32 * i) < E ? __expf(v[i] - mx) : 0.f;
    sum += v[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  float picked = 0.f;
  float w_out = 0.f;
  int i_out = 0;
  for (int j = 0; j < k; ++j) {
    float best = -1.f;
    int best_e = E;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = lane + 32 * i;
      if (v[i] > best || (v[i] == best && e < best_e)) { best = v[i]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if ((best_e & 31) == lane) v[best_e >> 5] = -1.f;      // remove the winner
    picked += best * inv;
    if (lane == j) { w_out = best * inv; i_out = best_e; }
  }
  if (lane < k) {
    weights[static_cast<size_t>(t) * k + lane] = normalize ? w_out / picked : w_out;
    indices[static_cast<size_t>(t) * k + lane] = i_out;
    if (counts != nullptr) atomicAdd(counts + i_out, 1);
  }
}

// ------------------------------------------------------------------------------------------------ quantisation
constexpr float E4M3_MAX = 448.f;

// one warp per (row, 128-column block): 4 elements per lane
__global__ void __launch_bounds__(256) quant_1x128_kernel(const bf16* __restrict__ x, __nv_fp8_e4m3* __restrict__ q,
                                                          float* __restrict__ scales, int64_t T, int H) {
  const int64_t w = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int nb = H / 128;
  if (w >= T * nb) return;
  const int64_t row = w / nb;
  const int kb = static_cast<int>(w % nb);
  const uint2 raw = *reinterpret_cast<const uint2*>(x + row * H + kb * 128 + lane * 4);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = fmaxf(amax, 1e-12f) / E4M3_MAX;
  const float inv = 1.f / scale;
  __nv_fp8_e4m3 o[4] = {__nv_fp8_e4m3(a.x * inv), __nv_fp8_e4m3(a.y * inv), __nv_fp8_e4m3(b.x * inv),
                        __nv_fp8_e4m3(b.y * inv)};
  *reinterpret_cast<uint32_t*>(q + row * H + kb * 128 + lane * 4) = *reinterpret_cast<uint32_t*>(o);
  if (lane == 0) scales[row * nb + kb] = scale;
}

// one CTA (256 threads) per 128 x 128 block of W [K, N]; writes the transposed block into Wt [N, K]
__global__ void __launch_bounds__(256) quant_128x128_t_kernel(const bf16* __restrict__ w, __nv_fp8_e4m3* __restrict__ wt,
                                                              float* __restrict__ scales, int K, int N) {
  __shared__ bf16 tile[128][130];
  __shared__ float red[8];
  const int kb = blockIdx.y, nb = blockIdx.x;
  float amax = 0.f;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = i >> 7, c = i & 127;
    const bf16 raw = w[static_cast<size_t>(kb * 128 + r) * N + nb * 128 + c];
    tile[r][c] = raw;
    amax = fmaxf(amax, fabsf(__bfloat162float(raw)));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float scale = fmaxf(amax, 1e-12f) / E4M3_MAX;
  const float inv = 1.f / scale;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int n = i >> 7, k = i & 127;      // output row n, column k  (k contiguous)
    wt[static_cast<size_t>(nb * 128 + n) * K + kb * 128 + k] = __nv_fp8_e4m3(__bfloat162float(tile[k][n]) * inv);
  }
  if (threadIdx.x == 0) scales[static_cast<size_t>(kb) * (N / 128) + nb] = scale;
}

// ------------------------------------------------------------------------------------------------ grouped fp8 GEMM
constexpr int BM = 128, BK = 128, STAGES = 4;
constexpr int SCALE_BLOCK = 128;                               // weight-scale granularity along N (and K)
constexpr int A_STAGE = BM * BK;                               // 16 KB (1 byte per element)
constexpr int MAX_EXPERTS = 64;
constexpr int OFF_SLOTS = 80;                                  // >= MAX_EXPERTS + 1, keeps the barriers 16-byte aligned
// NWG epilogue warpgroups own 128 accumulator columns each: the tile is 128 x (128 * NWG).  With one warpgroup the
// promotion (TMEM read + 128 FMAs per thread per 128-deep K block) takes about twice as long as the fp8 MMA of the
// block; two warpgroups on a 128 x 256 tile halve the promotion work per MMA cycle and bring the two into balance.
template <int NWG> struct Cfg {
  static constexpr int BN = SCALE_BLOCK * NWG;
  static constexpr int B_STAGE = BN * BK;
  static constexpr int THREADS = 128 * NWG + 64;
  static constexpr int SMEM = STAGES * (A_STAGE + B_STAGE) + 3 * OFF_SLOTS * 4 + 1024 + 256;
  static constexpr int TMEM_COLS = 2 * BN;                    // two accumulator buffers
};

struct Bars {
  uint64_t full[STAGES], empty[STAGES], tfull[2], tempty[2], drain;
  uint32_t tmem_base;
  int abort_flag;
  int verdict;
};

struct GParams {
  const int* offsets;       // [E + 1] row offsets of each expert in A / C
  const int* seg_ends;      // optional [E]: segment e covers rows [offsets[e], seg_ends[e]) - a layout with unused rows
                            // between segments (fixed-capacity receive buffers of the expert-parallel dispatch)
  const int* expert_map;    // optional [E]: weights / weight scales of segment e are those of expert expert_map[e]
                            // (several segments - one per source rank - share one expert)
  const float* a_scale;     // [M_total, K / 128]
  const float* b_scale;     // [E, K / 128, N / 128]
  bf16* c;                  // [M_total, N]
  int E, N, K, ldc;
  int* status;
};

// tile id -> (expert, first row, rows, n0); returns false when id is past the end
__device__ __forceinline__ bool locate(const int* offs, const int* ends, int E, int tiles_n, int bn, int id, int& e,
                                       int& m0, int& m_end, int& n0) {
  // Within an expert the row tiles vary fastest: the CTAs running at one time then share a few weight column
  // blocks (each read from HBM once and hit in L2 by the other row tiles) instead of streaming the whole weight
  // matrix once per row tile; the expert's activations (rows x K bytes) stay L2-resident either way.
  for (e = 0; e < E; ++e) {
    const int rows = max(ends[e] - offs[e], 0);
    const int tm = (rows + BM - 1) / BM;
    const int t = tm * tiles_n;
    if (id < t) {
      m0 = offs[e] + (id % tm) * BM;
      m_end = ends[e];
      n0 = (id / tm) * bn;
      return true;
    }
    id -= t;
  }
  return false;
}

template <int NWG>
__global__ void __launch_bounds__(Cfg<NWG>::THREADS, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GParams p) {
  constexpr int BN = Cfg<NWG>::BN, B_STAGE = Cfg<NWG>::B_STAGE, EPI_WARPS = 4 * NWG;
  constexpr int TMA_WARP = EPI_WARPS, MMA_WARP = EPI_WARPS + 1;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE;
  int* sOff = reinterpret_cast<int*>(sB + STAGES * B_STAGE);
  int* sEnd = sOff + OFF_SLOTS;
  int* sMap = sEnd + OFF_SLOTS;
  Bars* bars = reinterpret_cast<Bars*>(sMap + OFF_SLOTS);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = p.N / BN;
  const int KB = p.K / BK;

  for (int i = threadIdx.x; i <= p.E; i += Cfg<NWG>::THREADS) sOff[i] = p.offsets[i];
  for (int i = threadIdx.x; i < p.E; i += Cfg<NWG>::THREADS) {
    sEnd[i] = p.seg_ends != nullptr ? p.seg_ends[i] : p.offsets[i + 1];
    sMap[i] = p.expert_map != nullptr ? p.expert_map[i] : i;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tfull[a], 1);
      mbar_init(&bars->tempty[a], 128 * NWG);
    }
    mbar_init(&bars->drain, 1);
    bars->abort_flag = 0;
    bars->verdict = 0;
    fence_mbar_init();
  }
  if (warp == MMA_WARP) tmem_alloc(&bars->tmem_base, Cfg<NWG>::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == TMA_WARP) {
    if (lane == 0) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      int it = 0, armed = 0;
      bool ok = true;
      for (int id = blockIdx.x; ok; id += gridDim.x) {
        int e, m0, m_end, n0;
        if (!locate(sOff, sEnd, p.E, tiles_n, BN, id, e, m0, m_end, n0)) break;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&bars->empty[s], ((it / STAGES) & 1) ^ 1, abort_flag, p.status, 100 + s)) { ok = false; break; }
          mbar_expect_tx(&bars->full[s], A_STAGE + B_STAGE);
          tma_load_2d(sA + s * A_STAGE, &tmA, &bars->full[s], kb * BK, m0);            // box {128 k, 128 m}
#pragma unroll
          for (int g = 0; g < NWG; ++g)                                                  // box {128 k, 128 n, 1}
            tma_load_3d(sB + s * B_STAGE + g * (SCALE_BLOCK * BK), &tmB, &bars->full[s], kb * BK, n0 + g * SCALE_BLOCK, sMap[e]);
          armed = it + 1;
        }
      }
      if (!ok) {
        for (int i = max(0, armed - STAGES); i < armed; ++i) mbar_drain(&bars->full[i % STAGES], (i / STAGES) & 1);
      }
    }
    __syncwarp();
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN, false, false, 0, 0);        // e4m3 x e4m3, both K-major
      int it = 0;
      bool ok = true;
      for (int id = blockIdx.x; ok; id += gridDim.x) {
        int e, m0, m_end, n0;
        if (!locate(sOff, sEnd, p.E, tiles_n, BN, id, e, m0, m_end, n0)) break;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % STAGES, acc = it & 1;
          if (!mbar_wait(&bars->tempty[acc], ((it >> 1) & 1) ^ 1, abort_flag, p.status, 200 + acc)) { ok = false; break; }
          if (!mbar_wait(&bars->full[s], (it / STAGES) & 1, abort_flag, p.status, 300 + s)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * A_STAGE), b_addr = smem_u32(sB + s * B_STAGE);
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)
            umma_f8_ss(tmem_base + acc * BN, make_smem_desc_sw128(a_addr + k * 32, 16, 1024),
                       make_smem_desc_sw128(b_addr + k * 32, 16, 1024), idesc, k != 0 ? 1u : 0u);
          umma_commit(&bars->empty[s]);
          umma_commit(&bars->tfull[acc]);
        }
      }
      if (!ok) {
        umma_commit(&bars->drain);
        mbar_drain(&bars->drain, 0);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ promotion + store: thread = row, warpgroup = 128 columns
    const int wg = warp >> 2;
    const int tid = threadIdx.x & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int kbn = p.K / 128, nbn = p.N / 128;
    int it = 0;
    bool ok = true;
    for (int id = blockIdx.x; ok; id += gridDim.x) {
      int e, m0, m_end, n0;
      if (!locate(sOff, sEnd, p.E, tiles_n, BN, id, e, m0, m_end, n0)) break;
      const int row = m0 + tid;
      const bool live = row < m_end;
      float acc[SCALE_BLOCK];
#pragma unroll
      for (int i = 0; i < SCALE_BLOCK; ++i) acc[i] = 0.f;
      const float* as_row = p.a_scale + static_cast<size_t>(live ? row : m0) * kbn;
      const float* bs = p.b_scale + (static_cast<size_t>(sMap[e]) * kbn) * nbn + n0 / 128 + wg;
      // The scales of block kb + 1 are LOADED here and only multiplied at the top of the next iteration: issue is in
      // order, so using them now would park the warp on the load for a full memory latency every block.
      float a_nx = as_row[0], b_nx = bs[0];
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int a = it & 1;
        const float sc = a_nx * b_nx;
        if (kb + 1 < KB) {
          a_nx = as_row[kb + 1];
          b_nx = bs[static_cast<size_t>(kb + 1) * nbn];
        }
        int good = 1;
        if (lane == 0) good = mbar_wait(&bars->tfull[a], (it >> 1) & 1, abort_flag, p.status, 400 + a) ? 1 : 0;
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) { ok = false; break; }
#pragma unroll 1
        for (int i = 0; i < 1024 && !mbar_try_wait(&bars->tfull[a], (it >> 1) & 1); ++i) {
        }
        tc_fence_after();
        const uint32_t t_acc = tmem_base + lane_base + a * BN + wg * SCALE_BLOCK;
#pragma unroll
        for (int c = 0; c < SCALE_BLOCK / 64; ++c) {
          uint32_t r0[32], r1[32];                     // two TMEM reads in flight per wait
          tmem_ld_32x32(t_acc + c * 64, r0);
          tmem_ld_32x32(t_acc + c * 64 + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c * 64 + i] = fmaf(__uint_as_float(r0[i]), sc, acc[c * 64 + i]);
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c * 64 + 32 + i] = fmaf(__uint_as_float(r1[i]), sc, acc[c * 64 + 32 + i]);
        }
        tc_fence_before();
        mbar_arrive(&bars->tempty[a]);
      }
      if (!ok) break;
      if (live) {
        bf16* dst = p.c + static_cast<size_t>(row) * p.ldc + n0 + wg * SCALE_BLOCK;
#pragma unroll
        for (int j = 0; j < SCALE_BLOCK / 8; ++j) {
          uint4 v;
          v.x = pack_bf16x2(acc[8 * j + 0], acc[8 * j + 1]);
          v.y = pack_bf16x2(acc[8 * j + 2], acc[8 * j + 3]);
          v.z = pack_bf16x2(acc[8 * j + 4], acc[8 * j + 5]);
          v.w = pack_bf16x2(acc[8 * j + 6], acc[8 * j + 7]);
          *reinterpret_cast<uint4*>(dst + 8 * j) = v;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) tmem_dealloc(tmem_base, Cfg<NWG>::TMEM_COLS);
}

}  // namespace moe
}  // namespace pd

using namespace pd;
using namespace pd::moe;

// logits [T, E] fp32 -> weights [T, k] fp32, indices [T, k] int32, counts [E] int32 (added to; may be null)
PD_EXPORT int pd_moe_topk_softmax(const float* logits, int T, int E, int k, int normalize, float* weights, int* indices,
                                  int* counts, cudaStream_t stream) {
  if (T <= 0 || E <= 0 || E > 256 || k <= 0 || k > 8 || k > E) return kErrBadShape;
  const int blocks = (T * 32 + 255) / 256;
  topk_softmax_kernel<<<blocks, 256, 0, stream>>>(logits, T, E, k, normalize, weights, indices, counts);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

PD_EXPORT int pd_fp8_quant_1x128(const void* x, void* q, float* scales, int64_t T, int H, cudaStream_t stream) {
  if (T <= 0 || H <= 0 || (H % 128)) return kErrBadShape;
  if (!aligned16(x) || !aligned16(q)) return kErrAlignment;
  const int64_t warps = T * (H / 128);
  quant_1x128_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, stream>>>(
      (const bf16*)x, (__nv_fp8_e4m3*)q, scales, T, H);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

// w [K, N] bf16 -> wt [N, K] e4m3 (transposed: K contiguous) + scales [K/128, N/128]
PD_EXPORT int pd_fp8_quant_128x128_t(const void* w, void* wt, float* scales, int K, int N, cudaStream_t stream) {
  if (K <= 0 || N <= 0 || (K % 128) || (N % 128)) return kErrBadShape;
  quant_128x128_t_kernel<<<dim3(N / 128, K / 128), 256, 0, stream>>>((const bf16*)w, (__nv_fp8_e4m3*)wt, scales, K, N);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

static int launch_grouped(const CUtensorMap& tmA, const CUtensorMap& tmB, const GParams& p, int N, int max_tiles,
                          cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(grouped_gemm_fp8_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<1>::SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(grouped_gemm_fp8_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<2>::SMEM) != cudaSuccess)
      return kErrCuda;
    configured = true;
  }
  // max_tiles counts 128 x 128 tiles; the 128 x 256 kernel has half as many
  const bool wide = (N % Cfg<2>::BN) == 0;
  const int tiles = wide ? (max_tiles + 1) / 2 : max_tiles;
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (grid < 1) grid = 1;
  if (wide)
    grouped_gemm_fp8_kernel<2><<<grid, Cfg<2>::THREADS, Cfg<2>::SMEM, stream>>>(tmA, tmB, p);
  else
    grouped_gemm_fp8_kernel<1><<<grid, Cfg<1>::THREADS, Cfg<1>::SMEM, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

// A [M_total, K] e4m3 (rows sorted by expert), a_scale [M_total, K/128]; B [E, N, K] e4m3, b_scale [E, K/128, N/128];
// offsets [E + 1] int32 (device); C [M_total, N] bf16.  max_tiles: upper bound of sum_e ceil(rows_e / 128) * N / 128
// used to size the grid (for example ceil(M_total / 128) + E, times N / 128).
PD_EXPORT int pd_grouped_gemm_fp8(const void* A, const float* a_scale, const void* B, const float* b_scale,
                                  const int* offsets, void* C, int M_total, int N, int K, int E, int ldc, int max_tiles,
                                  int* status, cudaStream_t stream) {
  if (M_total <= 0 || N <= 0 || K <= 0 || E <= 0 || E > MAX_EXPERTS || (N % SCALE_BLOCK) || (K % BK)) return kErrBadShape;
  if (!aligned16(A) || !aligned16(B) || !aligned16(C) || (ldc % 8)) return kErrAlignment;
  CUtensorMap tmA, tmB;
  bool ok = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, A, K, M_total, uint64_t(K), BK, BM);
  uint64_t dims[3] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N), static_cast<uint64_t>(E)};
  uint64_t strides[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(K) * N};
  uint32_t box[3] = {BK, SCALE_BLOCK, 1};
  ok &= encode_tmap(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, B, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return kErrTensorMap;
  GParams p{offsets, nullptr, nullptr, a_scale, b_scale, (bf16*)C, E, N, K, ldc, status};
  return launch_grouped(tmA, tmB, p, N, max_tiles, stream);
}

// Segment form: rows of segment s are [seg_start[s], seg_end[s]) (unused rows may lie between segments) and its
// weights are those of expert expert_map[s]; n_seg <= 64, E_w = number of weight matrices in B.
PD_EXPORT int pd_grouped_gemm_fp8_seg(const void* A, const float* a_scale, const void* B, const float* b_scale,
                                      const int* seg_start, const int* seg_end, const int* expert_map, void* C,
                                      int M_total, int N, int K, int n_seg, int E_w, int ldc, int max_tiles, int* status,
                                      cudaStream_t stream) {
  if (M_total <= 0 || N <= 0 || K <= 0 || n_seg <= 0 || n_seg > MAX_EXPERTS || E_w <= 0 || (N % SCALE_BLOCK) || (K % BK))
    return kErrBadShape;
  if (!aligned16(A) || !aligned16(B) || !aligned16(C) || (ldc % 8)) return kErrAlignment;
  CUtensorMap tmA, tmB;
  bool ok = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, A, K, M_total, uint64_t(K), BK, BM);
  uint64_t dims[3] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N), static_cast<uint64_t>(E_w)};
  uint64_t strides[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(K) * N};
  uint32_t box[3] = {BK, SCALE_BLOCK, 1};
  ok &= encode_tmap(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, B, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return kErrTensorMap;
  // offsets[n_seg] is never read in this form (the ends come from seg_end)
  GParams p{seg_start, seg_end, expert_map, a_scale, b_scale, (bf16*)C, n_seg, N, K, ldc, status};
  return launch_grouped(tmA, tmB, p, N, max_tiles, stream);
}
