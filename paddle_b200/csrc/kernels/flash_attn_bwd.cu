// Flash-attention backward for sm_100a, head_dim 128, bf16, causal or full, GQA.
// (Reference: the external FA2 library behind paddle/phi/kernels/gpu/flash_attn_grad_kernel.cu:317.)
//
// One CTA owns a 128-row K/V tile of one kv head and walks over the query heads of its group and the
// 64-row query sub-tiles that can see it.  Every GEMM has M = 128 = the kv rows of the tile, so the
// per-row softmax threads coincide with TMEM lanes and P^T / dS^T feed the next GEMMs straight from
// TMEM (no shared-memory round trip):
//   (1) S^T  = K  Q_t^T          SS   N = 64      (2) dP^T = V dO_t^T          SS   N = 64
//   softmax warps: P^T = exp2(S^T*c - LSE), dS^T = P^T o (dP^T - Delta) * scale  -> TMEM (bf16) + smem
//   (3) dV  += P^T  dO_t         TS   N = 128     (4) dK  += dS^T Q_t           TS   N = 128
//   (5) dQ_t^T = K^T dS_t^T      SS   N = 64  -> drained by 4 extra warps, transposed in shared memory
//       and added to an fp32 dQ accumulator with a TMA reduce (cp.reduce.async.bulk.tensor .add).
// dK / dV stay in TMEM for the whole walk and are written once.  TMEM columns:
//   dK 0-127 | dV 128-255 | work buffer A 256-383 | work buffer B 384-511
// A work buffer holds S^T (cols 0-63) and dP^T (64-127) of one query sub-tile; after the softmax warps have read
// both into registers they write P^T (packed bf16, cols 0-31) and dS^T (32-63) over S^T, and GEMM (5) later puts
// dQ^T over dP^T.  Sub-tiles alternate between A and B, so GEMMs (1),(2) of sub-tile t+1 run on the tensor cores
// while the softmax warps work on sub-tile t, and GEMMs (3)-(5) of t overlap the softmax of t+1.  The per-column
// LSE / Delta values are staged in shared memory once per sub-tile and read as broadcasts.
// Warps: 0-3 softmax of query columns 0-31 (+ per-column statistics, final dK/dV store), 10-13 softmax of query columns
// 32-63 (the element-wise work needs no exchange between the halves: the log-sum-exp is an input), 4-7 dQ drain, 8 TMA
// producer, 9 MMA issuer.
#include <math.h>

#include "host_utils.h"
#include "sm100_prims.cuh"

namespace pd {
namespace fab {

constexpr int BKV = 128, BQ = 64, D = 128;
constexpr int KV_TILE = BKV * D * 2;          // 32 KB (two 16 KB boxes)
constexpr int KV_HALF = KV_TILE / 2;
constexpr int Q_TILE = BQ * D * 2;            // 16 KB (two 8 KB boxes)
constexpr int Q_HALF = Q_TILE / 2;
constexpr int STAGES = 3;
constexpr int DS_BYTES = BKV * BQ * 2;        // 16 KB
constexpr int DQ_STAGE_BYTES = BQ * D * 4;    // 32 KB fp32 [64 q][128 d]
constexpr int NUM_THREADS = 448;
constexpr int STATS_BYTES = 2 * 128 * 4;         // [2][lse2 x64 | delta x64]
constexpr int SMEM_BYTES = 2 * KV_TILE + STAGES * 2 * Q_TILE + 2 * DS_BYTES + DQ_STAGE_BYTES + STATS_BYTES + 1024 + 256;
constexpr uint32_t COL_DK = 0, COL_DV = 128, COL_BUF = 256;
constexpr uint32_t OFF_ST = 0, OFF_DPT = 64, OFF_PT = 0, OFF_DST = 32, OFF_DQT = 64;   // inside a 128-column work buffer

struct Barriers {
  uint64_t kv_full;
  uint64_t qdo_full[STAGES], qdo_empty[STAGES];
  uint64_t st_full[2], pds_full[2], dq_full[2], dq_empty[2], dkv_full, drain;
  uint32_t tmem_base;
  int abort_flag;
  int drain_decision;
};

struct Params {
  int B, Sq, Sk, Hq, Hkv, causal;
  float scale, scale_log2;
  const float* lse;     // [B, Hq, Sq] natural log
  const float* delta;   // [B, Hq, Sq]
  int* status;
  const int4* bounds;   // column-sparse mask, as in the forward kernel: [B, mask_heads, Sk] of {lts, lte, uts, ute}
  int mask_heads;
  const int4* tile_bounds;   // [B, mask_heads, ceil(Sk / 128)] of {max lts, min lte, max uts, min ute}
};

__device__ __forceinline__ bool warp_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                               int* status, int site) {
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
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <bool kMask>
__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                 const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                 const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmDK,
                 const __grid_constant__ CUtensorMap tmDV, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + KV_TILE;
  uint8_t* sQ = sV + KV_TILE;                       // STAGES x [Q tile | dO tile]
  uint8_t* sDS = sQ + STAGES * 2 * Q_TILE;
  uint8_t* sDQ = sDS + 2 * DS_BYTES;
  float* stats = reinterpret_cast<float*>(sDQ + DQ_STAGE_BYTES);
  Barriers* bars = reinterpret_cast<Barriers*>(sDQ + DQ_STAGE_BYTES + STATS_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jb = blockIdx.x, kv_head = blockIdx.y, batch = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int kv0 = jb * BKV;
  const int causal_off = p.Sk - p.Sq;
  const int n_sub = (p.Sq + BQ - 1) / BQ;
  int t0 = 0;
  if (p.causal) {
    const int first_q = kv0 - causal_off;            // first query row that sees kv row kv0
    t0 = first_q > 0 ? first_q / BQ : 0;
  }
  int t1 = n_sub;
  if (kMask && p.mask_heads != p.Hq) {
    // query sub-tiles outside [t0, t1) are masked as a whole for every column of this key tile: rows from max lts on
    // when the lower range is open-ended, rows below min ute when the upper range starts at row 0.  (With one mask per
    // query head the range would differ between the heads this CTA walks, so it is not narrowed then.)
    const int mh = p.mask_heads == 1 ? 0 : kv_head;
    const int4 tb = __ldg(p.tile_bounds + (static_cast<size_t>(batch) * p.mask_heads + mh) * gridDim.x + jb);
    if (tb.y >= p.Sq) t1 = min(t1, (max(tb.x, 0) + BQ - 1) / BQ);
    if (tb.z <= 0) t0 = max(t0, min(tb.w, p.Sq) / BQ);
  }
  const int per_head = t1 > t0 ? t1 - t0 : 0;
  const int n_it = per_head * group;

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->qdo_full[s], 1);
      mbar_init(&bars->qdo_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->st_full[b], 1);
      mbar_init(&bars->pds_full[b], 256);
      mbar_init(&bars->dq_full[b], 1);
      mbar_init(&bars->dq_empty[b], 128);
    }
    mbar_init(&bars->dkv_full, 1);
    mbar_init(&bars->drain, 1);
    bars->abort_flag = 0;
    bars->drain_decision = 0;
    fence_mbar_init();
  }
  if (warp == 9) tmem_alloc(&bars->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 8) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      prefetch_tmap(&tmQ);
      prefetch_tmap(&tmDO);
      mbar_expect_tx(&bars->kv_full, 2 * KV_TILE);
      tma_load_4d(sK, &tmK, &bars->kv_full, 0, kv_head, kv0, batch);
      tma_load_4d(sK + KV_HALF, &tmK, &bars->kv_full, 64, kv_head, kv0, batch);
      tma_load_4d(sV, &tmV, &bars->kv_full, 0, kv_head, kv0, batch);
      tma_load_4d(sV + KV_HALF, &tmV, &bars->kv_full, 64, kv_head, kv0, batch);
      bool ok = true;
      int issued = 0;
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(&bars->qdo_empty[s], ph ^ 1, abort_flag, p.status, 100 + s)) { ok = false; break; }
        const int qh = kv_head * group + it / per_head;
        const int q0 = (t0 + it % per_head) * BQ;
        uint8_t* dst = sQ + s * 2 * Q_TILE;
        mbar_expect_tx(&bars->qdo_full[s], 2 * Q_TILE);
        tma_load_4d(dst, &tmQ, &bars->qdo_full[s], 0, qh, q0, batch);
        tma_load_4d(dst + Q_HALF, &tmQ, &bars->qdo_full[s], 64, qh, q0, batch);
        tma_load_4d(dst + Q_TILE, &tmDO, &bars->qdo_full[s], 0, qh, q0, batch);
        tma_load_4d(dst + Q_TILE + Q_HALF, &tmDO, &bars->qdo_full[s], 64, qh, q0, batch);
        issued = it + 1;
      }
      if (!ok || *abort_flag || n_it == 0) {
        mbar_drain(&bars->kv_full, 0);
        for (int it = max(0, issued - STAGES); it < issued; ++it)
          mbar_drain(&bars->qdo_full[it % STAGES], (it / STAGES) & 1);
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_s = make_idesc(BKV, BQ, false, false);   // (1),(2)
      constexpr uint32_t idesc_kv = make_idesc(BKV, D, false, true);    // (3),(4)  A from TMEM
      constexpr uint32_t idesc_dq = make_idesc(D, BQ, true, true);      // (5)
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      bool ok = mbar_wait(&bars->kv_full, 0, abort_flag, p.status, 200);
      auto issue_s = [&](int it) -> bool {
        const int s = it % STAGES;
        if (!mbar_wait(&bars->qdo_full[s], (it / STAGES) & 1, abort_flag, p.status, 210 + s)) return false;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + s * 2 * Q_TILE), do_addr = q_addr + Q_TILE;
        const uint32_t buf = tmem + COL_BUF + (it & 1) * 128;
        // dP^T of this buffer's previous use now holds dQ^T: it must have been drained
        if (!mbar_wait(&bars->dq_empty[it & 1], ((it >> 1) & 1) ^ 1, abort_flag, p.status, 230 + (it & 1))) return false;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t offa = (ks >> 2) * KV_HALF + (ks & 3) * 32;
          const uint32_t offb = (ks >> 2) * Q_HALF + (ks & 3) * 32;
          umma_bf16_ss(buf + OFF_ST, make_smem_desc_sw128(k_addr + offa, 16, 1024),
                       make_smem_desc_sw128(q_addr + offb, 16, 1024), idesc_s, ks != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t offa = (ks >> 2) * KV_HALF + (ks & 3) * 32;
          const uint32_t offb = (ks >> 2) * Q_HALF + (ks & 3) * 32;
          umma_bf16_ss(buf + OFF_DPT, make_smem_desc_sw128(v_addr + offa, 16, 1024),
                       make_smem_desc_sw128(do_addr + offb, 16, 1024), idesc_s, ks != 0 ? 1u : 0u);
        }
        umma_commit(&bars->st_full[it & 1]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it % STAGES;
        const int b = it & 1;
        const uint32_t q_addr = smem_u32(sQ + s * 2 * Q_TILE), do_addr = q_addr + Q_TILE;
        const uint32_t buf = tmem + COL_BUF + b * 128;
        const uint32_t ds_addr = smem_u32(sDS + b * DS_BYTES);
        // S^T / dP^T of the NEXT sub-tile go to the other buffer now: they run while the softmax warps work
        if (it + 1 < n_it) {
          if (!issue_s(it + 1)) { ok = false; break; }
        }
        if (!mbar_wait(&bars->pds_full[b], (it >> 1) & 1, abort_flag, p.status, 220 + b)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BQ / 16; ++ks)   // (3) dV += P^T dO
          umma_bf16_ts(tmem + COL_DV, buf + OFF_PT + ks * 8,
                       make_smem_desc_sw128(do_addr + ks * 2048, Q_HALF, 1024), idesc_kv, (it | ks) != 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < BQ / 16; ++ks)   // (4) dK += dS^T Q
          umma_bf16_ts(tmem + COL_DK, buf + OFF_DST + ks * 8,
                       make_smem_desc_sw128(q_addr + ks * 2048, Q_HALF, 1024), idesc_kv, (it | ks) != 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < BKV / 16; ++ks)  // (5) dQ^T = K^T dS^T  (over this buffer's dP^T, already consumed)
          umma_bf16_ss(buf + OFF_DQT, make_smem_desc_sw128(k_addr + ks * 2048, KV_HALF, 1024),
                       make_smem_desc_sw128(ds_addr + ks * 2048, 16, 1024), idesc_dq, ks != 0 ? 1u : 0u);
        umma_commit(&bars->dq_full[b]);
        umma_commit(&bars->qdo_empty[s]);
      }
      if (ok) umma_commit(&bars->dkv_full);
      else {
        umma_commit(&bars->drain);
        mbar_drain(&bars->drain, 0);
      }
    }
    __syncwarp();
  } else if (warp < 4 || warp >= 10) {
    // ---------------------------------------------------------------- softmax warps: thread = kv row x column half
    // a warp may touch the TMEM lanes of its own quarter (warp index mod 4) only
    const int h = warp < 4 ? 0 : 1;                                 // query columns [32 h, 32 h + 32) of the sub-tile
    const int row = (warp & 3) * 32 + lane;
    const int kvi = kv0 + row;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int sw = row & 7;
    bool ok = true;
    auto load_stat = [&](int it) -> float {
      const int qh = kv_head * group + it / per_head;
      const int qi = (t0 + it % per_head) * BQ + (row & 63);
      const float* src = (row < 64 ? p.lse : p.delta) + (static_cast<size_t>(batch) * p.Hq + qh) * p.Sq;
      const bool in = qi < p.Sq;
      float v = in ? src[qi] : 0.f;
      if (row < 64) v = in ? v * 1.4426950408889634f : INFINITY;         // +inf -> p = 0 for padded rows
      return v;
    };
    float next_stat = (n_it > 0 && h == 0) ? load_stat(0) : 0.f;
    for (int it = 0; it < n_it; ++it) {
      const int qh = kv_head * group + it / per_head;
      const int q0 = (t0 + it % per_head) * BQ;
      const int b = it & 1;
      // per-column statistics of this sub-tile -> shared memory (threads 0-63: LSE in log2 units, 64-127: Delta).
      // The value was fetched one iteration ahead, so the global-memory latency never sits in front of the barrier.
      if (h == 0) {
        stats[b * 128 + row] = next_stat;
        if (it + 1 < n_it) next_stat = load_stat(it + 1);
      }
      named_bar_sync(1, 256);
      if (!warp_mbar_wait(&bars->st_full[b], (it >> 1) & 1, abort_flag, p.status, 300 + b)) { ok = false; break; }
      tc_fence_after();
      // visible iff kv <= q + off  <=>  q_local >= kvi - off - q0
      const int first_visible = p.causal ? (kvi - causal_off - q0) : 0;
      // this thread's key column carries its own masked query-row ranges (made local to the sub-tile here)
      int4 b4 = make_int4(0, 0, 0, 0);
      if (kMask && kvi < p.Sk) {
        const int mh = p.mask_heads == 1 ? 0 : (p.mask_heads == p.Hq ? qh : kv_head);
        b4 = __ldg(p.bounds + (static_cast<size_t>(batch) * p.mask_heads + mh) * p.Sk + kvi);
        b4.x -= q0; b4.y -= q0; b4.z -= q0; b4.w -= q0;
      }
      const uint32_t buf = tmem + lane_base + COL_BUF + b * 128;
      uint32_t s_r[32], dp_r[32];
      tmem_ld_32x32(buf + OFF_ST + h * 32, s_r);
      tmem_ld_32x32(buf + OFF_DPT + h * 32, dp_r);
      tmem_ld_wait();
      // P^T / dS^T go over S^T, and one half's outputs land on the columns the OTHER half reads its S^T from: nobody
      // writes before both halves hold their inputs in registers
      tc_fence_before();
      named_bar_sync(4, 256);
      tc_fence_after();
      const float* st = stats + b * 128;
      uint8_t* row_ptr = sDS + b * DS_BYTES + row * 128;
      {
        uint32_t pk_p[16], pk_ds[16];
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(st + h * 32 + c);
          const float4 d4 = *reinterpret_cast<const float4*>(st + 64 + h * 32 + c);
          const float l2[4] = {l4.x, l4.y, l4.z, l4.w}, dl[4] = {d4.x, d4.y, d4.z, d4.w};
          float pv[4], dsv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float pe = fast_exp2(fmaf(__uint_as_float(s_r[c + e]), p.scale_log2, -l2[e]));
            const int ql = h * 32 + c + e;
            if (ql < first_visible || (kMask && ((ql >= b4.x && ql < b4.y) || (ql >= b4.z && ql < b4.w)))) pe = 0.f;
            pv[e] = pe;
            dsv[e] = pe * (__uint_as_float(dp_r[c + e]) - dl[e]) * p.scale;
          }
          pk_p[c >> 1] = pack_bf16x2(pv[0], pv[1]);
          pk_p[(c >> 1) + 1] = pack_bf16x2(pv[2], pv[3]);
          pk_ds[c >> 1] = pack_bf16x2(dsv[0], dsv[1]);
          pk_ds[(c >> 1) + 1] = pack_bf16x2(dsv[2], dsv[3]);
        }
        tmem_st_32x16(buf + OFF_PT + h * 16, pk_p);
        tmem_st_32x16(buf + OFF_DST + h * 16, pk_ds);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
          *reinterpret_cast<uint4*>(row_ptr + (((h * 4 + jj) ^ sw) << 4)) =
              make_uint4(pk_ds[4 * jj], pk_ds[4 * jj + 1], pk_ds[4 * jj + 2], pk_ds[4 * jj + 3]);
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars->pds_full[b]);
    }
    // ---- final (first softmax warpgroup): dK, dV (fp32 in TMEM) -> bf16 -> swizzled staging (Q/dO ring is idle now)
    // -> TMA store
    if (h == 0 && ok && n_it > 0) ok = warp_mbar_wait(&bars->dkv_full, 0, abort_flag, p.status, 310);
    if (h == 0) named_bar_sync(3, 128);
    if (h == 0 && ok) {
      tc_fence_after();
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        uint8_t* stage = sQ + which * KV_TILE;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          if (n_it > 0) {
            tmem_ld_32x32(tmem + lane_base + (which == 0 ? COL_DK : COL_DV) + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          uint8_t* row_ptr = stage + (c >> 1) * KV_HALF + row * 128;
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * jj + 0]), __uint_as_float(r[8 * jj + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[8 * jj + 2]), __uint_as_float(r[8 * jj + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[8 * jj + 4]), __uint_as_float(r[8 * jj + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[8 * jj + 6]), __uint_as_float(r[8 * jj + 7]));
            *reinterpret_cast<uint4*>(row_ptr + ((((c & 1) * 4 + jj) ^ sw) << 4)) = v;
          }
        }
      }
      fence_proxy_async_smem();
    }
    if (h == 0) named_bar_sync(3, 128);
    if (h == 0 && ok && threadIdx.x == 0) {
      tma_store_4d(&tmDK, sQ, 0, kv_head, kv0, batch);
      tma_store_4d(&tmDK, sQ + KV_HALF, 64, kv_head, kv0, batch);
      tma_store_4d(&tmDV, sQ + KV_TILE, 0, kv_head, kv0, batch);
      tma_store_4d(&tmDV, sQ + KV_TILE + KV_HALF, 64, kv_head, kv0, batch);
      tma_commit_group();
      tma_wait_group<0>();
    }
  } else {
    // ---------------------------------------------------------------- dQ drain warps (4..7): thread = d
    const int dr = threadIdx.x - 128;                 // 0..127 = head-dim index = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    float* stage = reinterpret_cast<float*>(sDQ);
    for (int it = 0; it < n_it; ++it) {
      if (dr == 0) {
        const bool ok = mbar_wait(&bars->dq_full[it & 1], (it >> 1) & 1, abort_flag, p.status, 400 + (it & 1));
        if (ok) tma_wait_group_read<0>();             // previous reduce has read the staging tile
        bars->drain_decision = ok ? 1 : 0;
      }
      named_bar_sync(2, 128);
      if (bars->drain_decision == 0) break;
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld_32x32(tmem + lane_base + COL_BUF + (it & 1) * 128 + OFF_DQT, r0);
      tmem_ld_32x32(tmem + lane_base + COL_BUF + (it & 1) * 128 + OFF_DQT + 32, r1);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&bars->dq_empty[it & 1]);
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        stage[c * D + dr] = __uint_as_float(r0[c]);
        stage[(c + 32) * D + dr] = __uint_as_float(r1[c]);
      }
      fence_proxy_async_smem();
      named_bar_sync(2, 128);
      if (dr == 0) {
        const int qh = kv_head * group + it / per_head;
        const int q0 = (t0 + it % per_head) * BQ;
        tma_reduce_add_4d(&tmDQ, sDQ, 0, qh, q0, batch);
        tma_commit_group();
      }
    }
    if (dr == 0) tma_wait_group<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, 512);
}

// delta[b, h, s] = sum_d dO * O     (one warp per row)
__global__ void delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                             float* __restrict__ delta, int B, int S, int H, int64_t o_tok, int64_t o_batch,
                             int64_t do_tok, int64_t do_batch) {
  const int64_t w = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t total = static_cast<int64_t>(B) * S * H;
  if (w >= total) return;
  const int h = static_cast<int>(w % H);
  const int64_t bs = w / H;
  const int s = static_cast<int>(bs % S), b = static_cast<int>(bs / S);
  const uint2 a = *reinterpret_cast<const uint2*>(o + b * o_batch + s * o_tok + h * D + lane * 4);
  const uint2 g = *reinterpret_cast<const uint2*>(d_o + b * do_batch + s * do_tok + h * D + lane * 4);
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  const float2 g0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g.x));
  const float2 g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g.y));
  float acc = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[(static_cast<size_t>(b) * H + h) * S + s] = acc;
}

// dq (bf16, [B, S, H, 128] with token / batch strides) = dq_acc (fp32, contiguous); 32 threads per row
__global__ void dq_convert_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t rows,
                                  int S, int H, int64_t tok, int64_t batch) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < rows * 32;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i >> 5;
    const int c = static_cast<int>(i & 31) * 4;
    const int h = static_cast<int>(row % H);
    const int64_t bs = row / H;
    const int64_t s = bs % S, b = bs / S;
    const float4 v = *reinterpret_cast<const float4*>(src + row * D + c);
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(dst + b * batch + s * tok + static_cast<int64_t>(h) * D + c) = o;
  }
}

static bool make_map_bf16(CUtensorMap* m, const void* ptr, int B, int S, int H, int64_t tok, int64_t batch,
                          uint32_t rows) {
  uint64_t dims[4] = {D, static_cast<uint64_t>(H), static_cast<uint64_t>(S), static_cast<uint64_t>(B)};
  uint64_t strides[3] = {D * 2, static_cast<uint64_t>(tok) * 2, static_cast<uint64_t>(batch) * 2};
  uint32_t box[4] = {64, 1, rows, 1};
  return encode_tmap(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace fab
}  // namespace pd

// dq_acc: zero-initialised fp32 [B, Sq, Hq, 128] (contiguous); delta: fp32 [B, Hq, Sq] scratch;
// dq/dk/dv: bf16 outputs [B, S, H, 128] with their own token / batch strides (e.g. views of a packed dqkv).  `unused` keeps the argument list stable.
PD_EXPORT int pd_flash_attn_bwd(const void* d_o, const void* q, const void* k, const void* v, const void* o,
                                const float* lse, float* delta, float* dq_acc, void* unused, void* dq, void* dk,
                                void* dv, int B, int Sq, int Sk, int Hq, int Hkv, int64_t q_tok, int64_t q_batch,
                                int64_t k_tok, int64_t k_batch, int64_t v_tok, int64_t v_batch, int64_t o_tok,
                                int64_t o_batch, int64_t do_tok, int64_t do_batch, int64_t dq_tok, int64_t dq_batch,
                                int64_t dk_tok, int64_t dk_batch, int64_t dv_tok, int64_t dv_batch, float scale, int causal,
                                const void* bounds, const void* tile_bounds, int mask_heads, int* status,
                                cudaStream_t stream) {
  using namespace pd;
  using namespace pd::fab;
  (void)unused;
  if (B <= 0 || Sq <= 0 || Sk <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0) return kErrBadShape;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(d_o)) return kErrAlignment;
  if ((q_tok % 8) || (k_tok % 8) || (v_tok % 8) || (o_tok % 8) || (do_tok % 8)) return kErrAlignment;
  CUtensorMap tmQ, tmDO, tmK, tmV, tmDQ, tmDK, tmDV;
  bool ok = make_map_bf16(&tmQ, q, B, Sq, Hq, q_tok, q_batch, BQ) &&
            make_map_bf16(&tmDO, d_o, B, Sq, Hq, do_tok, do_batch, BQ) &&
            make_map_bf16(&tmK, k, B, Sk, Hkv, k_tok, k_batch, BKV) &&
            make_map_bf16(&tmV, v, B, Sk, Hkv, v_tok, v_batch, BKV) &&
            make_map_bf16(&tmDK, dk, B, Sk, Hkv, dk_tok, dk_batch, BKV) &&
            make_map_bf16(&tmDV, dv, B, Sk, Hkv, dv_tok, dv_batch, BKV);
  {
    uint64_t dims[4] = {D, static_cast<uint64_t>(Hq), static_cast<uint64_t>(Sq), static_cast<uint64_t>(B)};
    uint64_t strides[3] = {D * 4, static_cast<uint64_t>(Hq) * D * 4, static_cast<uint64_t>(Sq) * Hq * D * 4};
    uint32_t box[4] = {D, 1, BQ, 1};
    ok = ok && encode_tmap(&tmDQ, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dq_acc, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_NONE);
  }
  if (!ok) return kErrTensorMap;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(flash_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return kErrCuda;
    configured = true;
  }
  const int64_t rows = static_cast<int64_t>(B) * Sq * Hq;
  delta_kernel<<<static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, delta, B, Sq, Hq, o_tok, o_batch, do_tok, do_batch);
  if (bounds != nullptr && (mask_heads != 1 && mask_heads != Hq && mask_heads != Hkv)) return kErrBadShape;
  if (bounds != nullptr && (!aligned16(bounds) || tile_bounds == nullptr || !aligned16(tile_bounds))) return kErrAlignment;
  Params p{B, Sq, Sk, Hq, Hkv, causal, scale, scale * 1.4426950408889634f, lse, delta, status,
           static_cast<const int4*>(bounds), mask_heads, static_cast<const int4*>(tile_bounds)};
  dim3 grid((Sk + BKV - 1) / BKV, Hkv, B);
  if (bounds != nullptr) flash_bwd_kernel<true><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmQ, tmDO, tmK, tmV, tmDQ, tmDK, tmDV, p);
  else flash_bwd_kernel<false><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmQ, tmDO, tmK, tmV, tmDQ, tmDK, tmDV, p);
  int64_t blocks = (rows * 32 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  dq_convert_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(dq_acc, (__nv_bfloat16*)dq, rows, Sq, Hq, dq_tok,
                                                                       dq_batch);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}
