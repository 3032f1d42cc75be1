// Flash-attention forward for sm_100a, head_dim 128, bf16, causal or full, GQA.
//   O = softmax(Q K^T * scale [+ causal mask]) V,   LSE = log-sum-exp per query row (natural log)
// Layout [batch, seq, heads, 128] with arbitrary token/batch strides (q/k/v may be views into one
// packed qkv buffer), as in the reference API (python/paddle/nn/functional/flash_attention.py:358;
// the reference itself calls the external FA2 library: paddle/phi/kernels/gpu/flash_attn_kernel.cu:517).
//
// One CTA per (128-query tile, head, batch):
//   warp 4 : TMA producer (Q once, K/V tiles through two 2-stage rings, 128B swizzle)
//   warp 5 : tcgen05.mma issuer:  S_j = Q K_j^T (SS, both K-major) into a double-buffered TMEM tile,
//            O += P_j V_j (A = P from TMEM, B = V MN-major from smem)
//   warps 0-3 : softmax, one query row per thread (= one TMEM lane): tcgen05.ld S, online max /
//            exp2 / sum with lazy rescaling of the O accumulator in TMEM, P written back to TMEM as
//            packed bf16, final O / l through a swizzled staging tile and TMA store.
// The S_{j+1} GEMM is issued before the softmax of S_j finishes, so tensor cores and the softmax
// warps overlap.  TMEM columns: S0 0-127, S1 128-255, O 256-383, P0 384-447, P1 448-511.
#include <math.h>

#include "host_utils.h"
#include "sm100_prims.cuh"

namespace pd {
namespace fa {

constexpr int BQ = 128, BKV = 128, D = 128;
constexpr int TILE_BYTES = 128 * D * 2;       // 32 KB: two 16 KB swizzled boxes of [128 rows x 64 d]
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int KV_STAGES = 2;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = TILE_BYTES * (1 + 2 * KV_STAGES) + 1024 + 256;
constexpr uint32_t COL_S = 0, COL_O = 256, COL_P = 384;

struct Barriers {
  uint64_t q_full;
  uint64_t k_full[KV_STAGES], k_empty[KV_STAGES];
  uint64_t v_full[KV_STAGES], v_empty[KV_STAGES];
  uint64_t s_full[2], p_full[2];
  uint64_t o_full;
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
  int j_lo, j_hi;       // key tiles [j_lo, j_hi) are visited (mask-aware)
};

struct Params {
  int B, Sq, Sk, Hq, Hkv;
  int causal;
  float scale_log2;   // softmax scale * log2(e)
  float* lse;         // [B, Hq, Sq]
  int* status;
  // column-sparse mask (flashmask): per key column four query-row bounds {lts, lte, uts, ute}; query row r does not
  // see column c iff lts <= r < lte or uts <= r < ute.  [B, mask_heads, Sk] with mask_heads 1, Hkv or Hq; null = none.
  const int4* bounds;
  int mask_heads;
  // per 128-column key tile: {max lts, min lte, max uts, min ute} over its columns, [B, mask_heads, ceil(Sk / 128)];
  // a (query tile, key tile) pair is skipped when one of the two ranges covers every row of the query tile for every
  // column of the key tile
  const int4* tile_bounds;
};

// lane 0 performs the bounded wait, the verdict is shared so that the warp stays convergent for the
// warp-collective tcgen05.ld/st that follow; every lane then observes the completed phase itself.
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
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                 Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                               // also the output staging tile at the end
  uint8_t* sK = sQ + TILE_BYTES;
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(sV + KV_STAGES * TILE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qblocks = (p.Sq + BQ - 1) / BQ;
  const int qb = n_qblocks - 1 - static_cast<int>(blockIdx.x);   // heavy (late) causal tiles first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int q0 = qb * BQ;
  const int causal_off = p.Sk - p.Sq;                             // key j visible to query i iff j <= i + off
  int kv_len = p.Sk;
  if (p.causal) kv_len = min(p.Sk, q0 + BQ + causal_off);
  int n_kv = kv_len > 0 ? (kv_len + BKV - 1) / BKV : 0;
  int jbase = 0;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->p_full[s], 128);
    }
    mbar_init(&bars->o_full, 1);
    mbar_init(&bars->drain, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 5) tmem_alloc(&bars->tmem_base, 512);
  if (kMask && warp == 1) {
    // first and last key tile that is not masked out as a whole for this query tile
    const int mh = p.mask_heads == 1 ? 0 : (p.mask_heads == p.Hq ? head : kv_head);
    const int tiles_k = (p.Sk + BKV - 1) / BKV;
    const int4* tb = p.tile_bounds + (static_cast<size_t>(batch) * p.mask_heads + mh) * tiles_k;
    int lo = n_kv, hi = 0;
    for (int j = lane; j < n_kv; j += 32) {
      const int4 b = __ldg(tb + j);
      const bool dead = (b.x <= q0 && b.y >= q0 + BQ) || (b.z <= q0 && b.w >= q0 + BQ);
      if (!dead) {
        lo = min(lo, j);
        hi = max(hi, j + 1);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    if (lane == 0) {
      bars->j_lo = lo;
      bars->j_hi = hi;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  if (kMask) {
    jbase = bars->j_lo;
    n_kv = bars->j_hi > bars->j_lo ? bars->j_hi - bars->j_lo : 0;
  }

  if (warp == 4) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      prefetch_tmap(&tmQ);
      prefetch_tmap(&tmK);
      prefetch_tmap(&tmV);
      mbar_expect_tx(&bars->q_full, TILE_BYTES);
      tma_load_4d(sQ, &tmQ, &bars->q_full, 0, head, q0, batch);
      tma_load_4d(sQ + HALF_BYTES, &tmQ, &bars->q_full, 64, head, q0, batch);
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(&bars->k_empty[s], ph ^ 1, abort_flag, p.status, 100 + s)) { ok = false; break; }
        mbar_expect_tx(&bars->k_full[s], TILE_BYTES);
        tma_load_4d(sK + s * TILE_BYTES, &tmK, &bars->k_full[s], 0, kv_head, (jbase + j) * BKV, batch);
        tma_load_4d(sK + s * TILE_BYTES + HALF_BYTES, &tmK, &bars->k_full[s], 64, kv_head, (jbase + j) * BKV, batch);
        if (!mbar_wait(&bars->v_empty[s], ph ^ 1, abort_flag, p.status, 110 + s)) {
          mbar_drain(&bars->k_full[s], ph);
          ok = false;
          break;
        }
        mbar_expect_tx(&bars->v_full[s], TILE_BYTES);
        tma_load_4d(sV + s * TILE_BYTES, &tmV, &bars->v_full[s], 0, kv_head, (jbase + j) * BKV, batch);
        tma_load_4d(sV + s * TILE_BYTES + HALF_BYTES, &tmV, &bars->v_full[s], 64, kv_head, (jbase + j) * BKV, batch);
      }
      if (!ok || *abort_flag) {
        mbar_drain(&bars->q_full, 0);
        for (int j = max(0, n_kv - KV_STAGES); j < n_kv; ++j) {
          mbar_drain(&bars->k_full[j % KV_STAGES], (j / KV_STAGES) & 1);
          mbar_drain(&bars->v_full[j % KV_STAGES], (j / KV_STAGES) & 1);
        }
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t idesc_qk = make_idesc(BQ, BKV, false, false);
      constexpr uint32_t idesc_pv = make_idesc(BQ, D, false, true);
      const uint32_t q_addr = smem_u32(sQ);
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag, p.status, 200);
      tc_fence_after();
      auto issue_qk = [&](int j) -> bool {
        const int s = j % KV_STAGES;
        if (!mbar_wait(&bars->k_full[s], (j / KV_STAGES) & 1, abort_flag, p.status, 210 + s)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * TILE_BYTES);
        const uint32_t d_tmem = tmem + COL_S + (j & 1) * 128;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * HALF_BYTES + (ks & 3) * 32;
          umma_bf16_ss(d_tmem, make_smem_desc_sw128(q_addr + off, 16, 1024),
                       make_smem_desc_sw128(k_addr + off, 16, 1024), idesc_qk, ks != 0 ? 1u : 0u);
        }
        umma_commit(&bars->k_empty[s]);
        umma_commit(&bars->s_full[j & 1]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          if (!issue_qk(j + 1)) { ok = false; break; }
        }
        const int s = j % KV_STAGES;
        if (!mbar_wait(&bars->p_full[j & 1], (j >> 1) & 1, abort_flag, p.status, 220 + (j & 1))) { ok = false; break; }
        if (!mbar_wait(&bars->v_full[s], (j / KV_STAGES) & 1, abort_flag, p.status, 230 + s)) { ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + s * TILE_BYTES);
        const uint32_t p_tmem = tmem + COL_P + (j & 1) * 64;
#pragma unroll
        for (int ks = 0; ks < BKV / 16; ++ks) {
          umma_bf16_ts(tmem + COL_O, p_tmem + ks * 8, make_smem_desc_sw128(v_addr + ks * 2048, HALF_BYTES, 1024),
                       idesc_pv, (j | ks) != 0 ? 1u : 0u);
        }
        umma_commit(&bars->v_empty[s]);
        umma_commit(&bars->o_full);
      }
      if (!ok) {
        umma_commit(&bars->drain);
        mbar_drain(&bars->drain, 0);
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax + epilogue (warps 0..3)
    const int row = threadIdx.x;                 // query row within the tile == TMEM lane
    const int qi = q0 + row;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!warp_mbar_wait(&bars->s_full[j & 1], (j >> 1) & 1, abort_flag, p.status, 300 + (j & 1))) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_tmem = tmem + lane_base + COL_S + (j & 1) * 128;
      const uint32_t p_tmem = tmem + lane_base + COL_P + (j & 1) * 64;
      // highest visible key column (local to this tile) for this row
      const int col0 = (jbase + j) * BKV;          // first key column of this tile
      int col_limit = p.Sk - 1 - col0;
      if (p.causal) col_limit = min(col_limit, qi + causal_off - col0);
      const bool need_mask = col_limit < BKV - 1;
      // one TMEM read of the whole 128-column row: four loads in flight, one wait
      uint32_t r[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(s_tmem + c * 32, r[c]);
      tmem_ld_wait();
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (c * 32 + i > col_limit) r[c][i] = 0xff800000u;   // -inf: contributes exp2(-inf) = 0
          }
        }
      }
      if (kMask) {
        // every lane of the warp reads the same address: one broadcast transaction per column
        const int mh = p.mask_heads == 1 ? 0 : (p.mask_heads == p.Hq ? head : kv_head);
        const int4* bnd = p.bounds + (static_cast<size_t>(batch) * p.mask_heads + mh) * p.Sk + col0;
        const int cols = min(BKV, p.Sk - col0);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (c * 32 + i < cols) {
              const int4 b4 = __ldg(bnd + c * 32 + i);
              if ((qi >= b4.x && qi < b4.y) || (qi >= b4.z && qi < b4.w)) r[c][i] = 0xff800000u;
            }
          }
        }
      }
      // row maximum with eight independent chains
      float mxs[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mxs[i] = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
#pragma unroll
          for (int q = 0; q < 8; ++q) mxs[q] = fmaxf(mxs[q], __uint_as_float(r[c][i + q]));
        }
      }
      const float mx = fmaxf(fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])),
                             fmaxf(fmaxf(mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      // lazy rescale: only when some row of the warp moved its maximum by more than 2^8
      const bool want = (j == 0) || (m_new - m_used > 8.f);
      const bool warp_want = __any_sync(0xffffffffu, want);
      float factor = 1.f;
      if (warp_want) {
        factor = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
        l *= factor;
        m_used = m_new;
      }
      const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
      // probabilities -> TMEM (packed bf16), row sum in four independent chains
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float a = fast_exp2(fmaf(__uint_as_float(r[c][i]), p.scale_log2, -m_eff));
          const float b = fast_exp2(fmaf(__uint_as_float(r[c][i + 1]), p.scale_log2, -m_eff));
          if (((i >> 1) & 3) == 0) ls[0] += a + b;
          else if (((i >> 1) & 3) == 1) ls[1] += a + b;
          else if (((i >> 1) & 3) == 2) ls[2] += a + b;
          else ls[3] += a + b;
          pk[i >> 1] = pack_bf16x2(a, b);
        }
        tmem_st_32x16(p_tmem + c * 16, pk);
      }
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      tmem_st_wait();
      if (j > 0) {
        // PV_{j-1} must have landed in O before O is rescaled and before PV_j may be issued
        if (!warp_mbar_wait(&bars->o_full, (j - 1) & 1, abort_flag, p.status, 310)) { ok = false; break; }
        tc_fence_after();
        if (warp_want) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem + lane_base + COL_O + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
            tmem_st_32x32(tmem + lane_base + COL_O + c * 32, r);
          }
          tmem_st_wait();
        }
      }
      tc_fence_before();
      mbar_arrive(&bars->p_full[j & 1]);
    }
    // ---- epilogue: O / l -> bf16 -> swizzled staging (reuses the Q tile) -> TMA store; LSE
    if (ok && n_kv > 0) ok = warp_mbar_wait(&bars->o_full, (n_kv - 1) & 1, abort_flag, p.status, 320);
    named_bar_sync(1, 128);   // every softmax warp is past its last S read: the Q tile is free
    if (ok) {
      tc_fence_after();
      const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
      const int sw = row & 7;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        if (n_kv > 0) {
          tmem_ld_32x32(tmem + lane_base + COL_O + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        uint8_t* row_ptr = sQ + (c >> 1) * HALF_BYTES + row * 128;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(r[8 * jj + 0]) * inv_l, __uint_as_float(r[8 * jj + 1]) * inv_l);
          v.y = pack_bf16x2(__uint_as_float(r[8 * jj + 2]) * inv_l, __uint_as_float(r[8 * jj + 3]) * inv_l);
          v.z = pack_bf16x2(__uint_as_float(r[8 * jj + 4]) * inv_l, __uint_as_float(r[8 * jj + 5]) * inv_l);
          v.w = pack_bf16x2(__uint_as_float(r[8 * jj + 6]) * inv_l, __uint_as_float(r[8 * jj + 7]) * inv_l);
          *reinterpret_cast<uint4*>(row_ptr + ((((c & 1) * 4 + jj) ^ sw) << 4)) = v;
        }
      }
      if (qi < p.Sq && p.lse != nullptr) {
        const float lse = (l > 0.f) ? (m_used * 0.6931471805599453f + logf(l)) : -INFINITY;
        p.lse[(static_cast<size_t>(batch) * p.Hq + head) * p.Sq + qi] = lse;
      }
      fence_proxy_async_smem();
    }
    named_bar_sync(1, 128);
    if (ok && threadIdx.x == 0) {
      tma_store_4d(&tmO, sQ, 0, head, q0, batch);
      tma_store_4d(&tmO, sQ + HALF_BYTES, 64, head, q0, batch);
      tma_commit_group();
      tma_wait_group<0>();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, 512);
}

// 4-D map over [B, S, H, 128] bf16 with element strides (token, batch); box = {64, 1, 128 rows, 1}
static bool make_map(CUtensorMap* m, const void* ptr, int B, int S, int H, int64_t tok_stride,
                     int64_t batch_stride) {
  uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(H), static_cast<uint64_t>(S),
                      static_cast<uint64_t>(B)};
  uint64_t strides[3] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(tok_stride) * 2,
                         static_cast<uint64_t>(batch_stride) * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return encode_tmap(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace fa
}  // namespace pd

// q: [B, Sq, Hq, 128], k/v: [B, Sk, Hkv, 128], o: [B, Sq, Hq, 128] (bf16; strides in elements, head
// stride must be 128), lse: [B, Hq, Sq] fp32.  bounds: optional int32 [B, mask_heads, Sk, 4] column-sparse mask
// (see Params::bounds; python/paddle/nn/functional/flash_attention.py:1299 `flashmask_attention`).
PD_EXPORT int pd_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq,
                                int Sk, int Hq, int Hkv, int64_t q_tok, int64_t q_batch, int64_t k_tok,
                                int64_t k_batch, int64_t v_tok, int64_t v_batch, int64_t o_tok, int64_t o_batch,
                                float scale, int causal, const void* bounds, const void* tile_bounds, int mask_heads,
                                int* status, cudaStream_t stream) {
  using namespace pd;
  using namespace pd::fa;
  if (bounds != nullptr && (mask_heads != 1 && mask_heads != Hq && mask_heads != Hkv)) return kErrBadShape;
  if (bounds != nullptr && (!aligned16(bounds) || tile_bounds == nullptr || !aligned16(tile_bounds))) return kErrAlignment;
  if (B <= 0 || Sq <= 0 || Sk <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0) return kErrBadShape;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return kErrAlignment;
  if ((q_tok % 8) || (k_tok % 8) || (v_tok % 8) || (o_tok % 8) || (q_batch % 8) || (k_batch % 8) ||
      (v_batch % 8) || (o_batch % 8))
    return kErrAlignment;
  CUtensorMap tmQ, tmK, tmV, tmO;
  if (!make_map(&tmQ, q, B, Sq, Hq, q_tok, q_batch) || !make_map(&tmK, k, B, Sk, Hkv, k_tok, k_batch) ||
      !make_map(&tmV, v, B, Sk, Hkv, v_tok, v_batch) || !make_map(&tmO, o, B, Sq, Hq, o_tok, o_batch))
    return kErrTensorMap;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(flash_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return kErrCuda;
    configured = true;
  }
  Params p{B, Sq, Sk, Hq, Hkv, causal, scale * 1.4426950408889634f, lse, status, static_cast<const int4*>(bounds),
           mask_heads, static_cast<const int4*>(tile_bounds)};
  dim3 grid((Sq + BQ - 1) / BQ, Hq, B);
  if (bounds != nullptr) flash_fwd_kernel<true><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmQ, tmK, tmV, tmO, p);
  else flash_fwd_kernel<false><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmQ, tmK, tmV, tmO, p);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}
