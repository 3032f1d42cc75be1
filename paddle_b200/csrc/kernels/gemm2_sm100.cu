// Two-SM (cta_group::2) variant of the persistent bf16 GEMM for sm_100a:  C[M,N] (=|+=) op(A)[M,K] * op(B)[K,N]
//
// A cluster of two CTAs (one SM pair) owns a 256 x 256 output tile.  CTA r of the pair loads rows [128 r, 128 r + 128)
// of the A tile and columns [128 r, 128 r + 128) of the B tile into ITS OWN shared memory (plain per-CTA TMA loads, no
// cluster multicast), so every k-block costs each SM 32 KB of shared-memory fill instead of the 48 KB of the
// 128 x 256 single-CTA tile, and the tensor core reads half of B from the partner SM.  One thread of the leader CTA
// (cluster rank 0) issues tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 16); the accumulator rows 0-127 live in the
// leader's TMEM, rows 128-255 in the partner's, and each CTA's four epilogue warps drain their own half.
//
// Barriers (all waits bounded, see sm100_prims.cuh):
//   full[s]   leader only, 1 arrival + transaction bytes of BOTH CTAs (the partner's TMA loads complete on the
//             leader's barrier through the .cta_group::2 form of the load)
//   empty[s]  in both CTAs, released by tcgen05.commit.cta_group::2 with a CTA mask of both
//   tfull[a]  in both CTAs, same commit form: accumulator a is complete
//   tempty[a] leader only, 2 arrivals: each CTA's epilogue has drained its half of accumulator a
// Same operand-layout support, epilogues (bf16 store / fp32 store / fp32 reduce-add) and split-K slicing as
// gemm_sm100.cu; replaces the cuBLAS call behind matmul / linear
// (reference: paddle/phi/kernels/funcs/blas/blas_impl.cu.h:426).
#include "host_utils.h"
#include "sm100_prims.cuh"

namespace pd {
namespace gemm2 {

constexpr int BM = 128, BN_HALF = 128, BK = 64, STAGES = 6;
constexpr int TILE_M = 256, TILE_N = 256;
constexpr int A_STAGE_BYTES = BM * BK * 2;        // 16 KB
constexpr int B_STAGE_BYTES = BN_HALF * BK * 2;   // 16 KB
constexpr int C_CHUNK_BYTES = BM * 128;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 2 * C_CHUNK_BYTES + 1024 + 256;
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;   // clears the CTA-pair bit of a shared::cluster address -> leader CTA

enum Epi : int { kStoreBf16 = 0, kStoreF32 = 1, kAccumF32 = 2, kBiasAct = 3, kSwiglu = 4 };
// kBiasAct: C = act(A B + bias) as bf16 (bias bf16 [N] or null; act: 0 none, 1 relu, 2 gelu (erf), 3 gelu (tanh),
// 4 silu) - the reference's fused_gemm_epilogue (paddle/phi/kernels/fusion/gpu/fused_gemm_epilogue_kernel.cu).
// kSwiglu: the N columns hold (gate, up) pairs interleaved; C [M, N / 2] = silu(gate) * up as bf16, i.e. the first
// feed-forward GEMM with its activation, without the [M, N] intermediate ever reaching memory.
__device__ __forceinline__ float apply_act(float x, int act) {
  switch (act) {
    case 1: return fmaxf(x, 0.f);
    case 2: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case 3: return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    case 4: return x / (1.f + __expf(-x));
    default: return x;
  }
}

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tfull[2];
  uint64_t tempty[2];
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
  int epi_decision;
};

// ---- cluster / cta_group::2 primitives
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t cta) {
  uint32_t raddr;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(smem_u32(bar)), "r"(cta));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(raddr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_2cta(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_bf16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at this shared-memory offset in BOTH CTAs of the pair once all MMAs issued so far are complete
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}
// per-CTA tiled loads whose completion bytes are counted on the LEADER CTA's barrier (no data multicast)
__device__ __forceinline__ void tma2_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar) & PEER_BIT_MASK), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma2_load_3d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar) & PEER_BIT_MASK), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int G = 8;  // 256-row tiles per raster group: keeps a wave's A/B working set inside L2
  const int per_group = G * tiles_n;
  const int g = t / per_group;
  const int first_m = g * G;
  const int gsz = min(G, tiles_m - first_m);
  const int r = t - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

// a 128 x 64 operand block (rows = M or N index of this CTA's half) into one stage
template <bool MN>
__device__ __forceinline__ void load_half(void* dst, const CUtensorMap* tm, uint64_t* bar, int mn0, int k0, bool use3d) {
  if (!MN) {
    tma2_load_2d(dst, tm, bar, k0, mn0);                        // box {64 k, 128 rows}
  } else if (use3d) {
    tma2_load_3d(dst, tm, bar, 0, k0, mn0 >> 6);                // one box {64 mn, 64 k, 2 chunks}
  } else {
#pragma unroll
    for (int c = 0; c < 2; ++c)                                  // boxes {64 mn, 64 k}
      tma2_load_2d(static_cast<uint8_t*>(dst) + c * 8192, tm, bar, mn0 + c * 64, k0);
  }
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, int M, int N, int K, int mn3d, int splits, int* status,
                  const __nv_bfloat16* bias, int act) {
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared memory starts at the same offset in both CTAs, so the aligned carve-up is identical in both
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint8_t* sC = sB + STAGES * B_STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(sC + 2 * C_CHUNK_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();          // 0 = leader
  const bool leader = cta_rank == 0;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int tiles_m = (M + TILE_M - 1) / TILE_M, tiles_n = (N + TILE_N - 1) / TILE_N;
  const int KB_total = (K + BK - 1) / BK;
  const int KBS = (KB_total + splits - 1) / splits;
  const int num_tiles = tiles_m * tiles_n * splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tfull[a], 1);
      mbar_init(&bars->tempty[a], 2);
    }
    mbar_init(&bars->drain, 1);
    bars->abort_flag = 0;
    bars->epi_decision = 0;
    fence_mbar_init();
  }
  if (warp == 5) tmem_alloc_2cta(&bars->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // both CTAs' barriers are initialised before any remote arrive / remote completion
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer (one per CTA: its halves of A and B)
    if (lane == 0) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int issued = 0;
      for (int t = cluster_id; t < num_tiles && ok; t += n_clusters) {
        int tm, tn;
        tile_coords(t / splits, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * TILE_M + static_cast<int>(cta_rank) * BM;
        const int n0 = tn * TILE_N + static_cast<int>(cta_rank) * BN_HALF;
        const int kb0 = (t % splits) * KBS, kb1 = min(KB_total, kb0 + KBS);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_flag, status, 100 + s)) { ok = false; break; }
          if (leader) mbar_expect_tx(&bars->full[s], 2 * (A_STAGE_BYTES + B_STAGE_BYTES));
          const int k0 = kb * BK;
          load_half<A_MN>(sA + s * A_STAGE_BYTES, &tmA, &bars->full[s], m0, k0, (mn3d & 1) != 0);
          load_half<B_MN>(sB + s * B_STAGE_BYTES, &tmB, &bars->full[s], n0, k0, (mn3d & 2) != 0);
          ++issued;
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok && leader) {  // drain the loads that were armed but never consumed before the CTA may exit
        for (int i = 0; i < STAGES && i < issued; ++i) mbar_drain(&bars->full[i], 0), mbar_drain(&bars->full[i], 1);
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc(TILE_M, TILE_N, A_MN, B_MN);
      constexpr uint32_t a_kstep = A_MN ? 2048u : 32u;
      constexpr uint32_t b_kstep = B_MN ? 2048u : 32u;
      constexpr uint32_t a_lbo = A_MN ? 8192u : 16u;
      constexpr uint32_t b_lbo = B_MN ? 8192u : 16u;
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += n_clusters, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!mbar_wait(&bars->tempty[acc], acc_ph ^ 1, abort_flag, status, 200 + acc)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TILE_N;
        const int kb0 = (t % splits) * KBS, kb1 = min(KB_total, kb0 + KBS);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&bars->full[s], ph, abort_flag, status, 300 + s)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = make_smem_desc_sw128(a_addr + k * a_kstep, a_lbo, 1024);
            const uint64_t bd = make_smem_desc_sw128(b_addr + k * b_kstep, b_lbo, 1024);
            umma2_bf16_ss(d_tmem, ad, bd, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
          }
          umma2_commit_both(&bars->empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma2_commit_both(&bars->tfull[acc]);
      }
      if (!ok) {
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bars->drain))
                     : "memory");
        mbar_drain(&bars->drain, 0);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 0..3 of each CTA: its 128 rows)
    const int epi_tid = threadIdx.x;
    constexpr int CW = (EPI == kStoreBf16 || EPI == kBiasAct) ? 64 : (EPI == kSwiglu ? 128 : 32);
    constexpr int NCHUNK = TILE_N / CW;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    int it = 0;
    int chunk_counter = 0;
    for (int t = cluster_id; t < num_tiles; t += n_clusters, ++it) {
      int tm, tn;
      tile_coords(t / splits, tiles_m, tiles_n, tm, tn);
      const int m0 = tm * TILE_M + static_cast<int>(cta_rank) * BM, n0 = tn * TILE_N;
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      if (epi_tid == 0) {
        const bool ok = mbar_wait(&bars->tfull[acc], acc_ph, abort_flag, status, 400 + acc);
        bars->epi_decision = ok ? 1 : 0;
      }
      named_bar_sync(1, 128);
      if (bars->epi_decision == 0) break;
      tc_fence_after();
      const uint32_t t_acc = tmem_base + lane_base + acc * TILE_N;
      const bool rows_live = m0 < M;          // a partner half entirely below the matrix stores nothing
#pragma unroll 1
      for (int c = 0; c < NCHUNK; ++c, ++chunk_counter) {
        uint8_t* stage = sC + (chunk_counter & 1) * C_CHUNK_BYTES;
        if (epi_tid == 0) tma_wait_group_read<1>();
        named_bar_sync(1, 128);
        uint8_t* row_ptr = stage + epi_tid * 128;
        const int sw = epi_tid & 7;
        if (EPI == kSwiglu) {
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            uint32_t r[32];
            tmem_ld_32x32(t_acc + c * CW + h * 32, r);
            tmem_ld_wait();
            float o[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float g = __uint_as_float(r[2 * i]), u = __uint_as_float(r[2 * i + 1]);
              o[i] = g / (1.f + __expf(-g)) * u;
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              uint4 v;
              v.x = pack_bf16x2(o[8 * j + 0], o[8 * j + 1]);
              v.y = pack_bf16x2(o[8 * j + 2], o[8 * j + 3]);
              v.z = pack_bf16x2(o[8 * j + 4], o[8 * j + 5]);
              v.w = pack_bf16x2(o[8 * j + 6], o[8 * j + 7]);
              *reinterpret_cast<uint4*>(row_ptr + (((h * 2 + j) ^ sw) << 4)) = v;
            }
          }
        } else if (EPI == kStoreBf16 || EPI == kBiasAct) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld_32x32(t_acc + c * CW + h * 32, r);
            tmem_ld_wait();
            if (EPI == kBiasAct) {
              const int col0 = n0 + c * CW + h * 32;
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                float x = __uint_as_float(r[i]);
                if (bias != nullptr && col0 + i < N) x += __bfloat162float(__ldg(bias + col0 + i));
                r[i] = __float_as_uint(apply_act(x, act));
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
              v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
              v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
              v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
              *reinterpret_cast<uint4*>(row_ptr + (((h * 4 + j) ^ sw) << 4)) = v;
            }
          }
        } else {
          uint32_t r[32];
          tmem_ld_32x32(t_acc + c * CW, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 v = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            *reinterpret_cast<uint4*>(row_ptr + ((j ^ sw) << 4)) = v;
          }
        }
        if (c == NCHUNK - 1) tc_fence_before();
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (epi_tid == 0) {
          if (c == NCHUNK - 1) {   // this CTA's half of the accumulator is drained: tell the leader's MMA thread
            if (leader) mbar_arrive(&bars->tempty[acc]);
            else mbar_arrive_remote(&bars->tempty[acc], 0);
          }
          if (rows_live && n0 + c * CW < N) {
            if (EPI == kAccumF32) tma_reduce_add_2d(&tmC, stage, n0 + c * CW, m0);
            else if (EPI == kSwiglu) tma_store_2d(&tmC, stage, (n0 + c * CW) / 2, m0);
            else tma_store_2d(&tmC, stage, n0 + c * CW, m0);
          }
          tma_commit_group();
        }
      }
    }
    if (epi_tid == 0) tma_wait_group<0>();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // nobody leaves while the partner may still signal this CTA's barriers or read its tiles
  if (warp == 5) tmem_dealloc_2cta(tmem_base, 512);
}

template <bool A_MN, bool B_MN, int EPI>
static int launch_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, int M, int N, int K,
                          int mn3d, int* status, cudaStream_t stream, int max_ctas, int splits,
                          const __nv_bfloat16* bias = nullptr, int act = 0) {
  auto kfn = gemm2_bf16_kernel<A_MN, B_MN, EPI>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return kErrCuda;
    configured = true;
  }
  const int tiles = ((M + TILE_M - 1) / TILE_M) * ((N + TILE_N - 1) / TILE_N) * splits;
  int clusters = sm_count() / 2;
  if (max_ctas > 0 && clusters > max_ctas / 2) clusters = max_ctas / 2;
  if (clusters > tiles) clusters = tiles;
  if (clusters < 1) clusters = 1;
  kfn<<<clusters * 2, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, tmC, M, N, K, mn3d, splits, status, bias, act);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

}  // namespace gemm2
}  // namespace pd

// Same contract as pd_gemm_bf16 / pd_gemm_bf16_splitk (gemm_sm100.cu); splits = 1 for the plain form.
PD_EXPORT int pd_gemm_bf16_2cta(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                int a_mn_major, int b_mn_major, int epi, int max_ctas, int splits, int* status,
                                cudaStream_t stream) {
  using namespace pd;
  using namespace pd::gemm2;
  if (M <= 0 || N <= 0 || K <= 0 || splits < 1) return kErrBadShape;
  if (splits > 1 && epi != kAccumF32) return kErrBadShape;
  {
    const int kb_total = (K + BK - 1) / BK;
    if (splits > kb_total) splits = kb_total;
    const int kbs = (kb_total + splits - 1) / splits;
    splits = (kb_total + kbs - 1) / kbs;
  }
  if (!aligned16(A) || !aligned16(B) || !aligned16(C)) return kErrAlignment;
  if ((lda % 8) || (ldb % 8) || (epi == kStoreBf16 ? (ldc % 8) : (ldc % 4))) return kErrAlignment;
  CUtensorMap tmA, tmB, tmC;
  bool ok = true;
  int a3d = 0, b3d = 0;
  if (!a_mn_major) ok &= encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, A, K, M, uint64_t(lda) * 2, BK, BM);
  else ok &= encode_tmap_mn(&tmA, A, M, K, uint64_t(lda) * 2, BM / 64, BK, &a3d);
  if (!b_mn_major) ok &= encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, B, K, N, uint64_t(ldb) * 2, BK, BN_HALF);
  else ok &= encode_tmap_mn(&tmB, B, N, K, uint64_t(ldb) * 2, BN_HALF / 64, BK, &b3d);
  if (epi == kStoreBf16) ok &= encode_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, C, N, M, uint64_t(ldc) * 2, 64, BM);
  else ok &= encode_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, C, N, M, uint64_t(ldc) * 4, 32, BM);
  if (!ok) return kErrTensorMap;
#define PD_GEMM2_CASE(AM, BM_, E)                                                                  \
  if (a_mn_major == AM && b_mn_major == BM_ && epi == E)                                           \
    return launch_variant<AM, BM_, E>(tmA, tmB, tmC, M, N, K, a3d | (b3d << 1), status, stream, max_ctas, splits);
  PD_GEMM2_CASE(0, 0, 0) PD_GEMM2_CASE(0, 1, 0) PD_GEMM2_CASE(1, 0, 0) PD_GEMM2_CASE(1, 1, 0)
  PD_GEMM2_CASE(0, 0, 1) PD_GEMM2_CASE(0, 1, 1) PD_GEMM2_CASE(1, 0, 1) PD_GEMM2_CASE(1, 1, 1)
  PD_GEMM2_CASE(0, 0, 2) PD_GEMM2_CASE(0, 1, 2) PD_GEMM2_CASE(1, 0, 2) PD_GEMM2_CASE(1, 1, 2)
#undef PD_GEMM2_CASE
  return kErrBadShape;
}

// C = act(A B + bias) (swiglu = 0; C bf16 [M, N]) or C = silu(gate) * up over interleaved (gate, up) column pairs
// (swiglu = 1; C bf16 [M, N / 2], N a multiple of 16, bias must be null).  Operand layouts as pd_gemm_bf16_2cta.
PD_EXPORT int pd_gemm_bf16_2cta_epi(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                    int a_mn_major, int b_mn_major, const void* bias, int act, int swiglu, int* status,
                                    cudaStream_t stream) {
  using namespace pd;
  using namespace pd::gemm2;
  if (M <= 0 || N <= 0 || K <= 0 || act < 0 || act > 4) return kErrBadShape;
  if (swiglu && (bias != nullptr || (N % 16))) return kErrBadShape;
  if (!aligned16(A) || !aligned16(B) || !aligned16(C)) return kErrAlignment;
  if ((lda % 8) || (ldb % 8) || (ldc % 8)) return kErrAlignment;
  CUtensorMap tmA, tmB, tmC;
  bool ok = true;
  int a3d = 0, b3d = 0;
  if (!a_mn_major) ok &= encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, A, K, M, uint64_t(lda) * 2, BK, BM);
  else ok &= encode_tmap_mn(&tmA, A, M, K, uint64_t(lda) * 2, BM / 64, BK, &a3d);
  if (!b_mn_major) ok &= encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, B, K, N, uint64_t(ldb) * 2, BK, BN_HALF);
  else ok &= encode_tmap_mn(&tmB, B, N, K, uint64_t(ldb) * 2, BN_HALF / 64, BK, &b3d);
  ok &= encode_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, C, swiglu ? N / 2 : N, M, uint64_t(ldc) * 2, 64, BM);
  if (!ok) return kErrTensorMap;
  const __nv_bfloat16* bp = static_cast<const __nv_bfloat16*>(bias);
#define PD_GEMM2_EPI_CASE(AM, BM_)                                                                              \
  if (a_mn_major == AM && b_mn_major == BM_) {                                                                  \
    if (swiglu) return launch_variant<AM, BM_, kSwiglu>(tmA, tmB, tmC, M, N, K, a3d | (b3d << 1), status, stream, 0, 1); \
    return launch_variant<AM, BM_, kBiasAct>(tmA, tmB, tmC, M, N, K, a3d | (b3d << 1), status, stream, 0, 1, bp, act);   \
  }
  PD_GEMM2_EPI_CASE(0, 0) PD_GEMM2_EPI_CASE(0, 1) PD_GEMM2_EPI_CASE(1, 0) PD_GEMM2_EPI_CASE(1, 1)
#undef PD_GEMM2_EPI_CASE
  return kErrBadShape;
}
