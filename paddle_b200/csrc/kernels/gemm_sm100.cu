// Persistent, warp-specialised bf16 GEMM for sm_100a:  C[M,N] (=|+=) op(A)[M,K] * op(B)[K,N]
//
//   warp 4 (1 thread)  : TMA producer — A/B tiles into a 4-stage 128B-swizzled shared-memory ring
//   warp 5 (1 thread)  : tcgen05.mma issuer — 128x256x16 UMMAs into one of two 256-column TMEM
//                        accumulators; tcgen05.commit releases ring slots / publishes accumulators
//   warps 0-3          : epilogue — tcgen05.ld, convert, swizzled staging tile, TMA store or
//                        TMA reduce-add (fp32 accumulate into an existing buffer, e.g. main_grad)
//
// While the epilogue drains accumulator t, the MMA warp already fills accumulator t+1.
// Operand layouts: every combination of K-major / MN-major A and B is supported through the
// shared-memory descriptor, so no transposes are ever materialised:
//   forward   Y = X W        : A K-major,  B MN-major   (Paddle Linear weight is [in, out])
//   dgrad     dX = dY W^T    : A K-major,  B K-major
//   wgrad     dW += X^T dY   : A MN-major, B MN-major   (fp32 reduce-add epilogue)
// Role in the framework: replaces the cuBLAS call behind matmul/linear
// (reference: paddle/phi/kernels/funcs/blas/blas_impl.cu.h:426) and the beta=1 cublasLt call of
// fused_linear_param_grad_add (paddle/phi/kernels/fusion/gpu/fused_linear_param_grad_add_kernel.cu:36).
#include "host_utils.h"
#include "sm100_prims.cuh"

namespace pd {
namespace gemm {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;   // 32 KB
constexpr int C_CHUNK_BYTES = BM * 128;      // 128 rows x 128 B
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 2 * C_CHUNK_BYTES + 1024 /*align*/ + 256;

enum Epi : int { kStoreBf16 = 0, kStoreF32 = 1, kAccumF32 = 2 };

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

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int G = 16;  // m-tiles per raster group: keeps a wave's A/B working set inside L2
  const int per_group = G * tiles_n;
  const int g = t / per_group;
  const int first_m = g * G;
  const int gsz = min(G, tiles_m - first_m);
  const int r = t - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, int M, int N, int K, int mn3d, int splits, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint8_t* sC = sB + STAGES * B_STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(sC + 2 * C_CHUNK_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int KB_total = (K + BK - 1) / BK;
  // split-K: work item w = tile * splits + slice; each slice covers KBS k-blocks (fp32 reduce-add epilogue)
  const int KBS = (KB_total + splits - 1) / splits;
  const int num_tiles = tiles_m * tiles_n * splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tfull[a], 1);
      mbar_init(&bars->tempty[a], 1);
    }
    mbar_init(&bars->drain, 1);
    bars->abort_flag = 0;
    bars->epi_decision = 0;
    fence_mbar_init();
  }
  if (warp == 5) tmem_alloc(&bars->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      int s = 0;
      uint32_t ph = 0;
      uint32_t armed = 0;        // bit s set: full[s] was armed at least once
      uint32_t armed_parity = 0; // parity of the last armed phase of full[s]
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(t / splits, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        const int kb0 = (t % splits) * KBS, kb1 = min(KB_total, kb0 + KBS);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_flag, status, 100 + s)) { ok = false; break; }
          mbar_expect_tx(&bars->full[s], A_STAGE_BYTES + B_STAGE_BYTES);
          armed |= 1u << s;
          armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
          const int k0 = kb * BK;
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          if (!A_MN) {
            tma_load_2d(a_dst, &tmA, &bars->full[s], k0, m0);            // box {64 k, 128 m}
          } else if (mn3d & 1) {                                           // one box {64 m, 64 k, 2 chunks}
            tma_load_3d(a_dst, &tmA, &bars->full[s], 0, k0, m0 >> 6);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)                              // boxes {64 m, 64 k}
              tma_load_2d(a_dst + c * 8192, &tmA, &bars->full[s], m0 + c * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d(b_dst, &tmB, &bars->full[s], k0, n0);            // box {64 k, 256 n}
          } else if (mn3d & 2) {                                           // one box {64 n, 64 k, 4 chunks}
            tma_load_3d(b_dst, &tmB, &bars->full[s], 0, k0, n0 >> 6);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)                              // boxes {64 n, 64 k}
              tma_load_2d(b_dst + c * 8192, &tmB, &bars->full[s], n0 + c * 64, k0);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) {  // drain loads in flight before the CTA may exit
        for (int i = 0; i < STAGES; ++i)
          if (armed & (1u << i)) mbar_drain(&bars->full[i], (armed_parity >> i) & 1u);
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN, A_MN, B_MN);
      // byte advance of the descriptor start address per 16-wide K step
      constexpr uint32_t a_kstep = A_MN ? 2048u : 32u;
      constexpr uint32_t b_kstep = B_MN ? 2048u : 32u;
      constexpr uint32_t a_lbo = A_MN ? 8192u : 16u;
      constexpr uint32_t b_lbo = B_MN ? 8192u : 16u;
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!mbar_wait(&bars->tempty[acc], acc_ph ^ 1, abort_flag, status, 200 + acc)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
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
            umma_bf16_ss(d_tmem, ad, bd, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
          }
          umma_commit(&bars->empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&bars->tfull[acc]);
      }
      if (!ok) {  // make sure no MMA is still writing TMEM / reading smem before teardown
        umma_commit(&bars->drain);
        mbar_drain(&bars->drain, 0);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 0..3)
    const int epi_tid = threadIdx.x;          // 0..127, row of the tile
    constexpr int CW = (EPI == kStoreBf16) ? 64 : 32;   // columns per staging chunk (128 B rows)
    constexpr int NCHUNK = BN / CW;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    int it = 0;
    int chunk_counter = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
      int tm, tn;
      tile_coords(t / splits, tiles_m, tiles_n, tm, tn);
      const int m0 = tm * BM, n0 = tn * BN;
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      if (epi_tid == 0) {
        const bool ok = mbar_wait(&bars->tfull[acc], acc_ph, abort_flag, status, 400 + acc);
        bars->epi_decision = ok ? 1 : 0;
      }
      named_bar_sync(1, 128);
      if (bars->epi_decision == 0) break;
      tc_fence_after();
      const uint32_t t_acc = tmem_base + lane_base + acc * BN;
#pragma unroll 1
      for (int c = 0; c < NCHUNK; ++c, ++chunk_counter) {
        uint8_t* stage = sC + (chunk_counter & 1) * C_CHUNK_BYTES;
        // the store issued two chunks ago read this buffer: wait until it has been read
        if (epi_tid == 0) tma_wait_group_read<1>();
        named_bar_sync(1, 128);
        uint8_t* row_ptr = stage + epi_tid * 128;
        const int sw = epi_tid & 7;
        if (EPI == kStoreBf16) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld_32x32(t_acc + c * CW + h * 32, r);
            tmem_ld_wait();
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
        if (c == NCHUNK - 1) {  // accumulator fully read: hand it back to the MMA warp
          tc_fence_before();
        }
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (epi_tid == 0) {
          if (c == NCHUNK - 1) mbar_arrive(&bars->tempty[acc]);
          if (EPI == kAccumF32)
            tma_reduce_add_2d(&tmC, stage, n0 + c * CW, m0);
          else
            tma_store_2d(&tmC, stage, n0 + c * CW, m0);
          tma_commit_group();
        }
      }
    }
    if (epi_tid == 0) tma_wait_group<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, 512);
}

template <bool A_MN, bool B_MN, int EPI>
static int launch_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                          int M, int N, int K, int mn3d, int* status, cudaStream_t stream, int max_ctas, int splits = 1) {
  auto kfn = gemm_bf16_kernel<A_MN, B_MN, EPI>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return kErrCuda;
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * splits;
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  kfn<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, tmC, M, N, K, mn3d, splits, status);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

}  // namespace gemm
}  // namespace pd

// C[M,N] = / += op(A) op(B).
//   a_mn_major = 0: A stored [M,K] row-major (lda elements between rows); 1: A stored [K,M] (lda between k rows)
//   b_mn_major = 0: B stored [N,K] row-major;                              1: B stored [K,N]
//   epi: 0 = bf16 store, 1 = fp32 store, 2 = fp32 accumulate (C += ...)
//   max_ctas: 0 = all SMs; otherwise cap the persistent grid (used to leave SMs to a concurrent
//   communication kernel).
// Requirements: pointers 16-byte aligned; lda/ldb/ldc multiples of 8 elements (bf16) / 4 (fp32).
static int gemm_impl(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                     int a_mn_major, int b_mn_major, int epi, int max_ctas, int splits, int* status,
                     cudaStream_t stream) {
  using namespace pd;
  using namespace pd::gemm;
  if (M <= 0 || N <= 0 || K <= 0 || splits < 1) return kErrBadShape;
  if (splits > 1 && epi != kAccumF32) return kErrBadShape;
  {
    const int kb_total = (K + BK - 1) / BK;
    if (splits > kb_total) splits = kb_total;
    const int kbs = (kb_total + splits - 1) / splits;
    splits = (kb_total + kbs - 1) / kbs;      // no empty slices
  }
  if (!aligned16(A) || !aligned16(B) || !aligned16(C)) return kErrAlignment;
  if ((lda % 8) || (ldb % 8) || (epi == kStoreBf16 ? (ldc % 8) : (ldc % 4))) return kErrAlignment;
  CUtensorMap tmA, tmB, tmC;
  bool ok = true;
  int a3d = 0, b3d = 0;
  if (!a_mn_major)
    ok &= encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, A, K, M, uint64_t(lda) * 2, BK, BM);
  else
    ok &= encode_tmap_mn(&tmA, A, M, K, uint64_t(lda) * 2, BM / 64, BK, &a3d);
  if (!b_mn_major)
    ok &= encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, B, K, N, uint64_t(ldb) * 2, BK, BN);
  else
    ok &= encode_tmap_mn(&tmB, B, N, K, uint64_t(ldb) * 2, BN / 64, BK, &b3d);
  if (epi == kStoreBf16)
    ok &= encode_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, C, N, M, uint64_t(ldc) * 2, 64, BM);
  else
    ok &= encode_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, C, N, M, uint64_t(ldc) * 4, 32, BM);
  if (!ok) return kErrTensorMap;

#define PD_GEMM_CASE(AM, BM_, E)                                                                   \
  if (a_mn_major == AM && b_mn_major == BM_ && epi == E)                                           \
    return launch_variant<AM, BM_, E>(tmA, tmB, tmC, M, N, K, a3d | (b3d << 1), status, stream, max_ctas, splits);
  PD_GEMM_CASE(0, 0, 0) PD_GEMM_CASE(0, 1, 0) PD_GEMM_CASE(1, 0, 0) PD_GEMM_CASE(1, 1, 0)
  PD_GEMM_CASE(0, 0, 1) PD_GEMM_CASE(0, 1, 1) PD_GEMM_CASE(1, 0, 1) PD_GEMM_CASE(1, 1, 1)
  PD_GEMM_CASE(0, 0, 2) PD_GEMM_CASE(0, 1, 2) PD_GEMM_CASE(1, 0, 2) PD_GEMM_CASE(1, 1, 2)
#undef PD_GEMM_CASE
  return kErrBadShape;
}

PD_EXPORT int pd_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                           int ldc, int a_mn_major, int b_mn_major, int epi, int max_ctas, int* status,
                           cudaStream_t stream) {
  return gemm_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, epi, max_ctas, 1, status, stream);
}

// Split-K form for skinny problems (few output tiles, long K: decode-time projections): `splits` slices of K
// are reduced into the fp32 buffer C with TMA reduce-add, so C must hold the value to accumulate onto (zeros).
PD_EXPORT int pd_gemm_bf16_splitk(const void* A, const void* B, float* C, int M, int N, int K, int lda, int ldb,
                                  int ldc, int a_mn_major, int b_mn_major, int splits, int* status,
                                  cudaStream_t stream) {
  return gemm_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, 2, 0, splits, status, stream);
}
// Slices that fill the GPU about once for an [M,N,K] problem (at least 4 k-blocks of 64 per slice).
PD_EXPORT int pd_gemm_suggest_splits(int M, int N, int K) {
  using namespace pd::gemm;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int s = pd::sm_count() / (tiles > 0 ? tiles : 1);
  const int kb = (K + BK - 1) / BK;
  if (s > kb / 4) s = kb / 4;
  return s < 1 ? 1 : s;
}
