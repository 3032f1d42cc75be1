// GEMM -> all-reduce in ONE kernel for tensor-parallel decoding (row-parallel out / ffn2 projections):
//     out[M, N] = sum over ranks r of  X_r[M, K_r] W_r[K_r, N]   (+ residual),      M <= 128 tokens
// Reference sequence: cuBLAS GEMM, then ProcessGroupNCCL::AllReduce
// (paddle/phi/kernels/fusion/gpu/fused_multi_transformer_kernel.cu:809-816, :864-880).
//
// One CTA per 128-column slab of N (all CTAs are co-resident: N / 128 <= number of SMs), warp-specialised like
// the plain GEMM: warp 4 = TMA producer, warp 5 = tcgen05.mma issuer (128 x 128 fp32 accumulator in TMEM),
// warps 0-3 = epilogue.  The epilogue converts the slab to bf16, PUSHES it with plain peer stores into slot
// [epoch parity][this rank] of every rank's receive buffer (its own included), publishes one release-add on each
// rank's per-slab counter, waits (bounded) until its own counter shows all ranks' slabs of this epoch, then sums
// the n partials in fp32 (+ residual) and writes the final bf16 slab.  Transfer of slab t overlaps the MMA of the
// slabs still in flight on other SMs; there is no separate collective launch and no host synchronisation.
// In-switch form (multicast mapping available, 4 ranks or more): the slab is stored into this rank's OWN buffer only,
// the same notices are exchanged, and the reduction is one multimem.ld_reduce per 16 bytes - the NVSwitch adds the
// n copies - so nothing is pushed n - 1 times and no SM adds partials of other ranks.
//
// The epoch lives in device memory (state[0]; the last CTA of a launch advances it), so the kernel can be replayed
// from a CUDA graph with constant arguments.  Counters grow monotonically (expected = epoch * nranks * ARRIVAL_UNITS, independent of the K split); the two
// receive slots alternate so that a rank that runs ahead by one launch never overwrites data still being read.
#include <cuda_bf16.h>

#include "host_utils.h"
#include "sm100_prims.cuh"

namespace pd {
namespace gar {

typedef __nv_bfloat16 bf16;
constexpr int BM = 128, BN = 128, BK = 64, STAGES = 4;
constexpr int A_STAGE = BM * BK * 2, B_STAGE = BN * BK * 2;       // 16 KB each
constexpr int STAGE_TILE = BM * BN * 2;                            // 32 KB bf16 staging
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * (A_STAGE + B_STAGE) + STAGE_TILE + 1024 + 256;
constexpr int MAX_RANKS = 8;
constexpr int MAX_SPLITS = 4;
constexpr int ARRIVAL_UNITS = 12;      // divisible by every split count 1..MAX_SPLITS

struct Peers {
  bf16* recv[MAX_RANKS];     // each: [2 slots][nranks][m_cap][N] bf16
  int* cnt[MAX_RANKS];       // each: [N / 128] ints, monotonic
};

struct Bars {
  uint64_t full[STAGES], empty[STAGES], tfull, drain;
  uint32_t tmem_base;
  int abort_flag;
  int verdict;
};

template <int B3D>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_ar_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Peers peers,
               const bf16* __restrict__ residual, bf16* __restrict__ out, int M, int N, int K, int ldc, int rank,
               int nranks, int m_cap, int S, int* state, unsigned long long wait_ns, int* status,
               const bf16* __restrict__ mc_recv) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE;
  uint8_t* sC = sB + STAGES * B_STAGE;
  Bars* bars = reinterpret_cast<Bars*>(sC + STAGE_TILE);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // split-K: S CTAs share one slab, each pushes the partial of its K slice as one more addend of the reduction
  const int tile = blockIdx.x / S, ks = blockIdx.x % S, n0 = tile * BN;
  const int KB_total = (K + BK - 1) / BK, KBS = (KB_total + S - 1) / S;
  const int kb0 = ks * KBS, KB = max(0, min(KB_total, kb0 + KBS) - kb0);
  const int epoch = state[0] + 1;                  // read before anyone can advance it (only a finished launch does)
  const int slot = epoch & 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->tfull, 1);
    mbar_init(&bars->drain, 1);
    bars->abort_flag = 0;
    bars->verdict = 0;
    fence_mbar_init();
  }
  if (warp == 5) tmem_alloc(&bars->tmem_base, 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 4) {
    if (lane == 0) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      bool ok = true;
      int armed = 0;
      for (int kb = 0; kb < KB && ok; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1;
        if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_flag, status, 100 + s)) { ok = false; break; }
        mbar_expect_tx(&bars->full[s], A_STAGE + B_STAGE);
        tma_load_2d(sA + s * A_STAGE, &tmA, &bars->full[s], (kb0 + kb) * BK, 0);         // box {64 k, 128 m}
        if (B3D) {
          tma_load_3d(sB + s * B_STAGE, &tmB, &bars->full[s], 0, (kb0 + kb) * BK, n0 >> 6);   // box {64 n, 64 k, 2}
        } else {
          tma_load_2d(sB + s * B_STAGE, &tmB, &bars->full[s], n0, (kb0 + kb) * BK);
          tma_load_2d(sB + s * B_STAGE + 8192, &tmB, &bars->full[s], n0 + 64, (kb0 + kb) * BK);
        }
        armed = kb + 1;
      }
      if (!ok) {
        for (int kb = max(0, armed - STAGES); kb < armed; ++kb) mbar_drain(&bars->full[kb % STAGES], (kb / STAGES) & 1);
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN, false, true);
      bool ok = true;
      for (int kb = 0; kb < KB; ++kb) {
        const int s = kb % STAGES;
        if (!mbar_wait(&bars->full[s], (kb / STAGES) & 1, abort_flag, status, 200 + s)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(sA + s * A_STAGE), b_addr = smem_u32(sB + s * B_STAGE);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_bf16_ss(tmem_base, make_smem_desc_sw128(a_addr + k * 32, 16, 1024),
                       make_smem_desc_sw128(b_addr + k * 2048, 8192, 1024), idesc, (kb | k) != 0 ? 1u : 0u);
        umma_commit(&bars->empty[s]);
      }
      if (ok) {
        umma_commit(&bars->tfull);
      } else {
        umma_commit(&bars->drain);
        mbar_drain(&bars->drain, 0);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue: push, signal, wait, reduce
    const int tid = threadIdx.x;                 // 0..127 = accumulator row
    if (tid == 0) bars->verdict = mbar_wait(&bars->tfull, 0, abort_flag, status, 300) ? 1 : 0;
    named_bar_sync(1, 128);
    const bool mma_ok = bars->verdict != 0;
    if (mma_ok) {
      tc_fence_after();
      const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
      uint8_t* row_ptr = sC + tid * 256;
      const int sw = tid & 15;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_acc + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
          v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
          v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
          v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
          *reinterpret_cast<uint4*>(row_ptr + (((c * 4 + j) ^ sw) << 4)) = v;     // 16 chunks of 16 B per row
        }
      }
      tc_fence_before();
    }
    named_bar_sync(1, 128);
    if (mma_ok) {
      // coalesced push: half a warp per row (16 lanes x 16 B = the 256 B slab row), every rank's slot [slot][rank]
      const int half = lane >> 4, chunk = lane & 15;
      const size_t slot_off = (static_cast<size_t>(slot) * nranks * S + rank * S + ks) * m_cap * static_cast<size_t>(N);
      for (int r0 = warp * 2; r0 < M; r0 += 8) {
        const int row = r0 + half;
        if (row < M) {
          const uint4 v = *reinterpret_cast<const uint4*>(sC + row * 256 + ((chunk ^ (row & 15)) << 4));
          const size_t off = slot_off + static_cast<size_t>(row) * N + n0 + chunk * 8;
          if (mc_recv != nullptr) {
            // in-switch form: the partial stays in this rank's own buffer, at the same offset on every rank; the
            // reduction below reads the sum of all ranks' copies through the multicast address
            *reinterpret_cast<uint4*>(peers.recv[rank] + (static_cast<size_t>(slot) * nranks * S + ks) * m_cap * static_cast<size_t>(N) +
                                      static_cast<size_t>(row) * N + n0 + chunk * 8) = v;
          } else {
            for (int p = 0; p < nranks; ++p) {
              const int peer = (rank + p) % nranks;                     // spread the first stores over the links
              *reinterpret_cast<uint4*>(peers.recv[peer] + off) = v;
            }
          }
        }
      }
      __threadfence_system();
    }
    named_bar_sync(1, 128);
    if (tid == 0) {
      int ok = mma_ok ? 1 : 0;
      if (ok) {
        // one launch adds ARRIVAL_UNITS per rank to a slab's counter whatever its K split (a K slice adds
        // ARRIVAL_UNITS / S), so launches with different splits can share the counters and the epoch
        for (int p = 0; p < nranks; ++p) red_release_sys_add(peers.cnt[(rank + p) % nranks] + tile, ARRIVAL_UNITS / S);
        if (ks == 0)
          ok = flag_wait_ge(peers.cnt[rank] + tile, static_cast<int>(static_cast<unsigned>(epoch) * nranks * ARRIVAL_UNITS), wait_ns, status, 400) ? 1 : 0;
      }
      bars->verdict = ok;
    }
    named_bar_sync(1, 128);
    if (bars->verdict != 0 && ks == 0 && mc_recv != nullptr) {
      // in-switch form: a multimem.ld_reduce takes microseconds, so a thread first issues the loads of eight of its rows
      // (x S K-slices) and only then adds - up to 32 requests in flight per thread instead of one
      const int half = lane >> 4, chunk = lane & 15;
      const bf16* src = mc_recv + static_cast<size_t>(slot) * nranks * S * m_cap * static_cast<size_t>(N);
      constexpr int RB = 8;
      for (int rb = warp * 2 + half; rb < M; rb += 8 * RB) {
        uint4 v[RB][MAX_SPLITS];
#pragma unroll
        for (int i = 0; i < RB; ++i) {
          const int row = rb + 8 * i;
#pragma unroll
          for (int p = 0; p < MAX_SPLITS; ++p)
            if (row < M && p < S)
              v[i][p] = multimem_ld_reduce_bf16x8(src + static_cast<size_t>(p) * m_cap * N + static_cast<size_t>(row) * N + n0 + chunk * 8);
        }
#pragma unroll
        for (int i = 0; i < RB; ++i) {
          const int row = rb + 8 * i;
          if (row >= M) continue;
          float acc[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
          for (int p = 0; p < MAX_SPLITS; ++p) {
            if (p < S) {
              const uint32_t w[4] = {v[i][p].x, v[i][p].y, v[i][p].z, v[i][p].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                acc[2 * e] += __uint_as_float(w[e] << 16);
                acc[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
              }
            }
          }
          const size_t o = static_cast<size_t>(row) * ldc + n0 + chunk * 8;
          if (residual != nullptr) {
            const uint4 rv = *reinterpret_cast<const uint4*>(residual + o);
            const uint32_t w[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              acc[2 * e] += __uint_as_float(w[e] << 16);
              acc[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
            }
          }
          uint4 ov;
          ov.x = pack_bf16x2(acc[0], acc[1]);
          ov.y = pack_bf16x2(acc[2], acc[3]);
          ov.z = pack_bf16x2(acc[4], acc[5]);
          ov.w = pack_bf16x2(acc[6], acc[7]);
          *reinterpret_cast<uint4*>(out + o) = ov;
        }
      }
    } else if (bars->verdict != 0 && ks == 0) {
      const int half = lane >> 4, chunk = lane & 15;
      const int parts = nranks * S;
      const bf16* base = peers.recv[rank] + static_cast<size_t>(slot) * parts * m_cap * static_cast<size_t>(N);
      for (int r0 = warp * 2; r0 < M; r0 += 8) {
        const int row = r0 + half;
        if (row < M) {
          float acc[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = 0.f;
          const size_t off = static_cast<size_t>(row) * N + n0 + chunk * 8;
          for (int p = 0; p < parts; ++p) {
            const uint4 v = __ldcg(reinterpret_cast<const uint4*>(base + static_cast<size_t>(p) * m_cap * N + off));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              acc[2 * e] += __uint_as_float(w[e] << 16);
              acc[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
            }
          }
          const size_t o = static_cast<size_t>(row) * ldc + n0 + chunk * 8;
          if (residual != nullptr) {
            const uint4 v = *reinterpret_cast<const uint4*>(residual + o);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              acc[2 * e] += __uint_as_float(w[e] << 16);
              acc[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
            }
          }
          uint4 ov;
          ov.x = pack_bf16x2(acc[0], acc[1]);
          ov.y = pack_bf16x2(acc[2], acc[3]);
          ov.z = pack_bf16x2(acc[4], acc[5]);
          ov.w = pack_bf16x2(acc[6], acc[7]);
          *reinterpret_cast<uint4*>(out + o) = ov;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, 128);
  // the last CTA of the launch advances the epoch for the next launch (stream order makes it visible)
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(state + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      state[1] = 0;
      __threadfence();
      state[0] = epoch;
    }
  }
}

}  // namespace gar
}  // namespace pd

// A: X_r [M, K] row-major (lda), B: W_r [K, N] row-major (ldb), out/residual [M, N] (ldc).  peer_recv / peer_cnt:
// nranks device pointers (index = rank) into each rank's receive buffer ([2][nranks][m_cap][N] bf16) and counters
// ([N/128] int32, zero-initialised once); state: 2 local int32 (zero-initialised once).  N % 128 == 0, M <= 128,
// M <= m_cap, (N / 128) * splits <= number of SMs; the receive buffer holds [2][nranks * splits][m_cap][N] bf16 and
// every rank must pass the same `splits`.  mc_recv: multicast address of the receive buffers (0 = push form): each rank
// then keeps its partial slabs in its own buffer and the reduction reads the cross-rank sum with multimem.ld_reduce.
PD_EXPORT int pd_gemm_ar(const void* A, const void* B, void* out, const void* residual, int M, int N, int K, int lda,
                         int ldb, int ldc, int rank, int nranks, const unsigned long long* peer_recv,
                         const unsigned long long* peer_cnt, int m_cap, int splits, int* state, int wait_ms, int* status,
                         cudaStream_t stream, unsigned long long mc_recv) {
  using namespace pd;
  using namespace pd::gar;
  if (M <= 0 || M > BM || M > m_cap || N <= 0 || (N % BN) || K <= 0 || nranks < 1 || nranks > MAX_RANKS)
    return kErrBadShape;
  if (splits < 1) splits = 1;
  {
    const int kb_total = (K + BK - 1) / BK;
    if (splits > kb_total) splits = kb_total;
    const int kbs = (kb_total + splits - 1) / splits;
    splits = (kb_total + kbs - 1) / kbs;
  }
  if (splits > MAX_SPLITS) return kErrBadShape;
  if ((N / BN) * splits > sm_count()) return kErrTooLarge;      // every CTA must be resident: they wait on peers
  if (!aligned16(A) || !aligned16(B) || !aligned16(out) || (lda % 8) || (ldb % 8) || (ldc % 8) ||
      (residual && !aligned16(residual)))
    return kErrAlignment;
  CUtensorMap tmA, tmB;
  int b3d = 0;
  bool ok = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, A, K, M, uint64_t(lda) * 2, BK, BM);
  ok &= encode_tmap_mn(&tmB, B, N, K, uint64_t(ldb) * 2, BN / 64, BK, &b3d);
  if (!ok) return kErrTensorMap;
  Peers peers;
  for (int i = 0; i < MAX_RANKS; ++i) {
    peers.recv[i] = reinterpret_cast<bf16*>(peer_recv[i < nranks ? i : 0]);
    peers.cnt[i] = reinterpret_cast<int*>(peer_cnt[i < nranks ? i : 0]);
  }
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_ar_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_ar_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return kErrCuda;
    configured = true;
  }
  const unsigned long long wait_ns = static_cast<unsigned long long>(wait_ms) * 1000000ull;
  if (b3d)
    gemm_ar_kernel<1><<<(N / BN) * splits, NUM_THREADS, SMEM_BYTES, stream>>>(
        tmA, tmB, peers, (const bf16*)residual, (bf16*)out, M, N, K, ldc, rank, nranks, m_cap, splits, state, wait_ns,
        status, reinterpret_cast<const bf16*>(mc_recv));
  else
    gemm_ar_kernel<0><<<(N / BN) * splits, NUM_THREADS, SMEM_BYTES, stream>>>(
        tmA, tmB, peers, (const bf16*)residual, (bf16*)out, M, N, K, ldc, rank, nranks, m_cap, splits, state, wait_ns,
        status, reinterpret_cast<const bf16*>(mc_recv));
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}
