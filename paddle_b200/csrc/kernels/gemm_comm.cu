// Fused compute + collective GEMMs over NVLink peer memory (one kernel launch each, one process per GPU):
//
//   ag_gemm : all-gather -> GEMM.  A few "comm" CTAs push this rank's activation shard into every peer's
//             staging buffer with plain 16-byte peer stores, one flag per sub-chunk (st.release.sys); the
//             remaining CTAs run the persistent tcgen05 GEMM, consuming chunks in arrival order (local
//             shard first) — the TMA producer waits on the chunk flag (ld.acquire.sys, bounded) before it
//             loads tiles of that chunk from LOCAL memory.  Nothing is read twice over NVLink.
//   gemm_rs : GEMM -> reduce-scatter.  Tiles are computed destination by destination (remote first, own
//             shard last); the epilogue TMA-stores each bf16 partial tile straight into the destination
//             rank's receive buffer and bumps that tile's arrival counter (red.release.sys); every CTA then
//             reduces tiles of its own shard as soon as all ranks' partials have landed.
// These implement ColumnSequenceParallelLinear / RowSequenceParallelLinear forward and backward
// (python/paddle/distributed/fleet/utils/sequence_parallel_utils.py:429,564), where the reference issues
// a synchronous NCCL all-gather before / reduce-scatter after a cuBLAS GEMM (:58-82,543-549,669-678).
// No TMA multicast is used anywhere.  Every cross-rank wait is bounded and reports through the status word.
#include "host_utils.h"
#include "sm100_prims.cuh"

namespace pd {
namespace gc {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int C_CHUNK_BYTES = BM * 128;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 2 * C_CHUNK_BYTES + 1024 + 256;
constexpr int MAX_RANKS = 8;

struct Barriers {
  uint64_t full[STAGES], empty[STAGES], tfull[2], tempty[2], drain;
  uint32_t tmem_base;
  int abort_flag;
  int epi_decision;
};

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ void raster(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int G = 16;
  const int per_group = G * tiles_n;
  const int g = t / per_group;
  const int first_m = g * G;
  const int gsz = min(G, tiles_m - first_m);
  const int r = t - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

__device__ __forceinline__ void init_barriers(Barriers* bars) {
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

// MMA issuer loop shared by both kernels (identical to the plain GEMM).
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void mma_loop(Barriers* bars, uint8_t* sA, uint8_t* sB, uint32_t tmem_base, int my_tiles,
                                         int KB, int* status) {
  volatile int* abort_flag = &bars->abort_flag;
  constexpr uint32_t idesc = make_idesc(BM, BN, A_MN, B_MN);
  constexpr uint32_t a_kstep = A_MN ? 2048u : 32u, b_kstep = B_MN ? 2048u : 32u;
  constexpr uint32_t a_lbo = A_MN ? 8192u : 16u, b_lbo = B_MN ? 8192u : 16u;
  int s = 0;
  uint32_t ph = 0;
  bool ok = true;
  for (int it = 0; it < my_tiles && ok; ++it) {
    const int acc = it & 1;
    const uint32_t acc_ph = (it >> 1) & 1;
    if (!mbar_wait(&bars->tempty[acc], acc_ph ^ 1, abort_flag, status, 200 + acc)) { ok = false; break; }
    tc_fence_after();
    const uint32_t d_tmem = tmem_base + acc * BN;
    for (int kb = 0; kb < KB; ++kb) {
      if (!mbar_wait(&bars->full[s], ph, abort_flag, status, 300 + s)) { ok = false; break; }
      tc_fence_after();
      const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES), b_addr = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
      for (int k = 0; k < BK / 16; ++k)
        umma_bf16_ss(d_tmem, make_smem_desc_sw128(a_addr + k * a_kstep, a_lbo, 1024),
                     make_smem_desc_sw128(b_addr + k * b_kstep, b_lbo, 1024), idesc, (kb | k) != 0 ? 1u : 0u);
      umma_commit(&bars->empty[s]);
      if (++s == STAGES) { s = 0; ph ^= 1; }
    }
    if (ok) umma_commit(&bars->tfull[acc]);
  }
  if (!ok) {
    umma_commit(&bars->drain);
    mbar_drain(&bars->drain, 0);
  }
}

template <bool A_MN, bool B_MN>
__device__ __forceinline__ void load_stage(const CUtensorMap* tmA, const CUtensorMap* tmB, uint8_t* a_dst,
                                           uint8_t* b_dst, uint64_t* bar, int m0, int n0, int k0) {
  if (!A_MN) {
    tma_load_2d(a_dst, tmA, bar, k0, m0);
  } else {
#pragma unroll
    for (int c = 0; c < BM / 64; ++c) tma_load_2d(a_dst + c * 8192, tmA, bar, m0 + c * 64, k0);
  }
  if (!B_MN) {
    tma_load_2d(b_dst, tmB, bar, k0, n0);
  } else {
#pragma unroll
    for (int c = 0; c < BN / 64; ++c) tma_load_2d(b_dst + c * 8192, tmB, bar, n0 + c * 64, k0);
  }
}

template <bool A_MN>
__device__ __forceinline__ void load_a(const CUtensorMap* tm, uint8_t* dst, uint64_t* bar, int m0, int k0,
                                       bool use3d = false) {
  if (!A_MN) {
    tma_load_2d(dst, tm, bar, k0, m0);
  } else if (use3d) {
    tma_load_3d(dst, tm, bar, 0, k0, m0 >> 6);
  } else {
#pragma unroll
    for (int c = 0; c < BM / 64; ++c) tma_load_2d(dst + c * 8192, tm, bar, m0 + c * 64, k0);
  }
}
template <bool B_MN>
__device__ __forceinline__ void load_b(const CUtensorMap* tm, uint8_t* dst, uint64_t* bar, int n0, int k0,
                                       bool use3d = false) {
  if (!B_MN) {
    tma_load_2d(dst, tm, bar, k0, n0);
  } else if (use3d) {
    tma_load_3d(dst, tm, bar, 0, k0, n0 >> 6);
  } else {
#pragma unroll
    for (int c = 0; c < BN / 64; ++c) tma_load_2d(dst + c * 8192, tm, bar, n0 + c * 64, k0);
  }
}

// ============================================================================================ ag_gemm
struct AGParams {
  int gathered_b;      // wait_mode 1 only: the gathered (token-major) operand is B instead of A
  int mn3d;            // bit0/1/2: the A / B / local map is the 3-D (one box per operand) form
  int M, N, K;
  int rank, nranks;
  int rows_per_rank;   // token rows contributed by each rank
  int sub_rows;        // token rows per arrival flag (multiple of 128, divides rows_per_rank)
  int row_elems;       // elements per token row of the gathered matrix
  int n_comm;          // CTAs that push the local shard; the rest run the GEMM
  int epoch;           // call number on this slot (flags / acks hold the last completed epoch)
  int wait_mode;       // 0: tokens are the M dimension (wait per M tile); 1: tokens are the reduction dim
  int skip_push;       // 1: the gathered matrix of this epoch is already staged (second GEMM on the same data)
  int do_ack;          // 1: this launch is the last reader of the epoch's staged data -> acknowledge to all ranks
  int done_target;     // value of *local_done after every GEMM CTA of every acknowledging launch so far
  const int* bias;     // optional device int[2] added to {epoch, done_target}: lets a CUDA graph replay the launch
                       // (constant arguments) while the slot's epoch keeps advancing in device memory
  const void* x_shard; // [rows_per_rank, row_elems] bf16, local
  unsigned long long peer_stage[MAX_RANKS];  // staging buffer [nranks*rows_per_rank, row_elems] of every rank
  unsigned long long peer_flags[MAX_RANKS];  // int32 [nranks][n_sub] of every rank
  unsigned long long peer_ack[MAX_RANKS];    // int32 [nranks] of every rank
  int* local_done;
  int* status;
  unsigned long long wait_ns;
};

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmL,
               const __grid_constant__ AGParams p) {
  extern __shared__ uint8_t smem_raw[];
  const int epoch_v = p.epoch + (p.bias != nullptr ? __ldg(p.bias) : 0);
  const int done_target_v = p.done_target + (p.bias != nullptr ? __ldg(p.bias + 1) : 0);
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint8_t* sC = sB + STAGES * B_STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(sC + 2 * C_CHUNK_BYTES);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_sub = p.rows_per_rank / p.sub_rows;
  const int* flags_local = reinterpret_cast<const int*>(p.peer_flags[p.rank]);

  if (static_cast<int>(blockIdx.x) < p.n_comm) {
    // ------------------------------------------------------------------ comm CTA: push the local shard
    // One thread drives a ring of bulk copies: local HBM -> shared memory (cp.async.bulk + mbarrier), shared
    // memory -> the peer's staging buffer (cp.async.bulk store over NVLink).  Many KB stay in flight per CTA
    // without occupying load/store units, so a handful of CTAs saturate the link.
    if (p.skip_push || threadIdx.x != 0) return;
    // RING slots of PIECE_MAX bytes.  A slot is in one of two states: loaded and waiting for its store (at most
    // LOOKAHEAD pieces ahead; local HBM reads are fast, so a few suffice) or stored and still being read by the
    // copy engine (its bytes are on the wire).  Before piece q + LOOKAHEAD is loaded into the slot that piece
    // q + LOOKAHEAD - RING used, all but the newest RING - LOOKAHEAD - 1 stores must have finished reading shared
    // memory; that bound is what the wait below enforces, and it leaves RING - LOOKAHEAD - 1 pieces in flight.
    constexpr int RING = 12, LOOKAHEAD = 3, PIECE_MAX = 16384, FLAG_LAG = 3;
    constexpr int STORES_IN_FLIGHT = RING - LOOKAHEAD - 1;
    uint64_t* ring_bar = reinterpret_cast<uint64_t*>(smem + RING * PIECE_MAX);
    for (int i = 0; i < RING; ++i) mbar_init(&ring_bar[i], 1);
    fence_mbar_init();
    int dummy_abort = 0;
    const int* ack_local = reinterpret_cast<const int*>(p.peer_ack[p.rank]);
    const int npeers = p.nranks - 1;
    const int jobs = npeers * n_sub;                 // the local shard is read in place by the GEMM
    const int my_jobs = static_cast<int>(blockIdx.x) < jobs ? (jobs - static_cast<int>(blockIdx.x) + p.n_comm - 1) / p.n_comm : 0;
    const uint32_t row_bytes = static_cast<uint32_t>(p.row_elems) * 2;
    const int rows_per_piece = row_bytes >= PIECE_MAX ? 1 : PIECE_MAX / row_bytes;
    const int ppj = (p.sub_rows + rows_per_piece - 1) / rows_per_piece;     // pieces per job
    const int total = my_jobs * ppj;
    auto piece_info = [&](int q, int& peer, int& c, int& row0, uint32_t& bytes) {
      const int j = static_cast<int>(blockIdx.x) + (q / ppj) * p.n_comm;
      c = j / npeers;
      peer = (p.rank + 1 + j % npeers) % p.nranks;
      row0 = (q % ppj) * rows_per_piece;
      const int nrows = min(rows_per_piece, p.sub_rows - row0);
      bytes = static_cast<uint32_t>(nrows) * row_bytes;
    };
    auto issue_load = [&](int q) {
      int peer, c, row0;
      uint32_t bytes;
      piece_info(q, peer, c, row0, bytes);
      const int slot = q % RING;
      const uint8_t* src = static_cast<const uint8_t*>(p.x_shard) +
                           (static_cast<size_t>(c) * p.sub_rows + row0) * row_bytes;
      mbar_expect_tx(&ring_bar[slot], bytes);
      bulk_load(smem + slot * PIECE_MAX, src, bytes, &ring_bar[slot]);
    };
    for (int q = 0; q < total && q < LOOKAHEAD; ++q) issue_load(q);
    unsigned checked = 0;
    bool ok = true;
    int* pend_flag = nullptr;
    int pend_q = 0;
    for (int q = 0; q < total && ok; ++q) {
      if (q + LOOKAHEAD < total) {
        tma_wait_group_read<STORES_IN_FLIGHT>();   // the store that last read this slot has drained it
        issue_load(q + LOOKAHEAD);
      }
      int peer, c, row0;
      uint32_t bytes;
      piece_info(q, peer, c, row0, bytes);
      if (!(checked & (1u << peer))) {
        // the peer must have finished reading what the previous epoch put into this slot
        if (!flag_wait_ge(ack_local + peer, epoch_v - 1, p.wait_ns, p.status, 500 + peer)) { ok = false; break; }
        checked |= 1u << peer;
      }
      const int slot = q % RING;
      if (!mbar_wait(&ring_bar[slot], (q / RING) & 1, &dummy_abort, p.status, 510)) { ok = false; break; }
      uint8_t* dst = reinterpret_cast<uint8_t*>(p.peer_stage[peer]) +
                     ((static_cast<size_t>(p.rank) * n_sub + c) * p.sub_rows + row0) * row_bytes;
      bulk_store(dst, smem + slot * PIECE_MAX, bytes);
      tma_commit_group();
      // A chunk's flag is raised FLAG_LAG pieces after its last store was issued: by then waiting for "all but
      // the newest FLAG_LAG groups" costs nothing and guarantees the chunk has fully landed.
      if (pend_flag != nullptr && q - pend_q >= FLAG_LAG) {
        tma_wait_group<FLAG_LAG>();
        __threadfence_system();
        st_release_sys(pend_flag, epoch_v);
        pend_flag = nullptr;
      }
      if (q % ppj == ppj - 1) {
        if (pend_flag != nullptr) {                 // (only when a chunk has fewer than FLAG_LAG pieces)
          tma_wait_group<1>();
          __threadfence_system();
          st_release_sys(pend_flag, epoch_v);
        }
        pend_flag = reinterpret_cast<int*>(p.peer_flags[peer]) + p.rank * n_sub + c;
        pend_q = q;
      }
    }
    if (ok && pend_flag != nullptr) {
      tma_wait_group<0>();
      __threadfence_system();
      st_release_sys(pend_flag, epoch_v);
    }
    if (!ok) {                                       // drain what is still in flight before leaving
      tma_wait_group<0>();
      for (int q = 0; q < total; ++q) {
        const int slot = q % RING;
        mbar_drain(&ring_bar[slot], (q / RING) & 1);
        if (q >= RING) break;
      }
    }
    return;
  }

  // -------------------------------------------------------------------- GEMM CTA
  const int cta = blockIdx.x - p.n_comm, nct = gridDim.x - p.n_comm;
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int KB = (p.K + BK - 1) / BK;
  const int my_tiles = cta < num_tiles ? (num_tiles - cta + nct - 1) / nct : 0;
  const int tiles_per_src = p.rows_per_rank / BM;           // wait_mode 0
  const int kb_per_src = p.rows_per_rank / BK;              // wait_mode 1

  if (threadIdx.x == 0) init_barriers(bars);
  if (warp == 5) tmem_alloc(&bars->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 4) {
    if (lane == 0) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      prefetch_tmap(&tmL);
      // everything the loop needs is copied out of the parameter block once: a single thread issues every TMA
      // of this CTA, and re-reading parameters after each asm statement would put it on the critical path
      const int wait_mode = p.wait_mode, rank = p.rank, rows_per_rank = p.rows_per_rank, sub_rows = p.sub_rows;
      const int epoch = epoch_v, gathered_b = p.gathered_b, local_row0 = p.rank * p.rows_per_rank;
      const bool a3d = (p.mn3d & 1) != 0, b3d = (p.mn3d & 2) != 0, l3d = (p.mn3d & 4) != 0;
      const unsigned long long wait_ns = p.wait_ns;
      int* const status = p.status;
      int s = 0;
      uint32_t ph = 0, armed = 0, armed_parity = 0;
      bool ok = true;
      int last_chunk = -1;
      for (int t = cta; t < num_tiles && ok; t += nct) {
        int tm, tn;
        raster(t, tiles_m, tiles_n, tm, tn);
        if (wait_mode == 0) tm = (tm + rank * tiles_per_src) % tiles_m;   // local shard first
        const int m0 = tm * BM, n0 = tn * BN;
        // rows of this rank's own shard are read straight from x_shard (map tmL): no copy, no wait
        bool local_tile = false;
        if (wait_mode == 0) {
          local_tile = (m0 / rows_per_rank) == rank;
          const int chunk = m0 / sub_rows;      // == src * n_sub + sub-chunk
          if (!local_tile && chunk != last_chunk) {
            if (!flag_wait_ge(flags_local + chunk, epoch, wait_ns, status, 600)) { ok = false; *abort_flag = 1; break; }
            fence_proxy_async_all();
            last_chunk = chunk;
          }
        }
        for (int kbi = 0; kbi < KB; ++kbi) {
          int kb = kbi;
          bool local_k = false;
          if (wait_mode == 1) {
            kb = kbi + rank * kb_per_src;
            if (kb >= KB) kb -= KB;
            local_k = ((kb * BK) / rows_per_rank) == rank;
            const int chunk = (kb * BK) / sub_rows;
            if (!local_k && chunk != last_chunk) {
              if (!flag_wait_ge(flags_local + chunk, epoch, wait_ns, status, 610)) { ok = false; *abort_flag = 1; break; }
              fence_proxy_async_all();
              last_chunk = chunk;
            }
          }
          if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_flag, status, 100 + s)) { ok = false; break; }
          mbar_expect_tx(&bars->full[s], A_STAGE_BYTES + B_STAGE_BYTES);
          armed |= 1u << s;
          armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          const int k0 = kb * BK;
          if (wait_mode == 0) {
            if (local_tile) load_a<A_MN>(&tmL, a_dst, &bars->full[s], m0 - local_row0, k0);
            else load_a<A_MN>(&tmA, a_dst, &bars->full[s], m0, k0);
            load_b<B_MN>(&tmB, b_dst, &bars->full[s], n0, k0, b3d);
          } else {
            const int k0l = k0 - local_row0;
            if (local_k && !gathered_b) load_a<A_MN>(&tmL, a_dst, &bars->full[s], m0, k0l, l3d);
            else load_a<A_MN>(&tmA, a_dst, &bars->full[s], m0, k0, a3d);
            if (local_k && gathered_b) load_b<B_MN>(&tmL, b_dst, &bars->full[s], n0, k0l, l3d);
            else load_b<B_MN>(&tmB, b_dst, &bars->full[s], n0, k0, b3d);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok)
        for (int i = 0; i < STAGES; ++i)
          if (armed & (1u << i)) mbar_drain(&bars->full[i], (armed_parity >> i) & 1u);
    }
    __syncwarp();
  } else if (warp == 5) {
    if (lane == 0) mma_loop<A_MN, B_MN>(bars, sA, sB, tmem_base, my_tiles, KB, p.status);
    __syncwarp();
  } else {
    const int epi_tid = threadIdx.x;
    constexpr int CW = (EPI == 0) ? 64 : 32;
    constexpr int NCHUNK = BN / CW;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    int it = 0, chunk_counter = 0;
    bool alive = true;
    for (int t = cta; t < num_tiles; t += nct, ++it) {
      int tm, tn;
      raster(t, tiles_m, tiles_n, tm, tn);
      if (p.wait_mode == 0) tm = (tm + p.rank * tiles_per_src) % tiles_m;
      const int m0 = tm * BM, n0 = tn * BN;
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      if (epi_tid == 0) bars->epi_decision = mbar_wait(&bars->tfull[acc], acc_ph, abort_flag, p.status, 400 + acc) ? 1 : 0;
      named_bar_sync(1, 128);
      if (bars->epi_decision == 0) { alive = false; break; }
      tc_fence_after();
      const uint32_t t_acc = tmem_base + lane_base + acc * BN;
#pragma unroll 1
      for (int c = 0; c < NCHUNK; ++c, ++chunk_counter) {
        uint8_t* stage = sC + (chunk_counter & 1) * C_CHUNK_BYTES;
        if (epi_tid == 0) tma_wait_group_read<1>();
        named_bar_sync(1, 128);
        uint8_t* row_ptr = stage + epi_tid * 128;
        const int sw = epi_tid & 7;
        if (EPI == 0) {
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
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(row_ptr + ((j ^ sw) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
        if (c == NCHUNK - 1) tc_fence_before();
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (epi_tid == 0) {
          if (c == NCHUNK - 1) mbar_arrive(&bars->tempty[acc]);
          if (EPI == 2) tma_reduce_add_2d(&tmC, stage, n0 + c * CW, m0);
          else tma_store_2d(&tmC, stage, n0 + c * CW, m0);
          tma_commit_group();
        }
      }
    }
    if (epi_tid == 0) {
      tma_wait_group<0>();
      if (alive && p.do_ack) {
        // all staged data of this epoch has been consumed by this CTA: the last CTA acknowledges to every rank
        __threadfence();
        const int done = atomicAdd(p.local_done, 1) + 1;
        if (done == done_target_v)
          for (int r = 0; r < p.nranks; ++r)
            st_release_sys(reinterpret_cast<int*>(p.peer_ack[r]) + p.rank, epoch_v);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, 512);
}

// ============================================================================================ gemm_rs
struct RSParams {
  int M, N, K;
  int rank, nranks;
  int rows_per_rank;
  int epoch;
  const int* bias;     // optional device int[2]; bias[0] is added to epoch (CUDA-graph replay)
  int mn3d;
  unsigned long long peer_counters[MAX_RANKS];  // int32 [tiles_per_dst * tiles_n] on every rank
  unsigned long long peer_ack[MAX_RANKS];       // int32 [nranks] on every rank
  const void* recv_local;                       // bf16 [nranks][rows_per_rank][N]
  void* out;                                    // bf16 [rows_per_rank][N]
  int* local_done;
  int* status;
  unsigned long long wait_ns;
};
struct RSMaps {
  CUtensorMap dst[MAX_RANKS];   // partial-tile destination on rank d: [rows_per_rank, N] slab of this source
};

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ RSMaps maps, const __grid_constant__ RSParams p) {
  extern __shared__ uint8_t smem_raw[];
  const int epoch_v = p.epoch + (p.bias != nullptr ? __ldg(p.bias) : 0);
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint8_t* sC = sB + STAGES * B_STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(sC + 2 * C_CHUNK_BYTES);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, nct = gridDim.x;
  const int tiles_per_dst = (p.rows_per_rank + BM - 1) / BM;
  const int tiles_m = tiles_per_dst * p.nranks, tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int KB = (p.K + BK - 1) / BK;
  const int my_tiles = cta < num_tiles ? (num_tiles - cta + nct - 1) / nct : 0;
  const int tiles_dst_all = tiles_per_dst * tiles_n;     // tiles per destination

  if (threadIdx.x == 0) init_barriers(bars);
  if (warp == 5) tmem_alloc(&bars->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  // tile t -> destination-major order: remote destinations first (rank+1, rank+2, ...), own shard last
  auto decode = [&](int t, int& d, int& tml, int& tn) {
    const int di = t / tiles_dst_all, r = t % tiles_dst_all;
    d = (p.rank + 1 + di) % p.nranks;
    tml = r % tiles_per_dst;
    tn = r / tiles_per_dst;
  };

  if (warp == 4) {
    if (lane == 0) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      int s = 0;
      uint32_t ph = 0, armed = 0, armed_parity = 0;
      bool ok = true;
      const bool a3d = (p.mn3d & 1) != 0, b3d = (p.mn3d & 2) != 0;
      const int rows_per_rank = p.rows_per_rank;
      int* const status = p.status;
      for (int t = cta; t < num_tiles && ok; t += nct) {
        int d, tml, tn;
        decode(t, d, tml, tn);
        const int m0 = d * rows_per_rank + tml * BM, n0 = tn * BN;
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_flag, status, 100 + s)) { ok = false; break; }
          mbar_expect_tx(&bars->full[s], A_STAGE_BYTES + B_STAGE_BYTES);
          armed |= 1u << s;
          armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
          load_a<A_MN>(&tmA, sA + s * A_STAGE_BYTES, &bars->full[s], m0, kb * BK, a3d);
          load_b<B_MN>(&tmB, sB + s * B_STAGE_BYTES, &bars->full[s], n0, kb * BK, b3d);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok)
        for (int i = 0; i < STAGES; ++i)
          if (armed & (1u << i)) mbar_drain(&bars->full[i], (armed_parity >> i) & 1u);
    }
    __syncwarp();
  } else if (warp == 5) {
    if (lane == 0) mma_loop<A_MN, B_MN>(bars, sA, sB, tmem_base, my_tiles, KB, p.status);
    __syncwarp();
  } else {
    const int epi_tid = threadIdx.x;
    constexpr int CW = 64, NCHUNK = BN / CW;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int* ack_local = reinterpret_cast<const int*>(p.peer_ack[p.rank]);
    int it = 0, chunk_counter = 0;
    unsigned checked = 0;
    bool alive = true;
    int* pend_counter = nullptr;
    for (int t = cta; t < num_tiles; t += nct, ++it) {
      int d, tml, tn;
      decode(t, d, tml, tn);
      const int n0 = tn * BN;
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      if (epi_tid == 0) {
        bool ok = mbar_wait(&bars->tfull[acc], acc_ph, abort_flag, p.status, 400 + acc);
        if (ok && !(checked & (1u << d))) {
          // destination d must have finished reducing the previous epoch out of this slot
          ok = flag_wait_ge(ack_local + d, epoch_v - 1, p.wait_ns, p.status, 700 + d);
          if (!ok) *abort_flag = 1;
          checked |= 1u << d;
        }
        bars->epi_decision = ok ? 1 : 0;
      }
      named_bar_sync(1, 128);
      if (bars->epi_decision == 0) { alive = false; break; }
      tc_fence_after();
      const uint32_t t_acc = tmem_base + lane_base + acc * BN;
#pragma unroll 1
      for (int c = 0; c < NCHUNK; ++c, ++chunk_counter) {
        uint8_t* stage = sC + (chunk_counter & 1) * C_CHUNK_BYTES;
        if (epi_tid == 0) tma_wait_group_read<1>();
        named_bar_sync(1, 128);
        uint8_t* row_ptr = stage + epi_tid * 128;
        const int sw = epi_tid & 7;
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
        if (c == NCHUNK - 1) tc_fence_before();
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (epi_tid == 0) {
          if (c == NCHUNK - 1) mbar_arrive(&bars->tempty[acc]);
          tma_store_2d(&maps.dst[d], stage, n0 + c * CW, tml * BM);
          tma_commit_group();
          if (c == NCHUNK - 1) {
            // The arrival counter of a tile is bumped one tile later: by then "all but the newest NCHUNK
            // stores have completed" holds without stalling, and it means the tile has landed on rank d.
            if (pend_counter != nullptr) {
              tma_wait_group<NCHUNK>();
              __threadfence_system();
              red_release_sys_add(pend_counter, 1);
            }
            pend_counter = reinterpret_cast<int*>(p.peer_counters[d]) + tml * tiles_n + tn;
          }
        }
      }
    }
    if (epi_tid == 0 && pend_counter != nullptr) {
      tma_wait_group<0>();
      __threadfence_system();
      red_release_sys_add(pend_counter, 1);
    }
    // ---- reduce phase: out[tile] = sum over sources of the partial tiles received for my shard
    const int* counters = reinterpret_cast<const int*>(p.peer_counters[p.rank]);
    const __nv_bfloat16* recv = static_cast<const __nv_bfloat16*>(p.recv_local);
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
    const size_t slab = static_cast<size_t>(p.rows_per_rank) * p.N;
    for (int u = cta; u < tiles_dst_all && alive; u += nct) {
      const int tml = u % tiles_per_dst, tn = u / tiles_per_dst;
      if (epi_tid == 0)
        bars->epi_decision = flag_wait_ge(counters + tml * tiles_n + tn, p.nranks * epoch_v, p.wait_ns, p.status, 800) ? 1 : 0;
      named_bar_sync(1, 128);
      const int okd = bars->epi_decision;
      named_bar_sync(1, 128);
      if (!okd) { alive = false; break; }
      const int col = tn * BN + (epi_tid & 31) * 8;
      if (col < p.N) {
        // 4 rows x nranks sources of 16-byte loads are issued before any is consumed (latency hiding)
        constexpr int RU = 4;
        for (int rb = epi_tid >> 5; rb < BM; rb += 4 * RU) {
          uint4 v[RU][MAX_RANKS];
#pragma unroll
          for (int u = 0; u < RU; ++u) {
            const int row = tml * BM + rb + 4 * u;
#pragma unroll
            for (int s = 0; s < MAX_RANKS; ++s)
              if (s < p.nranks && row < p.rows_per_rank)
                v[u][s] = __ldcg(reinterpret_cast<const uint4*>(recv + s * slab + static_cast<size_t>(row) * p.N + col));
          }
#pragma unroll
          for (int u = 0; u < RU; ++u) {
            const int row = tml * BM + rb + 4 * u;
            if (row >= p.rows_per_rank) continue;
            float acc8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < MAX_RANKS; ++s) {
              if (s < p.nranks) {
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u][s]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 f = __bfloat1622float2(h[e]);
                  acc8[2 * e] += f.x;
                  acc8[2 * e + 1] += f.y;
                }
              }
            }
            uint4 o;
            o.x = pack_bf16x2(acc8[0], acc8[1]);
            o.y = pack_bf16x2(acc8[2], acc8[3]);
            o.z = pack_bf16x2(acc8[4], acc8[5]);
            o.w = pack_bf16x2(acc8[6], acc8[7]);
            *reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * p.N + col) = o;
          }
        }
      }
    }
    named_bar_sync(1, 128);
    if (epi_tid == 0 && alive) {
      __threadfence();
      const int done = atomicAdd(p.local_done, 1) + 1;
      if (done == nct * epoch_v)
        for (int r = 0; r < p.nranks; ++r) st_release_sys(reinterpret_cast<int*>(p.peer_ack[r]) + p.rank, epoch_v);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, 512);
}

template <typename KFn>
static int set_smem(KFn k) {
  return cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) == cudaSuccess ? 0 : -1;
}

static bool make_ab_maps(CUtensorMap* tmA, CUtensorMap* tmB, const void* A, const void* B, int M, int N, int K, int lda,
                         int ldb, int a_mn, int b_mn, int* mn3d) {
  bool ok = true;
  int a3 = 0, b3 = 0;
  if (!a_mn) ok &= encode_tmap_2d(tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, A, K, M, uint64_t(lda) * 2, BK, BM);
  else ok &= encode_tmap_mn(tmA, A, M, K, uint64_t(lda) * 2, BM / 64, BK, &a3);
  if (!b_mn) ok &= encode_tmap_2d(tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, B, K, N, uint64_t(ldb) * 2, BK, BN);
  else ok &= encode_tmap_mn(tmB, B, N, K, uint64_t(ldb) * 2, BN / 64, BK, &b3);
  *mn3d = a3 | (b3 << 1);
  return ok;
}

}  // namespace gc
}  // namespace pd

// All-gather -> GEMM.  A / B are the operand pointers the GEMM reads (the gathered one points into the LOCAL
// staging buffer peer_stage[rank]); see AGParams for the rest.  epi: 0 bf16 store, 1 fp32 store, 2 fp32 accumulate.
PD_EXPORT int pd_ag_gemm(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                         int a_mn, int b_mn, int epi, int gathered_b, const void* x_shard, int rows_per_rank, int sub_rows,
                         int row_elems, int rank, int nranks, int n_comm, int epoch, int wait_mode, int skip_push, int do_ack,
                         const unsigned long long* peer_stage, const unsigned long long* peer_flags,
                         const unsigned long long* peer_ack, int* local_done, int done_base, const int* bias, int wait_ms,
                         int* status, cudaStream_t stream) {
  using namespace pd;
  using namespace pd::gc;
  if (M <= 0 || N <= 0 || K <= 0 || nranks < 1 || nranks > MAX_RANKS) return kErrBadShape;
  if (rows_per_rank % sub_rows || sub_rows % BM || (wait_mode == 0 && rows_per_rank % BM)) return kErrBadShape;
  if ((lda % 8) || (ldb % 8) || (epi == 0 ? (ldc % 8) : (ldc % 4)) || (row_elems % 8)) return kErrAlignment;
  CUtensorMap tmA, tmB, tmC;
  int mn3d = 0, l3 = 0;
  bool ok = make_ab_maps(&tmA, &tmB, A, B, M, N, K, lda, ldb, a_mn, b_mn, &mn3d);
  if (epi == 0) ok &= encode_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, C, N, M, uint64_t(ldc) * 2, 64, BM);
  else ok &= encode_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, C, N, M, uint64_t(ldc) * 4, 32, BM);
  // map over this rank's own shard, in the role the gathered operand plays in this GEMM
  CUtensorMap tmL;
  if (wait_mode == 0) {
    ok &= encode_tmap_2d(&tmL, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x_shard, K, rows_per_rank, uint64_t(row_elems) * 2, BK, BM);
  } else if (!gathered_b) {
    ok &= encode_tmap_mn(&tmL, x_shard, M, rows_per_rank, uint64_t(row_elems) * 2, BM / 64, BK, &l3);
  } else {
    ok &= encode_tmap_mn(&tmL, x_shard, N, rows_per_rank, uint64_t(row_elems) * 2, BN / 64, BK, &l3);
  }
  if (!ok) return kErrTensorMap;
  AGParams p;
  p.M = M; p.N = N; p.K = K; p.rank = rank; p.nranks = nranks; p.rows_per_rank = rows_per_rank;
  p.sub_rows = sub_rows; p.row_elems = row_elems; p.n_comm = n_comm; p.epoch = epoch; p.wait_mode = wait_mode;
  p.gathered_b = gathered_b; p.mn3d = mn3d | (l3 << 2); p.skip_push = skip_push; p.do_ack = do_ack; p.x_shard = x_shard; p.local_done = local_done; p.status = status; p.bias = bias;
  p.wait_ns = static_cast<unsigned long long>(wait_ms) * 1000000ull;
  for (int i = 0; i < MAX_RANKS; ++i) {
    p.peer_stage[i] = i < nranks ? peer_stage[i] : 0;
    p.peer_flags[i] = i < nranks ? peer_flags[i] : 0;
    p.peer_ack[i] = i < nranks ? peer_ack[i] : 0;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int gemm_ctas = sm_count() - n_comm;
  if (gemm_ctas > tiles) gemm_ctas = tiles;
  if (gemm_ctas < 1) return kErrBadShape;
  const int grid = gemm_ctas + n_comm;
  p.done_target = 0;
  if (do_ack) {   // cumulative count of acknowledging GEMM CTAs on this slot, kept next to the counter on the host side
    p.done_target = done_base + gemm_ctas;
  }
#define PD_AG_CASE(AM, BM_, E)                                                                      \
  if (a_mn == AM && b_mn == BM_ && epi == E) {                                                      \
    static bool cfg = false;                                                                        \
    auto kfn = ag_gemm_kernel<AM, BM_, E>;                                                          \
    if (!cfg) { if (set_smem(kfn)) return kErrCuda; cfg = true; }                                   \
    kfn<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, tmC, tmL, p);                            \
    return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;                                \
  }
  PD_AG_CASE(0, 1, 0)   // forward:  Y = AG(X) W            (tokens = M)
  PD_AG_CASE(0, 0, 0)   // backward: dX = AG(dY) W^T        (tokens = M)
  PD_AG_CASE(1, 1, 2)   // wgrad:    dW += AG(X)^T dY / X^T AG(dY)   (tokens = reduction dim)
  PD_AG_CASE(1, 1, 0)
#undef PD_AG_CASE
  return kErrBadShape;
}

// GEMM -> reduce-scatter.  A: [M, K] (or [K, M] if a_mn), B as in pd_gemm_bf16, M = nranks * rows_per_rank.
// peer_recv[d]: receive buffer of rank d, bf16 [nranks][rows_per_rank][N]; out: [rows_per_rank, N] bf16.
PD_EXPORT int pd_gemm_rs(const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb, int a_mn,
                         int b_mn, int rows_per_rank, int rank, int nranks, int epoch,
                         const unsigned long long* peer_recv, const unsigned long long* peer_counters,
                         const unsigned long long* peer_ack, int* local_done, const int* bias, int wait_ms, int* status,
                         cudaStream_t stream) {
  using namespace pd;
  using namespace pd::gc;
  if (M <= 0 || N <= 0 || K <= 0 || nranks < 1 || nranks > MAX_RANKS || M != rows_per_rank * nranks) return kErrBadShape;
  if ((lda % 8) || (ldb % 8) || (N % 8)) return kErrAlignment;
  CUtensorMap tmA, tmB;
  int mn3d = 0;
  if (!make_ab_maps(&tmA, &tmB, A, B, M, N, K, lda, ldb, a_mn, b_mn, &mn3d)) return kErrTensorMap;
  RSMaps maps;
  const size_t slab_bytes = static_cast<size_t>(rows_per_rank) * N * 2;
  for (int d = 0; d < MAX_RANKS; ++d) {
    const int dd = d < nranks ? d : 0;
    void* base = reinterpret_cast<void*>(peer_recv[dd] + static_cast<size_t>(rank) * slab_bytes);
    if (!encode_tmap_2d(&maps.dst[d], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, N, rows_per_rank, uint64_t(N) * 2, 64, BM))
      return kErrTensorMap;
  }
  RSParams p;
  p.M = M; p.N = N; p.K = K; p.rank = rank; p.nranks = nranks; p.rows_per_rank = rows_per_rank; p.epoch = epoch;
  p.mn3d = mn3d;
  p.recv_local = reinterpret_cast<const void*>(peer_recv[rank]);
  p.out = out; p.local_done = local_done; p.status = status; p.bias = bias;
  p.wait_ns = static_cast<unsigned long long>(wait_ms) * 1000000ull;
  for (int i = 0; i < MAX_RANKS; ++i) {
    p.peer_counters[i] = i < nranks ? peer_counters[i] : 0;
    p.peer_ack[i] = i < nranks ? peer_ack[i] : 0;
  }
  const int tiles = ((rows_per_rank + BM - 1) / BM) * nranks * ((N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
#define PD_RS_CASE(AM, BM_)                                                                         \
  if (a_mn == AM && b_mn == BM_) {                                                                  \
    static bool cfg = false;                                                                        \
    auto kfn = gemm_rs_kernel<AM, BM_>;                                                             \
    if (!cfg) { if (set_smem(kfn)) return kErrCuda; cfg = true; }                                   \
    kfn<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, maps, p);                              \
    return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;                                \
  }
  PD_RS_CASE(0, 1)   // forward:  Y = X W  -> reduce-scatter
  PD_RS_CASE(0, 0)   // backward: dX = dY W^T -> reduce-scatter
#undef PD_RS_CASE
  return kErrBadShape;
}
