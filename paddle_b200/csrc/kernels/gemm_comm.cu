// Fused compute + collective GEMMs over NVLink peer memory (one kernel launch each, one process per GPU):
//
//   ag_gemm : all-gather -> GEMM.  A few "comm" CTAs push this rank's activation shard into every peer's
//             staging buffer; the remaining CTAs run the persistent tcgen05 GEMM, consuming chunks in arrival
//             order (local shard first) — the TMA producer waits on the chunk's arrival counter (ld.acquire.sys,
//             bounded) before it loads tiles of that chunk from LOCAL memory.  Nothing is read twice over
//             NVLink.  Three push forms (push_mode): 2 = one multimem.st per 16 bytes, replicated to every
//             peer by the NVSwitch (the SM issues 1/(n-1) of the stores); 1 = 16-byte stores to each peer from
//             all threads of the comm CTAs; 0 = one thread per comm CTA driving a ring of bulk copies.
//   gemm_rs : GEMM -> reduce-scatter.  Tiles are computed destination by destination (remote first, own
//             shard last); the epilogue TMA-stores each bf16 partial tile straight into the destination
//             rank's receive buffer and bumps that tile's arrival counter (red.release.sys); every CTA then
//             reduces tiles of its own shard as soon as all ranks' partials have landed.
//   gemm_rs_mc : the same contract over NVLS.  Every rank keeps its full partial product in its own
//             symmetric buffer (local TMA stores) and bumps the owner's per-tile counter; a few reducer CTAs
//             of the owner read each complete tile with multimem.ld_reduce, which sums the n copies inside
//             the switch, so a rank receives rows/n of the data instead of (n-1) slabs and no SM adds anything.
//             Tiles are produced row-block by row-block in the same order on every rank, so reduction runs
//             under the GEMM and only the last row block is a tail.
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
  uint64_t full[STAGES], empty[STAGES], tfull[2], tempty[2], drain, red[2];
  uint32_t tmem_base;
  int abort_flag;
  int epi_decision;
};

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

template <int G = 16>
__device__ __forceinline__ void raster(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = G * tiles_n;
  const int g = t / per_group;
  const int first_m = g * G;
  const int gsz = min(G, tiles_m - first_m);
  const int r = t - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

// Tile order of the all-gather GEMM when tokens are the M dimension.  Row blocks are visited in the order in which
// their data becomes available: first the rank's own shard (read in place, no wait), then the peers' 128-row chunks
// in ARRIVAL order - every peer pushes its chunk 0 first, then its chunk 1, ... - so that a CTA never waits for a
// chunk that is pushed late while earlier chunks lie unused.  Remote rows are rastered in groups of four row blocks:
// a group's tiles are dealt across all CTAs at once, so a larger group would make the whole GPU wait for the
// group's last chunk.
__device__ __forceinline__ void ag_tile(int t, int tiles_n, int tiles_per_src, int rank, int nranks, int& tm, int& tn) {
  const int local_tiles = tiles_per_src * tiles_n;
  if (t < local_tiles) {
    int i;
    raster<16>(t, tiles_per_src, tiles_n, i, tn);
    tm = rank * tiles_per_src + i;
    return;
  }
  int j;
  raster<4>(t - local_tiles, tiles_per_src * (nranks - 1), tiles_n, j, tn);
  const int c = j / (nranks - 1), k = j - c * (nranks - 1);
  int src = rank + 1 + k;
  if (src >= nranks) src -= nranks;
  tm = src * tiles_per_src + c;
}
// Same idea when tokens are the reduction dimension: k-blocks of the own shard first, then the peers' chunks in
// arrival order (a sum may run over k in any order).
__device__ __forceinline__ int ag_kblock(int kbi, int kb_per_src, int kb_per_chunk, int rank, int nranks) {
  if (kbi < kb_per_src) return rank * kb_per_src + kbi;
  const int j = kbi - kb_per_src;
  const int jj = j / kb_per_chunk, within = j - jj * kb_per_chunk;
  const int c = jj / (nranks - 1), k = jj - c * (nranks - 1);
  int src = rank + 1 + k;
  if (src >= nranks) src -= nranks;
  return src * kb_per_src + c * kb_per_chunk + within;
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
  mbar_init(&bars->red[0], 1);
  mbar_init(&bars->red[1], 1);
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

// Optional phase timestamps of the all-gather GEMM (diagnostics, globaltimer ns): per CTA {start, loads issued,
// ns spent waiting for arrival flags, epilogue done, push done (communication CTAs)}.  Off unless pd_ag_gemm_trace(1).
__device__ int g_ag_trace_on = 0;
__device__ unsigned long long g_ag_trace[256 * 8];
__device__ __forceinline__ void ag_trace(int slot, unsigned long long v) {
  if (g_ag_trace_on && blockIdx.x < 256) g_ag_trace[blockIdx.x * 8 + slot] = v;
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
  int push_mode;       // 0 bulk-copy ring (one thread), 1 vector stores to every peer, 2 multimem.st through mc_stage
  int parts;           // arrivals per chunk flag and epoch: a chunk's flag counts up to epoch * parts
  unsigned long long mc_stage;  // multicast address of the staging buffer (push_mode 2)
  const void* x_shard; // [rows_per_rank, row_elems] bf16, local
  unsigned long long peer_stage[MAX_RANKS];  // staging buffer [nranks*rows_per_rank, row_elems] of every rank
  unsigned long long peer_flags[MAX_RANKS];  // int32 [nranks][n_sub] of every rank
  unsigned long long peer_ack[MAX_RANKS];    // int32 [nranks] of every rank
  int* local_done;
  int* status;
  unsigned long long wait_ns;
};

struct AckPtrs {
  unsigned long long p[MAX_RANKS];
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
    if (p.skip_push) return;
    if (p.push_mode != 0) {
      // All threads copy: 16-byte loads from the local shard, then either one multimem.st (replicated to every
      // rank's staging buffer by the switch) or one plain store per peer.  A job is 1/parts of a 128-row chunk;
      // after a job every peer's arrival counter of that chunk is bumped once, so a chunk is complete at
      // epoch * parts.  Jobs are dealt chunk-major so that early chunks complete first.
      __shared__ int push_ok;
      const int* ack_local = reinterpret_cast<const int*>(p.peer_ack[p.rank]);
      if (threadIdx.x == 0) {
        bool ok = true;   // every peer must have finished reading what the previous epoch put into this slot
        for (int k = 1; k < p.nranks && ok; ++k) {
          const int peer = (p.rank + k) % p.nranks;
          ok = flag_wait_ge(ack_local + peer, epoch_v - 1, p.wait_ns, p.status, 500 + peer);
        }
        push_ok = ok ? 1 : 0;
      }
      __syncthreads();
      if (!push_ok) return;
      const uint32_t chunk_bytes = static_cast<uint32_t>(p.sub_rows) * static_cast<uint32_t>(p.row_elems) * 2u;
      const uint32_t part_bytes = chunk_bytes / static_cast<uint32_t>(p.parts);
      const int jobs = n_sub * p.parts;
      // 16 loads of 16 bytes in flight per thread (48 KB per CTA): the copy is bound by the latency of the local
      // reads, not by store issue
      constexpr int U = 16;
      constexpr uint32_t STEP = NUM_THREADS * 16;
      for (int job = blockIdx.x; job < jobs; job += p.n_comm) {
        const int c = job / p.parts, q = job - c * p.parts;
        const uint8_t* src = static_cast<const uint8_t*>(p.x_shard) + static_cast<size_t>(c) * chunk_bytes +
                             static_cast<size_t>(q) * part_bytes;
        const size_t dst_off = (static_cast<size_t>(p.rank) * n_sub + c) * chunk_bytes + static_cast<size_t>(q) * part_bytes;
        for (uint32_t i = threadIdx.x * 16; i < part_bytes; i += STEP * U) {
          uint4 v[U];
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (i + u * STEP < part_bytes) v[u] = ld_nc_v4(src + i + u * STEP);
          if (p.push_mode == 2) {
            uint8_t* dst = reinterpret_cast<uint8_t*>(p.mc_stage) + dst_off;
#pragma unroll
            for (int u = 0; u < U; ++u)
              if (i + u * STEP < part_bytes) multimem_st_v4(dst + i + u * STEP, v[u]);
          } else {
            for (int k = 1; k < p.nranks; ++k) {
              uint8_t* dst = reinterpret_cast<uint8_t*>(p.peer_stage[(p.rank + k) % p.nranks]) + dst_off;
#pragma unroll
              for (int u = 0; u < U; ++u)
                if (i + u * STEP < part_bytes) st_v4(dst + i + u * STEP, v[u]);
            }
          }
        }
        __syncthreads();           // every thread's stores of this job are issued and ordered before thread 0's release
        if (threadIdx.x == 0) {
          asm volatile("fence.acq_rel.sys;" ::: "memory");
          for (int k = 1; k < p.nranks; ++k)
            asm volatile("red.relaxed.sys.global.add.s32 [%0], 1;" ::"l"(
                             reinterpret_cast<int*>(p.peer_flags[(p.rank + k) % p.nranks]) + p.rank * n_sub + c)
                         : "memory");
        }
        // Nobody starts the next job before the arrival has been published: a system-scope fence completes only when
        // the SM's outstanding remote stores have drained, and stores of the next job issued meanwhile by the other
        // warps kept it (and with it every flag) waiting until the whole push was over.
        __syncthreads();
      }
      if (threadIdx.x == 0) ag_trace(4, globaltimer_ns());
      return;
    }
    if (threadIdx.x != 0) return;
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
    // A piece is either several whole rows (rows of up to PIECE_MAX bytes) or one PIECE_MAX-byte segment of a row
    // (wider rows, e.g. a gathered weight of 12288+ columns: a whole row would overrun its ring slot).
    const int segs = (row_bytes + PIECE_MAX - 1) / PIECE_MAX;               // segments per row
    const int rows_per_piece = segs > 1 ? 1 : PIECE_MAX / row_bytes;
    const int ppj = segs > 1 ? p.sub_rows * segs : (p.sub_rows + rows_per_piece - 1) / rows_per_piece;   // pieces per job
    const int total = my_jobs * ppj;
    auto piece_info = [&](int q, int& peer, int& c, int& row0, uint32_t& bytes, uint32_t& col_off) {
      const int j = static_cast<int>(blockIdx.x) + (q / ppj) * p.n_comm;
      c = j / npeers;
      peer = (p.rank + 1 + j % npeers) % p.nranks;
      if (segs > 1) {
        const int idx = q % ppj;
        row0 = idx / segs;
        col_off = static_cast<uint32_t>(idx % segs) * PIECE_MAX;
        bytes = min(static_cast<uint32_t>(PIECE_MAX), row_bytes - col_off);
      } else {
        row0 = (q % ppj) * rows_per_piece;
        col_off = 0;
        const int nrows = min(rows_per_piece, p.sub_rows - row0);
        bytes = static_cast<uint32_t>(nrows) * row_bytes;
      }
    };
    auto issue_load = [&](int q) {
      int peer, c, row0;
      uint32_t bytes, col_off;
      piece_info(q, peer, c, row0, bytes, col_off);
      const int slot = q % RING;
      const uint8_t* src = static_cast<const uint8_t*>(p.x_shard) +
                           (static_cast<size_t>(c) * p.sub_rows + row0) * row_bytes + col_off;
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
      uint32_t bytes, col_off;
      piece_info(q, peer, c, row0, bytes, col_off);
      if (!(checked & (1u << peer))) {
        // the peer must have finished reading what the previous epoch put into this slot
        if (!flag_wait_ge(ack_local + peer, epoch_v - 1, p.wait_ns, p.status, 500 + peer)) { ok = false; break; }
        checked |= 1u << peer;
      }
      const int slot = q % RING;
      if (!mbar_wait(&ring_bar[slot], (q / RING) & 1, &dummy_abort, p.status, 510)) { ok = false; break; }
      uint8_t* dst = reinterpret_cast<uint8_t*>(p.peer_stage[peer]) +
                     ((static_cast<size_t>(p.rank) * n_sub + c) * p.sub_rows + row0) * row_bytes + col_off;
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
  if (threadIdx.x == 0) ag_trace(0, globaltimer_ns());

  if (warp == 4) {
    if (lane == 0) {
      unsigned long long waited = 0;
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      prefetch_tmap(&tmL);
      // everything the loop needs is copied out of the parameter block once: a single thread issues every TMA
      // of this CTA, and re-reading parameters after each asm statement would put it on the critical path
      const int wait_mode = p.wait_mode, rank = p.rank, rows_per_rank = p.rows_per_rank, sub_rows = p.sub_rows;
      const int nranks = p.nranks, kb_per_chunk = p.sub_rows / BK;
      const int epoch = epoch_v * p.parts, gathered_b = p.gathered_b, local_row0 = p.rank * p.rows_per_rank;
      const bool a3d = (p.mn3d & 1) != 0, b3d = (p.mn3d & 2) != 0, l3d = (p.mn3d & 4) != 0;
      const unsigned long long wait_ns = p.wait_ns;
      int* const status = p.status;
      int s = 0;
      uint32_t ph = 0, armed = 0, armed_parity = 0;
      bool ok = true;
      int last_chunk = -1;
      // A chunk's arrival is checked once per CTA, not once per tile: the acquire load at system scope plus the proxy
      // fence cost about a microsecond, and with the tokens as the reduction dimension (weight gradients) a tile walks
      // every remote chunk, so re-checking stalled the four-stage ring for most of a tile.  Nothing is checked at all
      // when the matrix was staged by an earlier launch of this stream (skip_push): that launch consumed every chunk.
      const bool no_wait = p.skip_push != 0;
      unsigned long long seen = 0;
      for (int t = cta; t < num_tiles && ok; t += nct) {
        int tm, tn;
        if (wait_mode == 0 && nranks > 1) ag_tile(t, tiles_n, tiles_per_src, rank, nranks, tm, tn);
        else raster(t, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        // rows of this rank's own shard are read straight from x_shard (map tmL): no copy, no wait
        bool local_tile = false;
        if (wait_mode == 0) {
          local_tile = (m0 / rows_per_rank) == rank;
          const int chunk = m0 / sub_rows;      // == src * n_sub + sub-chunk
          if (!local_tile && chunk != last_chunk) {
            if (!no_wait && !(chunk < 64 && ((seen >> chunk) & 1ull))) {
              const unsigned long long w0 = g_ag_trace_on ? globaltimer_ns() : 0;
              if (!flag_wait_ge(flags_local + chunk, epoch, wait_ns, status, 600)) { ok = false; *abort_flag = 1; break; }
              if (g_ag_trace_on) waited += globaltimer_ns() - w0;
              fence_proxy_async_all();
              if (chunk < 64) seen |= 1ull << chunk;
            }
            last_chunk = chunk;
          }
        }
        for (int kbi = 0; kbi < KB; ++kbi) {
          int kb = kbi;
          bool local_k = false;
          if (wait_mode == 1) {
            kb = nranks > 1 ? ag_kblock(kbi, kb_per_src, kb_per_chunk, rank, nranks) : kbi;
            local_k = ((kb * BK) / rows_per_rank) == rank;
            const int chunk = (kb * BK) / sub_rows;
            if (!local_k && chunk != last_chunk) {
              if (!no_wait && !(chunk < 64 && ((seen >> chunk) & 1ull))) {
                const unsigned long long w0 = g_ag_trace_on ? globaltimer_ns() : 0;
                if (!flag_wait_ge(flags_local + chunk, epoch, wait_ns, status, 610)) { ok = false; *abort_flag = 1; break; }
                if (g_ag_trace_on) waited += globaltimer_ns() - w0;
                fence_proxy_async_all();
                if (chunk < 64) seen |= 1ull << chunk;
              }
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
      ag_trace(1, globaltimer_ns());
      ag_trace(2, waited);
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
      if (p.wait_mode == 0 && p.nranks > 1) ag_tile(t, tiles_n, tiles_per_src, p.rank, p.nranks, tm, tn);
      else raster(t, tiles_m, tiles_n, tm, tn);
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
      ag_trace(3, globaltimer_ns());
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

// Arrival signals of finished partial tiles, batched.  A system-scope fence costs microseconds (it waits until every
// earlier write of the SM is visible to all peers and the host), so issuing one per tile put ~20 us per tile on the
// epilogue's critical path.  Finished tiles are collected here and published together: wait for the bulk stores,
// ONE fence.acq_rel.sys, then one relaxed add per counter.  Used by epilogue thread 0 only.
struct SignalBatch {
  static constexpr int CAP = 8;
  int* ptr[CAP];
  int n = 0;
  __device__ __forceinline__ void flush() {
    if (n == 0) return;
    tma_wait_group<0>();                       // every store issued so far has been written
    asm volatile("fence.acq_rel.sys;" ::: "memory");
#pragma unroll
    for (int i = 0; i < CAP; ++i)
      if (i < n) asm volatile("red.relaxed.sys.global.add.s32 [%0], 1;" ::"l"(ptr[i]) : "memory");
    n = 0;
  }
  __device__ __forceinline__ void add(int* p) {
    if (n == CAP) flush();
#pragma unroll
    for (int i = 0; i < CAP; ++i)
      if (i == n) ptr[i] = p;
    ++n;
  }
};

// Optional phase timestamps of the reduce-scatter GEMM (diagnostics): per CTA {start, GEMM tiles done, arrivals
// published, reduction done, first reduce wait over, first tile reduced} in globaltimer nanoseconds.  Off unless pd_gemm_rs_trace(1) was called.
__device__ int g_rs_trace_on = 0;
__device__ unsigned long long g_rs_trace[256 * 8];
__device__ __forceinline__ void rs_trace(int slot) {
  if (g_rs_trace_on && blockIdx.x < 256) g_rs_trace[blockIdx.x * 8 + slot] = globaltimer_ns();
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
  if (threadIdx.x == 0) rs_trace(0);

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
    SignalBatch sig;
    int last_d = -1;
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
            // Arrivals are published in batches (see SignalBatch): when this CTA moves on to the tiles of its own
            // slab - the remote partials are then announced while the local tiles are computed - when the batch is
            // full, and at the end.
            if (d == p.rank && last_d != p.rank) sig.flush();
            last_d = d;
            sig.add(reinterpret_cast<int*>(p.peer_counters[d]) + tml * tiles_n + tn);
          }
        }
      }
    }
    if (epi_tid == 0) {
      rs_trace(1);
      sig.flush();
      rs_trace(2);
    }
    // ---- reduce phase: out = sum over sources of the partial tiles received for my shard (fp32, rank order).
    // The pass is fed by bulk copies instead of register loads: a unit is rows_u rows of one tile from all n sources
    // (rows_u = 128 / n rounded to a power of two, so that every thread issues exactly one 512-byte row copy), two
    // units of up to 64 KB are in flight per SM in the shared memory the GEMM pipeline no longer needs, and units are
    // dealt across ALL CTAs.  With plain loads (16 x 16 bytes per thread) one SM moved ~10 GB/s and a rank's 64 tiles at
    // 8 ranks kept 64 SMs busy for ~50 us while the others idled.
    const int* counters = reinterpret_cast<const int*>(p.peer_counters[p.rank]);
    const uint8_t* recv = static_cast<const uint8_t*>(p.recv_local);
    uint8_t* outb = static_cast<uint8_t*>(p.out);
    const size_t row_bytes = static_cast<size_t>(p.N) * 2;
    const size_t slab_bytes = static_cast<size_t>(p.rows_per_rank) * row_bytes;
    int np2 = 1;
    while (np2 < p.nranks) np2 <<= 1;
    const int rows_u = BM / np2, units_per_tile = np2;
    const int n_units = tiles_dst_all * units_per_tile;
    constexpr int SEG = BN * 2;                         // bytes of one tile row
    uint8_t* const rbuf0 = smem;                        // 2 x 64 KB inside the (now idle) A/B stage ring
    int last_tile = -1;
    // wait for the unit's tile to be complete, then issue its copies into buffer b; false = gave up
    auto stage_unit = [&](int u, int b) -> bool {
      const int tile = u / units_per_tile, g = u - tile * units_per_tile;
      const int tml = tile % tiles_per_dst, tn = tile / tiles_per_dst;
      if (epi_tid == 0) {
        int okf = 1;
        if (tile != last_tile)
          okf = flag_wait_ge(counters + tml * tiles_n + tn, p.nranks * epoch_v, p.wait_ns, p.status, 800) ? 1 : 0;
        bars->epi_decision = okf;
      }
      last_tile = tile;
      named_bar_sync(1, 128);
      const int okd = bars->epi_decision;
      named_bar_sync(1, 128);
      if (!okd) return false;
      const int row0 = tml * BM + g * rows_u, col0 = tn * BN;
      const int nrow = max(0, min(rows_u, p.rows_per_rank - row0));
      const uint32_t seg = static_cast<uint32_t>(min(BN, p.N - col0)) * 2u;
      uint8_t* buf = rbuf0 + b * 65536;
      fence_proxy_async_smem();                         // earlier generic reads of this buffer vs the async writes
      if (epi_tid == 0) mbar_expect_tx(&bars->red[b], static_cast<uint32_t>(nrow) * p.nranks * seg);
      const int src = epi_tid / rows_u, r = epi_tid - src * rows_u;
      if (src < p.nranks && r < nrow)
        bulk_load(buf + (src * rows_u + r) * SEG, recv + src * slab_bytes + static_cast<size_t>(row0 + r) * row_bytes + col0 * 2,
                  seg, &bars->red[b]);
      return true;
    };
    int iu = 0;
    if (alive && cta < n_units) alive = stage_unit(cta, 0);
    for (int u = cta; u < n_units && alive; u += nct, ++iu) {
      const int b = iu & 1;
      if (u + nct < n_units && !stage_unit(u + nct, b ^ 1)) { alive = false; break; }
      if (!mbar_wait(&bars->red[b], (iu >> 1) & 1, abort_flag, p.status, 810 + b)) { alive = false; break; }
      if (epi_tid == 0 && u == cta) rs_trace(4);
      const int tile = u / units_per_tile, g = u - tile * units_per_tile;
      const int tml = tile % tiles_per_dst, tn = tile / tiles_per_dst;
      const int row0 = tml * BM + g * rows_u, col0 = tn * BN;
      const int nrow = max(0, min(rows_u, p.rows_per_rank - row0));
      const int cvec = epi_tid & 31;
      const uint8_t* buf = rbuf0 + b * 65536;
      if (cvec * 8 < p.N - col0) {
        for (int r = epi_tid >> 5; r < nrow; r += 4) {
          float acc8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int src = 0; src < p.nranks; ++src) {
            const uint4 v = *reinterpret_cast<const uint4*>(buf + (src * rows_u + r) * SEG + cvec * 16);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(h[e]);
              acc8[2 * e] += f.x;
              acc8[2 * e + 1] += f.y;
            }
          }
          uint4 o;
          o.x = pack_bf16x2(acc8[0], acc8[1]);
          o.y = pack_bf16x2(acc8[2], acc8[3]);
          o.z = pack_bf16x2(acc8[4], acc8[5]);
          o.w = pack_bf16x2(acc8[6], acc8[7]);
          *reinterpret_cast<uint4*>(outb + static_cast<size_t>(row0 + r) * row_bytes + col0 * 2 + cvec * 16) = o;
        }
      }
      if (epi_tid == 0 && u == cta) rs_trace(5);
      named_bar_sync(1, 128);                           // buffer b may be refilled
    }
    named_bar_sync(1, 128);
    if (epi_tid == 0) rs_trace(3);
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

// ============================================================================================ gemm_rs_mc
struct RSMcParams {
  int M, N, K;
  int rank, nranks;
  int rows_per_rank;
  int epoch;
  const int* bias;     // optional device int[2]; bias[0] is added to epoch (CUDA-graph replay)
  int mn3d;
  int n_red;           // CTAs [0, n_red) reduce this rank's slab; the rest run the GEMM
  unsigned long long peer_counters[MAX_RANKS];  // int32 [tiles_per_dst * tiles_n] on every rank
  unsigned long long peer_ack[MAX_RANKS];       // int32 [nranks] on every rank
  unsigned long long mc_partial;                // multicast address of the partial buffers, bf16 [M][N] on every rank
  void* out;                                    // bf16 [rows_per_rank][N]
  int* local_done;
  int* status;
  unsigned long long wait_ns;
};

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_rs_mc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmP, const __grid_constant__ RSMcParams p) {
  extern __shared__ uint8_t smem_raw[];
  const int epoch_v = p.epoch + (p.bias != nullptr ? __ldg(p.bias) : 0);
  const int tiles_per_dst = (p.rows_per_rank + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles_dst_all = tiles_per_dst * tiles_n;

  if (static_cast<int>(blockIdx.x) < p.n_red) {
    // ------------------------------------------------------------------ reducer CTA
    // Tile u of this rank's slab (row-block major, the order in which every rank produces them) is complete when
    // its counter reaches nranks * epoch; the tile is then read once through the multicast address - the switch
    // returns the sum over all ranks' partial buffers - and written to `out`.
    __shared__ int red_ok;
    const int* counters = reinterpret_cast<const int*>(p.peer_counters[p.rank]);
    const uint8_t* mc = reinterpret_cast<const uint8_t*>(p.mc_partial);
    uint8_t* out = static_cast<uint8_t*>(p.out);
    bool alive = true;
    // A multimem.ld_reduce takes several microseconds (two NVLink hops plus the add in the switch), so throughput is
    // the number of loads in flight: thread t owns the 16-byte column (t % 32) of rows (t / 32) + 6 k of the tile and
    // keeps U of them outstanding.
    constexpr int U = 11;
    constexpr int ROW_STEP = NUM_THREADS / 32;          // 6 rows between a thread's consecutive loads
    const int cv = threadIdx.x & 31, r_first = threadIdx.x >> 5;
    const size_t row_bytes = static_cast<size_t>(p.N) * 2;
    for (int u = blockIdx.x; u < tiles_dst_all && alive; u += p.n_red) {
      const int tml = u / tiles_n, tn = u - tml * tiles_n;
      if (threadIdx.x == 0)
        red_ok = flag_wait_ge(counters + tml * tiles_n + tn, p.nranks * epoch_v, p.wait_ns, p.status, 800) ? 1 : 0;
      __syncthreads();
      const int okd = red_ok;
      __syncthreads();
      if (!okd) { alive = false; break; }
      const int row0 = tml * BM, col0 = tn * BN;
      const int nrow = min(BM, p.rows_per_rank - row0);
      if (col0 + cv * 8 >= p.N) continue;                      // N % 8 == 0: a vector is inside or outside as a whole
      const size_t base = (static_cast<size_t>(row0) * p.N + col0 + cv * 8) * 2;
      const uint8_t* src = mc + static_cast<size_t>(p.rank) * p.rows_per_rank * row_bytes + base;
      uint8_t* dst = out + base;
      for (int r = r_first; r < nrow; r += ROW_STEP * U) {
        uint4 v[U];
#pragma unroll
        for (int k = 0; k < U; ++k)
          if (r + k * ROW_STEP < nrow) v[k] = multimem_ld_reduce_bf16x8(src + static_cast<size_t>(r + k * ROW_STEP) * row_bytes);
#pragma unroll
        for (int k = 0; k < U; ++k)
          if (r + k * ROW_STEP < nrow) *reinterpret_cast<uint4*>(dst + static_cast<size_t>(r + k * ROW_STEP) * row_bytes) = v[k];
      }
    }
    __syncthreads();
    if (threadIdx.x == 0 && alive) {
      // every partial tile of this epoch has been read out of every rank's buffer: they may overwrite them
      __threadfence();
      // the last reducer of THIS launch acknowledges and re-arms the counter (launches on a slot are ordered on one
      // stream, so the count never mixes two launches and the number of reducers may differ from call to call)
      const int done = atomicAdd(p.local_done, 1) + 1;
      if (done == p.n_red) {
        atomicExch(p.local_done, 0);
        for (int r = 0; r < p.nranks; ++r) st_release_sys(reinterpret_cast<int*>(p.peer_ack[r]) + p.rank, epoch_v);
      }
    }
    return;
  }

  // -------------------------------------------------------------------- GEMM CTA
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint8_t* sC = sB + STAGES * B_STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(sC + 2 * C_CHUNK_BYTES);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x - p.n_red, nct = gridDim.x - p.n_red;
  const int num_tiles = tiles_dst_all * p.nranks;
  const int KB = (p.K + BK - 1) / BK;
  const int my_tiles = cta < num_tiles ? (num_tiles - cta + nct - 1) / nct : 0;

  if (threadIdx.x == 0) init_barriers(bars);
  if (warp == 5) tmem_alloc(&bars->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  // tile t -> (row block tml, destination d, column tile tn): the same order on every rank, so the n partial
  // copies of a tile are finished at about the same time and its owner can reduce it while the GEMM goes on
  auto decode = [&](int t, int& d, int& tml, int& tn) {
    const int per = p.nranks * tiles_n;
    tml = t / per;
    const int r = t - tml * per;
    d = r / tiles_n;
    tn = r - d * tiles_n;
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
    SignalBatch sig;
    for (int t = cta; t < num_tiles; t += nct, ++it) {
      int d, tml, tn;
      decode(t, d, tml, tn);
      const int n0 = tn * BN;
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      if (epi_tid == 0) {
        bool ok = mbar_wait(&bars->tfull[acc], acc_ph, abort_flag, p.status, 400 + acc);
        if (ok && !(checked & (1u << d))) {
          // owner d must have finished reading the previous epoch's partial tiles out of this rank's buffer
          ok = flag_wait_ge(ack_local + d, epoch_v - 1, p.wait_ns, p.status, 700 + d);
          if (!ok) *abort_flag = 1;
          checked |= 1u << d;
        }
        bars->epi_decision = ok ? 1 : 0;
      }
      named_bar_sync(1, 128);
      if (bars->epi_decision == 0) break;
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
          // rows beyond this destination's slab (rows_per_rank not a multiple of 128) would land in the next
          // destination's rows: the map is 3-D {N, rows_per_rank, nranks}, which clips them
          tma_store_3d(&tmP, stage, n0 + c * CW, tml * BM, d);
          tma_commit_group();
          if (c == NCHUNK - 1) {
            // arrivals are published four tiles at a time (see SignalBatch) and at the end
            sig.add(reinterpret_cast<int*>(p.peer_counters[d]) + tml * tiles_n + tn);
            if (sig.n >= 4) sig.flush();
          }
        }
      }
    }
    if (epi_tid == 0) {
      sig.flush();
      tma_wait_group<0>();
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
                         int push_mode, int parts, unsigned long long mc_stage, int* status, cudaStream_t stream) {
  using namespace pd;
  using namespace pd::gc;
  if (M <= 0 || N <= 0 || K <= 0 || nranks < 1 || nranks > MAX_RANKS) return kErrBadShape;
  if (push_mode < 0 || push_mode > 2 || parts < 1 || (push_mode == 0 && parts != 1)) return kErrBadShape;
  if (push_mode == 2 && mc_stage == 0) return kErrBadShape;
  if ((static_cast<long long>(sub_rows) * row_elems * 2) % (16ll * parts)) return kErrAlignment;
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
  p.push_mode = push_mode; p.parts = parts; p.mc_stage = mc_stage;
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

// Acknowledgement on its own: the staged matrix of `epoch` has been consumed by other launches of this stream (a plain
// GEMM reading the staging buffer), so the peers may overwrite it.  Counts as ONE acknowledging CTA in the slot's
// cumulative `local_done` bookkeeping (the host advances its base by one).
namespace pd {
namespace gc {
__global__ void ag_ack_kernel(int rank, int nranks, int epoch, AckPtrs ptrs, int* local_done, const int* bias) {
  // one lane per peer: the release stores (each of which orders the earlier reads of this GPU before it) go out side
  // by side instead of one after the other
  const int epoch_v = epoch + (bias != nullptr ? __ldg(bias) : 0);
  if (threadIdx.x == 0) atomicAdd(local_done, 1);
  if (static_cast<int>(threadIdx.x) < nranks) st_release_sys(reinterpret_cast<int*>(ptrs.p[threadIdx.x]) + rank, epoch_v);
}
}  // namespace gc
}  // namespace pd
PD_EXPORT int pd_ag_ack(int rank, int nranks, int epoch, const unsigned long long* peer_ack, int* local_done, const int* bias,
                        cudaStream_t stream) {
  using namespace pd;
  using namespace pd::gc;
  if (nranks < 1 || nranks > MAX_RANKS) return kErrBadShape;
  AckPtrs ptrs;
  for (int i = 0; i < MAX_RANKS; ++i) ptrs.p[i] = i < nranks ? peer_ack[i] : 0;
  ag_ack_kernel<<<1, 32, 0, stream>>>(rank, nranks, epoch, ptrs, local_done, bias);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
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
  PD_RS_CASE(1, 1)   // weight gradient of a row-sharded weight: dW = X^T dY -> reduce-scatter over the rows of W
#undef PD_RS_CASE
  return kErrBadShape;
}

// GEMM -> reduce-scatter over NVLS.  partial_local: this rank's bf16 [M][N] partial buffer inside a symmetric block
// whose multicast address is mc_partial (the same offset on every rank).  n_red reducer CTAs (may differ from call to call).
PD_EXPORT int pd_gemm_rs_mc(const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb, int a_mn,
                            int b_mn, int rows_per_rank, int rank, int nranks, int epoch, void* partial_local,
                            unsigned long long mc_partial, const unsigned long long* peer_counters,
                            const unsigned long long* peer_ack, int* local_done, const int* bias, int n_red, int wait_ms,
                            int* status, cudaStream_t stream) {
  using namespace pd;
  using namespace pd::gc;
  if (M <= 0 || N <= 0 || K <= 0 || nranks < 1 || nranks > MAX_RANKS || M != rows_per_rank * nranks) return kErrBadShape;
  if (n_red < 1 || mc_partial == 0) return kErrBadShape;
  if ((lda % 8) || (ldb % 8) || (N % 8)) return kErrAlignment;
  if (!aligned16(partial_local) || !aligned16(out) || (mc_partial & 15ull)) return kErrAlignment;
  CUtensorMap tmA, tmB, tmP;
  int mn3d = 0;
  if (!make_ab_maps(&tmA, &tmB, A, B, M, N, K, lda, ldb, a_mn, b_mn, &mn3d)) return kErrTensorMap;
  if (!encode_tmap_3d(&tmP, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, partial_local, N, rows_per_rank, nranks, uint64_t(N) * 2,
                      uint64_t(rows_per_rank) * N * 2, 64, BM, 1))
    return kErrTensorMap;
  RSMcParams p;
  p.M = M; p.N = N; p.K = K; p.rank = rank; p.nranks = nranks; p.rows_per_rank = rows_per_rank; p.epoch = epoch;
  p.mn3d = mn3d; p.n_red = n_red; p.mc_partial = mc_partial;
  p.out = out; p.local_done = local_done; p.status = status; p.bias = bias;
  p.wait_ns = static_cast<unsigned long long>(wait_ms) * 1000000ull;
  for (int i = 0; i < MAX_RANKS; ++i) {
    p.peer_counters[i] = i < nranks ? peer_counters[i] : 0;
    p.peer_ack[i] = i < nranks ? peer_ack[i] : 0;
  }
  const int tiles = ((rows_per_rank + BM - 1) / BM) * nranks * ((N + BN - 1) / BN);
  int gemm_ctas = sm_count() - n_red;
  if (gemm_ctas > tiles) gemm_ctas = tiles;
  if (gemm_ctas < 1) return kErrBadShape;
  const int grid = gemm_ctas + n_red;
#define PD_RSM_CASE(AM, BM_)                                                                        \
  if (a_mn == AM && b_mn == BM_) {                                                                  \
    static bool cfg = false;                                                                        \
    auto kfn = gemm_rs_mc_kernel<AM, BM_>;                                                          \
    if (!cfg) { if (set_smem(kfn)) return kErrCuda; cfg = true; }                                   \
    kfn<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, tmP, p);                               \
    return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;                                \
  }
  PD_RSM_CASE(0, 1)   // forward:  Y = X W  -> reduce-scatter
  PD_RSM_CASE(0, 0)   // backward: dX = dY W^T -> reduce-scatter
  PD_RSM_CASE(1, 1)   // weight gradient of a row-sharded weight
#undef PD_RSM_CASE
  return kErrBadShape;
}

// Diagnostics: switch the per-CTA phase timestamps of pd_gemm_rs on / off, and copy them out (256 x 4 values).
PD_EXPORT int pd_gemm_rs_trace(int on) {
  void* p = nullptr;
  if (on && cudaGetSymbolAddress(&p, pd::gc::g_rs_trace) == cudaSuccess) cudaMemset(p, 0, sizeof(unsigned long long) * 256 * 8);
  return cudaMemcpyToSymbol(pd::gc::g_rs_trace_on, &on, sizeof(int)) == cudaSuccess ? 0 : pd::kErrCuda;
}
PD_EXPORT int pd_gemm_rs_trace_read(unsigned long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, pd::gc::g_rs_trace, sizeof(unsigned long long) * 256 * 8) == cudaSuccess
             ? 0 : pd::kErrCuda;
}
PD_EXPORT int pd_ag_gemm_trace(int on) {
  void* p = nullptr;
  if (on && cudaGetSymbolAddress(&p, pd::gc::g_ag_trace) == cudaSuccess) cudaMemset(p, 0, sizeof(unsigned long long) * 256 * 8);
  return cudaMemcpyToSymbol(pd::gc::g_ag_trace_on, &on, sizeof(int)) == cudaSuccess ? 0 : pd::kErrCuda;
}
PD_EXPORT int pd_ag_gemm_trace_read(unsigned long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, pd::gc::g_ag_trace, sizeof(unsigned long long) * 256 * 8) == cudaSuccess
             ? 0 : pd::kErrCuda;
}
