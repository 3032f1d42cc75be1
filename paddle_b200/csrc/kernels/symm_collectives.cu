// Standalone collectives over symmetric (peer-mapped) memory for small and medium messages, where a library
// collective is dominated by launch and protocol latency:
//   pd_symm_all_reduce     : one-shot - every rank pushes its whole vector into row [rank] of every peer's receive
//                            buffer, then sums the n rows it received (fp32 accumulation, rank order: deterministic)
//   pd_symm_all_gather     : every rank pushes its shard into slot [rank] of every peer's output buffer
//   pd_symm_reduce_scatter : every rank pushes slice d of its vector to rank d, which sums the n rows
//   pd_symm_all_to_all     : every rank pushes slice d of its vector to rank d, which lays the n rows out in rank order
// (reference: ProcessGroupNCCL::AllReduce / AllGather / ReduceScatter, paddle/fluid/distributed/collective/
// process_group_nccl.cc:241,197,408 - the NCCL calls remain the path for large messages).
// Same protocol as the fused kernels: plain peer stores, one release-add per chunk on the destination's counter,
// bounded acquire-wait on the own counters, device-resident epoch (CUDA-graph replayable), two alternating slots.
#include <cuda_bf16.h>

#include "host_utils.h"
#include "sm100_prims.cuh"

namespace pd {
namespace sc {

typedef __nv_bfloat16 bf16;
constexpr int CHUNK_BYTES = 16384;
constexpr int THREADS = 256;
constexpr int MAX_RANKS = 8;

struct Args {
  const uint8_t* in;             // local input
  uint8_t* out;                  // local output
  uint8_t* recv[MAX_RANKS];      // receive buffers: [2][nranks][row_bytes_padded]
  int* cnt[MAX_RANKS];           // per-chunk counters
  int64_t in_row_bytes;          // bytes this rank contributes per destination row
  int64_t row_pad;               // padded row size in the receive buffer
  int rank, nranks, chunks, kind, is_bf16;   // kind 0 all_reduce, 1 all_gather, 2 reduce_scatter
  int chunk_bytes;               // multiple of CHUNK_BYTES, the same on every rank for a given call
  int* state;
  int* seen;                     // local, per chunk: arrivals consumed so far (calls of different sizes touch different chunks)
  unsigned long long wait_ns;
  int* status;
};

// 16-byte copies with four loads in flight per thread before the first store: over NVLink the copy is bound by the
// number of outstanding requests, not by issue rate.
__device__ __forceinline__ void copy_bytes(uint8_t* dst, const uint8_t* src, int64_t n, bool src_is_peer_written) {
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | n) & 15u) == 0) {
    const int64_t step = static_cast<int64_t>(THREADS) * 16;
    int64_t i = threadIdx.x * 16;
    for (; i + 3 * step < n; i += 4 * step) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint4* p = reinterpret_cast<const uint4*>(src + i + u * step);
        v[u] = src_is_peer_written ? __ldcg(p) : *p;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) *reinterpret_cast<uint4*>(dst + i + u * step) = v[u];
    }
    for (; i < n; i += step) {
      const uint4* p = reinterpret_cast<const uint4*>(src + i);
      *reinterpret_cast<uint4*>(dst + i) = src_is_peer_written ? __ldcg(p) : *p;
    }
  } else {
    for (int64_t i = threadIdx.x; i < n; i += THREADS) dst[i] = src_is_peer_written ? __ldcg(src + i) : src[i];
  }
}

__device__ __forceinline__ void add_bf16x8(float* acc, const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    acc[2 * e] += __uint_as_float(w[e] << 16);
    acc[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
  }
}

__global__ void __launch_bounds__(THREADS) symm_collective_kernel(Args a) {
  __shared__ int verdict;
  const int epoch = a.state[0] + 1;
  const int64_t slot_off = static_cast<int64_t>(epoch & 1) * a.nranks * a.row_pad;
  // ---- push: item = (destination, chunk)
  const int items = a.nranks * a.chunks;
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    const int dst = (a.rank + 1 + it / a.chunks) % a.nranks;
    const int c = it % a.chunks;
    const int64_t b0 = static_cast<int64_t>(c) * a.chunk_bytes;
    const int64_t n = min(static_cast<int64_t>(a.chunk_bytes), a.in_row_bytes - b0);
    // all_reduce / all_gather send the same bytes to everybody; reduce_scatter and all_to_all send slice `dst`
    const uint8_t* src = a.in + (a.kind >= 2 ? static_cast<int64_t>(dst) * a.in_row_bytes : 0) + b0;
    copy_bytes(a.recv[dst] + slot_off + static_cast<int64_t>(a.rank) * a.row_pad + b0, src, n, false);
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) red_release_sys_add(a.cnt[dst] + c, 1);
  }
  // ---- consume the n rows that arrived here
  const uint8_t* base = a.recv[a.rank] + slot_off;
  for (int c = blockIdx.x; c < a.chunks; c += gridDim.x) {
    if (threadIdx.x == 0) {
      // expected arrivals are tracked per chunk, not derived from the epoch: a short message leaves the counters of
      // the higher chunks untouched while the epoch still advances
      const int target = a.seen[c] + a.nranks;
      verdict = flag_wait_ge(a.cnt[a.rank] + c, target, a.wait_ns, a.status, 800) ? 1 : 0;
      a.seen[c] = target;
    }
    __syncthreads();
    const bool ok = verdict != 0;
    __syncthreads();
    if (!ok) continue;
    const int64_t b0 = static_cast<int64_t>(c) * a.chunk_bytes;
    const int64_t n = min(static_cast<int64_t>(a.chunk_bytes), a.in_row_bytes - b0);
    if (a.kind == 1 || a.kind == 3) {
      for (int r = 0; r < a.nranks; ++r)
        copy_bytes(a.out + static_cast<int64_t>(r) * a.in_row_bytes + b0, base + static_cast<int64_t>(r) * a.row_pad + b0, n,
                   true);
    } else {
      uint8_t* o = a.out + b0;
      const bool vec = ((reinterpret_cast<uintptr_t>(o) | n) & 15u) == 0;      // rows start 256-byte aligned
      int64_t done = 0;
      if (vec) {
        for (int64_t i = threadIdx.x * 16; i < n; i += THREADS * 16) {
          if (a.is_bf16) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < a.nranks; ++r)
              add_bf16x8(acc, __ldcg(reinterpret_cast<const uint4*>(base + static_cast<int64_t>(r) * a.row_pad + b0 + i)));
            uint4 ov;
            ov.x = pack_bf16x2(acc[0], acc[1]);
            ov.y = pack_bf16x2(acc[2], acc[3]);
            ov.z = pack_bf16x2(acc[4], acc[5]);
            ov.w = pack_bf16x2(acc[6], acc[7]);
            *reinterpret_cast<uint4*>(o + i) = ov;
          } else {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < a.nranks; ++r) {
              const float4 t = __ldcg(reinterpret_cast<const float4*>(base + static_cast<int64_t>(r) * a.row_pad + b0 + i));
              acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
            }
            *reinterpret_cast<float4*>(o + i) = acc;
          }
        }
        done = n;
      }
      if (a.is_bf16) {
        bf16* ob = reinterpret_cast<bf16*>(o);
        for (int64_t i = done / 2 + threadIdx.x; i < n / 2; i += THREADS) {
          float s = 0.f;
          for (int r = 0; r < a.nranks; ++r)
            s += __bfloat162float(__ldcg(reinterpret_cast<const bf16*>(base + static_cast<int64_t>(r) * a.row_pad + b0) + i));
          ob[i] = __float2bfloat16(s);
        }
      } else {
        float* of = reinterpret_cast<float*>(o);
        for (int64_t i = done / 4 + threadIdx.x; i < n / 4; i += THREADS) {
          float s = 0.f;
          for (int r = 0; r < a.nranks; ++r)
            s += __ldcg(reinterpret_cast<const float*>(base + static_cast<int64_t>(r) * a.row_pad + b0) + i);
          of[i] = s;
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.state + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      a.state[1] = 0;
      __threadfence();
      a.state[0] = epoch;
    }
  }
}

}  // namespace sc
}  // namespace pd

PD_EXPORT int pd_symm_chunk_bytes() { return pd::sc::CHUNK_BYTES; }

// kind 0 all_reduce (in: row_bytes, out: row_bytes), 1 all_gather (in: row_bytes, out: nranks * row_bytes),
// 2 reduce_scatter (in: nranks * row_bytes, out: row_bytes), 3 all_to_all (in / out: nranks * row_bytes, slice d of
// the input goes to rank d, slice s of the output came from rank s).  peer_recv[r]: [2][nranks][row_pad] bytes on rank r,
// peer_cnt[r]: int32 [ceil(row_pad / 16384)] zeroed once; state: 2 local int32 zeroed once; seen: local int32
// [ceil(row_pad / 16384)] zeroed once.
PD_EXPORT int pd_symm_collective(int kind, const void* in, void* out, int64_t row_bytes, int64_t row_pad, int is_bf16,
                                 int rank, int nranks, const unsigned long long* peer_recv,
                                 const unsigned long long* peer_cnt, int* state, int* seen, int wait_ms, int* status,
                                 cudaStream_t stream) {
  using namespace pd;
  using namespace pd::sc;
  if (kind < 0 || kind > 3 || row_bytes <= 0 || row_pad < row_bytes || nranks < 1 || nranks > MAX_RANKS) return kErrBadShape;
  if (kind != 1 && kind != 3 && (row_bytes % (is_bf16 ? 2 : 4))) return kErrBadShape;
  Args a;
  a.in = static_cast<const uint8_t*>(in);
  a.out = static_cast<uint8_t*>(out);
  for (int i = 0; i < MAX_RANKS; ++i) {
    a.recv[i] = reinterpret_cast<uint8_t*>(peer_recv[i < nranks ? i : 0]);
    a.cnt[i] = reinterpret_cast<int*>(peer_cnt[i < nranks ? i : 0]);
  }
  a.in_row_bytes = row_bytes; a.row_pad = row_pad; a.rank = rank; a.nranks = nranks;
  // about four chunks per CTA and destination for large messages (fewer system-scope fences per byte), never
  // smaller than CHUNK_BYTES; every rank derives the same value from the same row_bytes
  {
    const int64_t want = row_bytes / (static_cast<int64_t>(sm_count()) * 2 * 4 / nranks + 1);
    int64_t cb = (want + CHUNK_BYTES - 1) / CHUNK_BYTES * CHUNK_BYTES;
    if (cb < CHUNK_BYTES) cb = CHUNK_BYTES;
    if (cb > 16 * CHUNK_BYTES) cb = 16 * CHUNK_BYTES;
    a.chunk_bytes = static_cast<int>(cb);
  }
  a.chunks = static_cast<int>((row_bytes + a.chunk_bytes - 1) / a.chunk_bytes);
  a.kind = kind; a.is_bf16 = is_bf16; a.state = state; a.seen = seen;
  a.wait_ns = static_cast<unsigned long long>(wait_ms) * 1000000ull;
  a.status = status;
  const int64_t items = static_cast<int64_t>(a.chunks) * nranks;
  const int cap = sm_count() * 2;
  symm_collective_kernel<<<static_cast<int>(items < cap ? items : cap), THREADS, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

// ------------------------------------------------------------------------------------------------ NVLS all-reduce
// Two-shot all-reduce through the NVSwitch (multicast mapping of a symmetric buffer): every rank copies its vector into
// its own buffer; CTA b of rank r then reads its 1/n share of block b with multimem.ld_reduce - the switch returns the
// sum over all ranks' copies - and writes the sum back with multimem.st, which the switch replicates into every rank's
// buffer; finally every rank copies the reduced block out.  Each GPU sends and receives about 1/n + 1/n of the vector
// per direction instead of (n-1)/n twice, and no SM adds anything.  The two cross-rank barriers are per block: CTA b
// only synchronises with CTA b of the peers (release-add on the peers' counter of block b, bounded acquire-wait on the
// own one), so CTAs of one GPU never wait for each other.  The count a block has reached so far is kept on the device
// (`seen`, private to this rank), so calls of different sizes can follow each other and a CUDA graph can replay the launch.
namespace pd {
namespace sc {

constexpr int NV_THREADS = 512;

struct NvlsArgs {
  const uint8_t* in;
  uint8_t* out;
  uint8_t* buf_local;            // this rank's symmetric buffer
  uint8_t* buf_mc;               // multicast address of the same buffer
  int* cnt[MAX_RANKS];           // per-block arrival counters on every rank: [2][max_blocks]
  int64_t bytes;                 // multiple of 16
  int64_t block_bytes;           // multiple of 16 * nranks
  int rank, nranks, blocks, is_bf16;
  int* seen;                     // [2][max_blocks] counts already consumed per block (this rank only)
  int max_blocks;
  unsigned long long wait_ns;
  int* status;
};

__global__ void __launch_bounds__(NV_THREADS) symm_all_reduce_nvls_kernel(NvlsArgs a) {
  __shared__ int verdict;
  for (int b = blockIdx.x; b < a.blocks; b += gridDim.x) {
    const int64_t b0 = static_cast<int64_t>(b) * a.block_bytes;
    const int64_t n = min(a.block_bytes, a.bytes - b0);
    // ---- 1: own contribution into the own symmetric buffer
    for (int64_t i = threadIdx.x * 16; i < n; i += NV_THREADS * 16)
      *reinterpret_cast<uint4*>(a.buf_local + b0 + i) = __ldg(reinterpret_cast<const uint4*>(a.in + b0 + i));
    __syncthreads();
    if (threadIdx.x == 0) {
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      for (int r = 0; r < a.nranks; ++r) red_release_sys_add(a.cnt[r] + b, 1);
      const int want = a.seen[b] + a.nranks;
      a.seen[b] = want;
      verdict = flag_wait_ge(a.cnt[a.rank] + b, want, a.wait_ns, a.status, 820) ? 1 : 0;
      asm volatile("fence.acq_rel.sys;" ::: "memory");
    }
    __syncthreads();
    const bool ok1 = verdict != 0;
    __syncthreads();
    // ---- 2: reduce my share of the block inside the switch, broadcast the sum
    if (ok1) {
      const int64_t share = (n / 16 + a.nranks - 1) / a.nranks * 16;       // 16-byte granules per rank
      const int64_t s0 = min(n, share * a.rank), s1 = min(n, s0 + share);
      constexpr int U = 4;                                                 // reductions in flight per thread
      for (int64_t i = s0 + threadIdx.x * 16; i < s1; i += NV_THREADS * 16 * U) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int64_t j = i + static_cast<int64_t>(u) * NV_THREADS * 16;
          if (j < s1) v[u] = a.is_bf16 ? multimem_ld_reduce_bf16x8(a.buf_mc + b0 + j) : multimem_ld_reduce_f32x4(a.buf_mc + b0 + j);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int64_t j = i + static_cast<int64_t>(u) * NV_THREADS * 16;
          if (j < s1) multimem_st_v4(a.buf_mc + b0 + j, v[u]);
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      for (int r = 0; r < a.nranks; ++r) red_release_sys_add(a.cnt[r] + a.max_blocks + b, 1);
      const int want = a.seen[a.max_blocks + b] + a.nranks;
      a.seen[a.max_blocks + b] = want;
      verdict = (ok1 && flag_wait_ge(a.cnt[a.rank] + a.max_blocks + b, want, a.wait_ns, a.status, 821)) ? 1 : 0;
      asm volatile("fence.acq_rel.sys;" ::: "memory");
    }
    __syncthreads();
    const bool ok2 = verdict != 0;
    __syncthreads();
    // ---- 3: the whole block is reduced in every rank's buffer
    if (ok2)
      for (int64_t i = threadIdx.x * 16; i < n; i += NV_THREADS * 16)
        *reinterpret_cast<uint4*>(a.out + b0 + i) = __ldcg(reinterpret_cast<const uint4*>(a.buf_local + b0 + i));
  }
}

}  // namespace sc
}  // namespace pd

// in / out: `bytes` (multiple of 16; fp32 or bf16 elements) on this rank; buf_local / buf_mc: this rank's symmetric
// buffer (>= bytes rounded up to the block size) and its multicast address; peer_cnt[r]: int32 [2 * blocks] on rank r,
// zeroed once; seen: int32 [2 * max_blocks] on this rank, zeroed once; blocks = ceil(bytes / block_bytes) with block_bytes from pd_symm_nvls_block_bytes (the same on every rank).
PD_EXPORT int64_t pd_symm_nvls_block_bytes(int64_t bytes, int nranks) {
  // about two blocks per SM for large vectors, never below 16 KB, a multiple of 16 * nranks
  const int64_t unit = 16ll * nranks;
  int64_t bb = bytes / (2ll * pd::sm_count()) + 1;
  if (bb < 16384) bb = 16384;
  return (bb + unit - 1) / unit * unit;
}
PD_EXPORT int pd_symm_all_reduce_nvls(const void* in, void* out, int64_t bytes, int is_bf16, void* buf_local,
                                      unsigned long long buf_mc, int rank, int nranks, const unsigned long long* peer_cnt,
                                      int max_blocks, int* seen, int wait_ms, int* status, cudaStream_t stream) {
  using namespace pd;
  using namespace pd::sc;
  if (bytes <= 0 || (bytes % 16) || nranks < 1 || nranks > MAX_RANKS || buf_mc == 0) return kErrBadShape;
  if (!aligned16(in) || !aligned16(out) || !aligned16(buf_local)) return kErrAlignment;
  NvlsArgs a;
  a.in = static_cast<const uint8_t*>(in);
  a.out = static_cast<uint8_t*>(out);
  a.buf_local = static_cast<uint8_t*>(buf_local);
  a.buf_mc = reinterpret_cast<uint8_t*>(buf_mc);
  for (int i = 0; i < MAX_RANKS; ++i) a.cnt[i] = reinterpret_cast<int*>(peer_cnt[i < nranks ? i : 0]);
  a.bytes = bytes;
  a.block_bytes = pd_symm_nvls_block_bytes(bytes, nranks);
  a.blocks = static_cast<int>((bytes + a.block_bytes - 1) / a.block_bytes);
  if (a.blocks > max_blocks) return kErrTooLarge;
  a.rank = rank; a.nranks = nranks; a.is_bf16 = is_bf16; a.seen = seen; a.max_blocks = max_blocks;
  a.wait_ns = static_cast<unsigned long long>(wait_ms) * 1000000ull;
  a.status = status;
  const int cap = sm_count() * 2;
  symm_all_reduce_nvls_kernel<<<a.blocks < cap ? a.blocks : cap, NV_THREADS, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

// ------------------------------------------------------------------------------------------------ vocab-parallel CE
// Second half of the vocab-parallel softmax cross entropy (reference: three all-reduces - MAX of the row maxima, SUM of
// the shifted exponent sums, SUM of the target logits - in paddle/phi/kernels/gpu/c_softmax_with_cross_entropy_kernel.cu
// :229,309,322).  Here the three fp32 statistics of a block of rows are written straight into slot [rank] of every
// peer's exchange buffer, one release-add per (block, peer) tells the peer, and after a bounded wait for the n arrivals
// the same CTA merges the n triples of its rows into log-sum-exp and loss.  One launch instead of two collectives and
// the element-wise glue between them; the arrival count per block lives on the device, so a CUDA graph can replay it.
namespace pd {
namespace sc {

constexpr int CE_ROWS = 256;       // rows per CTA and per arrival counter

struct CEArgs {
  const float* mx; const float* sm; const float* tg;
  const long long* labels;
  float* lse; float* loss;
  float* recv[MAX_RANKS];        // [2 parities][nranks][3][rows_pad]
  int* cnt[MAX_RANKS];           // [max_blocks]
  int* seen;                     // [max_blocks] local
  long long rows, rows_pad, ignore_index;
  int rank, nranks;
  unsigned long long wait_ns;
  int* status;
};

__global__ void __launch_bounds__(CE_ROWS) ce_combine_kernel(CEArgs a) {
  __shared__ int s_par, s_ok;
  const int b = blockIdx.x;
  const long long row = static_cast<long long>(b) * CE_ROWS + threadIdx.x;
  if (threadIdx.x == 0) s_par = (a.seen[b] / a.nranks) & 1;
  __syncthreads();
  const int par = s_par;
  const bool live = row < a.rows;
  if (live) {
    const float m = a.mx[row], s = a.sm[row], t = a.tg[row];
    for (int d = 0; d < a.nranks; ++d) {
      const int peer = (a.rank + d) % a.nranks;
      float* base = a.recv[peer] + (static_cast<long long>(par) * a.nranks + a.rank) * 3 * a.rows_pad;
      base[row] = m;
      base[a.rows_pad + row] = s;
      base[2 * a.rows_pad + row] = t;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    for (int r = 0; r < a.nranks; ++r) red_release_sys_add(a.cnt[r] + b, 1);
    const int want = a.seen[b] + a.nranks;
    a.seen[b] = want;
    s_ok = flag_wait_ge(a.cnt[a.rank] + b, want, a.wait_ns, a.status, 830) ? 1 : 0;
    asm volatile("fence.acq_rel.sys;" ::: "memory");
  }
  __syncthreads();
  if (!s_ok || !live) return;
  const float* mine = a.recv[a.rank] + static_cast<long long>(par) * a.nranks * 3 * a.rows_pad;
  float gm = -INFINITY;
  for (int r = 0; r < a.nranks; ++r) gm = fmaxf(gm, __ldcg(mine + static_cast<long long>(r) * 3 * a.rows_pad + row));
  float se = 0.f, tgt = 0.f;
  for (int r = 0; r < a.nranks; ++r) {           // rank order: every rank computes the same bits
    const float* p = mine + static_cast<long long>(r) * 3 * a.rows_pad;
    se += __ldcg(p + a.rows_pad + row) * __expf(__ldcg(p + row) - gm);
    tgt += __ldcg(p + 2 * a.rows_pad + row);
  }
  const float l = gm + __logf(se);
  a.lse[row] = l;
  a.loss[row] = (a.labels[row] == a.ignore_index) ? 0.f : l - tgt;
}

}  // namespace sc
}  // namespace pd

// mx / sm / tg: fp32 [rows] statistics of this rank's vocabulary shard (pd_ce_stats); labels: int64 [rows];
// peer_recv[r]: fp32 [2][nranks][3][rows_pad] on rank r; peer_cnt[r] / seen: int32 [ceil(rows_pad / 256)], zeroed once.
PD_EXPORT int pd_ce_combine(const float* mx, const float* sm, const float* tg, const long long* labels, float* lse,
                            float* loss, long long rows, long long rows_pad, long long ignore_index, int rank, int nranks,
                            const unsigned long long* peer_recv, const unsigned long long* peer_cnt, int* seen,
                            int wait_ms, int* status, cudaStream_t stream) {
  using namespace pd;
  using namespace pd::sc;
  if (rows <= 0 || rows > rows_pad || nranks < 1 || nranks > MAX_RANKS) return kErrBadShape;
  CEArgs a;
  a.mx = mx; a.sm = sm; a.tg = tg; a.labels = labels; a.lse = lse; a.loss = loss;
  for (int i = 0; i < MAX_RANKS; ++i) {
    a.recv[i] = reinterpret_cast<float*>(peer_recv[i < nranks ? i : 0]);
    a.cnt[i] = reinterpret_cast<int*>(peer_cnt[i < nranks ? i : 0]);
  }
  a.seen = seen; a.rows = rows; a.rows_pad = rows_pad; a.ignore_index = ignore_index;
  a.rank = rank; a.nranks = nranks;
  a.wait_ns = static_cast<unsigned long long>(wait_ms) * 1000000ull;
  a.status = status;
  const int blocks = static_cast<int>((rows + CE_ROWS - 1) / CE_ROWS);
  ce_combine_kernel<<<blocks, CE_ROWS, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}

// ------------------------------------------------------------------------------------------------ vocab-parallel embedding
// Vocabulary-parallel embedding whose result is wanted sharded along the sequence (the input of a sequence-parallel
// decoder stack).  The reference looks the local rows up with zeros for foreign ids, all-reduces the full [T, H] result
// and slices it (c_embedding: paddle/phi/kernels/gpu/c_embedding_kernel.cu:31; mp_allreduce in
// python/paddle/distributed/fleet/layers/mpu/mp_layers.py:163-175; ScatterOp in fleet/utils/sequence_parallel_utils.py:85).
// Exactly one rank owns each token's row, so nothing has to be added: the owner of the ROW writes it straight into the
// sequence shard of the rank that owns the TOKEN (plain 16-byte peer stores), every CTA tells every peer once that it is
// done, and after a bounded wait for all n * grid notices each rank copies its complete shard out of the exchange buffer.
// (n - 1) / n * T/n * H bytes leave each GPU instead of an all-reduce of T * H.
namespace pd {
namespace sc {

constexpr int EMB_THREADS = 256;

struct EmbArgs {
  const long long* ids;          // [T]
  const uint4* weight;           // [rows_local, H] 16-byte units
  uint4* out;                    // [T / nranks, H] local result
  uint4* recv[MAX_RANKS];        // [2 parities][T_pad / nranks... rows_shard_pad][H] on every rank
  int* cnt[MAX_RANKS];           // one counter per rank
  int* seen;                     // local: [0] notices consumed so far, [1] calls so far (its parity picks the slot)
  long long T, vstart, rows_local, rows_shard, slot_units;
  int row_units;                 // H * element size / 16
  int rank, nranks;
  unsigned long long wait_ns;
  int* status;
};

__global__ void __launch_bounds__(EMB_THREADS) embedding_scatter_kernel(EmbArgs a) {
  __shared__ int s_ok, s_par;
  if (threadIdx.x == 0) s_par = a.seen[1] & 1;
  __syncthreads();
  const long long slot = static_cast<long long>(s_par) * a.slot_units;
  for (long long t = blockIdx.x; t < a.T; t += gridDim.x) {
    const long long local = a.ids[t] - a.vstart;
    if (local < 0 || local >= a.rows_local) continue;                     // another rank owns this row
    const int dst = static_cast<int>(t / a.rows_shard);
    const uint4* src = a.weight + local * a.row_units;
    uint4* d = a.recv[dst] + slot + (t - dst * a.rows_shard) * a.row_units;
    for (int i = threadIdx.x; i < a.row_units; i += EMB_THREADS) d[i] = __ldg(src + i);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    for (int r = 0; r < a.nranks; ++r) red_release_sys_add(a.cnt[r], 1);
    const int want = a.seen[0] + a.nranks * static_cast<int>(gridDim.x);
    s_ok = flag_wait_ge(a.cnt[a.rank], want, a.wait_ns, a.status, 840) ? 1 : 0;
    asm volatile("fence.acq_rel.sys;" ::: "memory");
  }
  __syncthreads();
  if (s_ok) {
    const uint4* mine = a.recv[a.rank] + slot;
    const long long units = a.rows_shard * a.row_units;
    for (long long i = static_cast<long long>(blockIdx.x) * EMB_THREADS + threadIdx.x; i < units;
         i += static_cast<long long>(gridDim.x) * EMB_THREADS)
      a.out[i] = __ldcg(mine + i);
  }
}

// every CTA has read seen[0] before any of them may advance it: a second, single-thread launch does it
__global__ void embedding_scatter_advance(int* seen, int by) {
  seen[0] += by;
  seen[1] += 1;
}

}  // namespace sc
}  // namespace pd

// ids: int64 [T] (every id inside the global vocabulary; T a multiple of nranks); weight: [rows_local, H] with
// H * elem_bytes a multiple of 16; out: [T / nranks, H]; peer_recv[r]: [2][T / nranks][H] elements on rank r (slot_bytes
// apart); peer_cnt[r]: one int32, zeroed once; seen: two local int32, zeroed once.  `grid` must be the same on all ranks and small
// enough for all its CTAs to be resident at once (each waits for the notices of all the others).
PD_EXPORT int pd_embedding_scatter(const long long* ids, const void* weight, void* out, long long T, long long vstart,
                                   long long rows_local, int row_bytes, long long slot_bytes, int rank, int nranks,
                                   const unsigned long long* peer_recv, const unsigned long long* peer_cnt, int* seen,
                                   int grid, int wait_ms, int* status, cudaStream_t stream) {
  using namespace pd;
  using namespace pd::sc;
  if (T <= 0 || T % nranks || row_bytes <= 0 || row_bytes % 16 || slot_bytes % 16 || nranks < 1 || nranks > MAX_RANKS ||
      grid < 1 || slot_bytes < T / nranks * row_bytes)
    return kErrBadShape;
  if (!aligned16(weight) || !aligned16(out)) return kErrAlignment;
  EmbArgs a;
  a.ids = ids; a.weight = static_cast<const uint4*>(weight); a.out = static_cast<uint4*>(out);
  for (int i = 0; i < MAX_RANKS; ++i) {
    a.recv[i] = reinterpret_cast<uint4*>(peer_recv[i < nranks ? i : 0]);
    a.cnt[i] = reinterpret_cast<int*>(peer_cnt[i < nranks ? i : 0]);
  }
  a.seen = seen; a.T = T; a.vstart = vstart; a.rows_local = rows_local; a.rows_shard = T / nranks;
  a.slot_units = slot_bytes / 16; a.row_units = row_bytes / 16; a.rank = rank; a.nranks = nranks;
  a.wait_ns = static_cast<unsigned long long>(wait_ms) * 1000000ull;
  a.status = status;
  embedding_scatter_kernel<<<grid, EMB_THREADS, 0, stream>>>(a);
  embedding_scatter_advance<<<1, 1, 0, stream>>>(seen, nranks * grid);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}
