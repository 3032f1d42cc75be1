// Standalone collectives over symmetric (peer-mapped) memory for small and medium messages, where a library
// collective is dominated by launch and protocol latency:
//   pd_symm_all_reduce     : one-shot - every rank pushes its whole vector into row [rank] of every peer's receive
//                            buffer, then sums the n rows it received (fp32 accumulation, rank order: deterministic)
//   pd_symm_all_gather     : every rank pushes its shard into slot [rank] of every peer's output buffer
//   pd_symm_reduce_scatter : every rank pushes slice d of its vector to rank d, which sums the n rows
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
  int* state;
  unsigned long long wait_ns;
  int* status;
};

__device__ __forceinline__ void copy_bytes(uint8_t* dst, const uint8_t* src, int64_t n) {
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | n) & 15u) == 0) {
    for (int64_t i = threadIdx.x * 16; i < n; i += THREADS * 16)
      *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
  } else {
    for (int64_t i = threadIdx.x; i < n; i += THREADS) dst[i] = src[i];
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
    const int64_t b0 = static_cast<int64_t>(c) * CHUNK_BYTES;
    const int64_t n = min(static_cast<int64_t>(CHUNK_BYTES), a.in_row_bytes - b0);
    // all_reduce / all_gather send the same bytes to everybody; reduce_scatter sends slice `dst`
    const uint8_t* src = a.in + (a.kind == 2 ? static_cast<int64_t>(dst) * a.in_row_bytes : 0) + b0;
    copy_bytes(a.recv[dst] + slot_off + static_cast<int64_t>(a.rank) * a.row_pad + b0, src, n);
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) red_release_sys_add(a.cnt[dst] + c, 1);
  }
  // ---- consume the n rows that arrived here
  const uint8_t* base = a.recv[a.rank] + slot_off;
  for (int c = blockIdx.x; c < a.chunks; c += gridDim.x) {
    if (threadIdx.x == 0)
      verdict = flag_wait_ge(a.cnt[a.rank] + c, epoch * a.nranks, a.wait_ns, a.status, 800) ? 1 : 0;
    __syncthreads();
    const bool ok = verdict != 0;
    __syncthreads();
    if (!ok) continue;
    const int64_t b0 = static_cast<int64_t>(c) * CHUNK_BYTES;
    const int64_t n = min(static_cast<int64_t>(CHUNK_BYTES), a.in_row_bytes - b0);
    if (a.kind == 1) {
      for (int r = 0; r < a.nranks; ++r) {
        const uint8_t* row = base + static_cast<int64_t>(r) * a.row_pad + b0;
        uint8_t* dst = a.out + static_cast<int64_t>(r) * a.in_row_bytes + b0;
        if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(row) | n) & 15u) == 0) {
          for (int64_t i = threadIdx.x * 16; i < n; i += THREADS * 16)
            *reinterpret_cast<uint4*>(dst + i) = __ldcg(reinterpret_cast<const uint4*>(row + i));
        } else {
          for (int64_t i = threadIdx.x; i < n; i += THREADS) dst[i] = __ldcg(row + i);
        }
      }
    } else if (a.is_bf16) {
      const int64_t ne = n / 2;
      bf16* o = reinterpret_cast<bf16*>(a.out + b0);
      for (int64_t i = threadIdx.x; i < ne; i += THREADS) {
        float s = 0.f;
        for (int r = 0; r < a.nranks; ++r)
          s += __bfloat162float(__ldcg(reinterpret_cast<const bf16*>(base + static_cast<int64_t>(r) * a.row_pad + b0) + i));
        o[i] = __float2bfloat16(s);
      }
    } else {
      const int64_t ne = n / 4;
      float* o = reinterpret_cast<float*>(a.out + b0);
      for (int64_t i = threadIdx.x; i < ne; i += THREADS) {
        float s = 0.f;
        for (int r = 0; r < a.nranks; ++r)
          s += __ldcg(reinterpret_cast<const float*>(base + static_cast<int64_t>(r) * a.row_pad + b0) + i);
        o[i] = s;
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
// 2 reduce_scatter (in: nranks * row_bytes, out: row_bytes).  peer_recv[r]: [2][nranks][row_pad] bytes on rank r,
// peer_cnt[r]: int32 [ceil(row_bytes / 16384)] zeroed once; state: 2 local int32 zeroed once.
PD_EXPORT int pd_symm_collective(int kind, const void* in, void* out, int64_t row_bytes, int64_t row_pad, int is_bf16,
                                 int rank, int nranks, const unsigned long long* peer_recv,
                                 const unsigned long long* peer_cnt, int* state, int wait_ms, int* status,
                                 cudaStream_t stream) {
  using namespace pd;
  using namespace pd::sc;
  if (kind < 0 || kind > 2 || row_bytes <= 0 || row_pad < row_bytes || nranks < 1 || nranks > MAX_RANKS) return kErrBadShape;
  if (kind != 1 && (row_bytes % (is_bf16 ? 2 : 4))) return kErrBadShape;
  Args a;
  a.in = static_cast<const uint8_t*>(in);
  a.out = static_cast<uint8_t*>(out);
  for (int i = 0; i < MAX_RANKS; ++i) {
    a.recv[i] = reinterpret_cast<uint8_t*>(peer_recv[i < nranks ? i : 0]);
    a.cnt[i] = reinterpret_cast<int*>(peer_cnt[i < nranks ? i : 0]);
  }
  a.in_row_bytes = row_bytes; a.row_pad = row_pad; a.rank = rank; a.nranks = nranks;
  a.chunks = static_cast<int>((row_bytes + CHUNK_BYTES - 1) / CHUNK_BYTES);
  a.kind = kind; a.is_bf16 = is_bf16; a.state = state;
  a.wait_ns = static_cast<unsigned long long>(wait_ms) * 1000000ull;
  a.status = status;
  const int64_t items = static_cast<int64_t>(a.chunks) * nranks;
  const int cap = sm_count() * 2;
  symm_collective_kernel<<<static_cast<int>(items < cap ? items : cap), THREADS, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}
