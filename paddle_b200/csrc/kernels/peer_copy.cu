// Device-to-peer copy kernels used by the symmetric-memory runtime (standalone all-gather / broadcast
// building block) and to measure which store path saturates NVLink:
//   mode 0: plain 16-byte loads + stores issued by every thread (grid-stride)
//   mode 1: one thread per CTA driving a ring of cp.async.bulk copies (HBM -> smem -> peer)
//   mode 2: bulk loads into shared memory, stores issued by all threads from shared memory
#include "host_utils.h"
#include "sm100_prims.cuh"

namespace pd {
namespace pc {

constexpr int THREADS = 256;
constexpr int PIECE = 16384;
constexpr int RING = 12;

__global__ void __launch_bounds__(THREADS) copy_plain_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                                             size_t nvec) {
  size_t i = blockIdx.x * static_cast<size_t>(THREADS) + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * THREADS;
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    dst[i] = a; dst[i + stride] = b; dst[i + 2 * stride] = c; dst[i + 3 * stride] = d;
  }
  for (; i < nvec; i += stride) dst[i] = src[i];
}

__global__ void __launch_bounds__(THREADS) copy_bulk_kernel(uint8_t* dst, const uint8_t* src, size_t bytes, int mode,
                                                            int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + RING * PIECE);
  __shared__ int decision;
  const size_t pieces = (bytes + PIECE - 1) / PIECE;
  const size_t per = (pieces + gridDim.x - 1) / gridDim.x;
  const size_t p0 = blockIdx.x * per, p1 = min(pieces, p0 + per);
  if (p0 >= p1) return;
  const int total = static_cast<int>(p1 - p0);
  if (threadIdx.x == 0) {
    for (int i = 0; i < RING; ++i) mbar_init(&bars[i], 1);
    fence_mbar_init();
  }
  __syncthreads();
  int dummy = 0;
  auto piece_bytes = [&](int q) { return static_cast<uint32_t>(min(static_cast<size_t>(PIECE), bytes - (p0 + q) * PIECE)); };
  if (mode == 1) {
    if (threadIdx.x != 0) return;
    constexpr int LOOK = RING - 2;
    for (int q = 0; q < total && q < LOOK; ++q) {
      mbar_expect_tx(&bars[q % RING], piece_bytes(q));
      bulk_load(smem + (q % RING) * PIECE, src + (p0 + q) * PIECE, piece_bytes(q), &bars[q % RING]);
    }
    for (int q = 0; q < total; ++q) {
      if (q + LOOK < total) {
        tma_wait_group_read<1>();
        const int s = (q + LOOK) % RING;
        mbar_expect_tx(&bars[s], piece_bytes(q + LOOK));
        bulk_load(smem + s * PIECE, src + (p0 + q + LOOK) * PIECE, piece_bytes(q + LOOK), &bars[s]);
      }
      if (!mbar_wait(&bars[q % RING], (q / RING) & 1, &dummy, status, 900)) break;
      bulk_store(dst + (p0 + q) * PIECE, smem + (q % RING) * PIECE, piece_bytes(q));
      tma_commit_group();
    }
    tma_wait_group<0>();
    return;
  }
  // mode 2: thread 0 keeps the load ring full, everyone stores
  constexpr int LOOK = RING - 1;
  if (threadIdx.x == 0)
    for (int q = 0; q < total && q < LOOK; ++q) {
      mbar_expect_tx(&bars[q % RING], piece_bytes(q));
      bulk_load(smem + (q % RING) * PIECE, src + (p0 + q) * PIECE, piece_bytes(q), &bars[q % RING]);
    }
  for (int q = 0; q < total; ++q) {
    if (threadIdx.x == 0) decision = mbar_wait(&bars[q % RING], (q / RING) & 1, &dummy, status, 901) ? 1 : 0;
    __syncthreads();
    if (!decision) break;
    const uint4* s4 = reinterpret_cast<const uint4*>(smem + (q % RING) * PIECE);
    uint4* d4 = reinterpret_cast<uint4*>(dst + (p0 + q) * PIECE);
    const int nv = piece_bytes(q) >> 4;
    for (int i = threadIdx.x; i < nv; i += THREADS) d4[i] = s4[i];
    __syncthreads();   // slot (q % RING) fully read
    if (threadIdx.x == 0 && q + LOOK < total) {
      // slot (q + LOOK) % RING == (q - 1) % RING was released by the previous iteration's barrier
      const int s = (q + LOOK) % RING;
      mbar_expect_tx(&bars[s], piece_bytes(q + LOOK));
      bulk_load(smem + s * PIECE, src + (p0 + q + LOOK) * PIECE, piece_bytes(q + LOOK), &bars[s]);
    }
  }
}

}  // namespace pc
}  // namespace pd

// Copy `bytes` (multiple of 16, both pointers 16-byte aligned; dst may be peer memory) with `nctas` CTAs.
PD_EXPORT int pd_peer_copy(void* dst, const void* src, int64_t bytes, int mode, int nctas, int* status,
                           cudaStream_t stream) {
  using namespace pd;
  using namespace pd::pc;
  if (bytes <= 0 || (bytes % 16) || !aligned16(dst) || !aligned16(src) || nctas <= 0) return kErrAlignment;
  if (mode == 0) {
    copy_plain_kernel<<<nctas, THREADS, 0, stream>>>((uint4*)dst, (const uint4*)src, static_cast<size_t>(bytes) >> 4);
  } else {
    const int smem = RING * PIECE + 256 + 128;
    static bool cfg = false;
    if (!cfg) {
      if (cudaFuncSetAttribute(copy_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return kErrCuda;
      cfg = true;
    }
    copy_bulk_kernel<<<nctas, THREADS, smem, stream>>>((uint8_t*)dst, (const uint8_t*)src, static_cast<size_t>(bytes),
                                                       mode, status);
  }
  return cudaGetLastError() == cudaSuccess ? kLaunchOk : kErrCuda;
}
