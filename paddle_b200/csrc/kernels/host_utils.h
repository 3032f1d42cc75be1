// Host-side helpers shared by the kernel launchers: TMA tensor-map encoding through the driver
// entry point (no link-time dependency on libcuda), error codes, device properties.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define PD_EXPORT extern "C" __attribute__((visibility("default")))

namespace pd {

// Launcher return codes (0 = launched).  Negative values are host-side argument / API errors.
enum LaunchError : int {
  kLaunchOk = 0,
  kErrBadShape = -1,
  kErrAlignment = -2,
  kErrTensorMap = -3,
  kErrCuda = -4,
  kErrTooLarge = -5,
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Encode a tiled map over a row-major tensor of `rank` dims.  dims[0] is the contiguous one.
// strides_bytes[i] is the stride of dims[i+1] (rank-1 entries).  Returns false on failure.
inline bool encode_tmap(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base,
                        const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                        CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  // The encoder is a driver-API call and needs a context bound to THIS thread.  The runtime binds the primary context
  // lazily, on a thread's first runtime call that needs it; a worker thread (the autograd engine's) whose first CUDA
  // work is one of these launchers has none yet, and the encoder answers CUDA_ERROR_INVALID_CONTEXT.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  cuuint64_t d[5], s[4];
  cuuint32_t b[5], e[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
  CUresult r = fn(out, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, s, b, e,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {   // say which map was refused: the launcher only returns kErrTensorMap
    fprintf(stderr, "[pd] cuTensorMapEncodeTiled failed (%d): base %p rank %d dims", static_cast<int>(r), base, rank);
    for (int i = 0; i < rank; ++i) fprintf(stderr, " %llu", static_cast<unsigned long long>(d[i]));
    fprintf(stderr, " strides");
    for (int i = 0; i + 1 < rank; ++i) fprintf(stderr, " %llu", static_cast<unsigned long long>(s[i]));
    fprintf(stderr, " box");
    for (int i = 0; i < rank; ++i) fprintf(stderr, " %u", b[i]);
    fprintf(stderr, "\n");
  }
  return r == CUDA_SUCCESS;
}

inline bool encode_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, const void* base,
                           uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                           uint32_t box_inner, uint32_t box_outer,
                           CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  uint64_t dims[2] = {inner, outer};
  uint64_t strides[1] = {row_stride_bytes};
  uint32_t box[2] = {box_inner, box_outer};
  return encode_tmap(out, dt, 2, base, dims, strides, box, swz);
}

// dims {inner, mid, outer} with byte strides of mid and outer; box {box_inner, box_mid, box_outer}.
inline bool encode_tmap_3d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t mid,
                           uint64_t outer, uint64_t mid_stride_bytes, uint64_t outer_stride_bytes, uint32_t box_inner,
                           uint32_t box_mid, uint32_t box_outer, CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  uint64_t dims[3] = {inner, mid, outer};
  uint64_t strides[2] = {mid_stride_bytes, outer_stride_bytes};
  uint32_t box[3] = {box_inner, box_mid, box_outer};
  return encode_tmap(out, dt, 3, base, dims, strides, box, swz);
}

// Map for an MN-major bf16 operand stored [k_extent rows][mn_extent contiguous].  When mn_extent is a multiple of
// 64 the matrix is viewed as [mn/64][k][64] so that ONE box {64, box_k, chunks} fills `chunks` consecutive
// 128B-swizzled 64-column slabs of shared memory (*is3d = 1); otherwise a plain 2-D map with box {64, box_k}
// is produced and the kernel issues one load per slab.
inline bool encode_tmap_mn(CUtensorMap* out, const void* base, uint64_t mn_extent, uint64_t k_extent,
                           uint64_t row_stride_bytes, uint32_t chunks, uint32_t box_k, int* is3d) {
  if (mn_extent % 64 == 0) {
    uint64_t dims[3] = {64, k_extent, mn_extent / 64};
    uint64_t strides[2] = {row_stride_bytes, 128};
    uint32_t box[3] = {64, box_k, chunks};
    *is3d = 1;
    return encode_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  }
  *is3d = 0;
  return encode_tmap_2d(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, mn_extent, k_extent, row_stride_bytes, 64, box_k);
}

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace pd
