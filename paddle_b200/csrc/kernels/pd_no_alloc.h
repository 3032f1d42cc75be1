// Allocation-free entry point of libpd_kernels.so.  This has no counterpart in the reference framework.
//
// Who needs it: code that drives these kernels from a place where device memory cannot be requested —
// a host process embedding the library behind its own fixed memory plan, a plug-in running inside another
// runtime's stream callback or capture region where allocator calls are forbidden, a real-time serving loop
// that pre-plans every byte.  Such callers can hand over inputs and outputs but cannot provide the temporary
// buffer that the regular pd_rms_norm_bwd asks for, and the library must not call cudaMalloc / cudaFree (or any
// allocating routine, PyTorch's included) on their behalf.
//
// pd_rms_norm_bwd_static computes exactly what pd_rms_norm_bwd computes (dx, and dw either stored or
// accumulated).  Its temporary — the per-CTA partial sums of the weight gradient — is a file-scope
// `static __device__` array of 128 x 8192 floats (4 MiB) that every GPU loading the library holds until
// the process exits.
//
// Limits and rules:
//   * H (row length) must be a multiple of 8 and at most 8192; larger sizes return -5 (size beyond the
//     supported maximum) without launching anything.  rows may be anything up to 2^31 - 1 (larger counts also
//     return -5): at most 128 CTAs share the work.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
//     device current).  Make that first call outside any stream capture.  Host threads may make their first
//     calls on a device concurrently: the cached address is an atomic and every thread stores the same value.
//   * All calls share the one array.  Nothing in it has to start at zero — each call overwrites the rows it
//     later sums — but two calls whose kernels overlap on the GPU (different streams, no ordering) race on it.
//     Serialise them on one stream or with events.
//   * Return value: 0 on success, negative launcher codes otherwise (host_utils.h).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int pd_rms_norm_bwd_static(const void* dy, const void* x, const void* w, int w_is_f32, const float* inv_rms,
                           void* dx, const void* dx_add, float* dw, int dw_accumulate, int64_t rows, int H,
                           cudaStream_t stream);

#ifdef __cplusplus
}
#endif
