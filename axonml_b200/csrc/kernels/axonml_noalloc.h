// Entry points of libaxonml_cuda.so that never allocate.
//
// This header has no counterpart in the reference project: it exists for callers of this library
// that are not allowed to call cudaMalloc (or any allocating routine, torch's caching allocator
// included) at the point where they need the kernel - graph-captured or latency-critical loops,
// plugins living inside a host application's fixed arena, processes whose device memory is managed
// by another runtime.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// LayerNorm (rms = 0) / RMSNorm (rms = 1) backward.  Same maths and arguments as ax_norm_bwd, but
// the per-CTA partial sums of the weight/bias gradients are kept in a fixed 4 MiB array inside the
// library (64 slots x 2 x 8192 floats) instead of a caller-provided scratch buffer.
//
//   dtype codes: 0 = fp32, 1 = bf16 (activations / weights); D must be a multiple of 8.
//   dy, x, dx: [rows, D]; w, dw, db: [D]; mean, rstd: [rows] fp32; dres (optional): [rows, D].
//
// Returns 0 on success, -1 for a bad shape, -2 when D exceeds the built-in scratch (8192), -3 for
// a device ordinal >= 64, otherwise a cudaError_t value.
//
// * The first call on each device looks up the array's device address with
//   cudaGetSymbolAddress (that device must be current); make that call outside stream capture.
// * All calls share the array, so calls that may run concurrently on the GPU race with each
//   other: issue them on one stream or order them with events.
// * The array is part of the loaded module: every GPU that loads the library holds the 4 MiB
//   until the process exits.  No call here reaches cudaMalloc, cudaFree or an allocating library.
int ax_norm_bwd_noalloc(int rms, int act_dtype, int w_dtype, const void* dy, const void* x,
                        const void* w, const float* mean, const float* rstd, const void* dres,
                        void* dx, void* dw, void* db, int rows, int D, cudaStream_t stream);

// Reports the compiled-in limits (largest D, number of partial slots).
int ax_norm_bwd_noalloc_limits(int* max_d, int* max_groups);

#ifdef __cplusplus
}
#endif
