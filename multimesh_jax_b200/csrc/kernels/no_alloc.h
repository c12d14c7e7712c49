// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project. It exists for code that
// runs where an allocation is impossible or forbidden: inside a region that an outer
// framework has frozen (its memory pool is handed out in advance and nothing may be
// requested from the driver any more), in a library-initialisation path that runs before
// the host application has chosen its allocator, or in a latency-critical loop where a
// call into the allocator could block on another thread. The ordinary entry point
// `mm_rmsnorm_bwd` needs a caller-provided scratch buffer for the per-block partial sums
// of the weight gradient; this variant keeps that scratch in a fixed array that is part of
// the library image instead, so the caller passes only inputs and outputs.
//
// Limits and rules
//   * hidden size D: a multiple of 8, at most MM_NOALLOC_MAX_D (8192). Larger or
//     unaligned sizes are refused with a message on stderr and a non-zero return code.
//   * up to 2^31 - 1 rows (more are refused); at most MM_NOALLOC_MAX_PARTS (128) blocks share
//     the rows, so the scratch is MM_NOALLOC_MAX_PARTS * MM_NOALLOC_MAX_D floats = 4 MiB. Every
//     GPU that loads the library holds this array until the process exits.
//   * the first call on each device is a set-up call: it looks up the device address of the
//     array (one `cudaGetSymbolAddress`, with that device current) and remembers it. With lazy
//     module loading that look-up, or the first kernel launch, can make the CUDA driver load
//     the library's code image onto the device - the 4 MiB array included - which is an
//     allocation made by the driver. So make one call per device during ordinary start-up:
//     before the region in which nothing may be allocated begins, and before any stream
//     capture on that device.
//   * apart from that driver-side loading on the first call, the function itself calls no
//     cudaMalloc, no cudaFree and no library routine that allocates.
//   * all calls on a device share the one array, and it keeps whatever the previous call
//     left in it. The kernels overwrite every element they later read, so nothing has to
//     be cleared, but two calls whose kernels overlap on the GPU (different streams
//     without an ordering between them) race on it: keep such calls ordered.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define MM_NOALLOC_MAX_D 8192
#define MM_NOALLOC_MAX_PARTS 128

#ifdef __cplusplus
extern "C" {
#endif

// dx[rows, D] (bf16) = d/dx of RMSNorm given x, weight w, upstream dy and the saved rstd;
// dw_out[D] (fp32) = weight gradient (added to the existing contents if accumulate_dw != 0).
// With add_to_dx != 0 the input gradient is added into dx instead of overwriting it.
// Returns 0 on success.
int mm_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                           float* dw_out, int64_t rows, int D, int accumulate_dw, int add_to_dx,
                           cudaStream_t stream);

#ifdef __cplusplus
}
#endif
