// An entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference; it is an addition of this library.
//
// Who needs it: code that runs where cudaMalloc (or any allocating library
// call, torch's caching allocator included) is off limits.  Examples are a
// plugin that runs inside a framework that has handed all device memory to
// its own pool, a real-time
// loop that may not take the allocator's locks, and a process that is close
// to the memory limit of a shared GPU and cannot risk an out-of-memory error
// in the middle of a step.  dsw_layernorm_bwd needs a scratch array for its
// per-block partial column sums; its normal callers allocate that array.
// dsw_layernorm_bwd_noalloc does the same computation with the scratch held
// in a fixed array that is part of the library image.
//
// Cost and limit: the array is DSW_NOALLOC_LN_MAX_BLOCKS * 3 *
// DSW_NOALLOC_LN_MAX_D floats = 6.9 MiB, and every GPU that loads the library
// carries it until the process exits, whether or not this entry point is used.
// Rows of up to DSW_NOALLOC_LN_MAX_D elements are supported (any number of
// rows); a larger d is refused with DSW_NOALLOC_TOO_LARGE and a message on
// stderr, and the caller should fall back to dsw_layernorm_bwd.
//
// Set-up: the first call on each device looks up the array's device address
// (cudaGetSymbolAddress, with that device current) and caches it.  Make that
// first call outside any stream capture.  No call allocates or frees memory.
//
// Sharing: all calls on a device use the same array.  Each call overwrites the
// part it uses before reading it, so nothing has to be cleared between calls,
// but two calls that can run at the same time on one GPU (different streams)
// race on it: keep calls on one stream or order them with events.
//
// Arguments and results are those of dsw_layernorm_bwd without `scratch`:
//   dy, x, dres (optional), dx : bf16 [M, d] row-major, 16-byte aligned
//   gamma, mean, rstd          : fp32 [d], [M], [M]
//   dgamma, dbeta (optional), dres_sum (optional) : fp32 [d], accumulated (+=)
// Returns 0, one of the codes below, or the negative code of dsw_layernorm_bwd.
#pragma once
#include <cuda_runtime.h>

#define DSW_NOALLOC_LN_MAX_D 2048
#define DSW_NOALLOC_LN_MAX_BLOCKS 296

#define DSW_NOALLOC_BAD_SHAPE (-20)
#define DSW_NOALLOC_TOO_LARGE (-21)
#define DSW_NOALLOC_NO_DEVICE (-22)
#define DSW_NOALLOC_NO_SYMBOL (-23)

#ifdef __cplusplus
extern "C" {
#endif

int dsw_layernorm_bwd_noalloc(const void* dy, const void* x, const float* gamma, const float* mean,
                              const float* rstd, const void* dres, void* dx, float* dgamma, float* dbeta,
                              float* dres_sum, int M, int d, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
