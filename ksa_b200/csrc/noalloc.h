// Entry point of the kernel library that never allocates memory.
//
// This has no counterpart in the reference: it exists for callers of this library that
// are not allowed to allocate device memory at the time of the call.  Examples: code that
// runs inside a memory pool it must not grow, a real-time or serving loop with a fixed
// memory budget decided at start-up, and host programs that embed the library through its
// C symbols and own every byte of device memory themselves.  Such callers cannot hand the
// RMSNorm backward its scratch buffer ("dw_partial" of ksa_rmsnorm_bwd) without allocating
// one, so this variant carries the scratch inside the library instead.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in scratch array covers.
#define KSA_NOALLOC_RMSNORM_MAX_D 4096      /* hidden size (columns) */
#define KSA_NOALLOC_RMSNORM_MAX_PARTS 148   /* partial rows = CTAs used */

// RMSNorm backward, same mathematics and argument meaning as ksa_rmsnorm_bwd:
//   dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres),   dw (+)= sum_rows dy * xhat
// with x, dy, dres, dx bf16 [rows, D]; w bf16 [D]; rstd fp32 [rows]; dw fp32 [D];
// dres may be null; accumulate_dw != 0 adds to dw instead of overwriting it.
//
// What differs from ksa_rmsnorm_bwd:
//   * no scratch argument: the per-CTA partial sums of dw go to an array of
//     KSA_NOALLOC_RMSNORM_MAX_PARTS x KSA_NOALLOC_RMSNORM_MAX_D floats (2.4 MB) that is part
//     of the library image.  Every GPU that loads the library holds that array until the
//     process exits, whether or not this function is ever called.
//   * D > KSA_NOALLOC_RMSNORM_MAX_D (or D not a multiple of 8, or rows < 0) is rejected with
//     a non-zero return code and a message in ksa_last_error(); nothing is launched.
//   * the function calls no cudaMalloc / cudaFree and no allocating library routine.  The
//     device that owns the buffers must already be current on the calling thread.
//   * the first call on each device looks up the device address of the array
//     (cudaGetSymbolAddress) and remembers it; make that first call before any stream
//     capture begins.  Where CUDA loads modules lazily, that first call may also be the one
//     that loads the module holding the array (the 2.4 MB appear then, once).
//   * all calls share the one array.  Nothing in it has to start at zero (every partial row
//     that is read was written by the same call), but two calls whose kernels overlap on the
//     GPU (different streams, no dependency between them) race on it and corrupt dw.
//     Serialise them on one stream or with events.
//
// Returns 0 on success.
__attribute__((visibility("default")))
int ksa_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const void* rstd, const void* dres,
                            void* dx, void* dw, int accumulate_dw, int rows, int D, void* stream);

#ifdef __cplusplus
}
#endif
