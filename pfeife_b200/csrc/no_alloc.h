// Norm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for embedders of this
// library that run where cudaMalloc is off limits: code executing inside a pre-sized memory
// arena they are not allowed to grow, plugins handed a fixed workspace by their host
// application, or latency-critical loops where an allocation (and the implicit device
// synchronisation it may cause) is not acceptable.
//
// pf_norm_bwd_static computes exactly what pf_norm_bwd computes (LayerNorm / RMSNorm backward:
// dx, dgamma, dbeta), but the per-CTA partial sums of dgamma / dbeta live in a fixed array that
// is part of the library image instead of a caller-provided scratch buffer.
//
//  * Limit: the partial sums need  pf_norm_bwd_ctas(rows, sm_count) * 2 * N  floats and the
//    built-in array holds PF_NORM_STATIC_SCRATCH_FLOATS (1 Mi floats = 4 MiB; e.g. N = 1408 on
//    a 148-SM device needs 0.83 Mi).  Larger problems are rejected with -3 and nothing is
//    launched.  Every GPU that loads the library holds these 4 MiB until the process exits.
//  * The call allocates nothing: no cudaMalloc / cudaFree, no allocating library routine.
//    Inputs and outputs are still the caller's buffers.
//  * The first call on each device looks up the array's device address (one
//    cudaGetSymbolAddress with that device current).  Make that first call before any stream
//    capture is started on the device, and OUTSIDE the region in which you may not allocate:
//    the CUDA runtime loads a library's device code lazily, so the first use of this
//    translation unit on a device can make the runtime itself allocate memory for the module
//    image (the 4 MiB array included).  From the second call on nothing is allocated.
//  * The looked-up addresses sit in a small per-device table that is filled without a lock.
//    Two host threads that make the first call for the same device at the same time both
//    store the same value, which is harmless; no other state is shared between host threads.
//  * All calls share the one array and it keeps the previous call's contents; the kernels
//    overwrite every element they later read, so nothing has to be cleared, but two calls that
//    overlap on the GPU (different streams, or graphs replayed concurrently) race on it.
//    Serialise them.
#pragma once
#include "api.h"

#define PF_NORM_STATIC_SCRATCH_FLOATS (1 << 20)

PF_DECL int pf_norm_bwd_static(const void* dy, const void* h, const void* gamma, const void* mean,
                               const void* rstd, const void* dres, void* dx, void* dgamma,
                               void* dbeta, long long rows, int N, int rms, int accumulate,
                               int dtype, int sm_count, void* stream);
