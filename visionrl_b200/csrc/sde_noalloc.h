// C entry point of the SDE step for callers that must not allocate.
//
// This function has no counterpart in the reference implementation.  It exists for hosts that
// drive the step from code where a device allocation is not allowed or not wanted: a C or C++
// serving loop without libtorch's caching allocator, a callback running inside a region whose
// memory footprint must stay fixed, or a real-time thread that may not take the allocator's
// locks.  The tensor-returning `sde_step_fwd` allocates its outputs and a per-call scratch
// buffer; this variant writes into caller-provided outputs and keeps its scratch in a fixed
// device array that is part of the loaded module.
#pragma once

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest scratch the entry point can serve, in floats:
//   batch * ceil(n / 4096) must not exceed this (n = elements per sample).
#define VRL_SDE_NOALLOC_MAX_SCRATCH_FLOATS 65536

// mean = a[s] x + b[s] v;  next = given `prev_in`, else mean + scale[s] * noise, or x + dt[s] v
// when `deterministic`;  logp[s] = Gaussian (or negative mean-square when !gaussian) log-density
// of `next` under N(mean, scale[s]^2), averaged over the n elements of sample s.
//
// All pointers are device pointers on the current device; v, x, noise / prev_in, next_out,
// mean_out hold batch * n floats, a, b, scale, dt, logp hold `batch` floats.  Exactly one of
// `prev_in` and `noise` may be null.  `stream` is a cudaStream_t (null = default stream).
//
// Returns 0 on success.  Non-zero: 1 bad argument, 2 the problem needs more scratch than
// VRL_SDE_NOALLOC_MAX_SCRATCH_FLOATS, 3 a CUDA call failed during set-up, 4 a launch failed, 5 an
// error from earlier, unrelated CUDA work was already pending (nothing is launched and the pending
// error is left in place for its owner to read).  When `err` is non-null a NUL-terminated description is written to it (at most `err_len` bytes).
//
// The function performs no device or host allocation.  The first call on each device looks up
// the address of the module's scratch array (one cudaGetSymbolAddress call with that device
// current) and caches it; make that first call outside of any stream capture.  Every element of
// the scratch that a call reads is written earlier in the same call, so nothing has to be
// zeroed.  All calls on one device share the one scratch array: calls whose kernels can overlap
// in time (different streams, or different host threads) race on it and must be serialised by
// the caller.
int vrl_sde_step_noalloc(const float* v, const float* x, const float* a, const float* b,
                         const float* scale, const float* dt, const float* prev_in,
                         const float* noise, float* next_out, float* mean_out, float* logp,
                         int batch, int64_t n, int deterministic, int gaussian, void* stream,
                         char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
