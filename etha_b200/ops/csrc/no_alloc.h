// Allocation-free entry point of the copy-table kernels.  It has no counterpart in the reference, whose
// executor allocates staging tensors on every transfer (src/etha/comm/ir.py:246-257).
//
// Who needs it: a weight-sync hook that runs inside an inference worker.  Such a worker has usually handed
// nearly all free device memory to its KV-cache pool before the first sync, so a cudaMalloc (or a torch
// allocation) at sync time can fail outright or evict/fragment the pool; the same holds for an agent that only
// maps other processes' tensors and owns no pool of its own.  These callers still own the tensors they want
// moved, so they pass sources and destinations as usual, and everything else the kernels need — the packed op
// table, the tile prefix sums, the CTA arrival counter and the error word — lives in one fixed array that is
// part of the loaded library image.
//
// Limits and rules:
//  * at most ETHA_NOALLOC_MAX_OPS ops per call; a larger request is refused with an error message, nothing
//    is launched;
//  * the array (ETHA_NOALLOC_SCRATCH_BYTES, 256-byte aligned) exists once per GPU that loads the library and
//    stays resident until the process exits;
//  * the first call on a device looks up the array's device address (no allocation, but a one-time runtime
//    query);
//  * never call it on a stream that is being captured, first call or later: each call copies its tables from
//    host arrays that belong to the calling thread, which a captured copy would re-read at replay time.  The
//    entry point checks and refuses a capturing stream (-101, nothing is enqueued);
//  * every call rewrites the table and zeroes the counters before launching, so nothing depends on what the
//    previous call left behind — but two calls that overlap on the GPU (different streams, different threads)
//    share the array and race.  Serialise them, or use the table API, which owns its buffers;
//  * no cudaMalloc / cudaFree / allocating library routine is called on any path of this entry point.
#pragma once
#include "m2n.h"

#define ETHA_NOALLOC_MAX_OPS 64
#define ETHA_NOALLOC_SCRATCH_BYTES (2048 + ETHA_NOALLOC_MAX_OPS * 320)

#ifdef __cplusplus
extern "C" {
#endif

// Packs `n_specs` op descriptions (same struct and validation as etha_pack_op), stores the table in the
// library's resident scratch array and enqueues the copy kernels on `stream`.  Returns 0, or a negative code
// with the reason in etha_last_error(): -100 too many ops, -101 bad argument, other codes from packing or
// from the CUDA runtime.  `ctas_per_sm` <= 0 selects the default (2).
int etha_m2n_run_noalloc(const struct M2NOpSpec* specs, uint32_t n_specs, int ctas_per_sm, void* stream);

// Reads the error word the kernels of the last call left in the scratch array (synchronises `stream`).
int etha_m2n_noalloc_status(uint32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
