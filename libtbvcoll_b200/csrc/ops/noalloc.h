// noalloc.h — an entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference library: it exists for users of THIS library
// who sit in a place where cudaMalloc is off limits.  Typical cases: a serving process that
// handed every free byte of the GPU to its KV-cache pool at start-up, so a later cudaMalloc
// simply fails; a latency-critical loop where an allocation would synchronise the whole
// device; a plug-in loaded into a host application whose rules forbid allocating after
// initialisation.  Such a caller can still do greedy sampling with the function below: it
// is the same two-stage arg-max as tbv_op_argmax, but the scratch it needs (per-row tickets
// and per-CTA partial maxima) lives in a fixed array inside the library image instead of a
// caller-provided workspace.
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest `tokens` (rows of logits) one call accepts.  The scratch array is sized for this
// and occupies about 193 KiB of device memory on every GPU that loads the library, from
// load until the process exits.
#define TBV_ARGMAX_NOALLOC_MAX_TOKENS 256

// Per row of logits [tokens, vocab] (bf16, row stride `ld` elements): out_val[row] = the
// largest logit as fp32, out_idx[row] = the lowest index holding it, plus index_offset.
// Same results, bit for bit, as tbv_op_argmax.
//
// Allocates nothing: no cudaMalloc / cudaFree, no torch, no library call that allocates.
// The caller passes inputs and outputs only.
//
// Returns 0 on success; -2 with a message on stderr when tokens exceeds
// TBV_ARGMAX_NOALLOC_MAX_TOKENS (or is negative / vocab is not positive); -1 when the set-up
// or the launch fails.
//
// The first call on each device looks up the device address of the scratch array (once per
// device, with that device current).  Make that first call before starting any stream
// capture on the device.
//
// All calls on a device share the one scratch array, and it keeps whatever the previous
// call left in it; each call clears the part that has to start at zero (the tickets) on the
// given stream before it launches.  Two calls whose kernels may run at the same time on one
// device — different streams with no ordering between them — race on the array and give
// wrong answers: order them.
int tbv_op_argmax_noalloc(const void* logits, int tokens, int vocab, int ld, long long index_offset, void* out_val,
                          void* out_idx, void* stream);

#ifdef __cplusplus
}
#endif
