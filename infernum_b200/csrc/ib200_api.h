/* C declarations of entry points of the "core" kernel library
 * (libib200_core_*.so) that are meant to be called from outside this package.
 * Pointers are device pointers, `stream` is a cudaStream_t, the return value
 * is 0 on success, a positive cudaError_t, or a negative refusal code
 * (-1 bad argument, -2 unsupported, -3 beyond the stated maximum,
 * -4 the per-device set-up failed). */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

/* Greedy token selection (largest logit, lowest index among equals) for
 * callers that cannot allocate device memory: a plug-in that is handed only
 * its input and output buffers by a host application and has to stay off
 * cudaMalloc (which synchronises the device, and can fail once cache pages
 * fill the GPU).  Same result as ib_argmax, whose wide-row variant needs a
 * caller-supplied scratch buffer; here the scratch is a 128 KiB array inside
 * the library, held by every GPU that loads it until the process exits.
 *
 *   logits  float32 [n_rows, ld], row r at logits + r * ld, V <= ld values used
 *   out     int32 [n_rows]
 *   n_rows  at most ib_argmax_noalloc_max_rows() (256); more is refused with -3
 *
 * The first call on each device looks up the scratch array's device address;
 * make that call before any stream capture begins.  All calls share the
 * array, so calls that overlap on the GPU race: keep them on one stream or
 * serialise them.  Nothing is allocated or freed.
 *
 * This entry point has no counterpart in the reference. */
int ib_argmax_noalloc(const float* logits, int ld, int n_rows, int V, int* out, void* stream);
int ib_argmax_noalloc_max_rows(void);

#ifdef __cplusplus
}
#endif
