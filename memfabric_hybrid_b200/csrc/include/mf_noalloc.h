/*
 * An all-reduce entry point that allocates nothing. It has no counterpart in the reference.
 *
 * Who it is for: code that runs where device memory must not be requested any more — inside a serving
 * engine after it has handed all free HBM to its KV cache, in a plugin whose host forbids cudaMalloc,
 * or on a path that must not disturb a caching allocator's bookkeeping. Such callers cannot give the
 * collective kernels the staging and flag memory they need, so this variant keeps that scratch in a
 * fixed array that is part of the library image.
 *
 * What it computes: `in` holds `world` equally long vectors stacked one after the other (the ranks of a
 * single-GPU, in-kernel-emulated group); every `out[r]` receives scale * reduce_r(in[r]) — the same
 * kernel, protocol and result as the regular one-shot all-reduce launched on an emulated heap.
 *
 * Limits and rules:
 *   - world is 1..MF_NOALLOC_MAX_WORLD and each vector is at most MF_NOALLOC_MAX_BYTES bytes; anything
 *     larger is refused with MF_NOALLOC_E_TOO_LARGE before any work is queued;
 *   - the scratch array (MF_NOALLOC_MAX_WORLD x 3 MiB) is held by every GPU that loads the library
 *     until the process exits;
 *   - the first call on a device looks up the array's device address, with that device current; make
 *     that first call outside any stream capture. Nothing is cleared: the array is zero when the library
 *     is loaded, and the only work queued is the kernel on the caller's stream;
 *   - all calls share the one array, which keeps what the previous call left in it (flags are epoch
 *     numbered, so they never need clearing); two calls that overlap on the GPU, from different streams
 *     or threads, race on it: serialise them;
 *   - it calls no cudaMalloc, cudaFree or allocating library routine;
 *   - every wait inside the kernel is bounded. A wait that runs out makes the kernel return without
 *     writing `out`; the launching call has long returned MF_NOALLOC_OK by then, so after synchronising
 *     the stream a careful caller asks mf_noalloc_status() whether that happened.
 */
#ifndef MF_B200_NOALLOC_H
#define MF_B200_NOALLOC_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MF_NOALLOC_MAX_WORLD 8
#define MF_NOALLOC_MAX_BYTES (1u << 20)

#define MF_NOALLOC_OK           0
#define MF_NOALLOC_E_ARG       -1  /* null pointer, bad dtype / op / world */
#define MF_NOALLOC_E_TOO_LARGE -2  /* a vector exceeds MF_NOALLOC_MAX_BYTES */
#define MF_NOALLOC_E_SETUP     -3  /* the scratch array's address could not be obtained on this device */
#define MF_NOALLOC_E_LAUNCH    -4  /* the kernel launch was refused */
#define MF_NOALLOC_E_TIMEOUT   -5  /* mf_noalloc_status: a bounded wait of an earlier call ran out */

/* dtype: 0 bf16, 1 fp16, 2 fp32, 3 int32. op: 0 sum, 1 max, 2 min, 3 prod. n: elements per vector. */
int mf_allreduce_stacked_noalloc(const void *in, void *out, int world, uint64_t n, int dtype, int op, float scale, void *stream);
const char *mf_noalloc_strerror(int code);

/* Reads the status words that the kernels of mf_allreduce_stacked_noalloc keep inside the built-in scratch
 * of the current device (it allocates nothing either). Call it after the stream of the all-reduce has been
 * synchronised. Returns MF_NOALLOC_OK with out = {0,0,0,0} when every call so far completed, else
 * MF_NOALLOC_E_TIMEOUT with out = {1 (time-out), where the first wait gave up, the call's sequence number,
 * how many waits gave up}. The words stay set until a call with clear != 0 resets them. It copies a few
 * bytes with a synchronous cudaMemcpy: do not call it while the current thread captures a stream. */
int mf_noalloc_status(uint32_t out[4], int clear);

#ifdef __cplusplus
}
#endif
#endif
