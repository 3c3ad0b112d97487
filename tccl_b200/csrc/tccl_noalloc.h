/*
 * An entry point of libtccl_b200 that allocates nothing.
 *
 * This function has no counterpart in the reference library; it exists for
 * callers that are not able to obtain device memory at the moment they need a
 * reduction:
 *   - a process that has already handed (nearly) all device memory to a
 *     framework's caching allocator or to a preallocating runtime, so that a
 *     direct cudaMalloc would fail;
 *   - a plug-in running inside a host application whose memory is all spoken for;
 *   - a latency-critical loop that must not pay cudaMalloc's implicit
 *     device-wide synchronisation.
 *
 * tccl_allreduce_local_noalloc() is the single-GPU form of the one-shot
 * all-reduce: `n_ranks` input buffers that live on the current device are summed
 * elementwise (fp32 accumulation, fixed order 0..n_ranks-1, one rounding) and the
 * sum is written to each of the `n_ranks` output buffers, exactly as
 * tccl_allreduce_oneshot_p2p does for ranks emulated on one GPU.  The kernel
 * needs scratch memory for its inter-block barriers (flag rows, epoch counters
 * and a status block per emulated rank).  Here that scratch is a file-scope
 * `static __device__` array inside the library, TCCL_NOALLOC_SCRATCH_BYTES long;
 * every GPU that loads the library holds it until the process exits.  The caller
 * passes only inputs and outputs.
 *
 * Limits (fixed by the size of the static scratch; larger values are rejected
 * with -TCCL_ESIZE and nothing is launched):
 *   n_ranks <= TCCL_NOALLOC_MAX_RANKS, ctas <= TCCL_NOALLOC_MAX_CTAS.
 * `numel` is not limited by the scratch.  Inputs and outputs must be 16-byte
 * aligned; `dtype` is a tccl_dtype.  No output may be one of the inputs (every
 * rank stores its sums while the others are still reading the inputs, so an
 * in-place call would race): such a call is rejected with -TCCL_EINVAL; partially
 * overlapping buffers are not detected and must be avoided by the caller.
 *
 * Set-up: the first call on each device looks up the device address of the
 * scratch array (cudaGetSymbolAddress, with that device current) and remembers
 * it.  Make that first call outside of any stream capture.  The look-up is
 * guarded by a mutex, so first calls from several host threads are safe.  No call
 * allocates or frees memory, in this library or through another one.
 *
 * Sharing: all calls on a device use the same scratch, and it keeps what the
 * previous call left there; each launch therefore clears the words that must
 * start at zero before it uses them.  Two calls that overlap on the GPU (for
 * example from two streams) race on the scratch and must be serialised by the
 * caller.
 *
 * Returns 0, a cudaError_t (> 0), or a negated tccl_arg_error; see
 * tccl_error_string().  A device-side wait that gives up is reported through
 * tccl_noalloc_last_status().
 */
#pragma once
#include <stdint.h>

#include "tccl_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define TCCL_NOALLOC_MAX_RANKS 8
#define TCCL_NOALLOC_MAX_CTAS 16
/* per emulated rank: barrier flag rows [ctas][TCCL_MAX_WORLD] + private state up to the status block */
#define TCCL_NOALLOC_FLAG_WORDS (TCCL_NOALLOC_MAX_CTAS * TCCL_MAX_WORLD)
#define TCCL_NOALLOC_LOCAL_WORDS (TCCL_LOCAL_STATUS + TCCL_ST_WORDS)
#define TCCL_NOALLOC_SCRATCH_BYTES \
  (TCCL_NOALLOC_MAX_RANKS * (TCCL_NOALLOC_FLAG_WORDS + TCCL_NOALLOC_LOCAL_WORDS) * 4)

int tccl_allreduce_local_noalloc(const void* const* in,  /* host array: n_ranks device pointers */
                                 void* const* out,       /* host array: n_ranks device pointers */
                                 int n_ranks, uint64_t numel, int dtype, int ctas, void* stream);

/* Copies the status words (TCCL_ST_WORDS of them) of emulated rank `rank` on the
 * current device into `words` (host memory) after synchronising `stream`. */
int tccl_noalloc_last_status(int rank, uint32_t* words, void* stream);

#ifdef __cplusplus
}
#endif
