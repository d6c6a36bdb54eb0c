/* spite_sample_noalloc: token sampling for callers that must not allocate.
 *
 * This entry point has no counterpart in giveen/spite; it is an addition of this
 * library.
 *
 * Who it is for.  `spite_sample` needs a float scratch row per row of logits,
 * which its caller allocates.  Some callers cannot do that at the moment they
 * sample: code running between the begin and end of a CUDA stream capture, a
 * host that handed all device memory to a pool of its own, a plugin loaded into
 * a process whose allocator must not be re-entered from this library, or a
 * real-time loop in which cudaMalloc's implicit device synchronisation is not
 * acceptable.  For them the scratch is a fixed array inside this library, and
 * the call allocates nothing: no cudaMalloc, no cudaFree, no allocating library
 * routine.
 *
 * The price.
 *  - The array is `SPITE_SAMPLE_NOALLOC_MAX_FLOATS` floats (8 MiB).  Every GPU
 *    on which this library is loaded holds it from the first use until the
 *    process exits.
 *  - rows * vocab must not exceed that size; a larger request is refused with
 *    status -2 and nothing is launched or written.
 *  - A row that fits the shared memory of a cluster of eight blocks (up to
 *    393,216 logits) is sampled there, as `spite_sample` does it, and the array
 *    is not touched; longer rows go through the array.  The size limit above
 *    holds either way, so that a caller need not know which applies.
 *  - All calls share the one array.  It keeps what the last call left in it;
 *    the kernel overwrites every element it reads before reading it, so nothing
 *    has to be cleared between calls.  Two calls that can run at the same time
 *    on one GPU (different streams, or different host threads on different
 *    streams) race on it: order them on one stream or with events.
 *  - The first call on a device looks the array's device address up
 *    (cudaGetSymbolAddress, once per device, with that device current) and
 *    remembers it.  Make that first call outside any stream capture.
 *
 * Inputs and outputs are the caller's, exactly as for `spite_sample`:
 * per-row option arrays may be null where `spite_sample` allows it, `rng_state`
 * is advanced in place for rows that draw, `out_tokens` receives one token per row.
 *
 * Returns 0 on success, -1 for a malformed argument, -2 for a size beyond the
 * fixed scratch, -3 if the address lookup or the launch failed.
 */
#pragma once

#define SPITE_SAMPLE_NOALLOC_MAX_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    const float* logits;               /* [rows, vocab], not modified */
    const float* temperature;          /* [rows]; <= 0: argmax */
    const int* top_k;                  /* [rows] or null; 0: off */
    const float* top_p;                /* [rows] or null; >= 1: off */
    const float* min_p;                /* [rows] or null; <= 0: off */
    const float* repetition_penalty;   /* [rows] or null; 1: off */
    const int* context;                /* tokens the penalty looks at, all rows, or null */
    const int* context_offsets;        /* [rows + 1] into context; required with context */
    unsigned long long* rng_state;     /* [rows], in and out */
    int* out_tokens;                   /* [rows], out */
    int rows;
    int vocab;
} SpiteSampleNoAllocArgs;

int spite_sample_noalloc(const SpiteSampleNoAllocArgs* args, void* stream);

#ifdef __cplusplus
}
#endif
