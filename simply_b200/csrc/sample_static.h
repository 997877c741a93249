/* Sampling for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in google-deepmind/simply.
 *
 * Who needs it: code that runs where cudaMalloc is off limits.  Examples are a host
 * thread inside a latency-critical serving loop that must never take the allocator's
 * lock or trigger an implicit device synchronisation, a process whose memory budget was
 * fixed at start-up and is policed (any later allocation is treated as a fault), and a
 * plug-in that is handed raw device pointers by a host application and has no
 * allocator of its own.  `sb_sample` (csrc/sampling.cu) asks its caller for a scratch
 * buffer, which those callers cannot provide; this variant brings its own.
 *
 * How: the scratch lives in one file-scope `static __device__` array inside the library
 * (SB_SAMPLE_STATIC_MAX_ROWS rows of SB_SAMPLE_STATIC_MAX_SLICES slices, about 133 KB).
 * Every GPU that loads the library holds that array until the process exits.  The
 * function calls no cudaMalloc, no cudaFree and no allocating library routine.
 *
 * Set-up: the first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current) and remembers it per device.  Make
 * that first call outside any stream capture.
 *
 * Sharing: all calls use the same array and find in it whatever the last call left.
 * The kernels write every word before they read it, so nothing needs clearing between
 * calls.  Two calls whose kernels overlap on the GPU (different streams, or different
 * host threads on one device) race on the array: serialise them.
 *
 * Inputs and outputs are the caller's, exactly as for `sb_sample`:
 *   logits  float32 [num_rows, vocab] on the device
 *   params  int32   [num_rows, 6] on the device: temperature (float bits), top_k,
 *           top_p (float bits), seed low word, seed high word, position of the sampled token
 *   out     int32   [num_rows] on the device: the sampled token ids
 *
 * Returns 0 on success, a positive cudaError_t if a CUDA call failed, or
 *   SB_SAMPLE_STATIC_TOO_MANY_ROWS   num_rows > SB_SAMPLE_STATIC_MAX_ROWS
 *   SB_SAMPLE_STATIC_BAD_ARGUMENT    a null pointer, num_rows < 0 or vocab <= 0; the current
 *                                    device's ordinal is 64 or more (the table of per-device
 *                                    addresses ends there); or the sampling kernels would cut a
 *                                    row into more than SB_SAMPLE_STATIC_MAX_SLICES slices (they
 *                                    never do: sb_sample_slices caps at the same number, and a
 *                                    static_assert in sampling.cu ties the two together)
 * (a line that names the limit is also written to stderr).
 */
#ifndef SIMPLY_B200_SAMPLE_STATIC_H_
#define SIMPLY_B200_SAMPLE_STATIC_H_

#include <cuda_runtime.h>

#define SB_SAMPLE_STATIC_MAX_ROWS 256
#define SB_SAMPLE_STATIC_MAX_SLICES 64
#define SB_SAMPLE_STATIC_TOO_MANY_ROWS (-21)
#define SB_SAMPLE_STATIC_BAD_ARGUMENT (-22)

#ifdef __cplusplus
extern "C" {
#endif

int sb_sample_static(const float* logits, const int* params, int* out, int num_rows, int vocab,
                     cudaStream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* SIMPLY_B200_SAMPLE_STATIC_H_ */
