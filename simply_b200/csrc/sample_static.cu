// sb_sample_static: the sampling kernels of sampling.cu with their scratch in a static
// device array, for callers that cannot allocate.  See sample_static.h for who they are,
// the limits and the rules of use.  No counterpart in google-deepmind/simply.
#include <stdio.h>

#include "sample_static.h"

// The existing entry point and its helper (sampling.cu).  It takes the scratch as an
// argument and does not allocate, so the variant only has to bring the scratch.
extern "C" int sb_sample(const float* logits, const int* params, int* out, int num_rows, int vocab,
                         void* scratch, cudaStream_t stream);
extern "C" int sb_sample_slices(int num_rows, int vocab);

// Per row: 1 threshold word (+1 of padding over all rows) and MAX_SLICES partial results of 2 words.
#define SB_SCRATCH_WORDS (SB_SAMPLE_STATIC_MAX_ROWS * (2 + 2 * SB_SAMPLE_STATIC_MAX_SLICES))

// In host code this name is only a handle for cudaGetSymbolAddress, not a device address.
static __device__ __align__(256) int sb_sample_scratch[SB_SCRATCH_WORDS];

#define SB_MAX_DEVICES 64
static void* g_scratch_address[SB_MAX_DEVICES];  // device address of the array, per device ordinal

extern "C" int sb_sample_static(const float* logits, const int* params, int* out, int num_rows, int vocab,
                                cudaStream_t stream) {
  if (!logits || !params || !out || num_rows < 0 || vocab <= 0) {
    fprintf(stderr, "sb_sample_static: null pointer, negative row count or empty vocabulary\n");
    return SB_SAMPLE_STATIC_BAD_ARGUMENT;
  }
  if (num_rows > SB_SAMPLE_STATIC_MAX_ROWS) {
    fprintf(stderr, "sb_sample_static: %d rows exceed the static scratch's limit of %d rows per call\n",
            num_rows, SB_SAMPLE_STATIC_MAX_ROWS);
    return SB_SAMPLE_STATIC_TOO_MANY_ROWS;
  }
  if (num_rows == 0) return 0;
  if (sb_sample_slices(num_rows, vocab) > SB_SAMPLE_STATIC_MAX_SLICES) {
    fprintf(stderr, "sb_sample_static: more than %d slices per row asked of the static scratch\n",
            SB_SAMPLE_STATIC_MAX_SLICES);
    return SB_SAMPLE_STATIC_BAD_ARGUMENT;
  }
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= SB_MAX_DEVICES) {
    fprintf(stderr, "sb_sample_static: device ordinal %d is beyond the %d this entry point keeps addresses for\n",
            device, SB_MAX_DEVICES);
    return SB_SAMPLE_STATIC_BAD_ARGUMENT;
  }
  if (g_scratch_address[device] == nullptr) {
    // Once per device, with that device current (it is: we just asked which one is).
    void* address = nullptr;
    e = cudaGetSymbolAddress(&address, sb_sample_scratch);
    if (e != cudaSuccess) return (int)e;
    g_scratch_address[device] = address;
  }
  return sb_sample(logits, params, out, num_rows, vocab, g_scratch_address[device], stream);
}
