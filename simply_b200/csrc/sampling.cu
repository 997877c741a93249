// Sampling from float32 logits.
//
// Semantics of simply/utils/sampling_lib.py:472-537:
//   temperature == 0 or top_k == 1 -> argmax (lowest index on ties)
//   otherwise logits / temperature, masked to the top-k entries (:427-431) and to
//   the top-p nucleus (:434-441; inside the top-k set when both are given,
//   :444-469), then one categorical draw.
// The draw is Gumbel-max, like jax.random.categorical, with counter-based noise:
// Philox-4x32-10 keyed by the request's 64-bit seed, counter (entry / 4, position
// of the sampled token, 0, 0), word entry % 4.  A request's draw therefore
// depends on nothing but its own seed, position and logits.
//
// Masks are found without sorting, by bisection on the order-preserving integer
// image of the scaled logits: the k-th largest value for top-k; for top-p the
// smallest value whose strictly-greater entries hold less than top_p of the
// probability mass.  Entries equal to the threshold are all kept (the
// reference's sort keeps the first of equal entries only).
#include <float.h>

#include "common.cuh"
#include "sample_static.h"

// Most slices a row of the vocabulary is cut into.  The static scratch of sb_sample_static is
// laid out for this many partial results per row.
#define SAMPLE_MAX_SLICES 64
static_assert(SAMPLE_MAX_SLICES == SB_SAMPLE_STATIC_MAX_SLICES,
              "sb_sample_static's scratch holds SB_SAMPLE_STATIC_MAX_SLICES partial results per row");

#define SAMPLE_THREADS 1024

__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t out[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ __forceinline__ float gumbel_from_bits(uint32_t bits) {
  const float u = ((float)(bits >> 8) + 0.5f) * 5.9604644775390625e-08f;  // 2^-24
  return -logf(-logf(u));
}

struct ArgMax {
  float v;
  int i;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ ArgMax block_argmax(ArgMax x, ArgMax* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = x;
  __syncthreads();
  if (warp == 0) {
    ArgMax y = lane < nwarps ? scratch[lane] : ArgMax{-FLT_MAX, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax z;
      z.v = __shfl_xor_sync(0xffffffffu, y.v, o);
      z.i = __shfl_xor_sync(0xffffffffu, y.i, o);
      y = better(y, z);
    }
    if (lane == 0) scratch[32] = y;
  }
  __syncthreads();
  return scratch[32];
}

__device__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -FLT_MAX;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// params per row (int32 words): temperature (float bits), top_k, top_p (float bits),
// seed low, seed high, position.
//
// Three launches: (1) one block per row finds the row's keep-threshold (0 when neither top-k
// nor top-p is set: the block leaves at once); (2) `slices` blocks per row each find the best
// entry of their slice of the vocabulary (plain argmax when greedy, argmax of scaled logit +
// Gumbel noise otherwise); (3) one warp per row picks the best slice, lowest index on ties.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_threshold_kernel(const float* __restrict__ logits, const int* __restrict__ params,
                        uint32_t* __restrict__ thresholds, int vocab) {
  pdl_wait_block();
  pdl_launch_dependents();
  __shared__ float fscratch[33];
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const int* p = params + r * 6;
  const float temperature = __int_as_float(p[0]);
  const int top_k = p[1];
  const float top_p = __int_as_float(p[2]);
  const bool greedy = temperature == 0.f || top_k == 1;
  const bool use_k = !greedy && top_k > 0 && top_k < vocab, use_p = !greedy && top_p < 1.f;
  if (!use_k && !use_p) {
    if (threadIdx.x == 0) thresholds[r] = 0;
    return;
  }
  uint32_t threshold = 0;  // keep entries whose key >= threshold
  if (use_k) {
    // Largest K with count(key >= K) >= top_k: the key of the k-th largest entry.
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = threshold | (1u << bit);
      float cnt = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) cnt += order_key(row[i] / temperature) >= cand ? 1.f : 0.f;
      cnt = block_sum(cnt, fscratch);
      if (cnt >= (float)top_k) threshold = cand;
    }
  }
  if (use_p) {
    float mx = -FLT_MAX;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float s = row[i] / temperature;
      if (order_key(s) >= threshold) mx = fmaxf(mx, s);
    }
    mx = block_max(mx, fscratch);
    float z = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float s = row[i] / temperature;
      if (order_key(s) >= threshold) z += expf(s - mx);
    }
    z = block_sum(z, fscratch);
    // Largest K with mass(key >= K) >= top_p (mass over the kept set, normalised).
    const float target = top_p * z;
    uint32_t k2 = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = k2 | (1u << bit);
      float mass = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float s = row[i] / temperature;
        const uint32_t key = order_key(s);
        if (key >= threshold && key >= cand) mass += expf(s - mx);
      }
      mass = block_sum(mass, fscratch);
      if (mass >= target) k2 = cand;
    }
    threshold = max(threshold, k2);
  }
  if (threadIdx.x == 0) thresholds[r] = threshold;
}

#define SLICE_THREADS 256

__global__ void __launch_bounds__(SLICE_THREADS)
sample_slice_kernel(const float* __restrict__ logits, const int* __restrict__ params,
                    const uint32_t* __restrict__ thresholds, ArgMax* __restrict__ partial, int vocab,
                    int slice_len) {
  pdl_wait_block();
  pdl_launch_dependents();
  __shared__ ArgMax ascratch[33];
  const int r = blockIdx.y, slice = blockIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const int* p = params + r * 6;
  const float temperature = __int_as_float(p[0]);
  const int top_k = p[1];
  const int lo = slice * slice_len, hi = min(lo + slice_len, vocab);  // slice_len is a multiple of 4
  ArgMax best{-FLT_MAX, 0x7fffffff};
  if (temperature == 0.f || top_k == 1) {
    // Four entries per load where the row allows it (lo is a multiple of 4), two loads in flight.
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
      const int hi4 = lo + (hi - lo) / 4 * 4;
      ArgMax other{-FLT_MAX, 0x7fffffff};
      int i = lo + threadIdx.x * 4;
      for (; i + (int)blockDim.x * 4 < hi4; i += blockDim.x * 8) {
        const float4 a = *reinterpret_cast<const float4*>(row + i);
        const float4 b = *reinterpret_cast<const float4*>(row + i + blockDim.x * 4);
        best = better(better(better(better(best, ArgMax{a.x, i}), ArgMax{a.y, i + 1}), ArgMax{a.z, i + 2}), ArgMax{a.w, i + 3});
        const int j = i + blockDim.x * 4;
        other = better(better(better(better(other, ArgMax{b.x, j}), ArgMax{b.y, j + 1}), ArgMax{b.z, j + 2}), ArgMax{b.w, j + 3});
      }
      for (; i < hi4; i += blockDim.x * 4) {
        const float4 a = *reinterpret_cast<const float4*>(row + i);
        best = better(better(better(better(best, ArgMax{a.x, i}), ArgMax{a.y, i + 1}), ArgMax{a.z, i + 2}), ArgMax{a.w, i + 3});
      }
      best = better(best, other);
      for (int k = hi4 + threadIdx.x; k < hi; k += blockDim.x) best = better(best, ArgMax{row[k], k});
    } else {
      for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) best = better(best, ArgMax{row[i], i});
    }
  } else {
    const uint32_t threshold = thresholds[r];
    const uint32_t seed_lo = (uint32_t)p[3], seed_hi = (uint32_t)p[4], position = (uint32_t)p[5];
    for (int blk = lo / 4 + threadIdx.x; blk * 4 < hi; blk += blockDim.x) {
      uint32_t bits[4];
      philox4x32_10((uint32_t)blk, position, 0u, 0u, seed_lo, seed_hi, bits);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = blk * 4 + e;
        if (i >= hi) break;
        const float s = row[i] / temperature;
        if (order_key(s) < threshold) continue;
        best = better(best, ArgMax{s + gumbel_from_bits(bits[e]), i});
      }
    }
  }
  best = block_argmax(best, ascratch);
  if (threadIdx.x == 0) partial[(size_t)r * gridDim.x + slice] = best;
}

__global__ void sample_final_kernel(const ArgMax* __restrict__ partial, int* __restrict__ out, int slices) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int r = blockIdx.x, lane = threadIdx.x;
  ArgMax best{-FLT_MAX, 0x7fffffff};
  for (int s = lane; s < slices; s += 32) best = better(best, partial[(size_t)r * slices + s]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax y;
    y.v = __shfl_xor_sync(0xffffffffu, best.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, best.i, o);
    best = better(best, y);
  }
  if (lane == 0) out[r] = best.i;
}

// Log-probability of the token that was drawn, under the distribution it was drawn from
// (simply/utils/sampling_lib.py:540-601): 0 when the row is greedy; otherwise the log-softmax of
// logits / temperature over the entries the masks keep, at the token.  One block per row; reads
// the keep-thresholds that sample_threshold_kernel left in the scratch of the same sb_sample call.
// With `step_counter` the result goes to row *step_counter of `out` (a burst's history).
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_logprob_kernel(const float* __restrict__ logits, const int* __restrict__ params,
                      const uint32_t* __restrict__ thresholds, const int* __restrict__ tokens,
                      float* __restrict__ out, const int* __restrict__ step_counter, int vocab) {
  pdl_wait_block();
  pdl_launch_dependents();
  __shared__ float fscratch[33];
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const int* p = params + r * 6;
  const float temperature = __int_as_float(p[0]);
  const int top_k = p[1];
  float* dst = out + (step_counter ? (size_t)*step_counter * gridDim.x : 0) + r;
  if (temperature == 0.f || top_k == 1) {
    if (threadIdx.x == 0) *dst = 0.f;
    return;
  }
  const uint32_t threshold = thresholds[r];
  float mx = -FLT_MAX;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float s = row[i] / temperature;
    if (order_key(s) >= threshold) mx = fmaxf(mx, s);
  }
  mx = block_max(mx, fscratch);
  float z = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float s = row[i] / temperature;
    if (order_key(s) >= threshold) z += expf(s - mx);
  }
  z = block_sum(z, fscratch);
  if (threadIdx.x == 0) {
    const int tok = tokens[r];
    const float s = (tok >= 0 && tok < vocab) ? row[tok] / temperature : -FLT_MAX;
    *dst = order_key(s) >= threshold ? s - mx - logf(z) : -FLT_MAX;
  }
}

// After sb_sample with the same arguments and scratch: out[r] (or out[*step_counter, r]) is the
// log-probability of tokens[r].
extern "C" int sb_sample_logprobs(const float* logits, const int* params, const int* tokens, float* out,
                                  const int* step_counter, int num_rows, int vocab, const void* scratch,
                                  cudaStream_t stream) {
  if (num_rows == 0) return 0;
  sb_launch(sample_logprob_kernel, num_rows, SAMPLE_THREADS, 0, stream, logits, params,
            reinterpret_cast<const uint32_t*>(scratch), tokens, out, step_counter, vocab);
  SB_LAUNCH_CHECK();
  return 0;
}

// scratch: at least num_rows * (1 + 2 * slices) 32-bit words, slices = sb_sample_slices(num_rows, vocab).
extern "C" int sb_sample_slices(int num_rows, int vocab) {
  int slices = (4 * 148 + num_rows - 1) / (num_rows > 0 ? num_rows : 1);
  if (slices > SAMPLE_MAX_SLICES) slices = SAMPLE_MAX_SLICES;
  const int most = (vocab + 1023) / 1024;  // at least about a thousand entries per slice
  if (slices > most) slices = most;
  return slices < 1 ? 1 : slices;
}

extern "C" int sb_sample(const float* logits, const int* params, int* out, int num_rows, int vocab,
                         void* scratch, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  const int slices = sb_sample_slices(num_rows, vocab);
  const int slice_len = ((vocab + slices - 1) / slices + 3) / 4 * 4;
  uint32_t* thresholds = reinterpret_cast<uint32_t*>(scratch);
  ArgMax* partial = reinterpret_cast<ArgMax*>(thresholds + num_rows + (num_rows & 1));
  sb_launch(sample_threshold_kernel, num_rows, SAMPLE_THREADS, 0, stream, logits, params, thresholds,
      vocab);
  SB_LAUNCH_CHECK();
  sb_launch(sample_slice_kernel, dim3(slices, num_rows), SLICE_THREADS, 0, stream, logits, params,
      thresholds, partial, vocab, slice_len);
  SB_LAUNCH_CHECK();
  sb_launch(sample_final_kernel, num_rows, 32, 0, stream, partial, out, slices);
  SB_LAUNCH_CHECK();
  return 0;
}
