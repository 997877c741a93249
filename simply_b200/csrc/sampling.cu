// Sampling from float32 logits, one block per row.
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
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const int* __restrict__ params, int* __restrict__ out,
              int vocab) {
  __shared__ float fscratch[33];
  __shared__ ArgMax ascratch[33];
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const int* p = params + r * 6;
  const float temperature = __int_as_float(p[0]);
  const int top_k = p[1];
  const float top_p = __int_as_float(p[2]);
  const uint32_t seed_lo = (uint32_t)p[3], seed_hi = (uint32_t)p[4];
  const uint32_t position = (uint32_t)p[5];

  if (temperature == 0.f || top_k == 1) {
    ArgMax best{-FLT_MAX, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = better(best, ArgMax{row[i], i});
    best = block_argmax(best, ascratch);
    if (threadIdx.x == 0) out[r] = best.i;
    return;
  }

  uint32_t threshold = 0;  // keep entries whose key >= threshold
  if (top_k > 0 && top_k < vocab) {
    // Largest K with count(key >= K) >= top_k: the key of the k-th largest entry.
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = threshold | (1u << bit);
      float cnt = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) cnt += order_key(row[i] / temperature) >= cand ? 1.f : 0.f;
      cnt = block_sum(cnt, fscratch);
      if (cnt >= (float)top_k) threshold = cand;
    }
  }
  if (top_p < 1.f) {
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

  ArgMax best{-FLT_MAX, 0x7fffffff};
  const int blocks4 = (vocab + 3) / 4;
  for (int blk = threadIdx.x; blk < blocks4; blk += blockDim.x) {
    uint32_t bits[4];
    philox4x32_10((uint32_t)blk, position, 0u, 0u, seed_lo, seed_hi, bits);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = blk * 4 + e;
      if (i >= vocab) break;
      const float s = row[i] / temperature;
      if (order_key(s) < threshold) continue;
      best = better(best, ArgMax{s + gumbel_from_bits(bits[e]), i});
    }
  }
  best = block_argmax(best, ascratch);
  if (threadIdx.x == 0) out[r] = best.i;
}

extern "C" int sb_sample(const float* logits, const int* params, int* out, int num_rows, int vocab,
                         cudaStream_t stream) {
  if (num_rows == 0) return 0;
  sample_kernel<<<num_rows, SAMPLE_THREADS, 0, stream>>>(logits, params, out, vocab);
  SB_LAUNCH_CHECK();
  return 0;
}
