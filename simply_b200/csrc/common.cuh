// Shared device helpers: storage types, conversions, reductions, error word.
//
// Every kernel computes in float32.  "T" is the storage type of activations and
// of the cache: float (the true 32-bit path) or __nv_bfloat16 (serving).  Vectors
// such as norm scales may be stored in either type whatever T is, so they come
// as an untyped pointer with a flag.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

#define SB_DTYPE_F32 0
#define SB_DTYPE_BF16 1

// Bits of the device-side error word (set, never trapped on).
#define SB_ERR_BAD_PAGE 1   // a block-table entry < 0 or >= num_pages was about to be followed
#define SB_ERR_BAD_TOKEN 2  // a token id outside the table
#define SB_ERR_BAD_ROW 4    // a gather row outside the batch

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float load_scalar(const void* p, int is_f32, int i) {
  return is_f32 ? reinterpret_cast<const float*>(p)[i]
                : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}

// 16-byte vectors of storage type T: 4 floats or 8 bfloat16, loaded to / stored from float registers.
template <typename T> struct Vec;
template <> struct Vec<float> {
  static constexpr int N = 4;
  __device__ __forceinline__ static void load(const float* p, float* out) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  }
  __device__ __forceinline__ static void store(float* p, const float* in) {
    *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
  }
};
template <> struct Vec<bf16> {
  static constexpr int N = 8;
  __device__ __forceinline__ static void load(const bf16* p, float* out) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      out[2 * i] = __uint_as_float(w[i] << 16);
      out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ static void store(bf16* p, const float* in) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// N consecutive scalars of a vector stored as float32 or bfloat16 (N = 4 or 8, i a multiple of N).
template <int N>
__device__ __forceinline__ void load_scalars(const void* p, int is_f32, int i, float* out) {
  if (is_f32) {
#pragma unroll
    for (int k = 0; k < N; k += 4) Vec<float>::load(reinterpret_cast<const float*>(p) + i + k, out + k);
  } else if (N == 8) {
    Vec<bf16>::load(reinterpret_cast<const bf16*>(p) + i, out);
  } else {
    const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(p) + i);
    out[0] = __uint_as_float(v.x << 16); out[1] = __uint_as_float(v.x & 0xffff0000u);
    out[2] = __uint_as_float(v.y << 16); out[3] = __uint_as_float(v.y & 0xffff0000u);
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block in a fixed order; every thread gets the result.  `scratch`
// holds at least 33 floats of shared memory.  blockDim.x is a multiple of 32.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Programmatic dependent launch.  Every kernel of the engine begins with
// `pdl_wait(); pdl_launch_dependents();` (or does work that depends on nothing written by
// earlier kernels, such as fetching weights, before the two).  The wait blocks until every
// earlier kernel has finished and its writes are visible; the trigger lets the next kernel of
// the stream start once all blocks of this one have passed it.  Trigger after wait: at most
// two kernels then overlap (this one, and the next up to its own wait).  Triggering before the
// wait lets a whole chain of kernels pile up on the device ahead of time, which was measured to
// slow a decode step by a fifth.  Launched without the attribute both are no-ops, so a kernel
// is always correct on its own.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// The same for a whole block, at a point all its threads reach: one thread waits, the others
// stand at the block's barrier.  (Thousands of threads each waiting out a long kernel before
// them slowed that kernel down: a norm of 8 rows, launched early behind a 60 us product, cost
// 50 us; with one waiting thread per block it costs nothing.)
__device__ __forceinline__ void pdl_wait_block() {
  if (threadIdx.x == 0) pdl_wait();
  __syncthreads();
}

#include <stdlib.h>

// SIMPLY_B200_PDL in the environment: 0 launches every kernel the plain way, 1 (the default)
// lets every kernel start early, 2 only those that have something to do before their inputs are
// ready (the weight-streaming products, attention over older keys).
inline int sb_pdl_level() {
  static int level = -1;
  if (level < 0) {
    const char* e = getenv("SIMPLY_B200_PDL");
    level = (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 1;
  }
  return level;
}

template <typename... KArgs, typename... Args>
inline cudaError_t sb_launch_level(int min_level, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                   cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  const int level = sb_pdl_level();
  config.numAttrs = (level == 1 || (level == 2 && min_level == 2)) ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

// A kernel that gains nothing from starting early.
template <typename... KArgs, typename... Args>
inline cudaError_t sb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
  return sb_launch_level(1, kernel, grid, block, smem, stream, args...);
}

// A kernel that fetches data no earlier kernel writes (weights) before it waits for its inputs.
template <typename... KArgs, typename... Args>
inline cudaError_t sb_launch_early(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                   cudaStream_t stream, Args... args) {
  return sb_launch_level(2, kernel, grid, block, smem, stream, args...);
}

#define SB_LAUNCH_CHECK()                      \
  do {                                         \
    cudaError_t e__ = cudaGetLastError();      \
    if (e__ != cudaSuccess) return (int)e__;   \
  } while (0)
