// Ragged paged attention, general form: any head size, page size, grouping and
// storage type.  One warp per (token, query head); keys are visited in tiles of
// 32 that start at a multiple of 32 of the absolute key position, so a token's
// result is the same whatever else the step holds.
//
//   s = q . k                 (q is already rotated and scaled)
//   s = cap * tanh(s / cap)   if cap > 0          simply/model_lib.py:621-626
//   keep k_pos <= q_pos and, with a window W, q_pos - k_pos < W
//                                                 simply/model_lib.py:469-515
//   p = softmax(s) in float32, o = p . v          simply/model_lib.py:633-637
//   query head n reads kv head n / (Hq / Hkv)     simply/model_lib.py:2306-2310
//
// This is the true 32-bit path's attention and the fallback of the bfloat16
// path for shapes its tensor-core kernels refuse.
#include <float.h>

#include "common.cuh"

#define GEN_WARPS 4
#define GEN_MAX_DPL 16  // dims per lane: head_dim <= 512

template <typename T> struct Vec16;  // 16-byte vector loads of storage type T
template <> struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* out) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  }
};
template <> struct Vec16<bf16> {
  static constexpr int N = 8;
  __device__ static void load(const bf16* p, float* out) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      out[2 * i] = __uint_as_float(w[i] << 16);
      out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

template <typename T>
__global__ void __launch_bounds__(GEN_WARPS * 32)
paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ cache,
                               const int* __restrict__ block_table, int max_pages,
                               const int* __restrict__ token_seq, const int* __restrict__ positions,
                               T* __restrict__ out, int num_tokens, int num_q_heads, int num_kv_heads,
                               int head_dim, int page_size, int num_pages, float cap, int window,
                               int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  extern __shared__ float smem[];  // per warp: head_dim floats of q
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long item = (long long)blockIdx.x * GEN_WARPS + warp;
  if (item >= (long long)num_tokens * num_q_heads) return;
  const int t = (int)(item / num_q_heads), n = (int)(item % num_q_heads);
  const int m = n / (num_q_heads / num_kv_heads);
  const int b = token_seq[t], pos = positions[t];
  float* qs = smem + warp * head_dim;
  const T* qp = q + ((size_t)t * num_q_heads + n) * head_dim;
  for (int d = lane; d < head_dim; d += 32) qs[d] = to_f32<T>(qp[d]);
  __syncwarp();

  const int lo = window > 0 ? max(pos - window + 1, 0) : 0;
  const float NEG = -0.5f * FLT_MAX;  // the reference's mask value, simply/utils/common.py:543-551
  float m_run = NEG, l_run = 0.f;
  float acc[GEN_MAX_DPL];
#pragma unroll
  for (int i = 0; i < GEN_MAX_DPL; ++i) acc[i] = 0.f;
  const size_t head_stride = (size_t)page_size * head_dim;
  const size_t kv_stride = (size_t)num_kv_heads * head_stride;
  constexpr int VN = Vec16<T>::N;

  for (int tile = (lo / 32) * 32; tile <= pos; tile += 32) {
    const int j = tile + lane;
    bool valid = j >= lo && j <= pos;
    long long page = -1;
    if (valid) {
      page = block_table[(size_t)b * max_pages + j / page_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(err, SB_ERR_BAD_PAGE);
        valid = false;
      }
    }
    const int off = j % page_size;
    float s = NEG;
    if (valid) {
      const T* kr = cache + ((size_t)page * 2) * kv_stride + m * head_stride + (size_t)off * head_dim;
      float dot = 0.f;
      int d = 0;
      if ((head_dim % VN) == 0) {
        for (; d < head_dim; d += VN) {
          float kf[VN];
          Vec16<T>::load(kr + d, kf);
#pragma unroll
          for (int e = 0; e < VN; ++e) dot = fmaf(qs[d + e], kf[e], dot);
        }
      } else {
        for (; d < head_dim; ++d) dot = fmaf(qs[d], to_f32<T>(kr[d]), dot);
      }
      s = cap > 0.f ? cap * tanhf(dot / cap) : dot;
    }
    const float m_new = fmaxf(m_run, warp_max(s));
    const float alpha = expf(m_run - m_new);
    const float p = valid ? expf(s - m_new) : 0.f;
    l_run = l_run * alpha + warp_sum(p);
    m_run = m_new;
#pragma unroll
    for (int i = 0; i < GEN_MAX_DPL; ++i) acc[i] *= alpha;
    const unsigned valid_mask = __ballot_sync(0xffffffffu, valid);
    for (int jj = 0; jj < 32; ++jj) {
      if (!((valid_mask >> jj) & 1u)) continue;  // uniform over the warp
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long pgj = __shfl_sync(0xffffffffu, page, jj);
      const int offj = (tile + jj) % page_size;
      const T* vr = cache + ((size_t)pgj * 2 + 1) * kv_stride + m * head_stride + (size_t)offj * head_dim;
#pragma unroll
      for (int i = 0; i < GEN_MAX_DPL; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) acc[i] = fmaf(pj, to_f32<T>(vr[d]), acc[i]);
      }
    }
  }
  T* op = out + ((size_t)t * num_q_heads + n) * head_dim;
  const float inv = 1.0f / l_run;
#pragma unroll
  for (int i = 0; i < GEN_MAX_DPL; ++i) {
    const int d = lane + 32 * i;
    if (d < head_dim) op[d] = from_f32<T>(acc[i] * inv);
  }
}

extern "C" int sb_paged_attention_generic(const void* q, int dtype, const void* cache, const int* block_table,
                                          int max_pages, const int* token_seq, const int* positions,
                                          void* out, int num_tokens, int num_q_heads, int num_kv_heads,
                                          int head_dim, int page_size, int num_pages, float cap, int window,
                                          int* err, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (head_dim <= 0 || head_dim > 32 * GEN_MAX_DPL) return -7;
  if (num_kv_heads <= 0 || num_q_heads % num_kv_heads) return -8;
  const long long items = (long long)num_tokens * num_q_heads;
  const unsigned blocks = (unsigned)((items + GEN_WARPS - 1) / GEN_WARPS);
  const size_t smem = (size_t)GEN_WARPS * head_dim * sizeof(float);
  if (dtype == SB_DTYPE_F32)
    sb_launch(paged_attention_generic_kernel<float>, blocks, GEN_WARPS * 32, smem, stream, (const float*)q,
        (const float*)cache, block_table, max_pages, token_seq, positions, (float*)out, num_tokens,
        num_q_heads, num_kv_heads, head_dim, page_size, num_pages, cap, window, err);
  else
    sb_launch(paged_attention_generic_kernel<bf16>, blocks, GEN_WARPS * 32, smem, stream, (const bf16*)q,
        (const bf16*)cache, block_table, max_pages, token_seq, positions, (bf16*)out, num_tokens,
        num_q_heads, num_kv_heads, head_dim, page_size, num_pages, cap, window, err);
  SB_LAUNCH_CHECK();
  return 0;
}
