// Row-wise and element-wise kernels: embedding, norms fused with the residual add,
// rotation tables, rotation + query scale + cache write, gated activation.
//
// Formulas (file:line in google-deepmind/simply):
//   embedding            simply/utils/module.py:450-481
//   RMS norm, (1 + w)    simply/model_lib.py:154-178
//   block order          simply/model_lib.py:2659-2708
//   rotation             simply/utils/position_encoding.py:83-110
//   query scale          simply/model_lib.py:2014-2019
//   gated activation     simply/model_lib.py:93-96, 722-726
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: out[t, :] = table[ids[t], :] * scale, float32 out (start of the residual stream).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float scale,
                             float* __restrict__ out, int width, int vocab, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_TOKEN);
    id = 0;
  }
  const T* row = table + (size_t)id * width;
  float* o = out + (size_t)t * width;
  constexpr int N = Vec<T>::N;
  if (width % N == 0) {
    for (int i = threadIdx.x * N; i < width; i += blockDim.x * N) {
      float v[N];
      Vec<T>::load(row + i, v);
#pragma unroll
      for (int k = 0; k < N; ++k) v[k] *= scale;
#pragma unroll
      for (int k = 0; k < N; k += 4) Vec<float>::store(o + i + k, v + k);
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = to_f32<T>(row[i]) * scale;
  }
}

extern "C" int sb_embed(const void* table, int table_dtype, const int* ids, float scale, float* out,
                        int num_tokens, int width, int vocab, int* err, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (table_dtype == SB_DTYPE_F32)
    sb_launch(embed_kernel<float>, num_tokens, 256, 0, stream, (const float*)table, ids, scale, out, width,
        vocab, err);
  else
    sb_launch(embed_kernel<bf16>, num_tokens, 256, 0, stream, (const bf16*)table, ids, scale, out, width,
        vocab, err);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Residual add fused with the norms around it.  One block per row.
//   b   = branch row                      (optional)
//   b   = b * rsqrt(mean(b^2) + eps_post) * (w_post [+ 1])   (if w_post)
//   h  += b                               (written back unless rows are gathered)
//   y   = h * rsqrt(mean(h^2) + eps_pre) * (w_pre [+ 1])     (if w_pre), stored as T
// With `rows`, block r works on row rows[r] and writes y[r]; h is left untouched.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void residual_norm_kernel(float* __restrict__ h, const T* __restrict__ branch,
                                     const void* __restrict__ w_post, int post_f32, float eps_post,
                                     int post_plus_one, const void* __restrict__ w_pre, int pre_f32,
                                     float eps_pre, int pre_plus_one, const int* __restrict__ rows,
                                     T* __restrict__ y, int width, int num_rows_total, int* err) {
  extern __shared__ float row[];  // width floats + 33 scratch
  float* scratch = row + width;
  const int r = blockIdx.x;
  constexpr int N = Vec<T>::N;
  const bool vec = width % N == 0;
  const bool one_chunk = vec && width <= (int)blockDim.x * N;
  // The norm scales are weights, which no kernel writes: they are fetched before the wait for
  // the kernel's inputs.
  float wp[N], wq[N];
#pragma unroll
  for (int k = 0; k < N; ++k) wp[k] = wq[k] = 0.f;
  if (one_chunk && (int)threadIdx.x * N < width) {
    if (branch && w_post) load_scalars<N>(w_post, post_f32, threadIdx.x * N, wp);
    if (w_pre) load_scalars<N>(w_pre, pre_f32, threadIdx.x * N, wq);
  }
  pdl_wait_block();
  pdl_launch_dependents();
  int src = rows ? rows[r] : r;
  if (src < 0 || src >= num_rows_total) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_ROW);
    src = 0;
  }
  float* hp = h + (size_t)src * width;
  const float post_one = post_plus_one ? 1.f : 0.f, pre_one = pre_plus_one ? 1.f : 0.f;
  if (one_chunk) {
    // The row fits one 16-byte chunk per thread: every load is issued before the first sum, so
    // the kernel pays one memory latency instead of one per pass.  Same arithmetic as below.
    const int i = threadIdx.x * N;
    const bool on = i < width;
    float b[N], v[N];
#pragma unroll
    for (int k = 0; k < N; ++k) b[k] = v[k] = 0.f;
    if (on) {
      if (branch) Vec<T>::load(branch + (size_t)src * width + i, b);
#pragma unroll
      for (int k = 0; k < N; k += 4) Vec<float>::load(hp + i + k, v + k);
    }
    if (branch) {
      float rstd_b = 1.f;
      if (w_post) {
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < N; ++k) ss += b[k] * b[k];
        ss = block_sum(ss, scratch);
        rstd_b = 1.0f / sqrtf(ss / (float)width + eps_post);
      }
#pragma unroll
      for (int k = 0; k < N; ++k) {
        float bb = b[k];
        if (w_post) bb = bb * rstd_b * (wp[k] + post_one);
        v[k] += bb;
      }
      if (!rows && on) {
#pragma unroll
        for (int k = 0; k < N; k += 4) Vec<float>::store(hp + i + k, v + k);
      }
    }
    if (w_pre) {
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < N; ++k) ss += v[k] * v[k];
      ss = block_sum(ss, scratch);
      const float rstd = 1.0f / sqrtf(ss / (float)width + eps_pre);
      if (on) {
        float o[N];
#pragma unroll
        for (int k = 0; k < N; ++k) o[k] = v[k] * rstd * (wq[k] + pre_one);
        Vec<T>::store(y + (size_t)r * width + i, o);
      }
    }
    return;
  }
  float rstd_b = 1.f;
  if (branch) {
    const T* bp = branch + (size_t)src * width;
    float ss = 0.f;
    if (vec) {
      for (int i = threadIdx.x * N; i < width; i += blockDim.x * N) {
        float b[N];
        Vec<T>::load(bp + i, b);
#pragma unroll
        for (int k = 0; k < N; ++k) {
          row[i + k] = b[k];
          ss += b[k] * b[k];
        }
      }
    } else {
      for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float b = to_f32<T>(bp[i]);
        row[i] = b;
        ss += b * b;
      }
    }
    if (w_post) {
      ss = block_sum(ss, scratch);
      rstd_b = 1.0f / sqrtf(ss / (float)width + eps_post);
    }
  }
  float ss = 0.f;
  if (vec) {
    for (int i = threadIdx.x * N; i < width; i += blockDim.x * N) {
      float v[N], w[N];
#pragma unroll
      for (int k = 0; k < N; k += 4) Vec<float>::load(hp + i + k, v + k);
      if (branch) {
        if (w_post) load_scalars<N>(w_post, post_f32, i, w);
#pragma unroll
        for (int k = 0; k < N; ++k) {
          float b = row[i + k];
          if (w_post) b = b * rstd_b * (w[k] + post_one);
          v[k] += b;
        }
        if (!rows) {
#pragma unroll
          for (int k = 0; k < N; k += 4) Vec<float>::store(hp + i + k, v + k);
        }
      }
#pragma unroll
      for (int k = 0; k < N; ++k) {
        row[i + k] = v[k];
        ss += v[k] * v[k];
      }
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float v = hp[i];
      if (branch) {
        float b = row[i];
        if (w_post) b = b * rstd_b * (load_scalar(w_post, post_f32, i) + post_one);
        v += b;
        if (!rows) hp[i] = v;
      }
      row[i] = v;
      ss += v * v;
    }
  }
  if (w_pre) {
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)width + eps_pre);
    T* yp = y + (size_t)r * width;
    if (vec) {
      for (int i = threadIdx.x * N; i < width; i += blockDim.x * N) {
        float w[N], o[N];
        load_scalars<N>(w_pre, pre_f32, i, w);
#pragma unroll
        for (int k = 0; k < N; ++k) o[k] = row[i + k] * rstd * (w[k] + pre_one);
        Vec<T>::store(yp + i, o);
      }
    } else {
      for (int i = threadIdx.x; i < width; i += blockDim.x)
        yp[i] = from_f32<T>(row[i] * rstd * (load_scalar(w_pre, pre_f32, i) + pre_one));
    }
  }
}

extern "C" int sb_residual_norm(float* h, const void* branch, int dtype, const void* w_post, int post_f32,
                                float eps_post, int post_plus_one, const void* w_pre, int pre_f32,
                                float eps_pre, int pre_plus_one, const int* rows, void* y, int num_rows,
                                int width, int num_rows_total, int* err, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  const int vec = dtype == SB_DTYPE_F32 ? 4 : 8;
  const size_t smem = (size_t)(width + 33) * sizeof(float);
  if (smem > 200 * 1024) return -2;  // refused: row does not fit shared memory
  // One 16-byte vector per thread where the row allows it: the kernel then issues all its loads
  // at once, and its small blocks fill the SMs whether the step has eight rows or thousands.
  // (One warp per row with the row in registers was tried for steps with many rows and is
  // slower: 170 registers per thread leave an SM too few warps.)
  int threads = width >= 2048 ? 512 : 256;
  if (width % vec == 0 && width / vec <= 1024) threads = ((width / vec + 31) / 32) * 32;
  if (threads < 64) threads = 64;
  if (dtype == SB_DTYPE_F32) {
    auto k = residual_norm_kernel<float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb_launch(k, num_rows, threads, smem, stream, h, (const float*)branch, w_post, post_f32, eps_post,
        post_plus_one, w_pre, pre_f32, eps_pre, pre_plus_one, rows, (float*)y, width, num_rows_total, err);
  } else {
    auto k = residual_norm_kernel<bf16>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb_launch(k, num_rows, threads, smem, stream, h, (const bf16*)branch, w_post, post_f32, eps_post,
        post_plus_one, w_pre, pre_f32, eps_pre, pre_plus_one, rows, (bf16*)y, width, num_rows_total, err);
  }
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Stand-alone RMS norm of rows stored as Tin, result stored as Tout.
// ---------------------------------------------------------------------------
template <typename Tin, typename Tout>
__global__ void rms_norm_kernel(const Tin* __restrict__ x, const void* __restrict__ w, int w_f32, float eps,
                                int plus_one, Tout* __restrict__ y, int width) {
  pdl_wait_block();
  pdl_launch_dependents();
  extern __shared__ float row[];
  float* scratch = row + width;
  const Tin* xp = x + (size_t)blockIdx.x * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = to_f32<Tin>(xp[i]);
    row[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rstd = 1.0f / sqrtf(ss / (float)width + eps);
  Tout* yp = y + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    yp[i] = from_f32<Tout>(row[i] * rstd * (load_scalar(w, w_f32, i) + (plus_one ? 1.f : 0.f)));
}

template <typename Tin, typename Tout>
static int launch_rms_norm(const void* x, const void* w, int w_f32, float eps, int plus_one, void* y,
                           int num_rows, int width, cudaStream_t stream) {
  const size_t smem = (size_t)(width + 33) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  auto k = rms_norm_kernel<Tin, Tout>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  sb_launch(k, num_rows, 256, smem, stream, (const Tin*)x, w, w_f32, eps, plus_one, (Tout*)y, width);
  SB_LAUNCH_CHECK();
  return 0;
}

extern "C" int sb_rms_norm(const void* x, int in_dtype, const void* w, int w_f32, float eps, int plus_one,
                           void* y, int out_dtype, int num_rows, int width, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  if (in_dtype == SB_DTYPE_F32 && out_dtype == SB_DTYPE_F32)
    return launch_rms_norm<float, float>(x, w, w_f32, eps, plus_one, y, num_rows, width, stream);
  if (in_dtype == SB_DTYPE_F32) return launch_rms_norm<float, bf16>(x, w, w_f32, eps, plus_one, y, num_rows, width, stream);
  if (out_dtype == SB_DTYPE_F32) return launch_rms_norm<bf16, float>(x, w, w_f32, eps, plus_one, y, num_rows, width, stream);
  return launch_rms_norm<bf16, bf16>(x, w, w_f32, eps, plus_one, y, num_rows, width, stream);
}

// ---------------------------------------------------------------------------
// Small helpers for norms the fused kernel does not know.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ rows, T* __restrict__ out,
                                   int width, int num_rows_total, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  int src = rows[blockIdx.x];
  if (src < 0 || src >= num_rows_total) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_ROW);
    src = 0;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    out[(size_t)blockIdx.x * width + i] = x[(size_t)src * width + i];
}

extern "C" int sb_gather_rows(const void* x, int dtype, const int* rows, void* out, int num_rows, int width,
                              int num_rows_total, int* err, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  if (dtype == SB_DTYPE_F32)
    sb_launch(gather_rows_kernel<float>, num_rows, 256, 0, stream, (const float*)x, rows, (float*)out,
        width, num_rows_total, err);
  else
    sb_launch(gather_rows_kernel<bf16>, num_rows, 256, 0, stream, (const bf16*)x, rows, (bf16*)out, width,
        num_rows_total, err);
  SB_LAUNCH_CHECK();
  return 0;
}

template <typename T>
__global__ void add_to_residual_kernel(float* __restrict__ h, const T* __restrict__ x, size_t n) {
  pdl_wait_block();
  pdl_launch_dependents();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) h[i] += to_f32<T>(x[i]);
}

extern "C" int sb_add_to_residual(float* h, const void* x, int dtype, long long n, cudaStream_t stream) {
  if (n == 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == SB_DTYPE_F32)
    sb_launch(add_to_residual_kernel<float>, blocks, 256, 0, stream, h, (const float*)x, (size_t)n);
  else
    sb_launch(add_to_residual_kernel<bf16>, blocks, 256, 0, stream, h, (const bf16*)x, (size_t)n);
  SB_LAUNCH_CHECK();
  return 0;
}

template <typename Tin, typename Tout>
__global__ void cast_kernel(const Tin* __restrict__ x, Tout* __restrict__ y, size_t n) {
  pdl_wait_block();
  pdl_launch_dependents();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = from_f32<Tout>(to_f32<Tin>(x[i]));
}

extern "C" int sb_cast(const void* x, int in_dtype, void* y, int out_dtype, long long n, cudaStream_t stream) {
  if (n == 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (in_dtype == SB_DTYPE_F32 && out_dtype == SB_DTYPE_BF16)
    sb_launch(cast_kernel<float, bf16>, blocks, 256, 0, stream, (const float*)x, (bf16*)y, (size_t)n);
  else if (in_dtype == SB_DTYPE_BF16 && out_dtype == SB_DTYPE_F32)
    sb_launch(cast_kernel<bf16, float>, blocks, 256, 0, stream, (const bf16*)x, (float*)y, (size_t)n);
  else
    return -3;
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Rotation tables for the step's tokens: angle = position / timescale / scale_factor,
// all float32, as the reference computes it; cos and sin are [T, half].
// ---------------------------------------------------------------------------
__global__ void rotation_tables_kernel(const int* __restrict__ positions, const float* __restrict__ timescale,
                                       float scale_factor, float* __restrict__ cos_out,
                                       float* __restrict__ sin_out, int num_tokens, int half) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= num_tokens * half) return;
  const int t = i / half, j = i - t * half;
  const float angle = (float)positions[t] / timescale[j] / scale_factor;
  float s, c;
  sincosf(angle, &s, &c);
  cos_out[i] = c;
  sin_out[i] = s;
}

extern "C" int sb_rotation_tables(const int* positions, const float* timescale, float scale_factor,
                                  float* cos_out, float* sin_out, int num_tokens, int half,
                                  cudaStream_t stream) {
  const int n = num_tokens * half;
  if (n == 0) return 0;
  sb_launch(rotation_tables_kernel, (n + 255) / 256, 256, 0, stream, positions, timescale, scale_factor,
      cos_out, sin_out, num_tokens, half);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// From the fused projection qkv [T, (Hq + 2 Hkv) * dh]:
//   q_out[t, n, :] = rotate(q) * q_scale
//   cache[page, 0, m, offset, :] = rotate(k);  cache[page, 1, m, offset, :] = v
// with page = block_table[seq(t), pos / page_size], offset = pos % page_size.
// The halves of a head rotate together: (a, b) -> (a cos - b sin, b cos + a sin).
// cos/sin may be null (no rotation).  Hkv_proj = 0: the projection holds q only.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rope_cache_write_kernel(const T* __restrict__ qkv, const float* __restrict__ cos_t,
                                        const float* __restrict__ sin_t, float q_scale, T* __restrict__ q_out,
                                        T* __restrict__ cache, const int* __restrict__ block_table,
                                        int max_pages, const int* __restrict__ token_seq,
                                        const int* __restrict__ positions, int num_q_heads, int num_kv_proj,
                                        int head_dim, int page_size, int num_pages, int write_cache, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int half = head_dim / 2;
  const int heads = num_q_heads + 2 * num_kv_proj;
  const T* in = qkv + (size_t)t * heads * head_dim;
  const int pos = positions[t];
  long long page = -1;
  int offset = 0;
  if (write_cache && num_kv_proj > 0) {
    page = block_table[(size_t)token_seq[t] * max_pages + pos / page_size];
    offset = pos % page_size;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_PAGE);
      page = -1;
    }
  }
  constexpr int N = Vec<T>::N;
  if (half % N == 0) {
    // N pairs (j, j + half) per thread and turn, 16-byte loads and stores.
    const int chunks = half / N;
    for (int i = threadIdx.x; i < heads * chunks; i += blockDim.x) {
      const int hh = i / chunks, j = (i - hh * chunks) * N;
      float a[N], b[N];
      Vec<T>::load(in + hh * head_dim + j, a);
      Vec<T>::load(in + hh * head_dim + half + j, b);
      if (hh < num_q_heads + num_kv_proj && cos_t) {
        float c[N], sn[N];
#pragma unroll
        for (int k = 0; k < N; k += 4) {
          Vec<float>::load(cos_t + (size_t)t * half + j + k, c + k);
          Vec<float>::load(sin_t + (size_t)t * half + j + k, sn + k);
        }
#pragma unroll
        for (int k = 0; k < N; ++k) {
          const float ra = a[k] * c[k] - b[k] * sn[k], rb = b[k] * c[k] + a[k] * sn[k];
          a[k] = ra;
          b[k] = rb;
        }
      }
      if (hh < num_q_heads) {
#pragma unroll
        for (int k = 0; k < N; ++k) {
          a[k] *= q_scale;
          b[k] *= q_scale;
        }
        T* o = q_out + ((size_t)t * num_q_heads + hh) * head_dim;
        Vec<T>::store(o + j, a);
        Vec<T>::store(o + half + j, b);
      } else if (page >= 0) {
        const int kv = hh < num_q_heads + num_kv_proj ? 0 : 1;
        const int m = hh - num_q_heads - kv * num_kv_proj;
        T* o = cache + ((((size_t)page * 2 + kv) * num_kv_proj + m) * page_size + offset) * head_dim;
        Vec<T>::store(o + j, a);
        Vec<T>::store(o + half + j, b);
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
    const int hh = i / half, j = i - hh * half;
    float a = to_f32<T>(in[hh * head_dim + j]);
    float b = to_f32<T>(in[hh * head_dim + half + j]);
    if (hh < num_q_heads + num_kv_proj && cos_t) {
      const float c = cos_t[(size_t)t * half + j], s = sin_t[(size_t)t * half + j];
      const float ra = a * c - b * s, rb = b * c + a * s;
      a = ra;
      b = rb;
    }
    if (hh < num_q_heads) {
      T* o = q_out + ((size_t)t * num_q_heads + hh) * head_dim;
      o[j] = from_f32<T>(a * q_scale);
      o[half + j] = from_f32<T>(b * q_scale);
    } else if (page >= 0) {
      const int kv = hh < num_q_heads + num_kv_proj ? 0 : 1;
      const int m = hh - num_q_heads - kv * num_kv_proj;
      T* o = cache + ((((size_t)page * 2 + kv) * num_kv_proj + m) * page_size + offset) * head_dim;
      o[j] = from_f32<T>(a);
      o[half + j] = from_f32<T>(b);
    }
  }
}

extern "C" int sb_rope_cache_write(const void* qkv, int dtype, const float* cos_t, const float* sin_t,
                                   float q_scale, void* q_out, void* cache, const int* block_table,
                                   int max_pages, const int* token_seq, const int* positions, int num_tokens,
                                   int num_q_heads, int num_kv_proj, int head_dim, int page_size,
                                   int num_pages, int write_cache, int* err, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (head_dim % 2) return -4;
  if (dtype == SB_DTYPE_F32)
    sb_launch(rope_cache_write_kernel<float>, num_tokens, 256, 0, stream, (const float*)qkv, cos_t, sin_t,
        q_scale, (float*)q_out, (float*)cache, block_table, max_pages, token_seq, positions, num_q_heads,
        num_kv_proj, head_dim, page_size, num_pages, write_cache, err);
  else
    sb_launch(rope_cache_write_kernel<bf16>, num_tokens, 256, 0, stream, (const bf16*)qkv, cos_t, sin_t,
        q_scale, (bf16*)q_out, (bf16*)cache, block_table, max_pages, token_seq, positions, num_q_heads,
        num_kv_proj, head_dim, page_size, num_pages, write_cache, err);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Gated activation: z[t, f] = act(gate_up[t, f]) * gate_up[t, F + f].
//   act 0: gelu, tanh form; 1: silu; 2: relu.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float apply_activation(float g, int act) {
  if (act == 0) {
    const float c = 0.7978845608028654f;  // sqrt(2 / pi)
    return 0.5f * g * (1.0f + tanhf(c * (g + 0.044715f * g * g * g)));
  }
  if (act == 1) return g / (1.0f + expf(-g));
  return fmaxf(g, 0.f);
}

// The bfloat16 path's gelu: 0.5 g (1 + tanh y) = g / (1 + exp(-2 y)), with the fast exponential
// and division (relative error about 1e-6, far below the rounding of the bfloat16 result).  With
// the accurate tanh the kernel is bound by instructions, not by memory.
template <typename T, int ACT>
__device__ __forceinline__ float gated_value(float g, float u) {
  if (ACT == 0 && sizeof(T) == 2) {
    const float c2 = 2.0f * 0.7978845608028654f;
    const float y2 = c2 * (g + 0.044715f * g * g * g);
    return __fdividef(g, 1.0f + __expf(-y2)) * u;
  }
  return apply_activation(g, ACT) * u;
}

// One block row per token (blockIdx.y), so that no thread divides.
template <typename T, int ACT>
__global__ void __launch_bounds__(256)
gated_activation_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ z, int hidden) {
  pdl_wait_block();
  pdl_launch_dependents();
  constexpr int N = Vec<T>::N;
  const int f = (blockIdx.x * blockDim.x + threadIdx.x) * N;
  if (f >= hidden) return;
  const T* row = gate_up + (size_t)blockIdx.y * 2 * hidden;
  float g[N], u[N];
  Vec<T>::load(row + f, g);
  Vec<T>::load(row + hidden + f, u);
#pragma unroll
  for (int k = 0; k < N; ++k) g[k] = gated_value<T, ACT>(g[k], u[k]);
  Vec<T>::store(z + (size_t)blockIdx.y * hidden + f, g);
}

template <typename T>
static void launch_gated_vec(const T* gate_up, T* z, int num_tokens, int hidden, int act, cudaStream_t stream) {
  constexpr int N = Vec<T>::N;
  // (grid.y holds at most 65535 rows: larger steps go in slabs.)
  for (int t0 = 0; t0 < num_tokens; t0 += 65535) {
    const dim3 grid((unsigned)((hidden / N + 255) / 256), (unsigned)min(65535, num_tokens - t0));
    const T* in = gate_up + (size_t)t0 * 2 * hidden;
    T* out = z + (size_t)t0 * hidden;
    if (act == 0) sb_launch(gated_activation_vec_kernel<T, 0>, grid, 256, 0, stream, in, out, hidden);
    else if (act == 1) sb_launch(gated_activation_vec_kernel<T, 1>, grid, 256, 0, stream, in, out, hidden);
    else sb_launch(gated_activation_vec_kernel<T, 2>, grid, 256, 0, stream, in, out, hidden);
  }
}

template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ gate_up, T* __restrict__ z, int hidden, int act,
                                        size_t n) {
  pdl_wait_block();
  pdl_launch_dependents();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t t = i / hidden, f = i - t * hidden;
  const float g = to_f32<T>(gate_up[t * 2 * hidden + f]);
  const float u = to_f32<T>(gate_up[t * 2 * hidden + hidden + f]);
  z[i] = from_f32<T>(apply_activation(g, act) * u);
}

extern "C" int sb_gated_activation(const void* gate_up, int dtype, void* z, int num_tokens, int hidden, int act,
                                   cudaStream_t stream) {
  const size_t n = (size_t)num_tokens * hidden;
  if (n == 0) return 0;
  if (act < 0 || act > 2) return -5;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == SB_DTYPE_F32) {
    if (hidden % 4 == 0)
      launch_gated_vec<float>((const float*)gate_up, (float*)z, num_tokens, hidden, act, stream);
    else
      sb_launch(gated_activation_kernel<float>, blocks, 256, 0, stream, (const float*)gate_up, (float*)z,
          hidden, act, n);
  } else {
    if (hidden % 8 == 0)
      launch_gated_vec<bf16>((const bf16*)gate_up, (bf16*)z, num_tokens, hidden, act, stream);
    else
      sb_launch(gated_activation_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)gate_up, (bf16*)z,
          hidden, act, n);
  }
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Soft cap in place on float32 logits: x = cap * tanh(x / cap).  simply/model_lib.py:107-109.
// ---------------------------------------------------------------------------
// (The logits of the bfloat16 path's library product: tanh y = 1 - 2 / (exp(2y) + 1) through the
// fast exponential, absolute error about 1e-7 of a value in [-1, 1]; with the accurate tanhf and
// one value per thread the pass was bound by instructions at a third of the memory bandwidth.)
__device__ __forceinline__ float soft_cap_value(float v, float cap, float two_over_cap) {
  return cap * (1.0f - __fdividef(2.0f, __expf(v * two_over_cap) + 1.0f));
}

__global__ void soft_cap_kernel(float* __restrict__ x, float cap, size_t n) {
  pdl_wait_block();
  pdl_launch_dependents();
  const float two_over_cap = 2.0f / cap;
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 4 <= n) {
    float4 v = *reinterpret_cast<const float4*>(x + i);
    v.x = soft_cap_value(v.x, cap, two_over_cap);
    v.y = soft_cap_value(v.y, cap, two_over_cap);
    v.z = soft_cap_value(v.z, cap, two_over_cap);
    v.w = soft_cap_value(v.w, cap, two_over_cap);
    *reinterpret_cast<float4*>(x + i) = v;
  } else {
    for (size_t j = i; j < n; ++j) x[j] = soft_cap_value(x[j], cap, two_over_cap);
  }
}

// x must be 16-byte aligned (a whole tensor is).
extern "C" int sb_soft_cap(float* x, float cap, long long n, cudaStream_t stream) {
  if (n == 0 || cap <= 0.f) return 0;
  if (reinterpret_cast<uintptr_t>(x) % 16 != 0) return -4;
  sb_launch(soft_cap_kernel, (unsigned)(((n + 3) / 4 + 255) / 256), 256, 0, stream, x, cap, (size_t)n);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Between two decode steps that run without the host in between (the reference's
// on-device decode loop, simply/utils/ragged_paged_attention.py:2064-2102): the
// sampled token becomes the next input, every position moves on by one, and the
// token is recorded in history[step, :].
//   sample_params: [B, 6] int32 words, word 5 is the position of the token to sample.
// ---------------------------------------------------------------------------
__global__ void decode_advance_kernel(const int* __restrict__ sampled, int* __restrict__ token_ids,
                                      int* __restrict__ positions, int* __restrict__ q_start,
                                      int* __restrict__ sample_params, int* __restrict__ history,
                                      int* __restrict__ step_counter, int batch) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int step = *step_counter;
  if (i < batch) {
    const int tok = sampled[i];
    history[(size_t)step * batch + i] = tok;
    token_ids[i] = tok;
    positions[i] += 1;
    q_start[i] += 1;
    sample_params[i * 6 + 5] += 1;
  }
  __syncthreads();  // launched as a single block: every thread has read the counter by now
  if (threadIdx.x == 0) *step_counter = step + 1;
}

extern "C" int sb_decode_advance(const int* sampled, int* token_ids, int* positions, int* q_start,
                                 int* sample_params, int* history, int* step_counter, int batch,
                                 cudaStream_t stream) {
  if (batch <= 0 || batch > 1024) return -10;  // one block of 1024 threads covers the batch
  sb_launch(decode_advance_kernel, 1, 1024, 0, stream, sampled, token_ids, positions, q_start,
      sample_params, history, step_counter, batch);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Keeps the logits of one decode step of a burst: history[step, :] = logits, with `step` read
// from the burst's device-side counter (launched before decode_advance moves the counter on).
// Only used when the decode runner is asked to keep logits, so that tests can compare the rows a
// CUDA-graph replay produced with a plain model's.
// ---------------------------------------------------------------------------
__global__ void keep_logits_kernel(const float* __restrict__ logits, float* __restrict__ history,
                                   const int* __restrict__ step_counter, size_t n) {
  pdl_wait_block();
  pdl_launch_dependents();
  const size_t step = (size_t)*step_counter;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) history[step * n + i] = logits[i];
}

extern "C" int sb_keep_logits(const float* logits, float* history, const int* step_counter, long long n,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  sb_launch(keep_logits_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, logits, history, step_counter,
            (size_t)n);
  SB_LAUNCH_CHECK();
  return 0;
}
