// Weight-streaming matrix product for a handful of tokens (decode steps):
//   out[M, N] = x[M, K] . w[N, K]^T,  bfloat16 in, float32 accumulate, M <= 32
// (the kernel table sends the products of steps of up to 16 tokens here, and the output layer's
// rows in chunks of up to 32).
//
// With so few rows the product is bound by reading w once from HBM, so the kernel
// is built around that stream.  The weight matrix is the 16-row operand of
// mma.m16n8k16 and the tokens are the 8-column operand ("swapped"), both loaded
// straight from global memory into registers with 16-byte loads.  The sum over K
// does not care about order, so lane (g, t) of a warp takes the 8 consecutive k
// values [32 s + 8 t, 32 s + 8 t + 8) of step s for weight rows g and g + 8 and
// for token g, and feeds them to two mma's; no shared-memory staging or
// transposition is needed.  A block owns 16 weight rows; its warps split K and
// add their partial sums through shared memory in a fixed order.
//
// Epilogues: 0 store as bfloat16; 1 store float32 with an optional soft cap
// (simply/model_lib.py:107-109, the output layer); 2 gated activation: the block
// also owns rows [N/2 + n0, N/2 + n0 + 16) and stores act(gate) * up
// (simply/model_lib.py:722-726); 3 the fused q, k, v projection of an attention layer: a block
// owns 16 dims of a head and the 16 dims half a head further, rotates the pairs
// (simply/utils/position_encoding.py:83-110), scales the query (simply/model_lib.py:2014-2019)
// and stores queries to their buffer, keys and values into the pages of the cache.
#include "common.cuh"

// What epilogue 3 needs besides the product.  cos_t / sin_t: [M, head_dim / 2] float32 or null.
struct RopeStore {
  const float* cos_t;
  const float* sin_t;
  float q_scale;
  bf16* q_out;   // [M, num_q_heads, head_dim]
  bf16* cache;   // [pages, 2, num_kv_proj, page_size, head_dim] or null
  const int* block_table;
  int max_pages;
  const int* token_seq;
  const int* positions;
  int num_q_heads, num_kv_proj, head_dim, page_size, num_pages;
  int* err;
};

__device__ __forceinline__ float skinny_activation(float g, int act) {
  if (act == 0) {
    const float c = 0.7978845608028654f;
    return 0.5f * g * (1.0f + tanhf(c * (g + 0.044715f * g * g * g)));
  }
  if (act == 1) return g / (1.0f + expf(-g));
  return fmaxf(g, 0.f);
}

__device__ __forceinline__ void mma_bf16_16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_stream16(const bf16* p) {
  return __ldcs(reinterpret_cast<const uint4*>(p));
}

// MT: token tiles of 8.  WARPS: warps per block (split of K).  EPI: epilogue.
template <int MT, int WARPS, int EPI>
__global__ void __launch_bounds__(WARPS * 32)
skinny_gemm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, void* __restrict__ out, int M,
                   int N, int K, float cap, int act, const RopeStore rs) {
  constexpr int SETS = EPI >= 2 ? 2 : 1;
  __shared__ float partial[WARPS][SETS][MT][16][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n_out = EPI == 2 ? N / 2 : N;  // rows a block set ranges over
  // Epilogue 3: block (head, slice) owns rows head * head_dim + 16 * slice + [0, 16) and the rows
  // half a head further; the others: rows 16 * block + [0, 16) (and those N / 2 further).
  const int half = EPI == 3 ? rs.head_dim / 2 : 0;
  const int slices = EPI == 3 ? half / 16 : 1;
  const int head = EPI == 3 ? blockIdx.x / slices : 0;
  const int n0 = EPI == 3 ? head * rs.head_dim + (blockIdx.x - head * slices) * 16 : blockIdx.x * 16;
  const int set_stride = EPI == 3 ? half : n_out;
  // Rows past the end are clamped for loading and dropped when storing.
  const bf16* wr[SETS][2];
#pragma unroll
  for (int s = 0; s < SETS; ++s) {
    wr[s][0] = w + (size_t)min(s * set_stride + n0 + g, N - 1) * K;
    wr[s][1] = w + (size_t)min(s * set_stride + n0 + g + 8, N - 1) * K;
  }
  const bf16* xr[MT];
  bool xok[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    xok[mt] = mt * 8 + g < M;
    xr[mt] = x + (size_t)min(mt * 8 + g, M - 1) * K;
  }
  float acc[SETS][MT][4];
#pragma unroll
  for (int s = 0; s < SETS; ++s)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[s][mt][i] = 0.f;

  const int steps = (K + 31) / 32;
  constexpr int UNROLL = SETS == 2 ? 2 : 4;
  constexpr int STRIDE = WARPS * UNROLL;
  // Weights do not depend on earlier kernels: the first batch is fetched before the wait, so
  // the stream of weights starts while the kernel before this one still runs.
  uint4 wa[UNROLL][SETS][2];
  auto load_weights = [&](uint4 (&dst)[UNROLL][SETS][2], int s0) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (s0 + u * WARPS) * 32 + t * 8;
      const bool ok = k < K;  // K is a multiple of 8, so a chunk is whole or absent
#pragma unroll
      for (int s = 0; s < SETS; ++s) {
        dst[u][s][0] = ok ? load_stream16(wr[s][0] + k) : make_uint4(0, 0, 0, 0);
        dst[u][s][1] = ok ? load_stream16(wr[s][1] + k) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  load_weights(wa, warp);
  pdl_wait_block();
  pdl_launch_dependents();
  for (int s0 = warp; s0 < steps; s0 += STRIDE) {
    uint4 xv[UNROLL][MT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (s0 + u * WARPS) * 32 + t * 8;
      const bool ok = k < K;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
        xv[u][mt] = (ok && xok[mt]) ? __ldg(reinterpret_cast<const uint4*>(xr[mt] + k)) : make_uint4(0, 0, 0, 0);
    }
    uint4 wn[UNROLL][SETS][2];  // the next batch is in flight while this one is multiplied
    if (s0 + STRIDE < steps) load_weights(wn, s0 + STRIDE);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_bf16_16816(acc[s][mt], wa[u][s][0].x, wa[u][s][1].x, wa[u][s][0].y, wa[u][s][1].y, xv[u][mt].x,
                         xv[u][mt].y);
          mma_bf16_16816(acc[s][mt], wa[u][s][0].z, wa[u][s][1].z, wa[u][s][0].w, wa[u][s][1].w, xv[u][mt].z,
                         xv[u][mt].w);
        }
    if (s0 + STRIDE < steps) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
#pragma unroll
        for (int s = 0; s < SETS; ++s) {
          wa[u][s][0] = wn[u][s][0];
          wa[u][s][1] = wn[u][s][1];
        }
    }
  }
  // acc[..][0,1]: weight row g, tokens 2t, 2t+1; acc[..][2,3]: weight row g + 8.
#pragma unroll
  for (int s = 0; s < SETS; ++s)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      partial[warp][s][mt][g][2 * t] = acc[s][mt][0];
      partial[warp][s][mt][g][2 * t + 1] = acc[s][mt][1];
      partial[warp][s][mt][g + 8][2 * t] = acc[s][mt][2];
      partial[warp][s][mt][g + 8][2 * t + 1] = acc[s][mt][3];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < MT * 16 * 8; i += WARPS * 32) {
    // Consecutive threads take consecutive weight rows: consecutive addresses of `out`.
    const int row = i % 16, tok8 = (i / 16) % 8, mt = i / 128;
    const int token = mt * 8 + tok8, n = n0 + row;
    if (token >= M || n >= n_out) continue;
    float v[SETS];
#pragma unroll
    for (int s = 0; s < SETS; ++s) {
      float sum = 0.f;
#pragma unroll
      for (int wi = 0; wi < WARPS; ++wi) sum += partial[wi][s][mt][row][tok8];
      v[s] = sum;
    }
    const size_t o = (size_t)token * n_out + n;
    if (EPI == 3) {
      // Round to bfloat16 first, as the unfused path stores the projection before it rotates.
      float a = __bfloat162float(__float2bfloat16_rn(v[0]));
      float b = __bfloat162float(__float2bfloat16_rn(v[SETS - 1]));
      const int j = n - head * rs.head_dim;  // the dim inside the head, below half
      if (head < rs.num_q_heads + rs.num_kv_proj && rs.cos_t != nullptr) {
        const float c = rs.cos_t[(size_t)token * half + j], sn = rs.sin_t[(size_t)token * half + j];
        const float ra = a * c - b * sn, rb = b * c + a * sn;
        a = ra;
        b = rb;
      }
      bf16* dst = nullptr;
      if (head < rs.num_q_heads) {
        a *= rs.q_scale;
        b *= rs.q_scale;
        dst = rs.q_out + ((size_t)token * rs.num_q_heads + head) * rs.head_dim;
      } else if (rs.cache != nullptr) {
        const int pos = rs.positions[token];
        const long long page = rs.block_table[(size_t)rs.token_seq[token] * rs.max_pages + pos / rs.page_size];
        if (page < 0 || page >= rs.num_pages) {
          atomicOr(rs.err, SB_ERR_BAD_PAGE);
        } else {
          const int kv = head < rs.num_q_heads + rs.num_kv_proj ? 0 : 1;
          const int m = head - rs.num_q_heads - kv * rs.num_kv_proj;
          dst = rs.cache + ((((size_t)page * 2 + kv) * rs.num_kv_proj + m) * rs.page_size + pos % rs.page_size) * rs.head_dim;
        }
      }
      if (dst != nullptr) {
        dst[j] = __float2bfloat16_rn(a);
        dst[j + half] = __float2bfloat16_rn(b);
      }
    } else if (EPI == 0) {
      reinterpret_cast<bf16*>(out)[o] = __float2bfloat16_rn(v[0]);
    } else if (EPI == 1) {
      reinterpret_cast<float*>(out)[o] = cap > 0.f ? cap * tanhf(v[0] / cap) : v[0];
    } else {
      // Round gate and up to bfloat16 first, as the unfused path stores them.
      const float gate = __bfloat162float(__float2bfloat16_rn(v[0]));
      const float up = __bfloat162float(__float2bfloat16_rn(v[SETS - 1]));
      reinterpret_cast<bf16*>(out)[o] = __float2bfloat16_rn(skinny_activation(gate, act) * up);
    }
  }
}

template <int MT, int WARPS>
static int launch_skinny(const bf16* x, const bf16* w, void* out, int M, int N, int K, int epilogue, float cap,
                         int act, cudaStream_t stream, const RopeStore& rs = RopeStore{}) {
  const int n_out = epilogue == 2 ? N / 2 : N;
  const unsigned blocks = epilogue == 3 ? (unsigned)(N / 32) : (unsigned)((n_out + 15) / 16);
  // Every block reads all of x through L1 just before it multiplies, so the stream of weights
  // stands still for the length of an L2 access whenever x is not there.  Attention kernels leave
  // the SMs split in favour of shared memory, and a kernel launched programmatically behind them
  // inherits that split (nothing drains the SMs in between): ask for no more shared memory than
  // the resident blocks' partial sums need, and so for the largest L1 beside it.
  static bool carveout_set = false;
  if (!carveout_set) {
    constexpr int SETS_MAX = 2;
    constexpr int resident = 512 / (WARPS * 32) > 0 ? 512 / (WARPS * 32) : 1;
    constexpr int needed = resident * (int)(sizeof(float) * WARPS * SETS_MAX * MT * 16 * 8 + 1024);
    const int percent = min(100, needed * 100 / (227 * 1024) + 1);
    cudaFuncSetAttribute(skinny_gemm_kernel<MT, WARPS, 0>, cudaFuncAttributePreferredSharedMemoryCarveout, percent);
    cudaFuncSetAttribute(skinny_gemm_kernel<MT, WARPS, 1>, cudaFuncAttributePreferredSharedMemoryCarveout, percent);
    cudaFuncSetAttribute(skinny_gemm_kernel<MT, WARPS, 2>, cudaFuncAttributePreferredSharedMemoryCarveout, percent);
    cudaFuncSetAttribute(skinny_gemm_kernel<MT, WARPS, 3>, cudaFuncAttributePreferredSharedMemoryCarveout, percent);
    carveout_set = true;
  }
  if (epilogue == 0)
    sb_launch_early(skinny_gemm_kernel<MT, WARPS, 0>, blocks, WARPS * 32, 0, stream, x, w, out, M, N, K, cap,
        act, rs);
  else if (epilogue == 1)
    sb_launch_early(skinny_gemm_kernel<MT, WARPS, 1>, blocks, WARPS * 32, 0, stream, x, w, out, M, N, K, cap,
        act, rs);
  else if (epilogue == 2)
    sb_launch_early(skinny_gemm_kernel<MT, WARPS, 2>, blocks, WARPS * 32, 0, stream, x, w, out, M, N, K, cap,
        act, rs);
  else
    sb_launch_early(skinny_gemm_kernel<MT, WARPS, 3>, blocks, WARPS * 32, 0, stream, x, w, out, M, N, K, cap,
        act, rs);
  SB_LAUNCH_CHECK();
  return 0;
}

// Returns -9 when the shape is outside what the kernel takes (the caller then
// uses the library product): M > 32, K not a multiple of 8, N odd for the gated epilogue.
extern "C" int sb_gemm_skinny_bf16(const void* x, const void* w, void* out, int M, int N, int K, int epilogue,
                                   float cap, int act, int warps_override, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M > 32 || K % 8 != 0 || K <= 0 || epilogue < 0 || epilogue > 2) return -9;
  if (epilogue == 2 && (N % 2 != 0 || act < 0 || act > 2)) return -9;
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)w;
  const int n_out = epilogue == 2 ? N / 2 : N;
  // Warps per block (the split of K).  All blocks should be resident at once, so that the
  // stream of weights never waits for a second wave: about 100 registers per thread let an SM
  // hold 512 threads, i.e. 148 blocks of 16 warps, 296 of 8 or 592 of 4.  `warps_override`
  // (4, 8 or 16) is for experiments.
  const int blocks = (n_out + 15) / 16;
  int warps = blocks <= 148 ? 16 : blocks <= 296 ? 8 : 4;
  if (K < warps * 32 * 4) warps = K >= 8 * 32 * 4 ? 8 : 4;  // every warp should have a full batch of loads
  if (warps_override == 4 || warps_override == 8 || warps_override == 16) warps = warps_override;
  if (M <= 8) {
    if (warps == 16) return launch_skinny<1, 16>(xp, wp, out, M, N, K, epilogue, cap, act, stream);
    if (warps == 8) return launch_skinny<1, 8>(xp, wp, out, M, N, K, epilogue, cap, act, stream);
    return launch_skinny<1, 4>(xp, wp, out, M, N, K, epilogue, cap, act, stream);
  }
  if (M <= 16) {
    if (warps == 16) return launch_skinny<2, 16>(xp, wp, out, M, N, K, epilogue, cap, act, stream);
    if (warps == 8) return launch_skinny<2, 8>(xp, wp, out, M, N, K, epilogue, cap, act, stream);
    return launch_skinny<2, 4>(xp, wp, out, M, N, K, epilogue, cap, act, stream);
  }
  // (8 warps at most: with 16 the partial sums of the gated epilogue outgrow static shared memory.)
  if (warps == 4) return launch_skinny<4, 4>(xp, wp, out, M, N, K, epilogue, cap, act, stream);
  return launch_skinny<4, 8>(xp, wp, out, M, N, K, epilogue, cap, act, stream);
}

// The fused q, k, v projection of an attention layer for at most 16 tokens: product, rotation,
// query scale, and the stores of queries (q_out) and of keys and values (pages of `cache`).
// w: [(num_q_heads + 2 * num_kv_proj) * head_dim, K], heads in the order q, k, v.
// cos_t / sin_t null: no rotation; cache null: keys and values are not stored.
// Returns -9 for shapes it does not take (M > 16, K % 8 != 0, head_dim % 32 != 0).
extern "C" int sb_qkv_rope_skinny(const void* x, const void* w, int M, int K, const float* cos_t,
                                  const float* sin_t, float q_scale, void* q_out, void* cache,
                                  const int* block_table, int max_pages, const int* token_seq,
                                  const int* positions, int num_q_heads, int num_kv_proj, int head_dim,
                                  int page_size, int num_pages, int* err, int warps_override,
                                  cudaStream_t stream) {
  if (M == 0) return 0;
  if (M > 16 || K % 8 != 0 || K <= 0 || head_dim <= 0 || head_dim % 32 != 0 || num_q_heads <= 0) return -9;
  RopeStore rs{cos_t, sin_t, q_scale, (bf16*)q_out, (bf16*)cache, block_table, max_pages, token_seq, positions,
               num_q_heads, num_kv_proj, head_dim, page_size, num_pages, err};
  const int N = (num_q_heads + 2 * num_kv_proj) * head_dim;
  const int blocks = N / 32;
  int warps = blocks <= 148 ? 16 : blocks <= 296 ? 8 : 4;
  if (K < warps * 32 * 2) warps = K >= 8 * 32 * 2 ? 8 : 4;
  if (warps_override == 4 || warps_override == 8 || warps_override == 16) warps = warps_override;
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)w;
  if (M <= 8) {
    if (warps == 16) return launch_skinny<1, 16>(xp, wp, nullptr, M, N, K, 3, 0.f, 0, stream, rs);
    if (warps == 8) return launch_skinny<1, 8>(xp, wp, nullptr, M, N, K, 3, 0.f, 0, stream, rs);
    return launch_skinny<1, 4>(xp, wp, nullptr, M, N, K, 3, 0.f, 0, stream, rs);
  }
  if (warps == 16) return launch_skinny<2, 16>(xp, wp, nullptr, M, N, K, 3, 0.f, 0, stream, rs);
  if (warps == 8) return launch_skinny<2, 8>(xp, wp, nullptr, M, N, K, 3, 0.f, 0, stream, rs);
  return launch_skinny<2, 4>(xp, wp, nullptr, M, N, K, 3, 0.f, 0, stream, rs);
}
