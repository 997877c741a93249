// Ragged paged attention on tensor cores (bfloat16 in, float32 softmax and accumulate),
// compiled once per head size (-DSB_HEAD_DIM=N, N a multiple of 16 up to 256).
//
//   s = q . k                 (q is already rotated and scaled)
//   s = cap * tanh(s / cap)   if cap > 0          simply/model_lib.py:621-626
//   keep k_pos <= q_pos and, with a window W, q_pos - k_pos < W
//                                                 simply/model_lib.py:469-515
//   p = softmax(s) in float32, o = p . v          simply/model_lib.py:633-637
//   query head n reads kv head n / G              simply/model_lib.py:2306-2310
//
// Two kernels share the tile code.
//  * prefill: a block owns 64 query rows of one (sequence, kv head): the G query heads
//    of the group for 64 / G consecutive tokens, so a key/value tile that is brought
//    to shared memory once serves the whole group.  Four warps own 16 rows each and
//    walk the key tiles (64 keys) with an online softmax.
//  * decode (at most 16 query rows per sequence and kv head, i.e. one or a few new
//    tokens): the keys are cut into chunks at fixed absolute positions; a persistent
//    grid draws (chunk, kv head) pairs from a counter; a block's warps split every key
//    tile between them, merge, and store a partial result (max, sum, normalised
//    output) that `combine` merges over chunks in a fixed order.
// Keys and values come from the paged cache through the block table with 16-byte
// cp.async copies; rows outside what the request holds are zero-filled, never read.
#include <cuda.h>
#include <float.h>
#include <string.h>

#include "common.cuh"

#ifndef SB_HEAD_DIM
#define SB_HEAD_DIM 256
#endif

namespace {

constexpr int DH = SB_HEAD_DIM;
constexpr int PITCH = DH + 8;  // elements; the 16-byte pad spreads 8 consecutive rows over all banks
constexpr int BN = 64;         // keys per tile
constexpr int CPR = DH / 8;    // 16-byte chunks per row
constexpr int NT = 128;        // threads per block
constexpr float LOG2E = 1.4426950408889634f;

static_assert(DH % 16 == 0 && DH >= 16 && DH <= 256, "head size must be a multiple of 16 up to 256");

struct AttnParams {
  const bf16* q;      // [T, Hq, DH]
  const bf16* cache;  // [P, 2, Hkv, page, DH]
  const int* block_table;
  int max_pages;
  const int* cu_q;     // [B + 1]
  const int* q_start;  // [B]
  bf16* out;           // [T, Hq * DH]
  int num_q_heads, num_kv_heads, page_size, num_pages;
  float cap;
  int window;
  const int* items;  // prefill: (sequence, first token of the tile); decode: (sequence, chunk)
  int chunk;         // decode: keys per chunk (a multiple of BN)
  float* part_o;     // decode: [items, Hkv, rows_max, DH]
  float* part_ml;    // decode: [items, Hkv, rows_max, 2]
  int rows_max;
  int older_keys_settled;  // decode: keys below q_start were written before the kernel just before this one
  int* err;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: nothing is read, the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t r[4], const bf16* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t r[4], const bf16* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void mma16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Brings keys [tile, tile + TILE) of (sequence b, kv head m) to shared memory; positions
// outside [kv_lo, kv_hi) and pages the request does not hold are zero-filled.  The block
// first works out where each of the TILE rows lives (one block-table lookup per row, into
// `row_src`, TILE entries of shared memory), then copies 16 bytes per thread and turn.
// Ends with the copies issued, not committed.  Contains one __syncthreads.
template <int TILE, int THREADS>
__device__ __forceinline__ void load_kv_tile(const AttnParams& p, bf16* sk, bf16* sv, long long* row_src,
                                             int tile, int kv_lo, int kv_hi, int b, int m) {
  const size_t head_stride = (size_t)p.page_size * DH;
  const size_t v_offset = (size_t)p.num_kv_heads * head_stride;
  for (int row = threadIdx.x; row < TILE; row += THREADS) {
    const int j = tile + row;
    long long src = -1;
    if (j >= kv_lo && j < kv_hi) {
      const int page_index = j / p.page_size;
      const long long page = p.block_table[(size_t)b * p.max_pages + page_index];
      if (page < 0 || page >= p.num_pages)
        atomicOr(p.err, SB_ERR_BAD_PAGE);
      else
        src = (long long)(((size_t)page * 2 * p.num_kv_heads + m) * head_stride +
                          (size_t)(j - page_index * p.page_size) * DH);
    }
    row_src[row] = src;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < TILE * CPR; i += THREADS) {
    const int row = i / CPR, c = i - row * CPR;
    const long long src = row_src[row];
    const bool valid = src >= 0;
    const bf16* g = p.cache + (valid ? src : 0) + c * 8;
    cp_async16(sk + row * PITCH + c * 8, g, valid);
    cp_async16(sv + row * PITCH + c * 8, g + v_offset, valid);
  }
}

// Scores of one warp's 16 query rows against NKT * 8 keys that start at row `key0` of the tile.
template <int NKT>
__device__ __forceinline__ void scores(float (&s)[NKT][4], const bf16* sq_rows, const bf16* sk, int key0) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < NKT; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
#pragma unroll
  for (int ks = 0; ks < DH / 16; ++ks) {
    uint32_t a[4];
    ldmatrix_x4(a, sq_rows + (lane & 15) * PITCH + ks * 16 + (lane >> 4) * 8);
#pragma unroll
    for (int np = 0; np < NKT / 2; ++np) {
      uint32_t r[4];
      ldmatrix_x4(r, sk + (key0 + np * 16 + (lane >> 4) * 8 + (lane & 7)) * PITCH + ks * 16 + ((lane >> 3) & 1) * 8);
      mma16816(s[2 * np], a, r[0], r[1]);
      mma16816(s[2 * np + 1], a, r[2], r[3]);
    }
  }
}

// Soft cap, mask, online softmax update and P.V for one warp.  `pos_a`, `pos_b`: positions of
// the thread's two query rows (-1 for a padding row).  `j0`: position of the first of the
// NKT * 8 keys.  m_* are kept in log2 units.
template <int NKT>
__device__ __forceinline__ void softmax_pv(float (&s)[NKT][4], float (&o)[DH / 8][4], float& m_a, float& m_b,
                                           float& l_a, float& l_b, int pos_a, int pos_b, int j0, float cap,
                                           int window, const bf16* sv, int key0, bool need_mask = true) {
  const int lane = threadIdx.x & 31, t = lane & 3;
  const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
  float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
  for (int i = 0; i < NKT; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int j = j0 + i * 8 + 2 * t + (e & 1);
      const int pos = e < 2 ? pos_a : pos_b;
      float v = s[i][e];
      if (cap > 0.f) v = cap * fast_tanh(v * inv_cap);
      // need_mask is false (for the whole warp) when every key of the tile is visible to every row.
      const bool keep = !need_mask || (j <= pos && (window <= 0 || pos - j < window));
      v = keep ? v * LOG2E : -INFINITY;
      s[i][e] = v;
      if (e < 2) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
    }
  mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
  mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
  mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
  mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
  const float new_a = fmaxf(m_a, mx_a), new_b = fmaxf(m_b, mx_b);
  const float use_a = new_a == -INFINITY ? 0.f : new_a, use_b = new_b == -INFINITY ? 0.f : new_b;
  const float alpha_a = fast_exp2(m_a - use_a), alpha_b = fast_exp2(m_b - use_b);
  m_a = new_a;
  m_b = new_b;
  float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
  for (int i = 0; i < NKT; ++i) {
    s[i][0] = fast_exp2(s[i][0] - use_a);
    s[i][1] = fast_exp2(s[i][1] - use_a);
    s[i][2] = fast_exp2(s[i][2] - use_b);
    s[i][3] = fast_exp2(s[i][3] - use_b);
    sum_a += s[i][0] + s[i][1];
    sum_b += s[i][2] + s[i][3];
  }
  l_a = l_a * alpha_a + sum_a;  // per-thread share of the row sum; the quad is added up at the end
  l_b = l_b * alpha_b + sum_b;
  if (__any_sync(0xffffffffu, alpha_a != 1.f || alpha_b != 1.f)) {  // the running maxima rarely move
#pragma unroll
    for (int d = 0; d < DH / 8; ++d) {
      o[d][0] *= alpha_a;
      o[d][1] *= alpha_a;
      o[d][2] *= alpha_b;
      o[d][3] *= alpha_b;
    }
  }
#pragma unroll
  for (int kk = 0; kk < NKT / 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < DH / 16; ++dp) {
      uint32_t r[4];
      ldmatrix_x4_trans(r, sv + (key0 + kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * PITCH + dp * 16 + (lane >> 4) * 8);
      mma16816(o[2 * dp], a, r[0], r[1]);
      mma16816(o[2 * dp + 1], a, r[2], r[3]);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Prefill: grid (items, kv heads).  A block owns WM * 16 query rows; its WM * WN warps are
// laid out as WM row groups of 16 rows times WN key groups that split every 64-key tile
// between them (WN = 2: two warps per scheduler to switch between; their partial results
// are merged through shared memory at the end).
// ---------------------------------------------------------------------------------------
template <int WM, int WN>
__global__ void __launch_bounds__(WM * WN * 32) attn_prefill_kernel(const AttnParams p) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int BM = WM * 16, THREADS = WM * WN * 32, KEYS = BN / WN;  // keys of a tile per warp
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sq = reinterpret_cast<bf16*>(smem_raw);  // [BM][PITCH]
  bf16* sk = sq + BM * PITCH;                    // [2][BN][PITCH]
  bf16* sv = sk + 2 * BN * PITCH;                // [2][BN][PITCH]
  __shared__ long long row_src[2][BN];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int wm = warp % WM, wn = warp / WM;
  const int b = p.items[2 * blockIdx.x], i0 = p.items[2 * blockIdx.x + 1], m = blockIdx.y;
  const int group = p.num_q_heads / p.num_kv_heads;
  const int tokens_per_tile = BM / group;
  const int row0 = p.cu_q[b], q_len = p.cu_q[b + 1] - row0, qs = p.q_start[b];
  const int ntok = min(tokens_per_tile, q_len - i0);
  const int rows_valid = ntok * group;

  for (int i = threadIdx.x; i < BM * CPR; i += THREADS) {
    const int row = i / CPR, c = i - row * CPR;
    const bool valid = row < rows_valid;
    const int tok = valid ? i0 + row / group : i0, h = m * group + (valid ? row % group : 0);
    cp_async16(sq + row * PITCH + c * 8, p.q + ((size_t)(row0 + tok) * p.num_q_heads + h) * DH + c * 8, valid);
  }
  const int p0 = qs + i0, p1 = qs + i0 + ntok - 1;
  const int kv_lo = p.window > 0 ? max(qs - p.window + 1, 0) : 0;  // lowest key the request still holds
  const int lo = p.window > 0 ? max(p0 - p.window + 1, 0) : 0;     // lowest key this tile can see
  const int kv_hi = p1 + 1;
  const int tile0 = (lo / BN) * BN;
  const int n_tiles = (kv_hi - tile0 + BN - 1) / BN;
  load_kv_tile<BN, THREADS>(p, sk, sv, row_src[0], tile0, kv_lo, kv_hi, b, m);
  cp_async_commit();

  const int ra = wm * 16 + g, rb = ra + 8;
  const int pos_a = ra < rows_valid ? p0 + ra / group : -1;
  const int pos_b = rb < rows_valid ? p0 + rb / group : -1;
  // Positions of this warp's first and last row, for deciding whether a tile needs masking.
  const bool rows_full = wm * 16 + 15 < rows_valid;
  const int warp_pos_lo = p0 + (wm * 16) / group, warp_pos_hi = p0 + (wm * 16 + 15) / group;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  float o[DH / 8][4];
#pragma unroll
  for (int d = 0; d < DH / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

  for (int it = 0; it < n_tiles; ++it) {
    const int stage = it & 1;
    if (it + 1 < n_tiles) {
      load_kv_tile<BN, THREADS>(p, sk + (stage ^ 1) * BN * PITCH, sv + (stage ^ 1) * BN * PITCH, row_src[stage ^ 1],
                                tile0 + (it + 1) * BN, kv_lo, kv_hi, b, m);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int j0 = tile0 + it * BN + wn * KEYS;  // this warp's first key of the tile
    // Every key visible to every row of the warp: below the lowest row's position, inside the
    // highest row's window.
    const bool need_mask = !rows_full || j0 + KEYS - 1 > warp_pos_lo || (p.window > 0 && warp_pos_hi - j0 >= p.window);
    float s[KEYS / 8][4];
    scores<KEYS / 8>(s, sq + wm * 16 * PITCH, sk + stage * BN * PITCH, wn * KEYS);
    softmax_pv<KEYS / 8>(s, o, m_a, m_b, l_a, l_b, pos_a, pos_b, j0, p.cap, p.window, sv + stage * BN * PITCH,
                         wn * KEYS, need_mask);
    __syncthreads();
  }
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  if (WN > 1) {
    // The key groups of a row group merge: warps of group 1 hand (max, sum, output) to group 0.
    float* xm = reinterpret_cast<float*>(sk);  // [BM] max, [BM] sum, then [BM][DH] (the tiles are no longer needed)
    float* xl = xm + BM;
    float* xo = xl + BM;
    if (wn == 1) {
      if (t == 0) {
        xm[ra] = m_a; xm[rb] = m_b;
        xl[ra] = l_a; xl[rb] = l_b;
      }
#pragma unroll
      for (int d = 0; d < DH / 8; ++d) {
        *reinterpret_cast<float2*>(xo + (size_t)ra * DH + d * 8 + 2 * t) = make_float2(o[d][0], o[d][1]);
        *reinterpret_cast<float2*>(xo + (size_t)rb * DH + d * 8 + 2 * t) = make_float2(o[d][2], o[d][3]);
      }
    }
    __syncthreads();
    if (wn == 1) return;
    const float om_a = xm[ra], om_b = xm[rb];
    const float nm_a = fmaxf(m_a, om_a), nm_b = fmaxf(m_b, om_b);
    const float ua = nm_a == -INFINITY ? 0.f : nm_a, ub = nm_b == -INFINITY ? 0.f : nm_b;
    const float sa = fast_exp2(m_a - ua), sb = fast_exp2(m_b - ub);     // scale of this warp's part
    const float ta = fast_exp2(om_a - ua), tb = fast_exp2(om_b - ub);   // scale of the other's
    l_a = l_a * sa + xl[ra] * ta;
    l_b = l_b * sb + xl[rb] * tb;
#pragma unroll
    for (int d = 0; d < DH / 8; ++d) {
      const float2 oa = *reinterpret_cast<const float2*>(xo + (size_t)ra * DH + d * 8 + 2 * t);
      const float2 ob = *reinterpret_cast<const float2*>(xo + (size_t)rb * DH + d * 8 + 2 * t);
      o[d][0] = o[d][0] * sa + oa.x * ta;
      o[d][1] = o[d][1] * sa + oa.y * ta;
      o[d][2] = o[d][2] * sb + ob.x * tb;
      o[d][3] = o[d][3] * sb + ob.y * tb;
    }
  }
  const float inv_a = l_a > 0.f ? 1.0f / l_a : 0.f, inv_b = l_b > 0.f ? 1.0f / l_b : 0.f;
  if (ra < rows_valid) {
    bf16* op = p.out + ((size_t)(row0 + i0 + ra / group) * p.num_q_heads + m * group + ra % group) * DH;
#pragma unroll
    for (int d = 0; d < DH / 8; ++d)
      *reinterpret_cast<uint32_t*>(op + d * 8 + 2 * t) = pack_bf16(o[d][0] * inv_a, o[d][1] * inv_a);
  }
  if (rb < rows_valid) {
    bf16* op = p.out + ((size_t)(row0 + i0 + rb / group) * p.num_q_heads + m * group + rb % group) * DH;
#pragma unroll
    for (int d = 0; d < DH / 8; ++d)
      *reinterpret_cast<uint32_t*>(op + d * 8 + 2 * t) = pack_bf16(o[d][2] * inv_b, o[d][3] * inv_b);
  }
}

// ---------------------------------------------------------------------------------------
// Decode: a persistent grid; blocks draw (item, kv head) pairs from a counter until none is
// left, so short and long chunks balance out.  A block has DEC_BN / 16 warps; warp w owns
// keys [16 w, 16 w + 16) of every tile.  Tiles of 32 keys for head sizes above 128 keep the
// block's shared memory below half an SM's, so two blocks run side by side and one's start
// and end overlap the other's stream of tiles.
// ---------------------------------------------------------------------------------------
constexpr int DEC_BN = DH > 128 ? 32 : 64;
constexpr int DEC_WARPS = DEC_BN / 16;
constexpr int DEC_NT = DEC_WARPS * 32;
constexpr int DEC_STAGES = 3;

__global__ void __launch_bounds__(DEC_NT) attn_decode_kernel(const AttnParams p, int* work_counter, int total_work) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sq = reinterpret_cast<bf16*>(smem_raw);  // [16][PITCH]
  bf16* sk = sq + 16 * PITCH;                    // [STAGES][DEC_BN][PITCH]
  bf16* sv = sk + DEC_STAGES * DEC_BN * PITCH;   // [STAGES][DEC_BN][PITCH]
  __shared__ int s_work;
  __shared__ long long row_src[DEC_STAGES][DEC_BN];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int group = p.num_q_heads / p.num_kv_heads;
  for (;;) {
    if (threadIdx.x == 0) s_work = atomicAdd(work_counter, 1);
    __syncthreads();
    const int work = s_work;
    __syncthreads();  // everyone has read s_work; shared memory of the last item is free
    if (work >= total_work) break;
    const int item = work / p.num_kv_heads, m = work - item * p.num_kv_heads;
    const int b = p.items[2 * item], chunk_index = p.items[2 * item + 1];
    if (b < 0) continue;  // filler item of a fixed-size work list
    const int row0 = p.cu_q[b], q_len = p.cu_q[b + 1] - row0, qs = p.q_start[b];
    const int rows_valid = q_len * group;  // <= 16 by the host's routing
    const int kv_lo = p.window > 0 ? max(qs - p.window + 1, 0) : 0;
    const int kv_hi = qs + q_len;
    const int begin = max(chunk_index * p.chunk, (kv_lo / 64) * 64);
    const int end = min((chunk_index + 1) * p.chunk, kv_hi);
    const int n_tiles = end > begin ? (end - begin + DEC_BN - 1) / DEC_BN : 0;

    for (int i = threadIdx.x; i < 16 * CPR; i += DEC_NT) {
      const int row = i / CPR, c = i - row * CPR;
      const bool valid = row < rows_valid;
      const int tok = valid ? row / group : 0, h = m * group + (valid ? row % group : 0);
      cp_async16(sq + row * PITCH + c * 8, p.q + ((size_t)(row0 + tok) * p.num_q_heads + h) * DH + c * 8, valid);
    }
#pragma unroll
    for (int st = 0; st < DEC_STAGES - 1; ++st) {
      if (st < n_tiles)  // uniform over the block
        load_kv_tile<DEC_BN, DEC_NT>(p, sk + st * DEC_BN * PITCH, sv + st * DEC_BN * PITCH, row_src[st],
                                     begin + st * DEC_BN, kv_lo, end, b, m);
      cp_async_commit();
    }
    const int pos_a = g < rows_valid ? qs + g / group : -1;
    const int pos_b = g + 8 < rows_valid ? qs + (g + 8) / group : -1;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    float o[DH / 8][4];
#pragma unroll
    for (int d = 0; d < DH / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

    for (int it = 0; it < n_tiles; ++it) {
      const int stage = it % DEC_STAGES;
      cp_async_wait<DEC_STAGES - 2>();
      __syncthreads();  // tile `it` has landed; everyone is done with tile it - 1
      if (it + DEC_STAGES - 1 < n_tiles) {
        const int st = (it + DEC_STAGES - 1) % DEC_STAGES;
        load_kv_tile<DEC_BN, DEC_NT>(p, sk + st * DEC_BN * PITCH, sv + st * DEC_BN * PITCH, row_src[st],
                                     begin + (it + DEC_STAGES - 1) * DEC_BN, kv_lo, end, b, m);
      }
      cp_async_commit();
      float s[2][4];
      scores<2>(s, sq, sk + stage * DEC_BN * PITCH, warp * 16);
      softmax_pv<2>(s, o, m_a, m_b, l_a, l_b, pos_a, pos_b, begin + it * DEC_BN + warp * 16, p.cap, p.window,
                    sv + stage * DEC_BN * PITCH, warp * 16);
    }
    cp_async_wait<0>();
    __syncthreads();
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

    // Merge the warps (each saw its share of every tile) through shared memory.
    float* wm = reinterpret_cast<float*>(sk);  // [W][16] max, [W][16] sum, then [W][rows_valid][DH]
    float* wl = wm + DEC_WARPS * 16;
    float* wo = wl + DEC_WARPS * 16;
    if (t == 0) {
      wm[warp * 16 + g] = m_a;
      wm[warp * 16 + g + 8] = m_b;
      wl[warp * 16 + g] = l_a;
      wl[warp * 16 + g + 8] = l_b;
    }
    if (g < rows_valid) {
#pragma unroll
      for (int d = 0; d < DH / 8; ++d) {
        wo[((size_t)warp * rows_valid + g) * DH + d * 8 + 2 * t] = o[d][0];
        wo[((size_t)warp * rows_valid + g) * DH + d * 8 + 2 * t + 1] = o[d][1];
      }
    }
    if (g + 8 < rows_valid) {
#pragma unroll
      for (int d = 0; d < DH / 8; ++d) {
        wo[((size_t)warp * rows_valid + g + 8) * DH + d * 8 + 2 * t] = o[d][2];
        wo[((size_t)warp * rows_valid + g + 8) * DH + d * 8 + 2 * t + 1] = o[d][3];
      }
    }
    __syncthreads();
    const size_t pidx = (size_t)item * p.num_kv_heads + m;
    for (int i = threadIdx.x; i < rows_valid * DH; i += DEC_NT) {
      const int r = i / DH, d = i - r * DH;
      float mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) mx = fmaxf(mx, wm[w * 16 + r]);
      float num = 0.f, den = 0.f;
      if (mx != -INFINITY) {
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
          const float sc = fast_exp2(wm[w * 16 + r] - mx);
          num += sc * wo[((size_t)w * rows_valid + r) * DH + d];
          den += sc * wl[w * 16 + r];
        }
      }
      p.part_o[(pidx * p.rows_max + r) * DH + d] = den > 0.f ? num / den : 0.f;
      if (d == 0) {
        p.part_ml[(pidx * p.rows_max + r) * 2] = mx;
        p.part_ml[(pidx * p.rows_max + r) * 2 + 1] = den;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Decode with at most 8 query rows per (sequence, kv head): the usual case of one new token
// and a group of up to 8 query heads.  Same persistent grid and chunks as above, but
//  * the product is turned round: scores^T[16 keys x 8 rows] = K . Q^T, so the 16-row operand
//    of the mma is a tile of keys and the 8-column operand is the queries, which stay in
//    registers for a whole chunk; out^T[16 dims x 8 rows] += V^T . P^T likewise.  Half the
//    tensor work, half the accumulator registers, no padding of 2 rows to 16;
//  * P^T becomes the 8-column operand by transposing its 8x8 blocks across the warp
//    (movmatrix), with no trip through shared memory;
//  * with USE_TMA, key/value tiles come in through the tensor memory accelerator: one
//    elected thread issues a few box copies per tile (`cp.async.bulk.tensor.2d`, 128-byte
//    swizzle, completion counted on an mbarrier per stage) instead of two thousand 16-byte
//    copies with their address arithmetic.  It needs a head size that is a multiple of 64 and
//    a page size that is a power of two; otherwise the 16-byte copies are used.
//    (One bulk copy per 512-byte row, without a tensor map, was measured slower than either.)
// Every wait on an mbarrier is bounded; on a time-out the block sets SB_ERR_TIMEOUT and leaves.
// ---------------------------------------------------------------------------------------
#define SB_ERR_TIMEOUT 8

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, int bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity; false after about half a second without success.
__device__ __forceinline__ unsigned long long sb_global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity) {
  // A try_wait may itself block for a while, so the bound is on time (half a second), not on
  // tries.  The clock is only read every 4096 tries: reading it, or sleeping, between two tries
  // would add its latency to every hand-over between the warps of a pipeline.
  unsigned long long start = 0;
  for (unsigned tries = 1;; ++tries) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((tries & 0xFFFu) == 0) {
      const unsigned long long now = sb_global_ns();
      if (start == 0) start = now;
      else if (now - start > 500000000ull) return false;
    }
  }
}
// One box of the tensor map (columns [col, col + 64), rows [row, row + box rows)) to shared memory.
__device__ __forceinline__ void tma_load_box(void* dst, const CUtensorMap* map, int col, int row, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(col), "r"(row), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}

constexpr int D8_BN = DH > 128 ? 32 : 64;  // keys per tile
constexpr int D8_WARPS = D8_BN / 16;
constexpr int D8_NT = D8_WARPS * 32;
constexpr int D8_STAGES = 2;
constexpr bool TMA_OK = DH % 64 == 0;        // 128-byte swizzled boxes of 64 columns
constexpr int SLABS = TMA_OK ? DH / 64 : 1;  // 64-column slabs of a tile in the swizzled layout
constexpr int SLAB_ELEMS = D8_BN * 64;       // elements of one slab of one tile

// Element (row, dim) of a tile.  Swizzled layout: [slab][row][64 columns], the 16-byte chunks of
// a 128-byte row XOR-ed with the row's low three bits (what the TMA's 128-byte swizzle writes).
template <bool USE_TMA>
__device__ __forceinline__ const bf16* tile_at(const bf16* tile, int row, int dim) {
  if (USE_TMA) return tile + (dim >> 6) * SLAB_ELEMS + row * 64 + ((((dim & 63) >> 3) ^ (row & 7)) << 3) + (dim & 7);
  return tile + row * PITCH + dim;
}

template <bool USE_TMA>
__global__ void __launch_bounds__(D8_NT)
attn_decode8_kernel(const AttnParams p, int* work_counter, int total_work, const __grid_constant__ CUtensorMap tmap,
                    int box_rows) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int TILE_ELEMS = USE_TMA ? D8_BN * DH : D8_BN * PITCH;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // The swizzle pattern is a function of the address: tiles start on a 1024-byte boundary
  // (the launch adds 1024 bytes of slack for this).
  unsigned char* aligned = smem_raw + (USE_TMA ? ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u) : 0u);
  bf16* sk = reinterpret_cast<bf16*>(aligned);  // [STAGES] key tiles
  bf16* sv = sk + D8_STAGES * TILE_ELEMS;        // [STAGES] value tiles
  __shared__ __align__(8) uint64_t full[D8_STAGES];
  __shared__ long long row_src[D8_STAGES][D8_BN];
  __shared__ int s_work;
  __shared__ int s_failed;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int group = p.num_q_heads / p.num_kv_heads;
  if (threadIdx.x == 0) {
    for (int st = 0; st < D8_STAGES; ++st) mbar_init(&full[st], 1);
    s_failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  unsigned tile_seq = 0;  // tiles this block has consumed so far: stage = seq % STAGES, parity from seq / STAGES

  for (;;) {
    if (threadIdx.x == 0) s_work = atomicAdd(work_counter, 1);
    __syncthreads();
    const int work = s_work;
    const bool failed = s_failed != 0;
    __syncthreads();  // everyone has read s_work; shared memory of the last item is free
    if (work >= total_work || failed) break;
    const int item = work / p.num_kv_heads, m = work - item * p.num_kv_heads;
    const int b = p.items[2 * item], chunk_index = p.items[2 * item + 1];
    if (b < 0) continue;  // filler item of a fixed-size work list
    const int row0 = p.cu_q[b], q_len = p.cu_q[b + 1] - row0, qs = p.q_start[b];
    const int rows_valid = q_len * group;  // <= 8 by the host's routing
    const int kv_lo = p.window > 0 ? max(qs - p.window + 1, 0) : 0;
    const int kv_hi = qs + q_len;
    const int begin = max(chunk_index * p.chunk, (kv_lo / 64) * 64);
    const int end = min((chunk_index + 1) * p.chunk, kv_hi);
    const int n_tiles = end > begin ? (end - begin + D8_BN - 1) / D8_BN : 0;

    auto issue_tile = [&](int tile_index, unsigned seq) {
      const int stage = seq % D8_STAGES;
      const int j0 = begin + tile_index * D8_BN;
      if (USE_TMA) {
        // One thread: a box per page piece and 64-column slab, for keys and for values.  Boxes of
        // pages the request does not hold, or wholly outside [kv_lo, end), are not fetched; the
        // consumers zero what they must not read.
        if (threadIdx.x != 0) return;
        int boxes = 0;
        for (int r = 0; r < D8_BN; r += box_rows) {
          const int j = j0 + r;
          if (j >= end || j + box_rows <= kv_lo) continue;
          const long long page = p.block_table[(size_t)b * p.max_pages + j / p.page_size];
          if (page >= 0 && page < p.num_pages) ++boxes;
        }
        mbar_arrive_expect_tx(&full[stage], boxes * 2 * SLABS * box_rows * 128);
        for (int r = 0; r < D8_BN; r += box_rows) {
          const int j = j0 + r;
          if (j >= end || j + box_rows <= kv_lo) continue;
          const long long page = p.block_table[(size_t)b * p.max_pages + j / p.page_size];
          if (page < 0 || page >= p.num_pages) {
            atomicOr(p.err, SB_ERR_BAD_PAGE);
            continue;
          }
          const long long krow = ((page * 2) * p.num_kv_heads + m) * p.page_size + (j & (p.page_size - 1));
          const long long vrow = krow + (long long)p.num_kv_heads * p.page_size;
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl) {
            tma_load_box(sk + (size_t)stage * TILE_ELEMS + sl * SLAB_ELEMS + r * 64, &tmap, sl * 64, (int)krow, &full[stage]);
            tma_load_box(sv + (size_t)stage * TILE_ELEMS + sl * SLAB_ELEMS + r * 64, &tmap, sl * 64, (int)vrow, &full[stage]);
          }
        }
      } else {
        load_kv_tile<D8_BN, D8_NT>(p, sk + (size_t)stage * TILE_ELEMS, sv + (size_t)stage * TILE_ELEMS, row_src[stage],
                                   j0, kv_lo, end, b, m);
      }
    };

    for (int st = 0; st < D8_STAGES - 1; ++st) {
      if (st < n_tiles) issue_tile(st, tile_seq + st);
      if (!USE_TMA) cp_async_commit();
    }

    // Queries: the 8-column operand, in registers for the whole chunk.  Column g is query row g.
    uint32_t qf[DH / 16][2];
    {
      const bool valid = g < rows_valid;
      const bf16* qrow = p.q + ((size_t)(row0 + (valid ? g / group : 0)) * p.num_q_heads + m * group +
                                (valid ? g % group : 0)) * DH;
#pragma unroll
      for (int ks = 0; ks < DH / 16; ++ks) {
        qf[ks][0] = valid ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t) : 0u;
        qf[ks][1] = valid ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t) : 0u;
      }
    }
    // This thread's two query rows are 2t and 2t + 1.
    const int pos0 = 2 * t < rows_valid ? qs + (2 * t) / group : -1;
    const int pos1 = 2 * t + 1 < rows_valid ? qs + (2 * t + 1) / group : -1;
    const float inv_cap = p.cap > 0.f ? 1.0f / p.cap : 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[DH / 16][4];  // out^T: [dims 16 blk + g | g + 8][rows 2t | 2t + 1]
#pragma unroll
    for (int d = 0; d < DH / 16; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

    bool ok = true;
    for (int it = 0; it < n_tiles; ++it) {
      const unsigned seq = tile_seq + it;
      const int stage = seq % D8_STAGES;
      bool landed = true;
      if (USE_TMA) {
        // The stage refilled here was read in the last iteration; the barrier at its end freed it.
        if (it + D8_STAGES - 1 < n_tiles) issue_tile(it + D8_STAGES - 1, seq + D8_STAGES - 1);
        // A thread whose wait ran out skips the arithmetic; the block agrees on leaving below.
        landed = mbar_wait_bounded(&full[stage], (seq / D8_STAGES) & 1);
      } else {
        cp_async_wait<D8_STAGES - 2>();
        __syncthreads();  // tile `it` has landed for every thread; the stage of tile it - 1 is free
        if (it + D8_STAGES - 1 < n_tiles) issue_tile(it + D8_STAGES - 1, seq + D8_STAGES - 1);
        cp_async_commit();
      }
      if (landed) {
        const bf16* kt = sk + (size_t)stage * TILE_ELEMS;
        const bf16* vt = sv + (size_t)stage * TILE_ELEMS;
        const int key0 = warp * 16;  // this warp's keys of the tile
        const int j_first = begin + it * D8_BN + key0;
        if (USE_TMA && (j_first < kv_lo || j_first + 16 > end)) {
          // Some of this warp's 16 keys are not the request's: their value rows must read as zeros
          // (0 * garbage could be NaN).  Only this warp reads these rows.
          for (int i = lane; i < 16 * (DH / 8); i += 32) {
            const int r = i / (DH / 8), c = i - r * (DH / 8);
            const int j = j_first + r;
            if (j < kv_lo || j >= end)
              *reinterpret_cast<uint4*>(const_cast<bf16*>(tile_at<true>(vt, key0 + r, c * 8))) = make_uint4(0, 0, 0, 0);
          }
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
          __syncwarp();
        }
        // scores^T for this warp's 16 keys; two accumulators halve the chain of dependent mma's
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < DH / 16; ks += 2) {
          uint32_t a[4], a2[4];
          ldmatrix_x4(a, tile_at<USE_TMA>(kt, key0 + (lane & 15), ks * 16 + (lane >> 4) * 8));
          mma16816(s0, a, qf[ks][0], qf[ks][1]);
          if (ks + 1 < DH / 16) {
            ldmatrix_x4(a2, tile_at<USE_TMA>(kt, key0 + (lane & 15), (ks + 1) * 16 + (lane >> 4) * 8));
            mma16816(s1, a2, qf[ks + 1][0], qf[ks + 1][1]);
          }
        }
        // s[0]: (key g, row 2t)  s[1]: (key g, row 2t+1)  s[2]: (key g+8, row 2t)  s[3]: (key g+8, row 2t+1)
        float sc[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s0[e] + s1[e];
          if (p.cap > 0.f) v = p.cap * fast_tanh(v * inv_cap);
          const int j = j_first + g + (e >> 1) * 8;
          const int pos = (e & 1) ? pos1 : pos0;
          const bool keep = j <= pos && (p.window <= 0 || pos - j < p.window);
          sc[e] = keep ? v * LOG2E : -INFINITY;
        }
        float mx0 = fmaxf(sc[0], sc[2]), mx1 = fmaxf(sc[1], sc[3]);
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
          mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
          mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        const float new0 = fmaxf(m0, mx0), new1 = fmaxf(m1, mx1);
        const float use0 = new0 == -INFINITY ? 0.f : new0, use1 = new1 == -INFINITY ? 0.f : new1;
        const float alpha0 = fast_exp2(m0 - use0), alpha1 = fast_exp2(m1 - use1);
        m0 = new0;
        m1 = new1;
        const float p0 = fast_exp2(sc[0] - use0), p1 = fast_exp2(sc[1] - use1);
        const float p2 = fast_exp2(sc[2] - use0), p3 = fast_exp2(sc[3] - use1);
        l0 = l0 * alpha0 + p0 + p2;  // this thread's keys only; the eight g-lanes are added at the end
        l1 = l1 * alpha1 + p1 + p3;
        if (__any_sync(0xffffffffu, alpha0 != 1.f || alpha1 != 1.f)) {
#pragma unroll
          for (int d = 0; d < DH / 16; ++d) {
            o[d][0] *= alpha0;
            o[d][1] *= alpha1;
            o[d][2] *= alpha0;
            o[d][3] *= alpha1;
          }
        }
        // P^T as the 8-column operand: (keys 2t, 2t+1 | 2t+8, 2t+9 ; row g) from (key g | g+8 ; rows 2t, 2t+1).
        const uint32_t b0 = movmatrix_trans(pack_bf16(p0, p1));
        const uint32_t b1 = movmatrix_trans(pack_bf16(p2, p3));
#pragma unroll
        for (int d = 0; d < DH / 16; ++d) {
          uint32_t a[4];
          ldmatrix_x4_trans(a, tile_at<USE_TMA>(vt, key0 + ((lane >> 4) & 1) * 8 + (lane & 7), d * 16 + ((lane >> 3) & 1) * 8));
          mma16816(o[d], a, b0, b1);
        }
      }
      if (USE_TMA) {
        // Everyone is done with this stage before it is filled again; and did everyone get its tile?
        if (!__syncthreads_and(landed ? 1 : 0)) {
          ok = false;
          break;
        }
      }
    }
    if (!USE_TMA) cp_async_wait<0>();
    if (!ok) {
      atomicOr(p.err, SB_ERR_TIMEOUT);
      s_failed = 1;
    }
    tile_seq += n_tiles;
    __syncthreads();
    if (s_failed) {
      // Copies of this block may still be in flight: give them a millisecond to land, then leave.
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
      break;
    }
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, off);
      l1 += __shfl_xor_sync(0xffffffffu, l1, off);
    }
    // Merge the warps through shared memory (the tiles are no longer needed).
    float* wm = reinterpret_cast<float*>(sk);  // [W][8] max, [W][8] sum, then [W][rows_valid][DH]
    float* wl = wm + D8_WARPS * 8;
    float* wo = wl + D8_WARPS * 8;
    if (g == 0) {
      wm[warp * 8 + 2 * t] = m0;
      wm[warp * 8 + 2 * t + 1] = m1;
      wl[warp * 8 + 2 * t] = l0;
      wl[warp * 8 + 2 * t + 1] = l1;
    }
#pragma unroll
    for (int d = 0; d < DH / 16; ++d) {
      if (2 * t < rows_valid) {
        wo[((size_t)warp * rows_valid + 2 * t) * DH + d * 16 + g] = o[d][0];
        wo[((size_t)warp * rows_valid + 2 * t) * DH + d * 16 + g + 8] = o[d][2];
      }
      if (2 * t + 1 < rows_valid) {
        wo[((size_t)warp * rows_valid + 2 * t + 1) * DH + d * 16 + g] = o[d][1];
        wo[((size_t)warp * rows_valid + 2 * t + 1) * DH + d * 16 + g + 8] = o[d][3];
      }
    }
    __syncthreads();
    const size_t pidx = (size_t)item * p.num_kv_heads + m;
    for (int i = threadIdx.x; i < rows_valid * DH; i += D8_NT) {
      const int r = i / DH, d = i - r * DH;
      float mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < D8_WARPS; ++w) mx = fmaxf(mx, wm[w * 8 + r]);
      float num = 0.f, den = 0.f;
      if (mx != -INFINITY) {
#pragma unroll
        for (int w = 0; w < D8_WARPS; ++w) {
          const float scale = fast_exp2(wm[w * 8 + r] - mx);
          num += scale * wo[((size_t)w * rows_valid + r) * DH + d];
          den += scale * wl[w * 8 + r];
        }
      }
      p.part_o[(pidx * p.rows_max + r) * DH + d] = den > 0.f ? num / den : 0.f;
      if (d == 0) {
        p.part_ml[(pidx * p.rows_max + r) * 2] = mx;
        p.part_ml[(pidx * p.rows_max + r) * 2 + 1] = den;
      }
    }
    // The generic-proxy writes above must not be overtaken by the next item's asynchronous copies.
    if (USE_TMA) asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
}

// ---------------------------------------------------------------------------------------
// The same kernel with a producer warp.  One extra warp does nothing but draw work items and
// issue their TMA copies, running ahead of the consumer warps across item boundaries, so
// the stream of tiles does not stop while the consumers merge one item and start the next.
//   work ring : the producer publishes item numbers (work_full / work_empty, 2 slots)
//   tiles     : full[stage] (tile landed, TMA) / empty[stage] (every consumer warp has left it)
// The consumers merge their partial results in the stage of the item's last tile and release
// that stage only afterwards, so no extra shared memory is needed.
// All waits are bounded; a wait that runs out sets SB_ERR_TIMEOUT and makes the warp leave.
// ---------------------------------------------------------------------------------------
constexpr int WS_STAGES = 2;
constexpr int WS_RING = 2;
constexpr int WS_NT = (D8_WARPS + 1) * 32;

struct WsItem {
  int b, m, begin, end, kv_lo, n_tiles, qs, q_len, row0;
};

__device__ __forceinline__ bool ws_item(const AttnParams& p, int work, WsItem& w) {
  const int item = work / p.num_kv_heads;
  w.m = work - item * p.num_kv_heads;
  w.b = p.items[2 * item];
  if (w.b < 0) return false;  // filler item of a fixed-size work list
  const int chunk_index = p.items[2 * item + 1];
  w.row0 = p.cu_q[w.b];
  w.q_len = p.cu_q[w.b + 1] - w.row0;
  w.qs = p.q_start[w.b];
  w.kv_lo = p.window > 0 ? max(w.qs - p.window + 1, 0) : 0;
  const int kv_hi = w.qs + w.q_len;
  w.begin = max(chunk_index * p.chunk, (w.kv_lo / 64) * 64);
  w.end = min((chunk_index + 1) * p.chunk, kv_hi);
  w.n_tiles = w.end > w.begin ? (w.end - w.begin + D8_BN - 1) / D8_BN : 0;
  return true;
}

__device__ __forceinline__ void mbar_arrive_one(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(WS_NT)
attn_decode8ws_kernel(const AttnParams p, int* work_counter, int total_work, const __grid_constant__ CUtensorMap tmap,
                      int box_rows) {
  constexpr int TILE_ELEMS = D8_BN * DH;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* aligned = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  bf16* sk = reinterpret_cast<bf16*>(aligned);  // [STAGES] key tiles
  bf16* sv = sk + WS_STAGES * TILE_ELEMS;       // [STAGES] value tiles
  __shared__ __align__(8) uint64_t full[WS_STAGES], empty[WS_STAGES], work_full[WS_RING], work_empty[WS_RING];
  __shared__ int work_ring[WS_RING];
  __shared__ float wm[D8_WARPS * 8], wl[D8_WARPS * 8];  // per warp and query row: running max, sum
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int group = p.num_q_heads / p.num_kv_heads;
  if (threadIdx.x == 0) {
    for (int i = 0; i < WS_STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], D8_WARPS);
    }
    for (int i = 0; i < WS_RING; ++i) {
      mbar_init(&work_full[i], 1);
      mbar_init(&work_empty[i], D8_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  // Launched early (programmatic dependent launch), the kernel before this one may still be
  // writing the queries and the newest keys and values.  Everything else this kernel reads (work
  // list, lengths, block table, older keys and values) is older than that kernel, so the producer
  // fetches tiles of older keys at once and waits only before a tile that may hold new ones; the
  // consumers wait before they read queries or write results.
  if (warp == D8_WARPS) {
    // ---- producer: one thread ------------------------------------------------------------
    if (lane != 0) return;
    unsigned seq = 0;  // tiles issued so far
    bool waited = false;
    if (!p.older_keys_settled) {  // the caller cannot vouch for the older keys: wait before any tile
      pdl_wait();
      waited = true;
    }
    for (unsigned wi = 0;; ++wi) {
      // The first item is the block's own index; further ones come from the counter.
      const int work = wi == 0 ? (int)blockIdx.x : (int)gridDim.x + atomicAdd(work_counter, 1);
      const int slot = wi % WS_RING;
      if (wi >= WS_RING && !mbar_wait_bounded(&work_empty[slot], (wi / WS_RING - 1) & 1)) {
        atomicOr(p.err, SB_ERR_TIMEOUT);
        return;
      }
      work_ring[slot] = work;
      mbar_arrive_one(&work_full[slot]);  // release: the consumers see the slot's content
      if (work >= total_work) return;
      WsItem w;
      if (!ws_item(p, work, w)) continue;
      for (int ti = 0; ti < w.n_tiles; ++ti, ++seq) {
        const int stage = seq % WS_STAGES;
        if (seq >= WS_STAGES && !mbar_wait_bounded(&empty[stage], (seq / WS_STAGES - 1) & 1)) {
          atomicOr(p.err, SB_ERR_TIMEOUT);
          return;
        }
        const int j0 = w.begin + ti * D8_BN;
        if (!waited && j0 + D8_BN > w.qs) {  // keys from position qs on are written by the step itself
          pdl_wait();
          waited = true;
        }
        int boxes = 0;
        for (int r = 0; r < D8_BN; r += box_rows) {
          const int j = j0 + r;
          if (j >= w.end || j + box_rows <= w.kv_lo) continue;
          const long long page = p.block_table[(size_t)w.b * p.max_pages + j / p.page_size];
          if (page >= 0 && page < p.num_pages) ++boxes;
        }
        mbar_arrive_expect_tx(&full[stage], boxes * 2 * SLABS * box_rows * 128);
        for (int r = 0; r < D8_BN; r += box_rows) {
          const int j = j0 + r;
          if (j >= w.end || j + box_rows <= w.kv_lo) continue;
          const long long page = p.block_table[(size_t)w.b * p.max_pages + j / p.page_size];
          if (page < 0 || page >= p.num_pages) {
            atomicOr(p.err, SB_ERR_BAD_PAGE);
            continue;
          }
          const long long krow = ((page * 2) * p.num_kv_heads + w.m) * p.page_size + (j & (p.page_size - 1));
          const long long vrow = krow + (long long)p.num_kv_heads * p.page_size;
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl) {
            tma_load_box(sk + (size_t)stage * TILE_ELEMS + sl * SLAB_ELEMS + r * 64, &tmap, sl * 64, (int)krow, &full[stage]);
            tma_load_box(sv + (size_t)stage * TILE_ELEMS + sl * SLAB_ELEMS + r * 64, &tmap, sl * 64, (int)vrow, &full[stage]);
          }
        }
      }
    }
  }

  // ---- consumers: D8_WARPS warps, 16 keys of every tile each ---------------------------------
  unsigned seq = 0;  // tiles consumed so far
  for (unsigned wi = 0;; ++wi) {
    const int slot = wi % WS_RING;
    if (!mbar_wait_bounded(&work_full[slot], (wi / WS_RING) & 1)) {
      if (lane == 0) atomicOr(p.err, SB_ERR_TIMEOUT);
      return;
    }
    const int work = work_ring[slot];
    __syncwarp();
    if (lane == 0) mbar_arrive_one(&work_empty[slot]);
    if (work >= total_work) return;
    WsItem w;
    if (!ws_item(p, work, w)) continue;
    const int rows_valid = w.q_len * group;  // <= 8 by the host's routing
    const size_t pidx = (size_t)(work / p.num_kv_heads) * p.num_kv_heads + w.m;
    pdl_wait();  // before the first read of a query and the first write of a result
    pdl_launch_dependents();
    if (w.n_tiles == 0) {
      // Nothing of this chunk is visible: an empty partial result.
      if (warp == 0) {
        for (int i = lane; i < rows_valid * DH; i += 32) p.part_o[pidx * p.rows_max * DH + i] = 0.f;
        if (lane < rows_valid) {
          p.part_ml[(pidx * p.rows_max + lane) * 2] = -INFINITY;
          p.part_ml[(pidx * p.rows_max + lane) * 2 + 1] = 0.f;
        }
      }
      continue;
    }
    uint32_t qf[DH / 16][2];
    {
      const bool valid = g < rows_valid;
      const bf16* qrow = p.q + ((size_t)(w.row0 + (valid ? g / group : 0)) * p.num_q_heads + w.m * group +
                                (valid ? g % group : 0)) * DH;
#pragma unroll
      for (int ks = 0; ks < DH / 16; ++ks) {
        qf[ks][0] = valid ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t) : 0u;
        qf[ks][1] = valid ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t) : 0u;
      }
    }
    const int pos0 = 2 * t < rows_valid ? w.qs + (2 * t) / group : -1;
    const int pos1 = 2 * t + 1 < rows_valid ? w.qs + (2 * t + 1) / group : -1;
    const float inv_cap = p.cap > 0.f ? 1.0f / p.cap : 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[DH / 16][4];
#pragma unroll
    for (int d = 0; d < DH / 16; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

    int last_stage = 0;
    for (int it = 0; it < w.n_tiles; ++it, ++seq) {
      const int stage = seq % WS_STAGES;
      last_stage = stage;
      if (!mbar_wait_bounded(&full[stage], (seq / WS_STAGES) & 1)) {
        if (lane == 0) atomicOr(p.err, SB_ERR_TIMEOUT);
        return;
      }
      const bf16* kt = sk + (size_t)stage * TILE_ELEMS;
      const bf16* vt = sv + (size_t)stage * TILE_ELEMS;
      const int key0 = warp * 16;
      const int j_first = w.begin + it * D8_BN + key0;
      if (j_first < w.kv_lo || j_first + 16 > w.end) {
        // Value rows of keys that are not the request's must read as zeros (only this warp reads them).
        for (int i = lane; i < 16 * (DH / 8); i += 32) {
          const int r = i / (DH / 8), c = i - r * (DH / 8);
          const int j = j_first + r;
          if (j < w.kv_lo || j >= w.end)
            *reinterpret_cast<uint4*>(const_cast<bf16*>(tile_at<true>(vt, key0 + r, c * 8))) = make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
      }
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < DH / 16; ks += 2) {
        uint32_t a[4], a2[4];
        ldmatrix_x4(a, tile_at<true>(kt, key0 + (lane & 15), ks * 16 + (lane >> 4) * 8));
        mma16816(s0, a, qf[ks][0], qf[ks][1]);
        if (ks + 1 < DH / 16) {
          ldmatrix_x4(a2, tile_at<true>(kt, key0 + (lane & 15), (ks + 1) * 16 + (lane >> 4) * 8));
          mma16816(s1, a2, qf[ks + 1][0], qf[ks + 1][1]);
        }
      }
      float sc[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s0[e] + s1[e];
        if (p.cap > 0.f) v = p.cap * fast_tanh(v * inv_cap);
        const int j = j_first + g + (e >> 1) * 8;
        const int pos = (e & 1) ? pos1 : pos0;
        const bool keep = j <= pos && (p.window <= 0 || pos - j < p.window);
        sc[e] = keep ? v * LOG2E : -INFINITY;
      }
      float mx0 = fmaxf(sc[0], sc[2]), mx1 = fmaxf(sc[1], sc[3]);
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
      }
      const float new0 = fmaxf(m0, mx0), new1 = fmaxf(m1, mx1);
      const float use0 = new0 == -INFINITY ? 0.f : new0, use1 = new1 == -INFINITY ? 0.f : new1;
      const float alpha0 = fast_exp2(m0 - use0), alpha1 = fast_exp2(m1 - use1);
      m0 = new0;
      m1 = new1;
      const float p0 = fast_exp2(sc[0] - use0), p1 = fast_exp2(sc[1] - use1);
      const float p2 = fast_exp2(sc[2] - use0), p3 = fast_exp2(sc[3] - use1);
      l0 = l0 * alpha0 + p0 + p2;
      l1 = l1 * alpha1 + p1 + p3;
      if (__any_sync(0xffffffffu, alpha0 != 1.f || alpha1 != 1.f)) {
#pragma unroll
        for (int d = 0; d < DH / 16; ++d) {
          o[d][0] *= alpha0;
          o[d][1] *= alpha1;
          o[d][2] *= alpha0;
          o[d][3] *= alpha1;
        }
      }
      const uint32_t b0 = movmatrix_trans(pack_bf16(p0, p1));
      const uint32_t b1 = movmatrix_trans(pack_bf16(p2, p3));
#pragma unroll
      for (int d = 0; d < DH / 16; ++d) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, tile_at<true>(vt, key0 + ((lane >> 4) & 1) * 8 + (lane & 7), d * 16 + ((lane >> 3) & 1) * 8));
        mma16816(o[d], a, b0, b1);
      }
      if (it + 1 < w.n_tiles) {  // the last tile's stage is kept for the merge
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // (after the zeroing above, if any)
        __syncwarp();
        if (lane == 0) mbar_arrive_one(&empty[stage]);
      }
    }
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, off);
      l1 += __shfl_xor_sync(0xffffffffu, l1, off);
    }
    // Merge the consumer warps in the last tile's stage: all have left it when the first
    // consumer barrier is passed (the producer cannot refill it before `empty` is signalled).
    asm volatile("bar.sync 1, %0;\n" ::"n"(D8_WARPS * 32) : "memory");
    float* wo = reinterpret_cast<float*>(sk + (size_t)last_stage * TILE_ELEMS);  // [W][rows_valid][DH]
    if (g == 0) {
      wm[warp * 8 + 2 * t] = m0;
      wm[warp * 8 + 2 * t + 1] = m1;
      wl[warp * 8 + 2 * t] = l0;
      wl[warp * 8 + 2 * t + 1] = l1;
    }
#pragma unroll
    for (int d = 0; d < DH / 16; ++d) {
      if (2 * t < rows_valid) {
        wo[((size_t)warp * rows_valid + 2 * t) * DH + d * 16 + g] = o[d][0];
        wo[((size_t)warp * rows_valid + 2 * t) * DH + d * 16 + g + 8] = o[d][2];
      }
      if (2 * t + 1 < rows_valid) {
        wo[((size_t)warp * rows_valid + 2 * t + 1) * DH + d * 16 + g] = o[d][1];
        wo[((size_t)warp * rows_valid + 2 * t + 1) * DH + d * 16 + g + 8] = o[d][3];
      }
    }
    asm volatile("bar.sync 1, %0;\n" ::"n"(D8_WARPS * 32) : "memory");
    for (int i = threadIdx.x; i < rows_valid * DH; i += D8_WARPS * 32) {
      const int r = i / DH, d = i - r * DH;
      float mx = -INFINITY;
#pragma unroll
      for (int x = 0; x < D8_WARPS; ++x) mx = fmaxf(mx, wm[x * 8 + r]);
      float num = 0.f, den = 0.f;
      if (mx != -INFINITY) {
#pragma unroll
        for (int x = 0; x < D8_WARPS; ++x) {
          const float scale = fast_exp2(wm[x * 8 + r] - mx);
          num += scale * wo[((size_t)x * rows_valid + r) * DH + d];
          den += scale * wl[x * 8 + r];
        }
      }
      p.part_o[(pidx * p.rows_max + r) * DH + d] = den > 0.f ? num / den : 0.f;
      if (d == 0) {
        p.part_ml[(pidx * p.rows_max + r) * 2] = mx;
        p.part_ml[(pidx * p.rows_max + r) * 2 + 1] = den;
      }
    }
    // Hand the stage back: the reads above are done, and the TMA must not overtake the writes.
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive_one(&empty[last_stage]);
  }
}

// Merges the chunks of every (token, query head): one block each.  Its warps take the
// chunks in turn (warp w: chunks w, w + 8, ...), then add up in a fixed order.
constexpr int COMBINE_WARPS = 8;
constexpr int DPL = (DH + 31) / 32;  // output elements per lane

__global__ void __launch_bounds__(COMBINE_WARPS * 32)
attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                    const int* __restrict__ token_seq, const int* __restrict__ cu_q,
                    const int* __restrict__ split_start, const int* __restrict__ split_count,
                    bf16* __restrict__ out, int num_q_heads, int num_kv_heads, int rows_max,
                    int* __restrict__ work_counter) {
  __shared__ float s_acc[COMBINE_WARPS][DH];
  __shared__ float s_den[COMBINE_WARPS];
  __shared__ float s_max[COMBINE_WARPS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tkn = blockIdx.x / num_q_heads, h = blockIdx.x - tkn * num_q_heads;
  // The step's own lists are older than the split-key kernel: read them while it still runs.
  const int b = token_seq[tkn];
  const int count = split_count[b];
  const int group = num_q_heads / num_kv_heads, m = h / group;
  const int r = (tkn - cu_q[b]) * group + h % group;
  const size_t base = ((size_t)split_start[b] * num_kv_heads + m) * rows_max + r;
  const size_t stride = (size_t)num_kv_heads * rows_max;  // from one chunk's partial to the next
  pdl_wait();
  pdl_launch_dependents();
  // The split-key kernel has finished: put its work counter back to zero for the next launch.
  if (blockIdx.x == 0 && threadIdx.x == 0) *work_counter = 0;
  if (count <= 0) return;  // this sequence went through the prefill kernel
  // One pass: every warp merges its share of the chunks with a running maximum (the loads of a
  // few chunks are in flight together), then the warps' results are merged through shared memory.
  float m_run = -INFINITY, den = 0.f;
  float acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
#pragma unroll 4
  for (int s = warp; s < count; s += COMBINE_WARPS) {
    const size_t pidx = base + s * stride;
    const float ms = part_ml[pidx * 2], ls = part_ml[pidx * 2 + 1];
    float o[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = lane + 32 * i;
      o[i] = d < DH ? part_o[pidx * DH + d] : 0.f;
    }
    if (ls > 0.f) {  // an empty chunk stored zeros
      const float m_new = fmaxf(m_run, ms);
      const float keep = fast_exp2(m_run - m_new);  // 0 for the first chunk
      const float w = ls * fast_exp2(ms - m_new);
      den = den * keep + w;
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[i] = fmaf(w, o[i], acc[i] * keep);
      m_run = m_new;
    }
  }
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + 32 * i;
    if (d < DH) s_acc[warp][d] = acc[i];
  }
  if (lane == 0) {
    s_den[warp] = den;
    s_max[warp] = m_run;
  }
  __syncthreads();
  float mx = -INFINITY;
#pragma unroll
  for (int w = 0; w < COMBINE_WARPS; ++w) mx = fmaxf(mx, s_max[w]);
  float scale[COMBINE_WARPS];
  den = 0.f;
#pragma unroll
  for (int w = 0; w < COMBINE_WARPS; ++w) {
    scale[w] = s_max[w] == -INFINITY ? 0.f : fast_exp2(s_max[w] - mx);
    den += s_den[w] * scale[w];
  }
  const float inv = den > 0.f ? 1.0f / den : 0.f;
  bf16* op = out + ((size_t)tkn * num_q_heads + h) * DH;
  for (int d = threadIdx.x; d < DH; d += COMBINE_WARPS * 32) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < COMBINE_WARPS; ++w) v = fmaf(s_acc[w][d], scale[w], v);
    op[d] = __float2bfloat16_rn(v * inv);
  }
}

constexpr size_t prefill_smem(int rows) { return (size_t)(rows + 4 * BN) * PITCH * sizeof(bf16); }
constexpr size_t DECODE_SMEM_KV = (size_t)(16 + 2 * DEC_STAGES * DEC_BN) * PITCH * sizeof(bf16);
constexpr size_t DECODE_SMEM_MERGE =
    16 * PITCH * sizeof(bf16) + (size_t)(2 * DEC_WARPS * 16 + DEC_WARPS * 16 * DH) * sizeof(float);
constexpr size_t DECODE_SMEM = DECODE_SMEM_KV > DECODE_SMEM_MERGE ? DECODE_SMEM_KV : DECODE_SMEM_MERGE;
constexpr size_t DECODE8_SMEM_KV = (size_t)(2 * D8_STAGES * D8_BN) * PITCH * sizeof(bf16);
constexpr size_t DECODE8_SMEM_TMA_KV = (size_t)(2 * D8_STAGES * D8_BN) * DH * sizeof(bf16);
constexpr size_t DECODE8_SMEM_MERGE = (size_t)(2 * D8_WARPS * 8 + D8_WARPS * 8 * DH) * sizeof(float);
constexpr size_t DECODE8_SMEM = DECODE8_SMEM_KV > DECODE8_SMEM_MERGE ? DECODE8_SMEM_KV : DECODE8_SMEM_MERGE;

}  // namespace

// Opts the kernel in to `smem` bytes of dynamic shared memory and reports how many of its
// blocks the device holds at once.
template <typename Kernel>
static int blocks_resident(Kernel kernel, int threads, size_t smem, int* out) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  int per_sm = 0, sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem);
  if (e != cudaSuccess) return (int)e;
  *out = (per_sm > 0 ? per_sm : 1) * (sms > 0 ? sms : 1);
  return 0;
}

#define SB_CONCAT2(a, b) a##b
#define SB_CONCAT(a, b) SB_CONCAT2(a, b)
#define SB_FN(name) SB_CONCAT(SB_CONCAT(name, _hd), SB_HEAD_DIM)

// Ragged prefill attention.  items: [num_items, 2] (sequence, first token of a tile of
// rows_per_tile / G tokens); rows_per_tile is 64 or 128.  Tiles of 64 rows run with two key
// groups (8 warps) unless single_key_group is set.
extern "C" int SB_FN(sb_attn_prefill)(const void* q, const void* cache, const int* block_table, int max_pages,
                                      const int* cu_q, const int* q_start, void* out, int num_q_heads,
                                      int num_kv_heads, int page_size, int num_pages, float cap, int window,
                                      const int* items, int num_items, int rows_per_tile, int single_key_group,
                                      int* err, cudaStream_t stream) {
  if (num_items == 0) return 0;
  if (num_kv_heads <= 0 || num_q_heads % num_kv_heads || num_q_heads / num_kv_heads > rows_per_tile) return -8;
  AttnParams p{};
  p.q = (const bf16*)q; p.cache = (const bf16*)cache; p.block_table = block_table; p.max_pages = max_pages;
  p.cu_q = cu_q; p.q_start = q_start; p.out = (bf16*)out; p.num_q_heads = num_q_heads;
  p.num_kv_heads = num_kv_heads; p.page_size = page_size; p.num_pages = num_pages; p.cap = cap;
  p.window = window; p.items = items; p.err = err;
  // The merge of two key groups needs [BM][DH] floats where the tiles were.
  constexpr bool split_fits = (size_t)(2 * 64 + 64 * DH) * sizeof(float) <= (size_t)4 * BN * PITCH * sizeof(bf16);
  if (rows_per_tile == 128) {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<8, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)prefill_smem(128));
      if (e != cudaSuccess) return (int)e;
      configured = true;
    }
    sb_launch(attn_prefill_kernel<8, 1>, dim3(num_items, num_kv_heads), 256, prefill_smem(128), stream, p);
  } else if (rows_per_tile == 64 && split_fits && !single_key_group) {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<4, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)prefill_smem(64));
      if (e != cudaSuccess) return (int)e;
      configured = true;
    }
    sb_launch(attn_prefill_kernel<4, 2>, dim3(num_items, num_kv_heads), 256, prefill_smem(64), stream, p);
  } else if (rows_per_tile == 64) {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<4, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)prefill_smem(64));
      if (e != cudaSuccess) return (int)e;
      configured = true;
    }
    sb_launch(attn_prefill_kernel<4, 1>, dim3(num_items, num_kv_heads), 128, prefill_smem(64), stream, p);
  } else {
    return -8;
  }
  SB_LAUNCH_CHECK();
  return 0;
}

// Split-key attention for sequences with at most 16 query rows per kv head, and the merge.
// items: [num_items, 2] (sequence or -1, chunk index); chunk: keys per chunk, a multiple of 64;
// part_o / part_ml: scratch of num_items * Hkv * rows_max * (DH | 2) floats;
// work_counter: one int that is zero before the first launch; the merge kernel zeroes it again;
// split_start / split_count: per sequence, its range of items (count 0: not handled here).
// older_keys_settled: the caller vouches that every key and value below q_start was written
// before the kernel launched just before this one (true inside the engine, where they come from
// earlier steps); the kernel may then fetch them before that kernel has finished.
extern "C" int SB_FN(sb_attn_decode)(const void* q, const void* cache, const int* block_table, int max_pages,
                                     const int* cu_q, const int* q_start, const int* token_seq, void* out,
                                     int num_tokens, int num_q_heads, int num_kv_heads, int page_size,
                                     int num_pages, float cap, int window, const int* items, int num_items,
                                     int chunk, float* part_o, float* part_ml, int* work_counter,
                                     int rows_max, const int* split_start, const int* split_count, int variant,
                                     const void* tensor_map, int older_keys_settled, int* err,
                                     cudaStream_t stream) {
  // variant: 0 picks the kernel by rows_max (<= 8: the turned-round kernel, fed by TMA through a
  // producer warp when a tensor map is given and the shapes allow); 1 forbids TMA; 2 uses TMA
  // without the producer warp; 16 forces the 16-row kernel.
  if (num_items == 0) return 0;
  if (num_kv_heads <= 0 || num_q_heads % num_kv_heads || rows_max > 16 || chunk % 64) return -8;
  AttnParams p{};
  p.q = (const bf16*)q; p.cache = (const bf16*)cache; p.block_table = block_table; p.max_pages = max_pages;
  p.cu_q = cu_q; p.q_start = q_start; p.out = (bf16*)out; p.num_q_heads = num_q_heads;
  p.num_kv_heads = num_kv_heads; p.page_size = page_size; p.num_pages = num_pages; p.cap = cap;
  p.window = window; p.items = items; p.chunk = chunk; p.part_o = part_o; p.part_ml = part_ml;
  p.rows_max = rows_max; p.older_keys_settled = older_keys_settled; p.err = err;
  const int total_work = num_items * num_kv_heads;
  const bool power_of_two_pages = (page_size & (page_size - 1)) == 0;
  constexpr size_t ws_merge = (size_t)(D8_WARPS * 8 * DH) * sizeof(float);
  constexpr bool ws_fits = ws_merge <= (size_t)D8_BN * DH * sizeof(bf16);  // the merge borrows one key tile
  if (rows_max <= 8 && (variant == 0 || variant == 3) && TMA_OK && ws_fits && tensor_map != nullptr && power_of_two_pages) {
    static int resident_ws = 0;
    constexpr size_t smem = (size_t)(2 * WS_STAGES * D8_BN) * DH * sizeof(bf16) + 1024;
    if (resident_ws == 0) {
      int rc = blocks_resident(attn_decode8ws_kernel, WS_NT, smem, &resident_ws);
      if (rc) return rc;
    }
    CUtensorMap map;
    memcpy(&map, tensor_map, sizeof(map));
    const int box_rows = page_size < D8_BN ? page_size : D8_BN;
    sb_launch_early(attn_decode8ws_kernel, total_work < resident_ws ? total_work : resident_ws, WS_NT, smem, stream,
        p, work_counter, total_work, map, box_rows);
  } else if (rows_max <= 8 && variant != 16 && TMA_OK && tensor_map != nullptr && power_of_two_pages && variant != 1) {
    static int resident_tma = 0;
    constexpr size_t smem = (DECODE8_SMEM_TMA_KV > DECODE8_SMEM_MERGE ? DECODE8_SMEM_TMA_KV : DECODE8_SMEM_MERGE) + 1024;
    if (resident_tma == 0) {
      int rc = blocks_resident(attn_decode8_kernel<true>, D8_NT, smem, &resident_tma);
      if (rc) return rc;
    }
    CUtensorMap map;
    memcpy(&map, tensor_map, sizeof(map));
    const int box_rows = page_size < D8_BN ? page_size : D8_BN;
    sb_launch(attn_decode8_kernel<true>, total_work < resident_tma ? total_work : resident_tma, D8_NT, smem, stream,
        p, work_counter, total_work, map, box_rows);
  } else if (rows_max <= 8 && variant != 16) {
    static int resident8 = 0;
    if (resident8 == 0) {
      int rc = blocks_resident(attn_decode8_kernel<false>, D8_NT, DECODE8_SMEM, &resident8);
      if (rc) return rc;
    }
    CUtensorMap map;
    memset(&map, 0, sizeof(map));
    sb_launch(attn_decode8_kernel<false>, total_work < resident8 ? total_work : resident8, D8_NT, DECODE8_SMEM, stream,
        p, work_counter, total_work, map, 0);
  } else {
    static int resident = 0;  // blocks of this kernel the device holds at once
    if (resident == 0) {
      int rc = blocks_resident(attn_decode_kernel, DEC_NT, DECODE_SMEM, &resident);
      if (rc) return rc;
    }
    sb_launch(attn_decode_kernel, total_work < resident ? total_work : resident, DEC_NT, DECODE_SMEM, stream,
        p, work_counter, total_work);
  }
  SB_LAUNCH_CHECK();
  sb_launch_early(attn_combine_kernel, (unsigned)(num_tokens * num_q_heads), COMBINE_WARPS * 32, 0, stream,
      part_o, part_ml, token_seq, cu_q, split_start, split_count, (bf16*)out, num_q_heads, num_kv_heads,
      rows_max, work_counter);
  SB_LAUNCH_CHECK();
  return 0;
}

// How many blocks of the split-key kernel for at most 8 query rows the device holds at once (the
// size of its persistent grid): the host cuts the keys into chunks so that the work items fill
// this many blocks evenly.  Returns the count, or a negative status.
extern "C" int SB_FN(sb_attn_decode_resident)(int with_tensor_map) {
  int resident = 0, rc;
  constexpr size_t ws_merge = (size_t)(D8_WARPS * 8 * DH) * sizeof(float);
  constexpr bool ws_fits = ws_merge <= (size_t)D8_BN * DH * sizeof(bf16);
  if (with_tensor_map && TMA_OK && ws_fits) {
    constexpr size_t smem = (size_t)(2 * WS_STAGES * D8_BN) * DH * sizeof(bf16) + 1024;
    rc = blocks_resident(attn_decode8ws_kernel, WS_NT, smem, &resident);
  } else {
    rc = blocks_resident(attn_decode8_kernel<false>, D8_NT, DECODE8_SMEM, &resident);
  }
  return rc ? (rc > 0 ? -rc : rc) : resident;
}

// Writes into `map_out` (128 bytes, host memory) the tensor map of one cache storage
// [pages, 2, heads, page_size, DH] seen as a matrix of total_rows x DH, fetched in boxes of
// box_rows x 64 elements with the 128-byte swizzle.  Returns 0, -11 when the head size does
// not allow it (not a multiple of 64), or -12 when the driver refuses.
extern "C" int SB_FN(sb_attn_tensor_map)(void* map_out, const void* cache, long long total_rows, int box_rows) {
  if (!TMA_OK || box_rows <= 0 || box_rows > 256) return -11;
  typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeTiled encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status) != cudaSuccess || !fn)
      return -12;
    encode = (EncodeTiled)fn;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)DH, (cuuint64_t)total_rows};
  const cuuint64_t strides[1] = {(cuuint64_t)DH * sizeof(bf16)};
  const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1u, 1u};
  CUtensorMap map;
  const CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box,
                            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -12;
  memcpy(map_out, &map, sizeof(map));
  return 0;
}
