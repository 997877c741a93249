// The last step of the weight-streaming product for a serving batch (gemm_stream_tc.cu): a block holds a tile of float32 sums [tokens][128 local rows] in shared
// memory; with k split over the blocks of a cluster every block holds such a tile of partial
// sums, and block `rank` finishes the tokens rank, rank + ks, ... by adding the tiles of all
// blocks in rank order through distributed shared memory (nothing is added atomically, so the
// result does not depend on timing).
//
// Local row r of the tile is weight row base0 + r for r < 64 and base0 + second + (r - 64)
// beyond.  Epilogues: 0 bfloat16; 1 float32 with soft cap (simply/model_lib.py:107-109, the
// output layer); 2 gated activation: rows r < 64 are gate rows, r + 64 their up rows
// (simply/model_lib.py:722-726); 3 the fused q, k, v projection: rows r < 64 are 64 dims of a
// head, r + 64 the dims half a head further; rotation (simply/utils/position_encoding.py:83-110),
// query scale (simply/model_lib.py:2014-2019), keys and values into the pages of the cache.
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"

namespace sbg {

constexpr int TILE_ROWS = 128;          // local rows of a tile of sums
constexpr int RSTRIDE = TILE_ROWS + 4;  // floats of a token's row in the tile (the 4 spread the banks)

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

// What a block needs to know about its tile.
struct TileGeometry {
  int base0, second, head, rows_end;
};

template <int EPI>
__device__ __forceinline__ TileGeometry tile_geometry(int tile, int N, const RopeStore& rs) {
  TileGeometry t;
  const int half = EPI == 3 ? rs.head_dim / 2 : 0;
  const int slices = EPI == 3 ? half / 64 : 1;
  t.head = EPI == 3 ? tile / slices : 0;
  t.base0 = EPI == 3 ? t.head * rs.head_dim + (tile - t.head * slices) * 64 : (EPI == 2 ? tile * 64 : tile * TILE_ROWS);
  t.second = EPI == 3 ? half : (EPI == 2 ? N / 2 : 64);
  t.rows_end = EPI == 2 ? N / 2 : N;
  return t;
}

__device__ __forceinline__ float gated_act(float g, int act) {
  if (act == 0) {
    const float c = 0.7978845608028654f;
    return 0.5f * g * (1.0f + tanhf(c * (g + 0.044715f * g * g * g)));
  }
  if (act == 1) return g / (1.0f + expf(-g));
  return fmaxf(g, 0.f);
}

// All threads of the block (and of every block of the cluster) call this once the block's tile
// `sums` [tokens][RSTRIDE] is written; it begins with the barrier that makes the tile visible (of
// the cluster when ks > 1).  The first 256 threads do the work: a thread owns one local row (or one
// pair of rows) and walks its tokens, a few at a time so that their loads are in flight together.
template <int EPI>
__device__ __forceinline__ void finish_tile(float* sums, int tokens, int M, int N, int ks, int rank,
                                            const TileGeometry& tg, void* out, float cap, int act,
                                            const RopeStore& rs) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const float* tp[8];  // (only ever indexed by unrolled constants: stays in registers)
  if (ks > 1) {
    cluster.sync();
#pragma unroll
    for (int q = 0; q < 8; ++q) tp[q] = q < ks ? cluster.map_shared_rank(sums, q) : sums;
  } else {
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 8; ++q) tp[q] = sums;
  }
  auto total = [&](int token, int r) {
    float v = tp[0][(size_t)token * RSTRIDE + r];
#pragma unroll
    for (int q = 1; q < 8; ++q)
      if (q < ks) v += tp[q][(size_t)token * RSTRIDE + r];
    return v;
  };
  constexpr int ROWS = (EPI >= 2) ? 64 : TILE_ROWS;  // rows (or pairs) a token has in this tile
  constexpr int PARTS = 256 / ROWS;                  // threads that share a row, each with its own tokens
  const int last = min(M, tokens);
  if (threadIdx.x < 256) {
    const int r = threadIdx.x % ROWS, part = threadIdx.x / ROWS;
    const int n = tg.base0 + r;
    const int half = EPI == 3 ? rs.head_dim / 2 : 0;
    // This block's tokens are rank, rank + ks, ...; the threads of a row take them in turn.
    if (EPI <= 1) {
      if (n < N) {
#pragma unroll 4
        for (int token = rank + ks * part; token < last; token += ks * PARTS) {
          const float v = total(token, r);
          const size_t o = (size_t)token * N + n;
          if (EPI == 0) reinterpret_cast<bf16*>(out)[o] = __float2bfloat16_rn(v);
          else reinterpret_cast<float*>(out)[o] = cap > 0.f ? cap * tanhf(v / cap) : v;
        }
      }
    } else if (EPI == 2) {
      if (n < tg.rows_end) {
#pragma unroll 4
        for (int token = rank + ks * part; token < last; token += ks * PARTS) {
          // Round gate and up to bfloat16 first, as the unfused path stores them.
          const float gate = __bfloat162float(__float2bfloat16_rn(total(token, r)));
          const float up = __bfloat162float(__float2bfloat16_rn(total(token, 64 + r)));
          reinterpret_cast<bf16*>(out)[(size_t)token * tg.rows_end + n] = __float2bfloat16_rn(gated_act(gate, act) * up);
        }
      }
    } else {
      const int head = tg.head;
      const int j = tg.base0 - head * rs.head_dim + r;  // the dim inside the head, below half
      const bool rotates = head < rs.num_q_heads + rs.num_kv_proj && rs.cos_t != nullptr;
#pragma unroll 2
      for (int token = rank + ks * part; token < last; token += ks * PARTS) {
        // Round to bfloat16 first, as the unfused path stores the projection before it rotates.
        float a = __bfloat162float(__float2bfloat16_rn(total(token, r)));
        float b = __bfloat162float(__float2bfloat16_rn(total(token, 64 + r)));
        if (rotates) {
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
      }
    }
  }
  if (ks > 1) cluster.sync();  // no block leaves while another still reads its sums
}

}  // namespace sbg
