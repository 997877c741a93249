// Ragged paged prefill attention by pairs of blocks (tcgen05 cta_group::2), compiled once per
// head size (-DSB_HEAD_DIM=N, N = 128 or 256).  The formulas are those of attention_tc.cu:
//
//   s = q . k                 (q is already rotated and scaled)
//   s = cap * tanh(s / cap)   if cap > 0          simply/model_lib.py:621-626
//   keep k_pos <= q_pos and, with a window W, q_pos - k_pos < W
//                                                 simply/model_lib.py:469-515
//   p = softmax(s) in float32, o = p . v          simply/model_lib.py:633-637
//   query head n reads kv head n / G              simply/model_lib.py:2306-2310
//
// A pair (a cluster of two blocks) owns 256 query rows of one (sequence, kv head): each block the G
// query heads of the group for 128 / G consecutive tokens, the second block the tokens after the
// first one's.  The pair walks the keys in tiles of 128, and every product is one instruction for
// both blocks:
//   S[256 x 128]  = Q . K^T    each block holds its 128 rows of Q and the K rows of 64 of the
//                              tile's keys; its 128 rows of S land in its own tensor memory
//   P             = softmax numerators of S as bfloat16, written over S in tensor memory
//   O[256 x DH]  += P . V      each block holds the V columns of DH / 2 dims for all 128 keys; its
//                              128 rows of O stay in its own tensor memory for the whole walk
// So a block fetches half the keys and values it would fetch alone, and one thread issues half as
// many instructions of twice the size (a thread cannot issue `tcgen05.mma` faster than about one
// per 52 cycles; a 128 x 64 x 16 product is 32 cycles of work, which is what limited the single
// blocks' walk).
// Roles in each block: warp 0 TMA producer of Q (once) and of its half of the key tiles, warp 2 of
// its half of the value tiles; in the pair's first block (rank 0) warps 1 and 3 issue Q.K^T and
// P.V for the pair (one thread each); warps 4..19 softmax and epilogue, four threads per query row
// with 32 of the tile's 128 columns each.
// Barriers.  Of rank 0: q_full, k_full[s] (both blocks' TMA count their bytes there), p_ready[b]
// (the softmax warps of both blocks arrive: P is written, and the block's value tile has landed).
// Of each block, reached by `tcgen05.commit` with multicast: s_full[b] (S of a tile is complete;
// its key stage is free), pv_done[b] (P.V of a tile is complete; S buffer and value stage are
// free), o_done.  Local: v_full[s] (the block's own value tile), x_bar, l_bar (the four threads of
// a row exchange maxima and sums).  Every wait is bounded; a wait that runs out sets
// SB_ERR_TIMEOUT, and both blocks still reach the cluster's barrier and release their tensor memory.
#include <float.h>

#include "common.cuh"
#include "tma_mbar.cuh"

#ifndef SB_HEAD_DIM
#define SB_HEAD_DIM 256
#endif

#if SB_HEAD_DIM == 128 || SB_HEAD_DIM == 256

namespace {

using namespace sbx;

constexpr int DH = SB_HEAD_DIM;
constexpr int BM = 128;         // query rows of a block
constexpr int BN = 128;         // keys of a tile
constexpr int KH = BN / 2;      // keys whose K rows a block holds
constexpr int VD = DH / 2;      // dims whose V columns a block holds
constexpr int SLABS = DH / 64;  // slabs of 64 dims of Q and K
constexpr int VSLABS = VD / 64;
constexpr int Q_BYTES = BM * DH * 2, K_BYTES = KH * DH * 2, V_BYTES = BN * VD * 2;
constexpr int STAGES = 2;
constexpr int SPLIT = 4;                 // softmax threads per query row
constexpr int CW = BN / SPLIT;           // columns of a key tile per softmax thread
constexpr int OW = DH / SPLIT;           // columns of O per softmax thread in the epilogue
static_assert(CW == 32 && OW % 16 == 0, "tensor-memory loads of 32 and 16 columns");
constexpr int PAIR_THREADS = 128 + 128 * SPLIT;
constexpr int S_COL0 = 0, O_COL0 = 2 * BN;  // two S buffers, O behind them
constexpr int TMEM_COLS = 512;
static_assert(O_COL0 + DH <= TMEM_COLS, "tensor memory has 512 columns");
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.f;
constexpr size_t PAIR_SMEM = (size_t)Q_BYTES + STAGES * (K_BYTES + V_BYTES) + 1024;

struct PairParams {
  const bf16* q;  // [T, Hq, DH]
  const int* block_table;
  int max_pages;
  const int* cu_q;
  const int* q_start;
  bf16* out;
  int num_q_heads, num_kv_heads, page_size, num_pages;
  float cap;
  int window;
  const int* items;  // per pair, in launch order: (sequence, first token of its 256 / G tokens, kv head)
  int* err;
};

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

__global__ void __launch_bounds__(PAIR_THREADS)
attn_prefill_pair_kernel(const PairParams p, const __grid_constant__ CUtensorMap map_q,
                         const __grid_constant__ CUtensorMap map_kv, const __grid_constant__ CUtensorMap map_out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sq = base;                          // [SLABS][128 rows][128 B]; at the end the result
  unsigned char* sk = sq + Q_BYTES;                  // [STAGES][SLABS][64 keys][128 B]
  unsigned char* sv = sk + STAGES * K_BYTES;         // [STAGES][VSLABS][128 keys][128 B]
  __shared__ __align__(8) uint64_t q_full, k_full[STAGES], v_full[STAGES], s_full[2], p_ready[2], pv_done[2], o_done,
      x_bar[4], l_bar[4];
  __shared__ float row_max[2][SPLIT][BM];  // the parts' row maxima of a tile, by tile parity
  __shared__ float row_sum[SPLIT][BM];     // at the end: the threads' partial row sums
  __shared__ uint32_t tmem_slot;
  __shared__ int s_failed;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int b = p.items[3 * pair], i0_pair = p.items[3 * pair + 1], m = p.items[3 * pair + 2];
  const int group = p.num_q_heads / p.num_kv_heads;
  const int tokens_per_tile = BM / group;
  const int row0 = p.cu_q[b], q_len = p.cu_q[b + 1] - row0, qs = p.q_start[b];
  const int i0 = i0_pair + rank * tokens_per_tile;                    // this block's first token
  const int ntok = max(min(tokens_per_tile, q_len - i0), 0);          // (none: the sequence ends in the first block)
  const int rows_valid = ntok * group;
  const int ntok_pair = min(2 * tokens_per_tile, q_len - i0_pair);
  const int p0 = qs + i0;                                             // this block's first position
  const int pair_p0 = qs + i0_pair, pair_p1 = qs + i0_pair + ntok_pair - 1;
  const int kv_lo = p.window > 0 ? max(qs - p.window + 1, 0) : 0;    // lowest key the request still holds
  const int lo = p.window > 0 ? max(pair_p0 - p.window + 1, 0) : 0;  // lowest key the pair can see
  const int kv_hi = pair_p1 + 1;
  const int tile0 = (lo / BN) * BN;
  const int n_tiles = (kv_hi - tile0 + BN - 1) / BN;

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 2);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&k_full[s], 2);
      mbar_init(&v_full[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 2 * 4 * SPLIT);  // the softmax warps of both blocks
      mbar_init(&pv_done[i], 1);
    }
    mbar_init(&o_done, 1);
    for (int q = 0; q < 4; ++q) {
      mbar_init(&x_bar[q], SPLIT);
      mbar_init(&l_bar[q], SPLIT);
    }
    s_failed = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, TMEM_COLS);  // the same columns in both blocks: each takes all there are
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the other block's barriers and tensor memory exist before anything arrives there
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  // The kernel before this one writes the queries and the newest keys and values: the producers
  // wait for it before their first copy, and everything the other warps do follows from those
  // copies (the set-up above ran beside that kernel's end).

  if (warp == 0 || warp == 2) {
    // ---- producers (one thread each, in both blocks): warp 0 brings Q and this block's half of the
    // key tiles, warp 2 its half of the value tiles.
    if (lane == 0) {
      const bool values = warp == 2;
      pdl_wait();
      pdl_launch_dependents();
      if (!values) {
        const uint32_t bar = mapa_shared(smem_u32(&q_full), 0);
        mbar_arrive_expect_tx_cluster(bar, Q_BYTES);
        for (int sl = 0; sl < SLABS; ++sl)  // box: 64 dims x G heads x 128 / G tokens, rows in (token, head) order
          tma_load_3d_pair(sq + sl * (BM * 128), &map_q, sl * 64, m * group, row0 + i0, bar);
      }
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % STAGES;
        if (j >= STAGES) {
          const int t = j - STAGES;  // the tile that used the stage before
          const bool freed = values ? mbar_wait_bounded(&pv_done[t & 1], (t / 2) & 1) : mbar_wait_bounded(&s_full[t & 1], (t / 2) & 1);
          if (!freed) {
            s_failed = 1;
            break;
          }
        }
        const int j0 = tile0 + j * BN;
        // Boxes of 64 keys: of K the one of this block's keys, of V both (for this block's dims).
        const int first = values ? 0 : rank, count = values ? 2 : 1;
        int boxes = 0;
        long long rows[2];
        for (int i = 0; i < count; ++i) {
          const int key = j0 + (first + i) * 64;
          rows[i] = -1;
          if (key >= kv_hi || key + 64 <= kv_lo) continue;
          const long long page = p.block_table[(size_t)b * p.max_pages + key / p.page_size];
          if (page < 0 || page >= p.num_pages) {
            atomicOr(p.err, SB_ERR_BAD_PAGE);
            continue;
          }
          rows[i] = ((page * 2 + (values ? 1 : 0)) * p.num_kv_heads + m) * p.page_size + (key & (p.page_size - 1));
          ++boxes;
        }
        if (values) {
          mbar_arrive_expect_tx(&v_full[s], boxes * VSLABS * 64 * 128);
          for (int i = 0; i < 2; ++i)
            if (rows[i] >= 0)
              for (int sl = 0; sl < VSLABS; ++sl)
                tma_load_2d(sv + s * V_BYTES + sl * (BN * 128) + i * 64 * 128, &map_kv, rank * VD + sl * 64, (int)rows[i], &v_full[s]);
        } else {
          const uint32_t bar = mapa_shared(smem_u32(&k_full[s]), 0);
          mbar_arrive_expect_tx_cluster(bar, boxes * SLABS * 64 * 128);
          if (rows[0] >= 0)
            for (int sl = 0; sl < SLABS; ++sl) tma_load_2d_pair(sk + s * K_BYTES + sl * (KH * 128), &map_kv, sl * 64, (int)rows[0], bar);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue of S = Q.K^T for the pair (one thread of rank 0) -----------------------------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_qk = idesc_bf16_f32(2 * BM, BN, false, false);
      bool ok = mbar_wait_bounded_cluster(&q_full, 0);
      const uint64_t q_desc0 = smem_desc_sw128(sq, 16, 1024);
      const uint64_t k_desc0 = smem_desc_sw128(sk, 16, 1024);
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int s = j % STAGES;
        // The tile's S buffer held S and then P of the tile before last: its P.V must be done.
        if (!mbar_wait_bounded_cluster(&k_full[s], (j / STAGES) & 1) ||
            (j >= 2 && !mbar_wait_bounded(&pv_done[j & 1], ((j - 2) / 2) & 1))) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint64_t k_desc = k_desc0 + (uint64_t)((s * K_BYTES) >> 4);
        const uint32_t s_tmem = tmem + S_COL0 + (j & 1) * BN;
#pragma unroll
        for (int ks = 0; ks < DH / 16; ++ks) {
          // 16 dims further = 32 bytes further inside a slab's 128-byte rows; the next 64 dims are one slab further
          const uint64_t adesc = q_desc0 + (uint64_t)(((ks / 4) * (BM * 128) + (ks % 4) * 32) >> 4);
          const uint64_t bdesc = k_desc + (uint64_t)(((ks / 4) * (KH * 128) + (ks % 4) * 32) >> 4);
          tc_mma_f16_pair(s_tmem, adesc, bdesc, idesc_qk, ks > 0);
        }
        tc_commit_pair(&s_full[j & 1]);  // also frees the key tile's stage, in both blocks
      }
      if (!ok) s_failed = 1;
    }
  } else if (warp == 3) {
    // ---- MMA issue of O += P.V for the pair (one thread of rank 0) --------------------------------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_pv = idesc_bf16_f32(2 * BM, DH, false, true);  // V: the N index (dims) is contiguous
      const uint64_t v_desc0 = smem_desc_sw128(sv, BN * 128, 1024);
      bool ok = true;
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int s = j % STAGES;
        if (!mbar_wait_bounded_cluster(&p_ready[j & 1], (j / 2) & 1)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          // P comes from tensor memory, where it overwrote the tile's S: 16 keys are 8 columns of
          // two bfloat16 each.  16 keys further in V = 16 rows of 128 bytes.
          const uint64_t bdesc = v_desc0 + (uint64_t)((s * V_BYTES + kk * 16 * 128) >> 4);
          tc_mma_f16_ts_pair(tmem + O_COL0, tmem + S_COL0 + (j & 1) * BN + kk * 8, bdesc, idesc_pv, j > 0 || kk > 0);
        }
        tc_commit_pair(&pv_done[j & 1]);  // also frees the value tile's stage and the S buffer
      }
      tc_commit_pair(&o_done);
      if (!ok) s_failed = 1;
    }
  } else if (warp >= 4) {
    // ---- softmax and epilogue (both blocks, each for its own 128 rows) --------------------------------
    // SPLIT threads share a query row, CW of the tile's columns each; a warp may only touch the 32
    // lanes of tensor memory that (warp % 4) names, so the threads of a row sit in the warps
    // quarter, quarter + 4, ...  All of them keep the row's running maximum and decide alike when
    // it moves; each keeps a partial row sum.
    const int quarter = warp & 3, part = (warp - 4) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int pos = r < rows_valid ? p0 + r / group : -1;
    const bool rows_full = quarter * 32 + 31 < rows_valid;
    const int warp_pos_lo = p0 + (quarter * 32) / group, warp_pos_hi = p0 + (quarter * 32 + 31) / group;
    const float inv_cap = p.cap > 0.f ? 1.0f / p.cap : 0.f;
    const float scale2 = p.cap > 0.f ? p.cap * LOG2E : LOG2E;  // from x (tanh's value, or the score) to log2 units
    const uint32_t ready0 = mapa_shared(smem_u32(&p_ready[0]), 0);  // rank 0's p_ready[0]; [1] is 8 bytes further
    float m_run = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      const int j0 = tile0 + j * BN;
      if (!mbar_wait_bounded(&s_full[sb], (j / 2) & 1)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      uint32_t sr[CW];
      tmem_load_32x32(tmem + lane_base + S_COL0 + sb * BN + part * CW, sr);
      tmem_wait_load();
      const bool need_mask = !rows_full || j0 + BN - 1 > warp_pos_lo || (p.window > 0 && warp_pos_hi - j0 >= p.window);
      float mx = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < CW; ++c) {
          float v = __uint_as_float(sr[c]);
          if (p.cap > 0.f) v = fast_tanh(v * inv_cap);
          const int key = j0 + part * CW + c;
          v = (key <= pos && (p.window <= 0 || pos - key < p.window)) ? v : -INFINITY;
          sr[c] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
      } else {
#pragma unroll
        for (int c = 0; c < CW; ++c) {
          float v = __uint_as_float(sr[c]);
          if (p.cap > 0.f) v = fast_tanh(v * inv_cap);
          sr[c] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
      }
      // The row's maximum over its parts.  While the other parts' maxima are on their way the
      // numerators are computed against the running maximum, which only moves when the row's
      // maximum has grown by more than the threshold (numerators up to 2^8 are kept, which
      // float32 and bfloat16 hold without loss): then they are computed again.
      row_max[sb][part][r] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(&x_bar[quarter]);
      uint32_t pw[CW / 2];
      float sum0 = 0.f, sum1 = 0.f;
      {
        const float neg_base = m_run == -INFINITY ? 0.f : -m_run;
#pragma unroll
        for (int c = 0; c < CW; c += 2) {
          const float e0 = fast_exp2(fmaf(__uint_as_float(sr[c]), scale2, neg_base));
          const float e1 = fast_exp2(fmaf(__uint_as_float(sr[c + 1]), scale2, neg_base));
          sum0 += e0;
          sum1 += e1;
          pw[c / 2] = pack_bf16(e0, e1);
        }
      }
      if (!mbar_wait_bounded(&x_bar[quarter], j & 1)) {
        ok = false;
        break;
      }
#pragma unroll
      for (int q = 0; q < SPLIT; ++q) mx = fmaxf(mx, row_max[sb][q][r]);
      mx *= scale2;
      float alpha = 1.f;
      if (mx > m_run + RESCALE_THRESHOLD || (m_run == -INFINITY && mx != -INFINITY)) {
        alpha = fast_exp2(m_run - mx);  // 0 when there was no maximum yet
        m_run = mx;
        sum0 = sum1 = 0.f;
#pragma unroll
        for (int c = 0; c < CW; c += 2) {
          const float e0 = fast_exp2(fmaf(__uint_as_float(sr[c]), scale2, -mx));
          const float e1 = fast_exp2(fmaf(__uint_as_float(sr[c + 1]), scale2, -mx));
          sum0 += e0;
          sum1 += e1;
          pw[c / 2] = pack_bf16(e0, e1);
        }
      }
      l = l * alpha + sum0 + sum1;
      // O may only be rescaled between the last tile's P.V and this one's (which is not issued
      // before this thread has arrived at p_ready below).
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        if (!mbar_wait_bounded(&pv_done[(j - 1) & 1], ((j - 1) / 2) & 1)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll 1
        for (int c = part * OW; c < (part + 1) * OW; c += 16) {
          uint32_t o[16];
          tmem_load_32x16(tmem + lane_base + O_COL0 + c, o);
          tmem_wait_load();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_store_32x16(tmem + lane_base + O_COL0 + c, o);
        }
        tmem_wait_store();
      }
      // P as the 128-row operand of the next product, in tensor memory over the tile's S (all
      // parts have read their S by now: they exchanged maxima since): two keys per column.
      tmem_store_32x16(tmem + lane_base + S_COL0 + sb * BN + part * (CW / 2), pw);
      tmem_wait_store();
      // This block's value tile must have landed before rank 0 may issue the product; rows of
      // keys that are not the request's must read as zeros (0 * garbage could be NaN).  The
      // barrier's phase before this one is long complete: this tile's S only exists once the
      // P.V that read the stage before is done.
      if (!mbar_wait_bounded(&v_full[sb], (j / 2) & 1)) {
        ok = false;
        break;
      }
      if (j0 < kv_lo || j0 + BN > kv_hi) {
        for (int i = (quarter + 4 * part) * 32 + lane; i < BN * VSLABS * 8; i += 128 * SPLIT) {
          const int key_row = (i / 8) % BN, sl = i / (8 * BN), c = i % 8;
          const int key = j0 + key_row;
          if (key < kv_lo || key >= kv_hi)
            *reinterpret_cast<uint4*>(sv + sb * V_BYTES + sl * (BN * 128) + key_row * 128 + c * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();  // the zeroed value rows are visible to the tensor core's reads
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(ready0 + 8 * sb);
    }
    // The row's sum over its parts (all relative to the same maximum).
    if (ok) {
      row_sum[part][r] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(&l_bar[quarter]);
      ok = mbar_wait_bounded(&l_bar[quarter], 0);
      l = 0.f;
#pragma unroll
      for (int q = 0; q < SPLIT; ++q) l += row_sum[q][r];
    }
    if (ok && !mbar_wait_bounded(&o_done, 0)) ok = false;
    tc_fence_after_sync();
    // A full tile leaves through shared memory (Q's place, free by now) in the layout Q came in,
    // as TMA stores of whole lines; a tile that ends with its sequence is stored row by row: a
    // box would reach into the next sequence's rows.
    const bool staged = rows_valid == BM;
    if (ok && rows_valid > 0) {
      // Every lane takes part in the warp-wide tensor-memory loads; only rows of the sequence store.
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      const bool valid = r < rows_valid;
      bf16* op = p.out + ((size_t)(row0 + i0 + (valid ? r / group : 0)) * p.num_q_heads + m * group + (valid ? r % group : 0)) * DH;
#pragma unroll 1
      for (int c = part * OW; c < (part + 1) * OW; c += 16) {
        uint32_t o[16];
        tmem_load_32x16(tmem + lane_base + O_COL0 + c, o);
        tmem_wait_load();
        uint4 v[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          v[i].x = pack_bf16(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
          v[i].y = pack_bf16(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
          v[i].z = pack_bf16(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
          v[i].w = pack_bf16(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
        }
        if (staged) {
          unsigned char* srow = sq + (c / 64) * (BM * 128) + r * 128;
          const int piece = (c % 64) / 8;
          *reinterpret_cast<uint4*>(srow + ((piece ^ (r & 7)) << 4)) = v[0];
          *reinterpret_cast<uint4*>(srow + (((piece + 1) ^ (r & 7)) << 4)) = v[1];
        } else if (valid) {
          *reinterpret_cast<uint4*>(op + c) = v[0];
          *reinterpret_cast<uint4*>(op + c + 8) = v[1];
        }
      }
    }
    if (staged) {  // the same for every thread of the block, whether its waits ran out or not
      fence_proxy_async();
      asm volatile("bar.sync 1, %0;\n" ::"n"(128 * SPLIT) : "memory");  // the softmax warps
      if (warp == 4 && lane == 0 && !s_failed) {
        for (int sl = 0; sl < SLABS; ++sl) tma_store_3d(&map_out, sq + sl * (BM * 128), sl * 64, m * group, row0 + i0);
        tma_store_commit();
        tma_store_wait_read();  // shared memory has been read; the grid's end covers the writes
      }
    }
    if (!ok) s_failed = 1;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && s_failed) atomicOr(p.err, SB_ERR_TIMEOUT);
  // Neither block leaves while the other may still arrive at its barriers, read its shared
  // memory or multiply into its tensor memory.
  cluster_sync_all();
  if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace

#define SB_CONCAT2(a, b) a##b
#define SB_CONCAT(a, b) SB_CONCAT2(a, b)
#define SB_FN(name) SB_CONCAT(SB_CONCAT(name, _hd), SB_HEAD_DIM)

// Ragged prefill attention by pairs of blocks.  q: [T, Hq, DH]; cache: [pages, 2, Hkv, page_size, DH];
// items: [num_pairs, 3] (sequence, first token of a pair's 256 / G tokens, kv head), in the order
// in which the pairs are to start: the GPU holds 74 pairs at once and gives the next one to the SMs
// that finish first, so the order decides how evenly the walks fill them.  Returns -11 when the
// shapes do not allow it (the group must divide 128; the page size must be a power of two of at
// least 64).
extern "C" int SB_FN(sb_attn_prefill_pair)(const void* q, const void* cache, const int* block_table, int max_pages,
                                           const int* cu_q, const int* q_start, void* out, int num_tokens,
                                           int num_q_heads, int num_kv_heads, int page_size, int num_pages, float cap,
                                           int window, const int* items, int num_pairs, int* err,
                                           cudaStream_t stream) {
  if (num_pairs == 0) return 0;
  if (num_kv_heads <= 0 || num_q_heads % num_kv_heads) return -8;
  const int group = num_q_heads / num_kv_heads;
  if (group > BM || BM % group || (page_size & (page_size - 1)) || page_size < 64) return -11;
  SbEncodeTiled encode = sb_encode_tiled();
  if (!encode) return -12;
  CUtensorMap map_q, map_kv, map_out;
  for (int which = 0; which < 2; ++which) {  // q and out have the same shape
    const cuuint64_t dims[3] = {(cuuint64_t)DH, (cuuint64_t)num_q_heads, (cuuint64_t)num_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)DH * 2, (cuuint64_t)num_q_heads * DH * 2};
    const cuuint32_t box[3] = {64u, (cuuint32_t)group, (cuuint32_t)(BM / group)};
    const cuuint32_t elem[3] = {1u, 1u, 1u};
    if (encode(which == 0 ? &map_q : &map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
               which == 0 ? const_cast<void*>(q) : out, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return -12;
  }
  if (sb_make_map_2d(&map_kv, cache, (long long)num_pages * 2 * num_kv_heads * page_size, DH, 64) != 0) return -12;
  PairParams p{};
  p.q = (const bf16*)q;
  p.block_table = block_table; p.max_pages = max_pages; p.cu_q = cu_q; p.q_start = q_start; p.out = (bf16*)out;
  p.num_q_heads = num_q_heads; p.num_kv_heads = num_kv_heads; p.page_size = page_size; p.num_pages = num_pages;
  p.cap = cap; p.window = window; p.items = items; p.err = err;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PAIR_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)(2 * num_pairs));
  config.blockDim = dim3(PAIR_THREADS);
  config.dynamicSmemBytes = PAIR_SMEM;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  int n_attr = 0;
  if (sb_pdl_level() >= 1) {
    attribute[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  attribute[n_attr].id = cudaLaunchAttributeClusterDimension;
  attribute[n_attr].val.clusterDim.x = 2;
  attribute[n_attr].val.clusterDim.y = 1;
  attribute[n_attr].val.clusterDim.z = 1;
  ++n_attr;
  config.attrs = attribute;
  config.numAttrs = n_attr;
  cudaError_t e = cudaLaunchKernelEx(&config, attn_prefill_pair_kernel, p, map_q, map_kv, map_out);
  if (e != cudaSuccess) return (int)e;
  SB_LAUNCH_CHECK();
  return 0;
}

#endif  // other head sizes do not get this kernel
