// Ragged paged prefill attention on the fifth-generation tensor cores (tcgen05), compiled once
// per head size (-DSB_HEAD_DIM=N, N a multiple of 64 up to 256).
//
//   s = q . k                 (q is already rotated and scaled)
//   s = cap * tanh(s / cap)   if cap > 0          simply/model_lib.py:621-626
//   keep k_pos <= q_pos and, with a window W, q_pos - k_pos < W
//                                                 simply/model_lib.py:469-515
//   p = softmax(s) in float32, o = p . v          simply/model_lib.py:633-637
//   query head n reads kv head n / G              simply/model_lib.py:2306-2310
//
// A block owns 128 query rows of one (sequence, kv head): the G query heads of the group for
// 128 / G consecutive tokens.  It walks the keys in tiles of 64:
//   S[128 x 64]  = Q . K^T     tcgen05.mma, accumulator in tensor memory (three S buffers: this
//                              product runs two key tiles ahead of the one below)
//   P            = softmax numerators of S as bfloat16, written over S in tensor memory: the
//                  next product's 128-row operand comes from there
//   O[128 x DH] += P . V       tcgen05.mma, accumulator in tensor memory for the whole walk
// Roles: warp 0 TMA producer of Q (once) and of the key tiles, warp 2 of the value tiles (both
// from the paged cache through the block table), warps 1 and 3 MMA issue (one thread each: Q.K^T
// and P.V), warps 4..19
// softmax and epilogue: two groups of 8 warps that take the key tiles in turn, two threads per
// query row in a group with 32 of the tile's 64 columns each.  (One thread per row leaves each
// scheduler a single warp, and one group of warps has to finish a tile's softmax before it can
// start the next: both leave the tensor cores waiting for the softmax's instruction latency.)
// The running maximum is only moved when it grows by more than 8 (log2 units):
// O is then rescaled in tensor memory; otherwise numerators up to 2^8 are kept, which float32
// and bfloat16 hold without loss, and the final division by the row sum makes it exact.
// All waits are bounded; a wait that runs out sets SB_ERR_TIMEOUT and the block leaves after
// releasing its tensor memory.
#include <float.h>

#include "common.cuh"
#include "tma_mbar.cuh"

#ifndef SB_HEAD_DIM
#define SB_HEAD_DIM 256
#endif

#if SB_HEAD_DIM % 64 == 0

namespace {

using namespace sbx;

constexpr int DH = SB_HEAD_DIM;
constexpr int BM = 128, BN = 64, SLABS = DH / 64;
// With a head size of 256 the first 128 dims of Q live in tensor memory (as the 128-row operand of
// the first eight products of a tile, which then read only K from shared memory: with Q from
// shared memory a 128 x 64 x 16 product waits about 75 cycles for its operands, twice what it
// computes), the rest in shared memory, which leaves room for a third stage of keys.
constexpr int QT_DIMS = DH == 256 ? 128 : 0;          // dims of Q in tensor memory
constexpr int QT_COLS = QT_DIMS / 2;                  // two bfloat16 per column
constexpr int QS_SLABS = SLABS - QT_DIMS / 64;        // slabs of 64 dims of Q in shared memory
constexpr int Q_BYTES = BM * QS_SLABS * 128, KV_TILE_BYTES = BN * DH * 2;
constexpr int K_STAGES = 3, V_STAGES = 2;
constexpr int GROUPS = 2;          // softmax groups: group g takes the key tiles j with j % 2 == g
constexpr int SPLIT = 2;           // softmax threads per query row within a group
constexpr int CW = BN / SPLIT;     // columns of a key tile per softmax thread
constexpr int OW = DH / (GROUPS * SPLIT);  // columns of O per softmax thread in the epilogue
static_assert(CW == 32 && OW % 16 == 0, "tensor-memory loads of 32 and 16 columns");
constexpr int TC_THREADS = 128 + 128 * GROUPS * SPLIT;  // warps: key producer, MMA, value producer, spare, softmax
constexpr int S_BUFS = 3;                               // S buffers: Q.K^T runs two key tiles ahead of P.V
constexpr int S_COL0 = 0, O_COL0 = S_BUFS * BN;         // S buffers from column 0, O behind them
constexpr int QT_COL0 = O_COL0 + DH;                    // Q's first dims behind O
constexpr int TMEM_COLS = QT_COL0 + QT_COLS <= 256 ? 256 : 512;  // a power of two that holds the S buffers, O and Q's part
static_assert(QT_COL0 + QT_COLS <= 512, "tensor memory has 512 columns");
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.f;

struct TcParams {
  const bf16* q;  // [T, Hq, DH]
  const int* block_table;
  int max_pages;
  const int* cu_q;
  const int* q_start;
  bf16* out;
  int num_q_heads, num_kv_heads, page_size, num_pages;
  float cap;
  int window;
  const int* items;  // per block, in launch order: (sequence, first token of the tile of 128 / G tokens, kv head)
  int box_rows;      // rows per key/value TMA box: min(page_size, 64)
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

__global__ void __launch_bounds__(TC_THREADS)
attn_prefill_tc_kernel(const TcParams p, const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_kv, const __grid_constant__ CUtensorMap map_out) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sq = base;                               // [QS_SLABS][128 rows][128 B]
  unsigned char* sk = sq + Q_BYTES;                       // [K_STAGES][SLABS][64 keys][128 B]
  unsigned char* sv = sk + K_STAGES * KV_TILE_BYTES;      // [V_STAGES][SLABS][64 keys][128 B]
  __shared__ __align__(8) uint64_t q_full, qt_ready, k_full[K_STAGES], v_full[V_STAGES], s_full[2 * S_BUFS], p_ready[4], pv_done[S_BUFS], o_done, x_bar[GROUPS][4], m_bar[2][4], l_bar[4];
  __shared__ float row_max[GROUPS][SPLIT][BM];  // the parts' row maxima of a group's tile
  __shared__ float row_m[2][BM];                // the running maximum after a tile, by tile parity
  __shared__ float row_sum[GROUPS * SPLIT][BM]; // at the end: the threads' partial row sums
  __shared__ uint32_t tmem_slot;
  __shared__ int s_failed;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = p.items[3 * blockIdx.x], i0 = p.items[3 * blockIdx.x + 1], m = p.items[3 * blockIdx.x + 2];
  const int group = p.num_q_heads / p.num_kv_heads;
  const int tokens_per_tile = BM / group;
  const int row0 = p.cu_q[b], q_len = p.cu_q[b + 1] - row0, qs = p.q_start[b];
  const int ntok = min(tokens_per_tile, q_len - i0);
  const int rows_valid = ntok * group;
  const int p0 = qs + i0, p1 = qs + i0 + ntok - 1;
  const int kv_lo = p.window > 0 ? max(qs - p.window + 1, 0) : 0;  // lowest key the request still holds
  const int lo = p.window > 0 ? max(p0 - p.window + 1, 0) : 0;     // lowest key this tile can see
  const int kv_hi = p1 + 1;
  const int tile0 = (lo / BN) * BN;
  const int n_tiles = (kv_hi - tile0 + BN - 1) / BN;

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    mbar_init(&qt_ready, 4 * GROUPS * SPLIT);
    for (int s = 0; s < K_STAGES; ++s) mbar_init(&k_full[s], 1);
    for (int s = 0; s < V_STAGES; ++s) mbar_init(&v_full[s], 1);
    for (int s = 0; s < 2 * S_BUFS; ++s) mbar_init(&s_full[s], 1);
    for (int q = 0; q < 4; ++q) {
      for (int g = 0; g < GROUPS; ++g) mbar_init(&x_bar[g][q], SPLIT);
      mbar_init(&m_bar[0][q], SPLIT);
      mbar_init(&m_bar[1][q], SPLIT);
      mbar_init(&l_bar[q], GROUPS * SPLIT);
    }
    for (int q = 0; q < 4; ++q) mbar_init(&p_ready[q], 4 * SPLIT);
    for (int q = 0; q < S_BUFS; ++q) mbar_init(&pv_done[q], 1);
    mbar_init(&o_done, 1);
    s_failed = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;

  if (warp == 0 || warp == 2) {
    // ---- producers (one thread each): warp 0 brings Q and the key tiles, warp 2 the value tiles.
    // Keys and values have rings of their own: a key tile is free as soon as its Q.K^T is done,
    // long before the value tile of the same keys, so the next keys arrive early.
    // A stage of keys is free once the Q.K^T that read it is done (s_full of that tile), a stage of
    // values once its P.V is (pv_done): the producers wait on those barriers, each on every phase.
    if (lane == 0) {
      const bool values = warp == 2;
      uint64_t* full = values ? v_full : k_full;
      unsigned char* ring = values ? sv : sk;
      const int stages = values ? V_STAGES : K_STAGES;
      if (!values && QS_SLABS > 0) {
        mbar_arrive_expect_tx(&q_full, Q_BYTES);
        for (int sl = 0; sl < QS_SLABS; ++sl)  // box: 64 dims x G heads x 128 / G tokens, rows in (token, head) order
          tma_load_3d(sq + sl * (BM * 128), &map_q, (sl + QT_DIMS / 64) * 64, m * group, row0 + i0, &q_full);
      }
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % stages;
        if (j >= stages) {
          const int t = j - stages;  // the tile that used the stage before
          const bool freed = values ? mbar_wait_bounded(&pv_done[t % S_BUFS], (t / S_BUFS) & 1)
                                    : mbar_wait_bounded(&s_full[t % (2 * S_BUFS)], (t / (2 * S_BUFS)) & 1);
          if (!freed) {
            s_failed = 1;
            break;
          }
        }
        const int j0 = tile0 + j * BN;
        int boxes = 0;
        for (int r = 0; r < BN; r += p.box_rows) {
          const int key = j0 + r;
          if (key >= kv_hi || key + p.box_rows <= kv_lo) continue;
          const long long page = p.block_table[(size_t)b * p.max_pages + key / p.page_size];
          if (page >= 0 && page < p.num_pages) ++boxes;
        }
        mbar_arrive_expect_tx(&full[s], boxes * SLABS * p.box_rows * 128);
        for (int r = 0; r < BN; r += p.box_rows) {
          const int key = j0 + r;
          if (key >= kv_hi || key + p.box_rows <= kv_lo) continue;
          const long long page = p.block_table[(size_t)b * p.max_pages + key / p.page_size];
          if (page < 0 || page >= p.num_pages) {
            atomicOr(p.err, SB_ERR_BAD_PAGE);
            continue;
          }
          const long long row = ((page * 2 + (values ? 1 : 0)) * p.num_kv_heads + m) * p.page_size + (key & (p.page_size - 1));
          for (int sl = 0; sl < SLABS; ++sl)
            tma_load_2d(ring + s * KV_TILE_BYTES + sl * (BN * 128) + r * 128, &map_kv, sl * 64, (int)row, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue of S = Q.K^T (one thread) ----------------------------------------------------------
    // Two threads issue the products, this one and warp 3's below: one thread alone spends about
    // 70 cycles per instruction on the sixteen 128 x 64 x 16 products of a tile (they wait for Q
    // and K from shared memory) and cannot feed the tensor cores.
    // S(j) goes to buffer j % 3, which held S and then P of tile j - 3: its P.V must be done
    // (pv_done[j % 3]: one barrier per buffer, since P.V may complete up to the tile before the one
    // this thread is at, and a barrier shared by tiles j - 3 and j - 1 could then pass two phases
    // before this thread looks, which a wait by phase parity cannot tell from none).
    // The tile's barrier is s_full[j % 6], which only the softmax group of tile j waits on (a
    // barrier that both groups waited on in turn would show each of them only every other phase,
    // which a wait by phase parity cannot tell apart).
    if (lane == 0) {
      const uint32_t idesc_qk = idesc_bf16_f32(BM, BN, false, false);
      bool ok = (QS_SLABS == 0 || mbar_wait_bounded(&q_full, 0)) && (QT_DIMS == 0 || mbar_wait_bounded(&qt_ready, 0));
      // Descriptors are a base plus a constant per step of 16 dims (the start address is the
      // descriptor's low field, in units of 16 bytes), so that between two products of a tile
      // this thread has one addition to do: it is the thread the whole block waits for.
      const uint64_t q_desc0 = smem_desc_sw128(sq, 16, 1024);
      const uint64_t k_desc0 = smem_desc_sw128(sk, 16, 1024);
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int s = j % K_STAGES;
        if (!mbar_wait_bounded(&k_full[s], (j / K_STAGES) & 1) ||
            (j >= S_BUFS && !mbar_wait_bounded(&pv_done[j % S_BUFS], ((j - S_BUFS) / S_BUFS) & 1))) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint64_t k_desc = k_desc0 + (uint64_t)((s * KV_TILE_BYTES) >> 4);
        const uint32_t s_tmem = tmem + S_COL0 + (j % S_BUFS) * BN;
#pragma unroll
        for (int ks = 0; ks < DH / 16; ++ks) {
          const uint64_t bdesc = k_desc + (uint64_t)(((ks / 4) * (BN * 128) + (ks % 4) * 32) >> 4);
          if (ks < QT_DIMS / 16) {
            // 16 dims of Q are 8 columns of two bfloat16 each
            tc_mma_f16_ts(s_tmem, tmem + QT_COL0 + ks * 8, bdesc, idesc_qk, ks > 0);
          } else {
            const int kq = ks - QT_DIMS / 16;
            tc_mma_f16(s_tmem, q_desc0 + (uint64_t)(((kq / 4) * (BM * 128) + (kq % 4) * 32) >> 4), bdesc, idesc_qk, ks > 0);
          }
        }
        tc_commit(&s_full[j % (2 * S_BUFS)]);  // also frees the key tile's stage
      }
      if (!ok) s_failed = 1;
    }
  } else if (warp == 3) {
    // ---- MMA issue of O += P.V (one thread) ---------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc_pv = idesc_bf16_f32(BM, DH, false, true);  // V: the N index (dims) is contiguous
      const uint64_t v_desc0 = smem_desc_sw128(sv, BN * 128, 1024);
      bool ok = true;
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int s = j % V_STAGES;
        // p_ready[j % 4]: the softmax may be two tiles ahead of this thread (S exists as soon as the
        // P.V three tiles back is done), so tiles j and j + 2 must not share a barrier.
        if (!mbar_wait_bounded(&p_ready[j % 4], (j / 4) & 1) || !mbar_wait_bounded(&v_full[s], (j / V_STAGES) & 1)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          // P comes from tensor memory, where it overwrote the tile's S: 16 keys are 8 columns of
          // two bfloat16 each.  16 keys further in V = 16 rows of 128 bytes; the next 64 dims are
          // one slab (BN * 128 bytes) further.
          const uint64_t bdesc = v_desc0 + (uint64_t)((s * KV_TILE_BYTES + kk * 16 * 128) >> 4);
          tc_mma_f16_ts(tmem + O_COL0, tmem + S_COL0 + (j % S_BUFS) * BN + kk * 8, bdesc, idesc_pv, j > 0 || kk > 0);
        }
        tc_commit(&pv_done[j % S_BUFS]);  // also frees the value tile's stage
      }
      tc_commit(&o_done);  // every product into O is complete (a barrier of its own: the softmax
                           // warps skip phases of pv_done, and the last one must not be mistaken)
      if (!ok) s_failed = 1;
    }
  } else if (warp >= 4) {
    // ---- softmax and epilogue ---------------------------------------------------------------------
    // Two groups of 8 warps; group g takes the key tiles j with j % 2 == g, so that the softmax of
    // one tile runs while the other group's tile is still on its way (one group alone is bound by
    // the latency of its own instruction chain).  Within a group SPLIT threads share a query row,
    // CW of the tile's 64 columns each; a warp may only touch the 32 lanes of tensor memory that
    // (warp % 4) names, so the threads of a row sit in the warps quarter, quarter + 4, ...
    // A barrier that both groups wait on in turn exists once per tile parity (m_bar): a thread then
    // waits on every phase of it, never on every other one, which a wait by phase parity could not
    // tell apart.
    // What passes from tile to tile is the row's running maximum: the group of tile j publishes it
    // (row_m, m_bar) as soon as it has seen the tile's maxima, long before its P is written.  Row
    // sums stay partial in every thread, each relative to the maximum that thread saw last.
    const int quarter = warp & 3, sw = (warp - 4) >> 2;  // sw: 0 .. GROUPS * SPLIT - 1
    const int grp = sw / SPLIT, part = sw % SPLIT;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int pos = r < rows_valid ? p0 + r / group : -1;
    // Positions of this warp's first and last row, for deciding whether a tile needs masking.
    const bool rows_full = quarter * 32 + 31 < rows_valid;
    const int warp_pos_lo = p0 + (quarter * 32) / group, warp_pos_hi = p0 + (quarter * 32 + 31) / group;
    const float inv_cap = p.cap > 0.f ? 1.0f / p.cap : 0.f;
    const float scale2 = p.cap > 0.f ? p.cap * LOG2E : LOG2E;  // from x (tanh's value, or the score) to log2 units
    float m_own = -INFINITY, l = 0.f;  // the maximum this thread's sum is relative to; the sum
    bool ok = true;
    if (QT_DIMS > 0) {
      // Q's first dims to tensor memory: row = lane, this thread's 32 of them as 16 columns.
      const bool valid = r < rows_valid;
      const bf16* qrow = p.q + ((size_t)(row0 + i0 + (valid ? r / group : 0)) * p.num_q_heads + m * group + (valid ? r % group : 0)) * DH +
                         sw * (QT_DIMS / (GROUPS * SPLIT));
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 v = valid ? *reinterpret_cast<const uint4*>(qrow + i * 8) : make_uint4(0, 0, 0, 0);
        w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
      }
      tmem_store_32x16(tmem + lane_base + QT_COL0 + sw * (QT_COLS / (GROUPS * SPLIT)), w);
      tmem_wait_store();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&qt_ready);
    }
    for (int j = grp; j < n_tiles; j += GROUPS) {
      const int sb = j % S_BUFS, s = j % V_STAGES;
      const int j0 = tile0 + j * BN;
      const int use = j / GROUPS;  // how often this group's barriers have been used
      if (!mbar_wait_bounded(&s_full[j % (2 * S_BUFS)], (j / (2 * S_BUFS)) & 1)) {
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
      // The row's maximum over the group's parts.
      row_max[grp][part][r] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(&x_bar[grp][quarter]);
      if (!mbar_wait_bounded(&x_bar[grp][quarter], use & 1)) {
        ok = false;
        break;
      }
#pragma unroll
      for (int q = 0; q < SPLIT; ++q) mx = fmaxf(mx, row_max[grp][q][r]);
      mx *= scale2;
      // The running maximum after the tile before this one (the other group's), then after this
      // one: it only moves when it grows by more than the threshold.  Every part of the group
      // decides alike and publishes; the other group waits for it at its next tile.
      float m_prev = -INFINITY;
      if (j > 0) {
        if (!mbar_wait_bounded(&m_bar[(j - 1) & 1][quarter], ((j - 1) / 2) & 1)) {
          ok = false;
          break;
        }
        m_prev = row_m[(j - 1) & 1][r];
      }
      float m_use = m_prev;
      if (mx > m_prev + RESCALE_THRESHOLD || (m_prev == -INFINITY && mx != -INFINITY)) m_use = mx;
      if (part == 0) row_m[j & 1][r] = m_use;
      __syncwarp();
      if (lane == 0) mbar_arrive(&m_bar[j & 1][quarter]);
      const float alpha = m_use == m_prev ? 1.f : fast_exp2(m_prev - m_use);  // for O; 0 when there was no maximum yet
      if (m_use != m_own) {
        l *= m_own == -INFINITY ? 0.f : fast_exp2(m_own - m_use);
        m_own = m_use;
      }
      const float neg_base = m_use == -INFINITY ? 0.f : -m_use;
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int c = 0; c < CW; c += 2) {
        const float e0 = fast_exp2(fmaf(__uint_as_float(sr[c]), scale2, neg_base));
        const float e1 = fast_exp2(fmaf(__uint_as_float(sr[c + 1]), scale2, neg_base));
        sum0 += e0;
        sum1 += e1;
        sr[c / 2] = pack_bf16(e0, e1);
      }
      l += sum0 + sum1;
      // O may only be rescaled between the last tile's P.V and this one's.  (The phases of this
      // barrier that are skipped here are long complete: a tile's S only exists once the P.V
      // three tiles back is done.)
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        if (!mbar_wait_bounded(&pv_done[(j - 1) % S_BUFS], ((j - 1) / S_BUFS) & 1)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll 1
        for (int c = part * (DH / SPLIT); c < (part + 1) * (DH / SPLIT); c += 16) {
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
      // parts have read their S by now: they exchanged maxima since): row = lane, two keys per column.
      {
        uint32_t pw[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) pw[c] = sr[c];
        tmem_store_32x16(tmem + lane_base + S_COL0 + sb * BN + part * (CW / 2), pw);
        tmem_wait_store();
      }
      // Value rows of keys that are not the request's must read as zeros (0 * garbage could be NaN):
      // only in tiles that reach beyond [kv_lo, kv_hi).
      if (j0 < kv_lo || j0 + BN > kv_hi) {
        // The value tile's barrier is only looked at in such tiles; its phase before this one is
        // known to be complete once the P.V two tiles back is (whose phase before is complete in
        // turn, as this tile's S exists).
        if ((j >= V_STAGES && !mbar_wait_bounded(&pv_done[(j - 2) % S_BUFS], ((j - 2) / S_BUFS) & 1)) ||
            !mbar_wait_bounded(&v_full[s], (j / V_STAGES) & 1)) {
          ok = false;
          break;
        }
        for (int i = (quarter + 4 * part) * 32 + lane; i < BN * SLABS * 8; i += 128 * SPLIT) {
          const int key_row = (i / 8) % BN, sl = i / (8 * BN), c = i % 8;
          const int key = j0 + key_row;
          if (key < kv_lo || key >= kv_hi)
            *reinterpret_cast<uint4*>(sv + s * KV_TILE_BYTES + sl * (BN * 128) + key_row * 128 + c * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();  // the zeroed value rows are visible to the tensor core's reads
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[j % 4]);
    }
    // The row's sum over all threads that share it, each brought to the final maximum.
    if (ok && n_tiles > 0) {
      ok = mbar_wait_bounded(&m_bar[(n_tiles - 1) & 1][quarter], ((n_tiles - 1) / 2) & 1);
      const float m_final = ok ? row_m[(n_tiles - 1) & 1][r] : 0.f;
      row_sum[sw][r] = (m_own == -INFINITY || m_final == -INFINITY) ? 0.f : l * fast_exp2(m_own - m_final);
      __syncwarp();
      if (lane == 0) mbar_arrive(&l_bar[quarter]);
      ok = ok && mbar_wait_bounded(&l_bar[quarter], 0);
      l = 0.f;
#pragma unroll
      for (int q = 0; q < GROUPS * SPLIT; ++q) l += row_sum[q][r];
    }
    if (ok && !mbar_wait_bounded(&o_done, 0)) ok = false;
    tc_fence_after_sync();
    // A full tile leaves through shared memory (the key stages, free by now) in the layout Q came
    // in, as TMA stores of whole lines: stored straight from registers, 16 bytes per lane at a
    // row's stride, the 64 KB of a tile took 3.7 us of a block's time.  A tile that ends with its
    // sequence is stored row by row: a box would reach into the next sequence's rows.
    const bool staged = rows_valid == BM;
    if (ok) {
      // Every lane takes part in the warp-wide tensor-memory loads; only rows of the sequence store.
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      const bool valid = r < rows_valid;
      bf16* op = p.out + ((size_t)(row0 + i0 + (valid ? r / group : 0)) * p.num_q_heads + m * group + (valid ? r % group : 0)) * DH;
#pragma unroll 1
      for (int c = sw * OW; c < (sw + 1) * OW; c += 16) {
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
          // slab of 64 dims, row of 128 bytes, 16-byte pieces swizzled as the TMA expects
          unsigned char* srow = sk + (c / 64) * (BM * 128) + r * 128;
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
      asm volatile("bar.sync 1, %0;\n" ::"n"(128 * GROUPS * SPLIT) : "memory");  // the softmax warps
      if (warp == 4 && lane == 0 && !s_failed) {
        for (int sl = 0; sl < SLABS; ++sl) tma_store_3d(&map_out, sk + sl * (BM * 128), sl * 64, m * group, row0 + i0);
        tma_store_commit();
        tma_store_wait_read();  // shared memory has been read; the grid's end covers the writes
      }
    }
    if (!ok) s_failed = 1;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && s_failed) atomicOr(p.err, SB_ERR_TIMEOUT);
  if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

constexpr size_t TC_SMEM = (size_t)Q_BYTES + (K_STAGES + V_STAGES) * KV_TILE_BYTES + 1024;
static_assert(QT_DIMS == 0 || QT_DIMS / (GROUPS * SPLIT) == 32, "each softmax thread stores 32 dims of Q");
static_assert(V_STAGES == 2, "the zeroing of value rows looks two tiles back");

}  // namespace

#define SB_CONCAT2(a, b) a##b
#define SB_CONCAT(a, b) SB_CONCAT2(a, b)
#define SB_FN(name) SB_CONCAT(SB_CONCAT(name, _hd), SB_HEAD_DIM)

// Ragged prefill attention on tcgen05.  q: [T, Hq, DH]; cache: [pages, 2, Hkv, page_size, DH];
// items: [num_items, 3] (sequence, first token of a tile of 128 / G tokens, kv head), in the order in
// which the blocks are to start (longest walk first over all heads, so that the SMs that are free
// first take the longest walks left).  Returns -11 when
// the shapes do not allow it (the group must divide 128, the page size must be a power of two).
extern "C" int SB_FN(sb_attn_prefill_tc)(const void* q, const void* cache, const int* block_table, int max_pages,
                                         const int* cu_q, const int* q_start, void* out, int num_tokens,
                                         int num_q_heads, int num_kv_heads, int page_size, int num_pages, float cap,
                                         int window, const int* items, int num_items, int* err, cudaStream_t stream) {
  if (num_items == 0) return 0;
  if (num_kv_heads <= 0 || num_q_heads % num_kv_heads) return -8;
  const int group = num_q_heads / num_kv_heads;
  if (group > BM || BM % group || (page_size & (page_size - 1))) return -11;
  SbEncodeTiled encode = sb_encode_tiled();
  if (!encode) return -12;
  CUtensorMap map_q, map_kv, map_out;
  for (int which = 0; which < 2; ++which) {  // q and out have the same shape
    const cuuint64_t dims[3] = {(cuuint64_t)DH, (cuuint64_t)num_q_heads, (cuuint64_t)num_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)DH * 2, (cuuint64_t)num_q_heads * DH * 2};
    const cuuint32_t box[3] = {64u, (cuuint32_t)group, (cuuint32_t)(BM / group)};
    const cuuint32_t elem[3] = {1u, 1u, 1u};
    if (encode(which == 0 ? &map_q : &map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, which == 0 ? const_cast<void*>(q) : out, dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return -12;
  }
  const int box_rows = page_size < BN ? page_size : BN;
  if (sb_make_map_2d(&map_kv, cache, (long long)num_pages * 2 * num_kv_heads * page_size, DH, box_rows) != 0) return -12;
  TcParams p{};
  p.q = (const bf16*)q;
  p.block_table = block_table; p.max_pages = max_pages; p.cu_q = cu_q; p.q_start = q_start; p.out = (bf16*)out;
  p.num_q_heads = num_q_heads; p.num_kv_heads = num_kv_heads; p.page_size = page_size; p.num_pages = num_pages;
  p.cap = cap; p.window = window; p.items = items; p.box_rows = box_rows; p.err = err;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  sb_launch(attn_prefill_tc_kernel, dim3(num_items), TC_THREADS, TC_SMEM, stream, p, map_q, map_kv, map_out);
  SB_LAUNCH_CHECK();
  return 0;
}

#endif  // head sizes that are no multiple of 64 do not get this kernel
