// Gated feed-forward product for many tokens (a prompt's portion) on the fifth-generation tensor cores:
//   out[M, F] = act(x[M, K] . w[0:F, K]^T) * (x[M, K] . w[F:2F, K]^T),  bfloat16 in and out,
// float32 accumulation in tensor memory.  The activation runs on the accumulators, so the [M, 2F]
// product never goes to memory and back.
//
// One persistent block per SM walks over output tiles of 128 tokens x 128 features.  A tile's
// accumulator is 128 lanes x 256 columns of tensor memory: the gate rows of w are columns 0..127
// and the up rows of the same features columns 128..255, one `tcgen05.mma` of 128 x 256 x 16 per
// 16 of k.  Tensor memory holds two such accumulators, so the products of the next tile run while
// the last one is read back.  Roles:
//   warp 0: TMA producer (one thread): per 64 of k one box of x and two boxes of w (128-byte
//           swizzle) into a ring of shared-memory stages
//   warp 1: tensor-memory allocation, MMA issue (one thread)
//   warps 2..9: epilogue: read an accumulator (`tcgen05.ld`), one 32-lane quarter and half of the
//           tile's features each, apply the activation and store bfloat16 rows.  (Four warps, one
//           per scheduler, took longer over a tile's activations than the tensor core over its
//           products.)
// Barriers: full[s] / empty[s] for the stages, acc_full[b] / acc_empty[b] for the accumulators.
// Every wait is bounded; a wait that runs out sets SB_ERR_TIMEOUT, and the block still releases
// its tensor memory before it leaves.
// Tiles are numbered tokens first: blocks that run at the same time read the same few weight
// tiles, which then come from L2.
// F must be a multiple of 128 and K a multiple of 8 (16-byte rows for the TMA); rows beyond M and
// columns beyond K read as zero.
#include <mutex>
#include <unordered_map>

#include "gemm_epilogue.cuh"
#include "tma_mbar.cuh"

namespace {

using namespace sbx;

constexpr int BM = 128, BF = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;      // tokens
constexpr int B_BYTES = 2 * BF * BK * 2;  // gate rows, then up rows
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 4;
constexpr int EPI_WARPS = 8;  // two per 32-lane quarter of tensor memory, 64 features each
constexpr int THREADS = (2 + EPI_WARPS) * 32;
constexpr int ACC_COLS = 2 * BF;  // columns of one accumulator
// Results leave through shared memory: a warp's 32 tokens x 64 features (rows of 128 bytes, 128-byte
// swizzle) go out as one TMA store of whole lines.  (Stored straight from registers, 16 bytes per
// lane at a row's stride, they cost the kernel 7 % more time than the loads and products alone.)
constexpr int OUT_WARP_BYTES = 32 * 128;
constexpr int OUT_BYTES = EPI_WARPS * OUT_WARP_BYTES;
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + OUT_BYTES + 1024;

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// A block's (or pair's) walk over its tiles and their blocks of k, without a division per step.
struct TileWalk {
  int tile, stride, tiles_m, nkb, rows;  // rows: tokens of a tile
  int m0, f0, kb;
  __device__ TileWalk(int first, int stride_, int tiles_m_, int nkb_, int rows_)
      : tile(first), stride(stride_), tiles_m(tiles_m_), nkb(nkb_), rows(rows_), kb(0) {
    place();
  }
  __device__ void place() { m0 = (tile % tiles_m) * rows, f0 = (tile / tiles_m) * BF; }
  __device__ void next() {
    if (++kb == nkb) {
      kb = 0;
      tile += stride;
      place();
    }
  }
};

// The gate's activation.  The tanh form of GELU is written as g / (1 + exp(-2 y)) with
// y = sqrt(2 / pi) (g + 0.044715 g^3), which is the same function (0.5 (1 + tanh y) = 1 / (1 + exp(-2 y)))
// at two special-function instructions (ex2, rcp) instead of a library tanh; both are exact to a
// few units in the last place of float32, far below the bfloat16 rounding that follows.
__device__ __forceinline__ float gate_act(float g, int act) {
  if (act == 0) {
    constexpr float A = -2.0f * 1.4426950408889634f * 0.7978845608028654f;  // exp(-2 y) = 2^(g (A + B g^2))
    constexpr float B = A * 0.044715f;
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(e) : "f"(g * fmaf(g * g, B, A)));
    return __fdividef(g, 1.0f + e);
  }
  return sbg::gated_act(g, act);
}

// A warp's part of a tile: 32 tokens (this warp's lanes of tensor memory) x 64 features from
// feature c0 of the tile.  Gate and up sums from the accumulator at `acc`, the activation,
// bfloat16 results to the warp's own 4 KB of shared memory (`stage`: 32 rows of 128 bytes, 16-byte
// pieces swizzled as the TMA expects), then one TMA store to out[row0.., f0 + c0..].
__device__ __forceinline__ void store_gated_rows(uint32_t acc, int c0, unsigned char* stage, const CUtensorMap* map_out,
                                                 int row0, int f0, int act) {
  const int lane = threadIdx.x & 31;
  if (lane == 0) tma_store_wait_read();  // the store of the tile before has read the stage
  __syncwarp();
#pragma unroll 1
  for (int c = 0; c < BF / 2; c += 16) {
    uint32_t g[16], u[16];
    tmem_load_32x16(acc + c0 + c, g);
    tmem_load_32x16(acc + BF + c0 + c, u);
    tmem_wait_load();
    uint32_t packed[8];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      // The projections are rounded to bfloat16 before the activation, as a product that
      // stores them would (two per conversion; a bfloat16 is the upper half of its float32).
      const uint32_t gp = pack_bf16(__uint_as_float(g[i]), __uint_as_float(g[i + 1]));
      const uint32_t up = pack_bf16(__uint_as_float(u[i]), __uint_as_float(u[i + 1]));
      const float g0 = __uint_as_float(gp << 16), g1 = __uint_as_float(gp & 0xFFFF0000u);
      const float u0 = __uint_as_float(up << 16), u1 = __uint_as_float(up & 0xFFFF0000u);
      packed[i / 2] = pack_bf16(gate_act(g0, act) * u0, gate_act(g1, act) * u1);
    }
    unsigned char* srow = stage + lane * 128;
    const int piece = c / 8;  // 16-byte pieces of the row: two per 16 features
    *reinterpret_cast<uint4*>(srow + ((piece ^ (lane & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    *reinterpret_cast<uint4*>(srow + (((piece + 1) ^ (lane & 7)) << 4)) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
  }
  fence_proxy_async();  // the rows are visible to the TMA
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(map_out, stage, f0 + c0, row0);
    tma_store_commit();
  }
}

__global__ void __launch_bounds__(THREADS, 1)
gated_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                const __grid_constant__ CUtensorMap map_out, int M, int F, int K, int act, int* err) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* tiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int s_failed;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_f = F / BF;
  const int num_tiles = tiles_m * tiles_f;
  const int nkb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], EPI_WARPS);
    }
    s_failed = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_base_slot, 2 * ACC_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_slot;
  // What the kernel before this one wrote (x) or may still read (out) is only touched by the
  // producer and the epilogue warps: they wait for it, the rest of the set-up ran beside it.

  if (warp == 0 && lane == 0) {
    // ---- producer -------------------------------------------------------------------------
    // Weights depend on no earlier kernel: those of the first stages are asked for before
    // `griddepcontrol.wait`, x after it.  (Only this thread waits and triggers: everything the
    // other warps do follows from its loads, and many threads polling for a long kernel before
    // them slow that kernel down.)
    const int my_tiles = blockIdx.x < num_tiles ? (num_tiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    const int total = my_tiles * nkb, pre = min(total, STAGES);
    TileWalk at(blockIdx.x, gridDim.x, tiles_m, nkb, BM);
    auto load_w = [&](const TileWalk& w, int s) {
      unsigned char* stage = tiles + s * STAGE_BYTES;
      tma_load_2d(stage + A_BYTES, &map_w, w.kb * BK, w.f0, &full[s]);
      tma_load_2d(stage + A_BYTES + B_BYTES / 2, &map_w, w.kb * BK, F + w.f0, &full[s]);
    };
    auto load_x = [&](const TileWalk& w, int s) {
      tma_load_2d(tiles + s * STAGE_BYTES, &map_x, w.kb * BK, w.m0, &full[s]);
    };
    TileWalk first = at;
    for (int it = 0; it < pre; ++it, at.next()) {
      mbar_arrive_expect_tx(&full[it], STAGE_BYTES);
      load_w(at, it);
    }
    pdl_wait();
    pdl_launch_dependents();
    for (int it = 0; it < pre; ++it, first.next()) load_x(first, it);
    for (int it = pre, s = pre % STAGES, use = pre / STAGES; it < total; ++it, at.next()) {
      if (!mbar_wait_bounded(&empty[s], (use - 1) & 1)) {
        s_failed = 1;
        break;
      }
      mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
      load_w(at, s);
      load_x(at, s);
      if (++s == STAGES) s = 0, ++use;
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issue ---------------------------------------------------------------------------
    const uint32_t idesc = idesc_bf16_f32(BM, ACC_COLS, false, false);
    // Descriptors are a base plus a constant per stage and per 16 of k (the start address is the
    // descriptor's low field, in units of 16 bytes): 16 columns of K further are 32 bytes
    // further inside the swizzled 128-byte rows.
    const uint64_t a_desc0 = smem_desc_sw128(tiles, 16, 1024);
    const uint64_t b_desc0 = smem_desc_sw128(tiles + A_BYTES, 16, 1024);
    int it = 0, t = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++t) {
      const int buf = t & 1;
      if (t >= 2) {  // the epilogue has read this accumulator's tile before last
        ok = mbar_wait_bounded(&acc_empty[buf], (t / 2 - 1) & 1);
        if (!ok) break;
        tc_fence_after_sync();
      }
      const uint32_t d = tmem + buf * ACC_COLS;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % STAGES;
        if (!mbar_wait_bounded(&full[s], (it / STAGES) & 1)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint64_t off = (uint64_t)((s * STAGE_BYTES) >> 4);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          tc_mma_f16(d, a_desc0 + off + (uint64_t)(k * 2), b_desc0 + off + (uint64_t)(k * 2), idesc, kb > 0 || k > 0);
        tc_commit(&empty[s]);  // the stage is free once these products are done
      }
      if (ok) tc_commit(&acc_full[buf]);
    }
    if (!ok) s_failed = 1;
  } else if (warp >= 2) {
    // ---- epilogue ----------------------------------------------------------------------------
    // A warp may only touch the 32 lanes of tensor memory that (warp % 4) names.
    const int quarter = warp & 3, c0 = ((warp - 2) >> 2) * (BF / 2);
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    unsigned char* out_stage = tiles + STAGES * STAGE_BYTES + (warp - 2) * OUT_WARP_BYTES;
    int t = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++t) {
      const int buf = t & 1;
      const int m0 = (tile % tiles_m) * BM, f0 = (tile / tiles_m) * BF;
      if (!mbar_wait_bounded_relaxed(&acc_full[buf], (t / 2) & 1)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      store_gated_rows(tmem + lane_base + buf * ACC_COLS, c0, out_stage, &map_out, m0 + quarter * 32, f0, act);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (lane == 0) tma_store_wait_read();  // shared memory has been read; the grid's end covers the writes
    if (!ok) s_failed = 1;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && s_failed) atomicOr(err, SB_ERR_TIMEOUT);
  if (warp == 1) tmem_dealloc(tmem, 2 * ACC_COLS);
}

// The same product by pairs of blocks (clusters of two): a pair's tile is 256 tokens x 128
// features, one `tcgen05.mma.cta_group::2` of 256 x 256 x 16 per 16 of k.  Each block fetches its
// own 128 tokens of x and one half of the tile's weights (rank 0 the gate rows, rank 1 the up
// rows), so a block reads a third less per product than alone, and its stages are smaller: six
// fit.  Its accumulator is its own 128 tokens x (128 gate + 128 up) columns, as above.
//   Both blocks' TMA count their bytes at rank 0's full[s]; one thread of rank 0 issues the
//   products for the pair; `tcgen05.commit` arrives at empty[s] and acc_full[b] of both blocks;
//   the epilogue warps of both blocks arrive at rank 0's acc_empty[b].
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_STAGE_BYTES = A_BYTES + B_BYTES / 2;
constexpr size_t PAIR_SMEM_BYTES = (size_t)PAIR_STAGES * PAIR_STAGE_BYTES + OUT_BYTES + 1024;

__global__ void __launch_bounds__(THREADS, 1)
gated_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                     const __grid_constant__ CUtensorMap map_out, int M, int F, int K, int act, int* err) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* tiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t full[PAIR_STAGES], empty[PAIR_STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int s_failed;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_f = F / BF;
  const int num_tiles = tiles_m * tiles_f;
  const int nkb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 2 * EPI_WARPS);
    }
    s_failed = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_base_slot, 2 * ACC_COLS);  // the same columns in both blocks: each takes all there are
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the other block's barriers and tensor memory exist before anything arrives there
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_slot;

  if (warp == 0 && lane == 0) {
    // ---- producer (both blocks) ------------------------------------------------------------
    // As above: weights of the first stages before `griddepcontrol.wait`, x after it.
    const int my_tiles = pair < num_tiles ? (num_tiles - 1 - pair) / num_pairs + 1 : 0;
    const int total = my_tiles * nkb, pre = min(total, PAIR_STAGES);
    TileWalk at(pair, num_pairs, tiles_m, nkb, 2 * BM);
    const uint32_t full0 = mapa_shared(smem_u32(&full[0]), 0);  // rank 0's full[0]; the others follow at 8 bytes each
    auto load_w = [&](const TileWalk& w, int s) {
      tma_load_2d_pair(tiles + s * PAIR_STAGE_BYTES + A_BYTES, &map_w, w.kb * BK, rank == 0 ? w.f0 : F + w.f0, full0 + 8 * s);
    };
    auto load_x = [&](const TileWalk& w, int s) {
      tma_load_2d_pair(tiles + s * PAIR_STAGE_BYTES, &map_x, w.kb * BK, w.m0 + rank * BM, full0 + 8 * s);
    };
    TileWalk first = at;
    for (int it = 0; it < pre; ++it, at.next()) {
      if (rank == 0) mbar_arrive_expect_tx(&full[it], 2 * PAIR_STAGE_BYTES);
      load_w(at, it);
    }
    pdl_wait();
    pdl_launch_dependents();
    for (int it = 0; it < pre; ++it, first.next()) load_x(first, it);
    for (int it = pre, s = pre % PAIR_STAGES, use = pre / PAIR_STAGES; it < total; ++it, at.next()) {
      if (!mbar_wait_bounded(&empty[s], (use - 1) & 1)) {
        s_failed = 1;
        break;
      }
      if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * PAIR_STAGE_BYTES);
      load_w(at, s);
      load_x(at, s);
      if (++s == PAIR_STAGES) s = 0, ++use;
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---- MMA issue (rank 0, for the pair) -----------------------------------------------------
    const uint32_t idesc = idesc_bf16_f32(2 * BM, ACC_COLS, false, false);
    const uint64_t a_desc0 = smem_desc_sw128(tiles, 16, 1024);
    const uint64_t b_desc0 = smem_desc_sw128(tiles + A_BYTES, 16, 1024);
    int it = 0, t = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < num_tiles; tile += num_pairs, ++t) {
      const int buf = t & 1;
      if (t >= 2) {
        ok = mbar_wait_bounded_cluster(&acc_empty[buf], (t / 2 - 1) & 1);
        if (!ok) break;
        tc_fence_after_sync();
      }
      const uint32_t d = tmem + buf * ACC_COLS;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % PAIR_STAGES;
        if (!mbar_wait_bounded(&full[s], (it / PAIR_STAGES) & 1)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint64_t off = (uint64_t)((s * PAIR_STAGE_BYTES) >> 4);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          tc_mma_f16_pair(d, a_desc0 + off + (uint64_t)(k * 2), b_desc0 + off + (uint64_t)(k * 2), idesc, kb > 0 || k > 0);
        tc_commit_pair(&empty[s]);
      }
      if (ok) tc_commit_pair(&acc_full[buf]);
    }
    if (!ok) s_failed = 1;
  } else if (warp >= 2) {
    // ---- epilogue (both blocks, each its own 128 tokens) ----------------------------------------
    const int quarter = warp & 3, c0 = ((warp - 2) >> 2) * (BF / 2);
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    unsigned char* out_stage = tiles + PAIR_STAGES * PAIR_STAGE_BYTES + (warp - 2) * OUT_WARP_BYTES;
    int t = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < num_tiles; tile += num_pairs, ++t) {
      const int buf = t & 1;
      const int m0 = (tile % tiles_m) * 2 * BM + rank * BM, f0 = (tile / tiles_m) * BF;
      if (!mbar_wait_bounded_relaxed(&acc_full[buf], (t / 2) & 1)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      store_gated_rows(tmem + lane_base + buf * ACC_COLS, c0, out_stage, &map_out, m0 + quarter * 32, f0, act);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&acc_empty[buf]), 0));
    }
    if (lane == 0) tma_store_wait_read();  // shared memory has been read; the grid's end covers the writes
    if (!ok) s_failed = 1;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && s_failed) atomicOr(err, SB_ERR_TIMEOUT);
  // Neither block leaves while the other may still arrive at its barriers or multiply into its
  // tensor memory.
  cluster_sync_all();
  if (warp == 1) tmem_dealloc(tmem, 2 * ACC_COLS);
}

// Tensor maps of weights are kept: a weight matrix stays where it is for the life of the model.
int weight_map(CUtensorMap* map, const void* w, long long rows, long long cols) {
  struct Key {
    const void* p;
    long long r, c;
    bool operator==(const Key& o) const { return p == o.p && r == o.r && c == o.c; }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      return std::hash<const void*>()(k.p) ^ (std::hash<long long>()(k.r) * 31) ^ (std::hash<long long>()(k.c) * 131);
    }
  };
  static std::mutex mu;
  static std::unordered_map<Key, CUtensorMap, Hash> maps;
  std::lock_guard<std::mutex> lock(mu);
  const Key key{w, rows, cols};
  auto it = maps.find(key);
  if (it == maps.end()) {
    CUtensorMap m;
    if (sb_make_map_2d(&m, w, rows, cols, BF) != 0) return -12;
    it = maps.emplace(key, m).first;
  }
  *map = it->second;
  return 0;
}

}  // namespace

// x: [M, K]; w: [2F, K] (gate rows, then up rows); out: [M, F].  Returns -9 for shapes the kernel
// does not take (the caller then uses another product): F not a multiple of 128, K not a
// multiple of 8, operands not 16-byte aligned.  blocks: 0 = one per SM.  pairs: 1 = blocks work in
// pairs on tiles of 256 tokens, 0 = each alone on tiles of 128.
extern "C" int sb_gemm_gated_tc(const void* x, const void* w, void* out, int M, int F, int K, int act, int blocks,
                                int pairs, int* err, cudaStream_t stream) {
  if (M == 0 || F == 0) return 0;
  if (F % BF != 0 || K % 8 != 0 || K <= 0 || act < 0 || act > 2) return -9;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15) return -9;
  static int configured = -1, num_sms = 0, max_pairs = 0;
  if (configured < 0) {
    int device = 0;
    cudaGetDevice(&device);
    if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || num_sms <= 0) num_sms = 1;
    configured = (int)cudaFuncSetAttribute(gated_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (configured == 0)
      configured = (int)cudaFuncSetAttribute(gated_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)PAIR_SMEM_BYTES);
    if (configured == 0) {
      // how many pairs the GPU holds at once (a pair lives inside one GPC)
      cudaLaunchConfig_t config = {};
      config.gridDim = dim3(2 * num_sms);
      config.blockDim = dim3(THREADS);
      config.dynamicSmemBytes = PAIR_SMEM_BYTES;
      cudaLaunchAttribute attribute[1];
      attribute[0].id = cudaLaunchAttributeClusterDimension;
      attribute[0].val.clusterDim.x = 2;
      attribute[0].val.clusterDim.y = 1;
      attribute[0].val.clusterDim.z = 1;
      config.attrs = attribute;
      config.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&max_pairs, gated_tc_pair_kernel, &config) != cudaSuccess) {
        cudaGetLastError();
        max_pairs = 0;
      }
    }
  }
  if (configured != 0) return configured;
  CUtensorMap map_x, map_w, map_out;
  if (weight_map(&map_w, w, 2LL * F, K) != 0) return -12;
  if (sb_make_map_2d(&map_x, x, M, K, BM) != 0) return -12;
  if (sb_make_map_2d(&map_out, out, M, F, 32) != 0) return -12;
  if (pairs && max_pairs > 0) {
    const int num_tiles = ((M + 2 * BM - 1) / (2 * BM)) * (F / BF);
    const int n = min(num_tiles, blocks > 0 ? max(blocks / 2, 1) : max_pairs);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)(2 * n));
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = PAIR_SMEM_BYTES;
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
    cudaError_t e = cudaLaunchKernelEx(&config, gated_tc_pair_kernel, map_x, map_w, map_out, M, F, K, act, err);
    if (e != cudaSuccess) return (int)e;
    SB_LAUNCH_CHECK();
    return 0;
  }
  const int num_tiles = ((M + BM - 1) / BM) * (F / BF);
  const int grid = min(num_tiles, blocks > 0 ? blocks : num_sms);
  cudaError_t e = sb_launch_early(gated_tc_kernel, dim3(grid), dim3(THREADS), SMEM_BYTES, stream, map_x, map_w,
                                  map_out, M, F, K, act, err);
  if (e != cudaSuccess) return (int)e;
  SB_LAUNCH_CHECK();
  return 0;
}
