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
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + 1024;

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// The gate's activation.  The tanh form of GELU is written as g / (1 + exp(-2 y)) with
// y = sqrt(2 / pi) (g + 0.044715 g^3), which is the same function (0.5 (1 + tanh y) = 1 / (1 + exp(-2 y)))
// at two special-function instructions instead of a library tanh; both are exact to a few units
// in the last place of float32, far below the bfloat16 rounding that follows.
__device__ __forceinline__ float gate_act(float g, int act) {
  if (act == 0) {
    const float y = 0.7978845608028654f * fmaf(0.044715f * g * g, g, g);
    return __fdividef(g, 1.0f + exp2f(-2.0f * 1.4426950408889634f * y));
  }
  return sbg::gated_act(g, act);
}

// One thread's row of a tile: gate and up sums of the features [c0, c1) from the accumulator at
// `acc` (this warp's lanes), the activation, bfloat16 results to out[row, f0 + c0 ..].  Every lane
// takes part in the warp-wide tensor-memory loads; only rows of the matrix store.
__device__ __forceinline__ void store_gated_rows(uint32_t acc, int c0, int c1, int row, int M, int F, int f0,
                                                 bf16* __restrict__ out, int act) {
  bf16* orow = out + (size_t)row * F + f0;
#pragma unroll 1
  for (int c = c0; c < c1; c += 16) {
    uint32_t g[16], u[16];
    tmem_load_32x16(acc + c, g);
    tmem_load_32x16(acc + BF + c, u);
    tmem_wait_load();
    uint32_t packed[8];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      // The projections are rounded to bfloat16 before the activation, as a product that
      // stores them would.
      const float g0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(g[i])));
      const float g1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(g[i + 1])));
      const float u0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[i])));
      const float u1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[i + 1])));
      packed[i / 2] = pack_bf16(gate_act(g0, act) * u0, gate_act(g1, act) * u1);
    }
    if (row < M) {
      *reinterpret_cast<uint4*>(orow + c) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      *reinterpret_cast<uint4*>(orow + c + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    }
  }
}

__global__ void __launch_bounds__(THREADS, 1)
gated_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                bf16* __restrict__ out, int M, int F, int K, int act, int* err) {
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
  pdl_wait_block();  // x is written by the kernel before this one, and out may still be read by it
  pdl_launch_dependents();

  if (warp == 0 && lane == 0) {
    // ---- producer -------------------------------------------------------------------------
    int it = 0;  // stages filled so far, over all tiles
    for (int tile = blockIdx.x; tile < num_tiles && !s_failed; tile += gridDim.x) {
      const int m0 = (tile % tiles_m) * BM, f0 = (tile / tiles_m) * BF;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % STAGES;
        if (it >= STAGES && !mbar_wait_bounded(&empty[s], (it / STAGES - 1) & 1)) {
          s_failed = 1;
          break;
        }
        unsigned char* stage = tiles + s * STAGE_BYTES;
        mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
        tma_load_2d(stage, &map_x, kb * BK, m0, &full[s]);
        tma_load_2d(stage + A_BYTES, &map_w, kb * BK, f0, &full[s]);
        tma_load_2d(stage + A_BYTES + B_BYTES / 2, &map_w, kb * BK, F + f0, &full[s]);
      }
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
    int t = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++t) {
      const int buf = t & 1;
      const int m0 = (tile % tiles_m) * BM, f0 = (tile / tiles_m) * BF;
      if (!mbar_wait_bounded(&acc_full[buf], (t / 2) & 1)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      store_gated_rows(tmem + lane_base + buf * ACC_COLS, c0, c0 + BF / 2, m0 + quarter * 32 + lane, M, F, f0, out, act);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
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
constexpr size_t PAIR_SMEM_BYTES = (size_t)PAIR_STAGES * PAIR_STAGE_BYTES + 1024;

__global__ void __launch_bounds__(THREADS, 1)
gated_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                     bf16* __restrict__ out, int M, int F, int K, int act, int* err) {
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
  pdl_wait_block();
  pdl_launch_dependents();

  if (warp == 0 && lane == 0) {
    // ---- producer (both blocks) ------------------------------------------------------------
    int it = 0;
    for (int tile = pair; tile < num_tiles && !s_failed; tile += num_pairs) {
      const int m0 = (tile % tiles_m) * 2 * BM + rank * BM, f0 = (tile / tiles_m) * BF;
      const int w_row = rank == 0 ? f0 : F + f0;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % PAIR_STAGES;
        if (it >= PAIR_STAGES && !mbar_wait_bounded_cluster(&empty[s], (it / PAIR_STAGES - 1) & 1)) {
          s_failed = 1;
          break;
        }
        unsigned char* stage = tiles + s * PAIR_STAGE_BYTES;
        const uint32_t bar = mapa_shared(smem_u32(&full[s]), 0);
        if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * PAIR_STAGE_BYTES);
        tma_load_2d_pair(stage, &map_x, kb * BK, m0, bar);
        tma_load_2d_pair(stage + A_BYTES, &map_w, kb * BK, w_row, bar);
      }
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
        if (!mbar_wait_bounded_cluster(&full[s], (it / PAIR_STAGES) & 1)) {
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
    int t = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < num_tiles; tile += num_pairs, ++t) {
      const int buf = t & 1;
      const int m0 = (tile % tiles_m) * 2 * BM + rank * BM, f0 = (tile / tiles_m) * BF;
      if (!mbar_wait_bounded_cluster(&acc_full[buf], (t / 2) & 1)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      store_gated_rows(tmem + lane_base + buf * ACC_COLS, c0, c0 + BF / 2, m0 + quarter * 32 + lane, M, F, f0, out, act);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&acc_empty[buf]), 0));
    }
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
  CUtensorMap map_x, map_w;
  if (weight_map(&map_w, w, 2LL * F, K) != 0) return -12;
  if (sb_make_map_2d(&map_x, x, M, K, BM) != 0) return -12;
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
    cudaError_t e = cudaLaunchKernelEx(&config, gated_tc_pair_kernel, map_x, map_w, (bf16*)out, M, F, K, act, err);
    if (e != cudaSuccess) return (int)e;
    SB_LAUNCH_CHECK();
    return 0;
  }
  const int num_tiles = ((M + BM - 1) / BM) * (F / BF);
  const int grid = min(num_tiles, blocks > 0 ? blocks : num_sms);
  cudaError_t e = sb_launch(gated_tc_kernel, dim3(grid), dim3(THREADS), SMEM_BYTES, stream, map_x, map_w, (bf16*)out, M,
                            F, K, act, err);
  if (e != cudaSuccess) return (int)e;
  SB_LAUNCH_CHECK();
  return 0;
}
