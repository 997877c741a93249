// Weight-streaming matrix product for a serving batch on the fifth-generation tensor cores:
//   out[M, N] = x[M, K] . w[N, K]^T,  bfloat16 in, float32 accumulate in tensor memory, M <= 128.
//
// With 17 to 128 tokens the product is still bound by reading w once from HBM, but the tokens are
// too many for the register-fed mma.sync kernel of smaller steps (gemm_skinny_bf16.cu): x would
// have to pass the load units once per 16 weight rows.  Here nothing passes registers on the way
// in.  The operands are swapped: 128 weight rows are the 128-row operand of `tcgen05.mma`, the
// tokens (32, 64 or 128, padded by the TMA's zero fill) are its N; both arrive by TMA (128-byte
// swizzle) in a ring of shared-memory stages and are read from there by the tensor core; the
// accumulator [128 weight rows x tokens] lives in tensor memory.  Roles:
//   warp 0: TMA producer (one thread).  It asks for the weights of its first stages before
//           `griddepcontrol.wait`: weights depend on no earlier kernel, so their stream starts
//           while the kernel before this one still runs; x follows after the wait.
//   warp 1: tensor-memory allocation, MMA issue (one thread)
//   warps 2..9: read the accumulator back (`tcgen05.ld`): one 32-lane quarter and half of the
//           token columns each
// When a product has too few 128-row tiles to fill the GPU (attention output, down projection),
// k is split over the blocks of a thread-block cluster; their partial sums meet through
// distributed shared memory in rank order (gemm_epilogue.cuh), where the epilogues are too
// (bfloat16; float32 with soft cap; gated activation; fused q, k, v rotation and cache write).
//
// Barriers: full[s] (a stage has landed), empty[s] (its MMAs are done: tcgen05.commit), done (the
// accumulator is ready).  Every wait is bounded; a wait that runs out sets SB_ERR_TIMEOUT, and the
// block still passes every barrier and releases its tensor memory before it leaves.
// K must be a multiple of 8 (16-byte rows for the TMA); rows and columns beyond M, N, K read as zero.
#include <mutex>
#include <unordered_map>

#include "gemm_epilogue.cuh"
#include "tma_mbar.cuh"

namespace {

using namespace sbx;
using sbg::RopeStore;
using sbg::RSTRIDE;

constexpr int BK = 64;                     // k of a stage: one 128-byte swizzled row
constexpr int A_BYTES = 128 * BK * 2;      // 128 weight rows
constexpr int THREADS = 320;  // producer warp, MMA warp, eight warps that read the accumulator back
constexpr int MAX_STAGES = 8;

template <int BNT, int STAGES, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
stream_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 void* __restrict__ out, int M, int N, int K, int kb_per_block, int ks, float cap, int act,
                 const RopeStore rs, int* err) {
  constexpr int B_BYTES = BNT * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  static_assert((size_t)STAGES * STAGE_BYTES >= (size_t)BNT * RSTRIDE * sizeof(float), "the sums reuse the stages");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* tiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t full[MAX_STAGES], empty[MAX_STAGES], done;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int s_failed;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / ks, rank = blockIdx.x - tile * ks;
  const sbg::TileGeometry tg = sbg::tile_geometry<EPI>(tile, N, rs);
  const int total_kb = (K + BK - 1) / BK;
  const int kb_begin = rank * kb_per_block;
  const int nkb = max(min(total_kb, kb_begin + kb_per_block) - kb_begin, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&done, 1);
    s_failed = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_base_slot, BNT);  // BNT columns of float32: a power of two >= 32
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_d = tmem_base_slot;

  if (warp == 0 && lane == 0) {
    // ---- producer -------------------------------------------------------------------------
    auto load_w = [&](int kb) {
      unsigned char* stage = tiles + (kb % STAGES) * STAGE_BYTES;
      const int k = (kb_begin + kb) * BK;
      tma_load_2d(stage, &map_w, k, tg.base0, &full[kb % STAGES]);                           // local rows 0..63
      tma_load_2d(stage + A_BYTES / 2, &map_w, k, tg.base0 + tg.second, &full[kb % STAGES]);  // local rows 64..127
    };
    auto load_x = [&](int kb) {
      tma_load_2d(tiles + (kb % STAGES) * STAGE_BYTES + A_BYTES, &map_x, (kb_begin + kb) * BK, 0, &full[kb % STAGES]);
    };
    const int pre = min(nkb, STAGES);
    for (int kb = 0; kb < pre; ++kb) {
      mbar_arrive_expect_tx(&full[kb], STAGE_BYTES);
      load_w(kb);
    }
    pdl_wait();  // x is written by the kernel before this one
    for (int kb = 0; kb < pre; ++kb) load_x(kb);
    for (int kb = pre; kb < nkb; ++kb) {
      const int s = kb % STAGES;
      if (!mbar_wait_bounded(&empty[s], (kb / STAGES - 1) & 1)) {
        s_failed = 1;
        break;
      }
      mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
      load_w(kb);
      load_x(kb);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issue ---------------------------------------------------------------------------
    const uint32_t idesc = idesc_bf16_f32(128, BNT, false, false);
    for (int kb = 0; kb < nkb; ++kb) {
      const int s = kb % STAGES;
      if (!mbar_wait_bounded(&full[s], (kb / STAGES) & 1)) {
        s_failed = 1;
        break;
      }
      tc_fence_after_sync();
      const unsigned char* a = tiles + s * STAGE_BYTES;
      const unsigned char* b = a + A_BYTES;
#pragma unroll
      for (int k = 0; k < BK / 16; ++k) {
        // 16 columns of K further = 32 bytes further inside the swizzled 128-byte rows
        tc_mma_f16(tmem_d, smem_desc_sw128(a + k * 32, 16, 1024), smem_desc_sw128(b + k * 32, 16, 1024), idesc,
                   kb > 0 || k > 0);
      }
      tc_commit(&empty[s]);  // the stage may be refilled once these MMAs have read it
    }
    tc_commit(&done);
  }
  // Every role has issued its work, and the producer is past its wait: the kernel after this one
  // may start (its own weights do not depend on this one's result).
  __syncthreads();
  pdl_wait();
  pdl_launch_dependents();

  // ---- the accumulator goes to shared memory as sums[token][local row] ----------------------
  float* sums = reinterpret_cast<float*>(tiles);  // the stages are free once `done` has completed
  if (warp >= 2) {
    const int quarter = warp & 3;            // the 32 lanes of tensor memory this warp may read
    const int c0 = ((warp - 2) >> 2) * (BNT / 2);  // its half of the token columns
    bool ok = true;
    if (nkb > 0) {
      ok = mbar_wait_bounded(&done, 0);
      if (!ok) s_failed = 1;
    }
    tc_fence_after_sync();
#pragma unroll
    for (int c = c0; c < c0 + BNT / 2; c += 16) {
      uint32_t r[16];
      if (nkb > 0 && ok) {
        tmem_load_32x16(tmem_d + ((uint32_t)(quarter * 32) << 16) + c, r);
        tmem_wait_load();
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = 0u;  // a block without k of its own adds nothing
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) sums[(size_t)(c + j) * RSTRIDE + quarter * 32 + lane] = __uint_as_float(r[j]);
    }
  }
  tc_fence_before_sync();
  sbg::finish_tile<EPI>(sums, BNT, M, N, ks, rank, tg, out, cap, act, rs);  // begins with a barrier
  __syncthreads();
  tc_fence_after_sync();
  if (threadIdx.x == 0 && s_failed) atomicOr(err, SB_ERR_TIMEOUT);
  if (warp == 1) tmem_dealloc(tmem_d, BNT);
}

// Tensor maps of weight matrices are kept: a weight's address, shape and box never change.
struct MapKey {
  const void* p;
  long long rows, cols;
  bool operator==(const MapKey& o) const { return p == o.p && rows == o.rows && cols == o.cols; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.p) ^ (std::hash<long long>()(k.rows) * 31) ^ (std::hash<long long>()(k.cols) * 131);
  }
};

int weight_map(CUtensorMap* map, const void* w, long long rows, long long cols) {
  static std::mutex lock;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> maps;
  std::lock_guard<std::mutex> guard(lock);
  const MapKey key{w, rows, cols};
  auto it = maps.find(key);
  if (it == maps.end()) {
    CUtensorMap m;
    if (sb_make_map_2d(&m, w, rows, cols, 64) != 0) return -12;
    if (maps.size() > 4096) maps.clear();  // (weights that were freed and replaced: start over)
    it = maps.emplace(key, m).first;
  }
  *map = it->second;
  return 0;
}

// The kernel needs more dynamic shared memory than a launch gets by default; said once per kernel,
// before anything asks how many of its blocks or clusters fit the GPU.
template <int BNT, int STAGES, int EPI>
int configure_kernel() {
  constexpr size_t smem_bytes = (size_t)STAGES * (A_BYTES + BNT * BK * 2) + 1024;
  static int status = -1;
  if (status < 0)
    status = (int)cudaFuncSetAttribute(stream_tc_kernel<BNT, STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem_bytes);
  return status;
}

template <int BNT, int STAGES, int EPI>
int max_active_clusters(int ks, size_t smem_bytes) {
  if (configure_kernel<BNT, STAGES, EPI>() != 0) return 0;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(ks * 64);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem_bytes;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = ks;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, stream_tc_kernel<BNT, STAGES, EPI>, &config) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  return n;
}

// Blocks of a cluster for a product with `tiles` row tiles: the size (at most 8) that brings the
// launch closest to one block on every SM without a second wave, given how many clusters of each
// size the GPU holds at once (clusters live inside one GPC, so a size that does not divide a GPC's
// SMs leaves some of them out: 18 tiles run as clusters of 6, not of 8).
template <int BNT, int STAGES, int EPI>
int choose_split(int tiles, int total_kb, size_t smem_bytes) {
  static int max_clusters[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};  // by cluster size
  static int num_sms = 0;
  if (num_sms == 0) {
    int device = 0;
    cudaGetDevice(&device);
    if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || num_sms <= 0) num_sms = 1;
  }
  int best = 1, best_blocks = tiles;
  for (int ks = 2; ks <= 8; ++ks) {
    if (total_kb / ks < 4) break;  // every block should have a few stages of k
    if (max_clusters[ks] < 0) max_clusters[ks] = max_active_clusters<BNT, STAGES, EPI>(ks, smem_bytes);
    if (tiles > max_clusters[ks]) continue;  // would need a second wave of clusters
    const int blocks = tiles * ks;
    if (blocks > best_blocks && blocks <= num_sms) {
      best = ks;
      best_blocks = blocks;
    }
  }
  return best;
}

template <int BNT, int STAGES, int EPI>
int launch_stream(const bf16* x, const bf16* w, void* out, int M, int N, int K, float cap, int act, int split_override,
                  int* err, cudaStream_t stream, const RopeStore& rs) {
  constexpr size_t smem_bytes = (size_t)STAGES * (A_BYTES + BNT * BK * 2) + 1024;
  if (const int e = configure_kernel<BNT, STAGES, EPI>()) return e;
  CUtensorMap map_w, map_x;
  if (weight_map(&map_w, w, N, K) != 0) return -12;
  if (sb_make_map_2d(&map_x, x, M, K, BNT) != 0) return -12;
  const int tiles = EPI == 3 ? N / 128 : (EPI == 2 ? (N / 2 + 63) / 64 : (N + 127) / 128);
  const int total_kb = (K + BK - 1) / BK;
  int ks = EPI == 1 ? 1 : choose_split<BNT, STAGES, EPI>(tiles, total_kb, smem_bytes);
  if (split_override >= 1 && split_override <= 8) ks = split_override;
  const int kb_per_block = (total_kb + ks - 1) / ks;

  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)(tiles * ks));
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  int n_attr = 0;
  if (sb_pdl_level() >= 1) {
    attribute[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  if (ks > 1) {
    attribute[n_attr].id = cudaLaunchAttributeClusterDimension;
    attribute[n_attr].val.clusterDim.x = ks;
    attribute[n_attr].val.clusterDim.y = 1;
    attribute[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  config.attrs = attribute;
  config.numAttrs = n_attr;
  cudaError_t e = cudaLaunchKernelEx(&config, stream_tc_kernel<BNT, STAGES, EPI>, map_w, map_x, out, M, N, K,
                                     kb_per_block, ks, cap, act, rs, err);
  if (e != cudaSuccess) return (int)e;
  SB_LAUNCH_CHECK();
  return 0;
}

template <int BNT, int DEEP, int SHALLOW, int EPI>
int launch_stream_depth(const bf16* x, const bf16* w, void* out, int M, int N, int K, float cap, int act,
                        int split_override, int stages, int* err, cudaStream_t stream, const RopeStore& rs) {
  // Stages: the deep ring (8; 6 with 128 tokens) gives one block the whole SM; the shallow one
  // keeps two blocks on an SM (this kernel's and the next one's, which then starts its weights
  // early).  Measured on the four products of a Gemma 2 2B layer, the deep ring is the faster one
  // where a block streams a few hundred KB of weights, the shallow one for the small products.
  bool deep = stages >= 6;
  if (stages == 0) {
    const int tiles = EPI == 3 ? N / 128 : (EPI == 2 ? (N / 2 + 63) / 64 : (N + 127) / 128);
    const int total_kb = (K + BK - 1) / BK;
    constexpr size_t smem_deep = (size_t)DEEP * (A_BYTES + BNT * BK * 2) + 1024;
    const int ks = (EPI == 1 || (split_override >= 1 && split_override <= 8))
                       ? (split_override >= 1 ? split_override : 1)
                       : choose_split<BNT, DEEP, EPI>(tiles, total_kb, smem_deep);
    deep = (total_kb + ks - 1) / ks >= 20;
  }
  return deep ? launch_stream<BNT, DEEP, EPI>(x, w, out, M, N, K, cap, act, split_override, err, stream, rs)
              : launch_stream<BNT, SHALLOW, EPI>(x, w, out, M, N, K, cap, act, split_override, err, stream, rs);
}

template <int EPI>
int launch_stream_rows(const bf16* x, const bf16* w, void* out, int M, int N, int K, float cap, int act,
                       int split_override, int stages, int* err, cudaStream_t stream, const RopeStore& rs = RopeStore{}) {
  if (M <= 32) return launch_stream_depth<32, 8, 4, EPI>(x, w, out, M, N, K, cap, act, split_override, stages, err, stream, rs);
  if (M <= 64) return launch_stream_depth<64, 8, 4, EPI>(x, w, out, M, N, K, cap, act, split_override, stages, err, stream, rs);
  return launch_stream_depth<128, 6, 3, EPI>(x, w, out, M, N, K, cap, act, split_override, stages, err, stream, rs);
}

}  // namespace

// Returns -9 when the shape is outside what the kernel takes (the caller then uses another
// product): M > 128, K not a multiple of 8, N odd for the gated epilogue, operands not 16-byte aligned.
// split_override: 0 lets the launch choose how many blocks share a tile's k; 1 to 8 fix it (tests).
// stages: 0 lets the launch choose the depth of the ring of stages; 8 the deep one, 4 the shallow one (tests).
extern "C" int sb_gemm_stream_tc(const void* x, const void* w, void* out, int M, int N, int K, int epilogue, float cap,
                                 int act, int split_override, int stages, int* err, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M > 128 || K % 8 != 0 || K <= 0 || epilogue < 0 || epilogue > 2) return -9;
  if (epilogue == 2 && (N % 2 != 0 || act < 0 || act > 2)) return -9;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return -9;
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)w;
  if (epilogue == 0) return launch_stream_rows<0>(xp, wp, out, M, N, K, cap, act, split_override, stages, err, stream);
  if (epilogue == 1) return launch_stream_rows<1>(xp, wp, out, M, N, K, cap, act, split_override, stages, err, stream);
  return launch_stream_rows<2>(xp, wp, out, M, N, K, cap, act, split_override, stages, err, stream);
}

// The fused q, k, v projection of an attention layer for up to 128 tokens (see sb_qkv_rope_skinny
// for the arguments).  Returns -9 for shapes it does not take (M > 128, K % 8 != 0, head_dim % 128 != 0).
extern "C" int sb_qkv_rope_stream_tc(const void* x, const void* w, int M, int K, const float* cos_t, const float* sin_t,
                                     float q_scale, void* q_out, void* cache, const int* block_table, int max_pages,
                                     const int* token_seq, const int* positions, int num_q_heads, int num_kv_proj,
                                     int head_dim, int page_size, int num_pages, int* err, int split_override,
                                     int stages, cudaStream_t stream) {
  if (M == 0) return 0;
  if (M > 128 || K % 8 != 0 || K <= 0 || head_dim <= 0 || head_dim % 128 != 0 || num_q_heads <= 0) return -9;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return -9;
  RopeStore rs{cos_t, sin_t, q_scale, (bf16*)q_out, (bf16*)cache, block_table, max_pages, token_seq, positions,
               num_q_heads, num_kv_proj, head_dim, page_size, num_pages, err};
  const int N = (num_q_heads + 2 * num_kv_proj) * head_dim;
  return launch_stream_rows<3>((const bf16*)x, (const bf16*)w, nullptr, M, N, K, 0.f, 0, split_override, stages, err,
                               stream, rs);
}
