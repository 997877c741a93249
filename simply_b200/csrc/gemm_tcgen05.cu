// Matrix product on the fifth-generation tensor cores:
//   out[M, N] = x[M, K] . w[N, K]^T, bfloat16 in, float32 accumulate in tensor memory.
//
// One block computes a 128 x BN tile of out.  Operand tiles of 64 columns of K arrive by TMA
// (128-byte swizzle) in a ring of shared-memory stages; one thread issues `tcgen05.mma`
// (128 x BN x 16 per instruction, four per stage) with the accumulator in tensor memory; four
// warps read the accumulator back with `tcgen05.ld` and store the tile.  Roles:
//   warp 0: TMA producer (one thread)      warp 1: tensor-memory allocation, MMA issue (one thread)
//   warps 2..5: epilogue, one 32-lane quarter of tensor memory each
// Barriers: full[s] (a stage has landed), empty[s] (its MMAs are done: tcgen05.commit),
// done (the whole accumulator is ready).  All waits are bounded; a wait that runs out sets
// SB_ERR_TIMEOUT, and the block still releases its tensor memory before it leaves.
//
// K must be a multiple of 8 (16-byte rows for the TMA); rows and columns beyond M, N, K read
// as zero and are not stored.  The soft cap of the output layer is an optional epilogue
// (simply/model_lib.py:107-109).
#include "common.cuh"
#include "tma_mbar.cuh"

namespace {

using namespace sbx;

constexpr int TC_BM = 128, TC_BK = 64, TC_STAGES = 4;
constexpr int TC_THREADS = 192;

template <int BN, bool OUT_F32>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               void* __restrict__ out, int M, int N, int K, float cap, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* tiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t full[TC_STAGES], empty[TC_STAGES], done;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int s_failed;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * BN;
  const int k_blocks = (K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&done, 1);
    s_failed = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_base_slot, BN);  // BN columns of float32: a power of two >= 32
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_d = tmem_base_slot;

  if (warp == 0 && lane == 0) {
    // ---- producer -------------------------------------------------------------------------
    for (int kb = 0; kb < k_blocks; ++kb) {
      const int s = kb % TC_STAGES;
      if (kb >= TC_STAGES && !mbar_wait_bounded(&empty[s], (kb / TC_STAGES - 1) & 1)) {
        s_failed = 1;
        break;
      }
      mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
      tma_load_2d(tiles + s * STAGE_BYTES, &map_x, kb * TC_BK, m0, &full[s]);
      tma_load_2d(tiles + s * STAGE_BYTES + A_BYTES, &map_w, kb * TC_BK, n0, &full[s]);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issue ---------------------------------------------------------------------------
    const uint32_t idesc = idesc_bf16_f32(TC_BM, BN, false, false);
    for (int kb = 0; kb < k_blocks; ++kb) {
      const int s = kb % TC_STAGES;
      if (!mbar_wait_bounded(&full[s], (kb / TC_STAGES) & 1)) {
        s_failed = 1;
        break;
      }
      tc_fence_after_sync();
      const unsigned char* a = tiles + s * STAGE_BYTES;
      const unsigned char* b = a + A_BYTES;
#pragma unroll
      for (int k = 0; k < TC_BK / 16; ++k) {
        // 16 columns of K further = 32 bytes further inside the swizzled 128-byte rows
        tc_mma_f16(tmem_d, smem_desc_sw128(a + k * 32, 16, 1024), smem_desc_sw128(b + k * 32, 16, 1024), idesc,
                   kb > 0 || k > 0);
      }
      tc_commit(&empty[s]);  // the stage may be refilled once these MMAs have read it
    }
    tc_commit(&done);
  } else if (warp >= 2) {
    // ---- epilogue ----------------------------------------------------------------------------
    const bool ok = mbar_wait_bounded(&done, 0);
    if (!ok) s_failed = 1;
    tc_fence_after_sync();
    const int quarter = warp & 3;  // the 32 lanes of tensor memory this warp may read
    const int row = m0 + quarter * 32 + lane;
    if (ok) {
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_load_32x32(tmem_d + ((uint32_t)(quarter * 32) << 16) + c, r);
        tmem_wait_load();
        if (row < M) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = n0 + c + j;
            if (col >= N) break;
            float v = __uint_as_float(r[j]);
            if (cap > 0.f) v = cap * tanhf(v / cap);
            if (OUT_F32)
              reinterpret_cast<float*>(out)[(size_t)row * N + col] = v;
            else
              reinterpret_cast<bf16*>(out)[(size_t)row * N + col] = __float2bfloat16_rn(v);
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && s_failed) atomicOr(err, SB_ERR_TIMEOUT);
  if (warp == 1) tmem_dealloc(tmem_d, BN);
}

template <int BN, bool OUT_F32>
int launch_tc(const CUtensorMap& mx, const CUtensorMap& mw, void* out, int M, int N, int K, float cap, int* err,
              cudaStream_t stream) {
  constexpr size_t smem = (size_t)TC_STAGES * (TC_BM + BN) * TC_BK * 2 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, OUT_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  sb_launch(gemm_tc_kernel<BN, OUT_F32>, dim3((N + BN - 1) / BN, (M + TC_BM - 1) / TC_BM), TC_THREADS, smem, stream,
            mx, mw, out, M, N, K, cap, err);
  SB_LAUNCH_CHECK();
  return 0;
}

}  // namespace

// out[M, N] = x[M, K] . w[N, K]^T.  out_f32: float32 output (with soft cap if cap > 0), else bfloat16.
// tile_n: 64, 128 or 256 columns per block.  Returns -9 for shapes it does not take (K % 8 != 0).
extern "C" int sb_gemm_tcgen05(const void* x, const void* w, void* out, int M, int N, int K, int out_f32, float cap,
                               int tile_n, int* err, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (K % 8 != 0 || K <= 0) return -9;
  CUtensorMap mx, mw;
  if (sb_make_map_2d(&mx, x, M, K, TC_BM) != 0) return -12;
  if (sb_make_map_2d(&mw, w, N, K, tile_n) != 0) return -12;
  if (tile_n == 64) return out_f32 ? launch_tc<64, true>(mx, mw, out, M, N, K, cap, err, stream)
                                   : launch_tc<64, false>(mx, mw, out, M, N, K, cap, err, stream);
  if (tile_n == 128) return out_f32 ? launch_tc<128, true>(mx, mw, out, M, N, K, cap, err, stream)
                                    : launch_tc<128, false>(mx, mw, out, M, N, K, cap, err, stream);
  if (tile_n == 256) return out_f32 ? launch_tc<256, true>(mx, mw, out, M, N, K, cap, err, stream)
                                    : launch_tc<256, false>(mx, mw, out, M, N, K, cap, err, stream);
  return -9;
}
