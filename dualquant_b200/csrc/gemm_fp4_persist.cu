// Block-scaled FP4 W4A4 GEMM for prefill-size batches: the persistent form of gemm_fp4_kernel.
//
//   Y[m,n] = r[n] * tw * tx[m] * sum_k ( qx[m,k] * sfx[m, k/B] ) * ( qw[n,k] * sfw[n, k/B] )
//
// Same operands, same instruction stream per stage (four tcgen05.mma kind::mxf4nvf4.block_scale of
// 128 x 256 x 64 with the block scales in tensor memory) and therefore the same results as the
// one-tile-per-CTA kernel; what changes is what happens between tiles.  One CTA per SM walks over
// tiles of 128 weight rows x 256 tokens: the producer, the scale-factor copiers and the rings they
// feed never stop at a tile boundary, so the next tile's operands are in shared memory while the
// accumulator of the finished one is drained, and the only time the tensor core idles per tile is
// that drain (eight epilogue warps: tensor memory -> registers -> [token][row] chunks in shared
// memory -> tiled bulk stores through a ring of four 16 KB buffers).  The one-tile kernel pays CTA
// launch, barrier and tensor-memory set-up, the first operand round trip and the drain on every
// tile - about as long as the K loop itself at K = 3584.
//
//   warp 0       TMA producer (one lane)            warp 1   UMMA issue (one lane), TMEM owner
//   warps 2, 3   scale factors shared -> tensor memory (tcgen05.cp): weights + activation rows 0-127,
//                activation rows 128-255 (a copy costs its thread ~70 cycles of issue)
//   warps 4-11   epilogue, two teams of four (one warp per TMEM lane quarter), alternate 32-token
//                chunks; a warp first moves all its columns to registers and hands the accumulator
//                back, then converts and stores while the next tile's UMMAs run
// Every barrier wait is bounded.
#include "dq_common.h"
#include "dq_ptx.cuh"
#include "gemm_fp4.cuh"

#include <cuda_bf16.h>
#include <string.h>

namespace dq {
namespace fp4p {

constexpr int kTok = 256;
constexpr int kStages = 3;
constexpr int kBBytes = kTok * 128;
constexpr int kOffA = 0;
constexpr int kOffB = kOffA + kStages * kFTileBytes;
constexpr int kOffSFA = kOffB + kStages * kBBytes;
constexpr int kOffSFB = kOffSFA + kStages * 2048;
constexpr int kOffOut = kOffSFB + kStages * 2 * 2048;
constexpr int kOutBuf = 32 * kFBN * 4;  // one chunk: 32 tokens x 128 rows of fp32 (bf16 uses half)
constexpr int kOffBar = kOffOut + 4 * kOutBuf;
constexpr int kNumBars = 3 * kStages + 2;
constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16;
constexpr int kThreads = 384;  // twelve warps: registers are granted to warps in fours, 168 per thread at this size
constexpr int kSfColsStage = 48;  // 16 columns of weight scale factors, 2 x 16 of activation scale factors
constexpr int kSfColBase = kTok;
constexpr uint32_t kTmemCols = 512;
static_assert(kSmemBytes <= 227 * 1024, "shared memory");
static_assert(kOffB % 1024 == 0 && kOffOut % 1024 == 0, "operand tiles on 1 KB boundaries");
static_assert(kSfColBase + kStages * kSfColsStage <= 512, "tensor memory columns");

enum { PSITE_TMA = 71, PSITE_MMA = 72, PSITE_SF = 73, PSITE_EPI = 74, PSITE_ACC = 75, PSITE_ALIGN = 76 };

__device__ __forceinline__ void bulk_wait_group_read1() {
  asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}

template <int NVFP4>
__global__ void __launch_bounds__(kThreads, 1)
gemm_fp4_persist_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                        const __grid_constant__ CUtensorMap tm_y, const uint8_t* __restrict__ sfw,
                        const uint8_t* __restrict__ sfx, const float* __restrict__ r,
                        const float* __restrict__ w_scale, const float* __restrict__ x_scale, int y_bf16, int M,
                        int N, int K, int row_tiles, int tok_tiles, int tok_block, int* status) {
  constexpr int kAtoms = NVFP4 ? 4 : 2;  // scale-factor atoms per operand block per stage
  constexpr uint32_t kSfBytes = kAtoms * 512;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(status, 0, PSITE_ALIGN);
    return;
  }
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint64_t* empty = full + kStages;
  uint64_t* sf_ready = empty + kStages;
  uint64_t* acc_full = sf_ready + kStages;
  uint64_t* acc_empty = acc_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nst = K / kFKStage;
  const int total_tiles = row_tiles * tok_tiles;
  const int my_tiles = (total_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                       static_cast<int>(gridDim.x);
  // token tiles in blocks of tok_block; inside a block all row tiles, tokens fastest: the CTAs running
  // at one time share a few weight tiles and a block's activations stay in L2
  const int full_block = tok_block * row_tiles;
  auto tile_of = [&](int it, int& row, int& tok) {
    const int t = static_cast<int>(blockIdx.x) + it * static_cast<int>(gridDim.x);
    const int b = t / full_block, rem = t - b * full_block;
    const int width = (tok_tiles - b * tok_block < tok_block) ? (tok_tiles - b * tok_block) : tok_block;
    row = rem / width;
    tok = b * tok_block + (rem - row * width);
  };

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
      mbar_init(&sf_ready[i], 2);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 8);  // the eight epilogue warps
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_y);
  }
  grid_dep_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol = l2_policy_evict_last();
      grid_dep_wait();  // the activation codes and scale factors come from the kernel before this one
      int gi = 0;
      bool ok = true;
      for (int it = 0; it < my_tiles && ok; ++it) {
        int row_tile, tok_tile;
        tile_of(it, row_tile, tok_tile);
        const int n0 = row_tile * kFBN, t0 = tok_tile * kTok;
        const int nblk = (M - t0 > kFTN) ? 2 : 1;
        const uint8_t* sfw_tile = sfw + static_cast<size_t>(row_tile) * nst * kSfBytes;
        const uint8_t* sfx_tile = sfx + static_cast<size_t>(t0 / kFTN) * nst * kSfBytes;
        const size_t sfx_block = static_cast<size_t>(nst) * kSfBytes;
        for (int i = 0; i < nst; ++i, ++gi) {
          const int s = gi % kStages;
          if (!mbar_wait(&empty[s], ((gi / kStages) & 1) ^ 1, abort_flag, PSITE_TMA)) { ok = false; break; }
          mbar_expect_tx(&full[s], kFTileBytes + kBBytes + (1 + nblk) * kSfBytes);
          tma_load_2d(smem + kOffA + s * kFTileBytes, &tm_w, i * 128, n0, &full[s], pol);
          tma_load_2d(smem + kOffB + s * kBBytes, &tm_x, i * 128, t0, &full[s], pol);
          bulk_load_1d(smem + kOffSFA + s * 2048, sfw_tile + static_cast<size_t>(i) * kSfBytes, kSfBytes, &full[s], pol);
          for (int b = 0; b < nblk; ++b)
            bulk_load_1d(smem + kOffSFB + (s * 2 + b) * 2048, sfx_tile + b * sfx_block + static_cast<size_t>(i) * kSfBytes,
                         kSfBytes, &full[s], pol);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issue
    if (lane == 0) {
      int gi = 0;
      bool ok = true;
      for (int it = 0; it < my_tiles && ok; ++it) {
        int row_tile, tok_tile;
        tile_of(it, row_tile, tok_tile);
        const int nblk = (M - tok_tile * kTok > kFTN) ? 2 : 1;
        // the accumulator of the previous tile has been read by all eight epilogue warps
        if (!mbar_wait(acc_empty, (it & 1) ^ 1, abort_flag, PSITE_ACC)) break;
        for (int i = 0; i < nst; ++i, ++gi) {
          const int s = gi % kStages;
          if (!mbar_wait(&full[s], (gi / kStages) & 1, abort_flag, PSITE_MMA)) { ok = false; break; }
          if (!mbar_wait(&sf_ready[s], (gi / kStages) & 1, abort_flag, PSITE_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sfa_t = tmem_base + kSfColBase + s * kSfColsStage;
          const uint32_t sfb_t = sfa_t + 16;
          const uint64_t da = umma_desc_k_sw128(smem_u32(smem + kOffA + s * kFTileBytes));
          const uint64_t db = umma_desc_k_sw128(smem_u32(smem + kOffB + s * kBBytes));
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // four K = 64 UMMAs: +32 bytes along K each
            const int atom = NVFP4 ? j : (j >> 1);
            const uint32_t sf_id = NVFP4 ? 0u : static_cast<uint32_t>((j & 1) * 2);
            const uint32_t idesc = umma_idesc_fp4(kFBN, nblk * kFTN, NVFP4 ? 0 : 1, sf_id);
            umma_fp4<NVFP4>(tmem_base, da + 2 * j, db + 2 * j, idesc, sfa_t + 4 * atom, sfb_t + 8 * atom,
                            (i > 0 || j > 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);
          if (i == nst - 1) umma_commit(acc_full);
        }
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ scale-factor copiers
    // warp 2: weight scale factors and those of activation rows 0-127; warp 3: activation rows 128-255
    if (lane == 0) {
      const bool second = (warp == 3);
      int gi = 0;
      bool ok = true;
      for (int it = 0; it < my_tiles && ok; ++it) {
        int row_tile, tok_tile;
        tile_of(it, row_tile, tok_tile);
        const bool present = !second || (M - tok_tile * kTok > kFTN);  // the second block may hold no tokens
        for (int i = 0; i < nst; ++i, ++gi) {
          const int s = gi % kStages;
          if (!mbar_wait(&full[s], (gi / kStages) & 1, abort_flag, PSITE_SF)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sf_t = tmem_base + kSfColBase + s * kSfColsStage;
          if (!second) {
            const uint32_t src_a = smem_u32(smem + kOffSFA + s * 2048);
#pragma unroll
            for (int at = 0; at < kAtoms; ++at) tmem_cp_32x128b_warpx4(sf_t + 4 * at, sf_atom_desc(src_a + at * 512));
          }
          if (present) {
            const int blk = second ? 1 : 0;
            const uint32_t src_b = smem_u32(smem + kOffSFB + (s * 2 + blk) * 2048);
#pragma unroll
            for (int at = 0; at < kAtoms; ++at)
              tmem_cp_32x128b_warpx4(sf_t + 16 + 8 * at + 4 * blk, sf_atom_desc(src_b + at * 512));
          }
          umma_commit(&sf_ready[s]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int team = (warp - 4) >> 2;  // 0: warps 4-7, 1: warps 8-11
    const int q = warp & 3;            // TMEM lane quarter
    const bool leader = (warp & 3) == 0 && lane == 0;
    int chunk_no = 0;                  // chunks this team has staged so far (buffer parity)
    for (int it = 0; it < my_tiles; ++it) {
      int row_tile, tok_tile;
      tile_of(it, row_tile, tok_tile);
      const int n0 = row_tile * kFBN, t0 = tok_tile * kTok;
      const int n = n0 + q * 32 + lane;
      int tok_cols = M - t0;
      if (tok_cols > kTok) tok_cols = kTok;
      const int col_end = (tok_cols + 31) & ~31;
      float rn = 0.f;
      if (n < N) {
        rn = (r != nullptr) ? r[n] : 1.f;
        if (w_scale != nullptr) rn *= *w_scale;
      }
      if (!mbar_wait(acc_full, it & 1, abort_flag, PSITE_EPI)) break;
      tc_fence_after();
      // all of this warp's columns (up to four chunks of 32) to registers, then the accumulator
      // goes back to the tensor core
      uint32_t v[4][32];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c0 = team * 32 + k * 64;
        if (c0 < col_end) tmem_ld_x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c0, v[k]);
      }
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c0 = team * 32 + k * 64;
        if (c0 < col_end) {  // uniform over the team
          uint8_t* buf = smem + kOffOut + (2 * team + (chunk_no & 1)) * kOutBuf;
          ++chunk_no;
          // the store that last used this buffer (two chunks ago) has finished reading it
          if (leader) bulk_wait_group_read1();
          if (team == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
          else asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int m = t0 + c0 + j;
            const float tx = (x_scale != nullptr && m < M) ? __ldg(x_scale + m) : 1.f;
            const float val = __uint_as_float(v[k][j]) * (rn * tx);
            if (y_bf16)
              reinterpret_cast<__nv_bfloat16*>(buf)[j * kFBN + q * 32 + lane] = __float2bfloat16_rn(val);
            else
              reinterpret_cast<float*>(buf)[j * kFBN + q * 32 + lane] = val;
          }
          fence_proxy_async_smem();
          if (team == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
          else asm volatile("bar.sync 2, 128;" ::: "memory");
          if (leader) {
            tma_store_2d(&tm_y, buf, n0, t0 + c0);
            bulk_commit_group();
          }
        }
      }
    }
    if (leader) bulk_wait_group_read0();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tid == 0 && *abort_flag != 0) atomicCAS(status, 0, *abort_flag);
}

}  // namespace fp4p

int init_gemm_fp4_persist_kernels() {
  cudaError_t e = cudaFuncSetAttribute(fp4p::gemm_fp4_persist_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       fp4p::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(fp4p::gemm_fp4_persist_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             fp4p::kSmemBytes);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "cudaFuncSetAttribute(gemm_fp4_persist) failed: %s", cudaGetErrorString(e));
  return DQ_OK;
}

// Prefill-size batches whose output the copy engine can address; the caller has validated the operands.
// Processes row tiles [0, row_tiles) of the weight (the caller may give the rest to the one-tile kernel).
int launch_gemm_fp4_persist(const uint8_t* x_codes, const uint8_t* x_sf_atoms, const float* x_scale,
                            const uint8_t* w_codes, const uint8_t* w_sf_atoms, const float* w_scale, const float* r,
                            int M, int N, int K, int nvfp4, void* y, int y_dtype, int row_tiles, cudaStream_t stream,
                            DeviceState* st) {
  CUtensorMap tm_w, tm_x, tm_y;
  int rc = make_tmap_2d_u8(&tm_w, w_codes, static_cast<uint64_t>(K) / 2, N, static_cast<uint64_t>(K) / 2, 128, kFBN,
                           CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != DQ_OK) return rc;
  rc = make_tmap_2d_u8(&tm_x, x_codes, static_cast<uint64_t>(K) / 2, M, static_cast<uint64_t>(K) / 2, 128, fp4p::kTok,
                       CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != DQ_OK) return rc;
  const int esz = (y_dtype == DQ_DTYPE_BF16) ? 2 : 4;
  rc = make_tmap_2d_out(&tm_y, y, esz, static_cast<uint64_t>(N), static_cast<uint64_t>(M), kFBN, 32);
  if (rc != DQ_OK) return rc;
  const int tok_tiles = (M + fp4p::kTok - 1) / fp4p::kTok;  // row_tiles: the first row tiles of the weight
  const int64_t tiles = static_cast<int64_t>(row_tiles) * tok_tiles;
  const int grid = static_cast<int>(tiles < st->sm_count ? tiles : st->sm_count);
  // a block of token tiles whose packed activations (K / 2 bytes per token) take about 40 MB of L2
  int tok_block = static_cast<int>((40ll << 20) / (static_cast<int64_t>(fp4p::kTok) * (K / 2)));
  if (tok_block < 1) tok_block = 1;
  if (tok_block > tok_tiles) tok_block = tok_tiles;
  const int bf = y_dtype == DQ_DTYPE_BF16 ? 1 : 0;
  cudaError_t e;
  if (nvfp4)
    e = launch_pdl(fp4p::gemm_fp4_persist_kernel<1>, dim3(grid), dim3(fp4p::kThreads), fp4p::kSmemBytes, stream, tm_w,
                   tm_x, tm_y, w_sf_atoms, x_sf_atoms, r, w_scale, x_scale, bf, M, N, K, row_tiles, tok_tiles,
                   tok_block, st->status_dev);
  else
    e = launch_pdl(fp4p::gemm_fp4_persist_kernel<0>, dim3(grid), dim3(fp4p::kThreads), fp4p::kSmemBytes, stream, tm_w,
                   tm_x, tm_y, w_sf_atoms, x_sf_atoms, r, w_scale, x_scale, bf, M, N, K, row_tiles, tok_tiles,
                   tok_block, st->status_dev);
  if (e != cudaSuccess) return set_error(DQ_ERR_CUDA, "gemm_fp4_persist launch failed: %s", cudaGetErrorString(e));
  return DQ_OK;
}

}  // namespace dq
