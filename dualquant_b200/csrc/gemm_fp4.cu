// Block-scaled FP4 W4A4 GEMM for sm_100a: tcgen05.mma kind::mxf4nvf4.block_scale.
//
//   Y[m,n] = r[n] * tw * tx[m] * sum_k ( qx[m,k] * sfx[m, k/B] ) * ( qw[n,k] * sfw[n, k/B] )
//
// MXFP4: B = 32, E8M0 scales, scale_vec::2X, tw = tx = 1.  NVFP4: B = 16, E4M3 scales,
// scale_vec::4X, tw = per-tensor weight scale, tx[m] = per-token second-level scale.
// The block scales are applied by the tensor core, so one fp32 accumulator in tensor memory
// runs over the whole K loop and is drained once.
//
// Orientation as in the int4 kernel: 128 weight rows = UMMA M (TMEM lanes), 128 tokens = UMMA N
// (TMEM columns).  A stage is 256 k: operand tiles of 128 rows x 128 bytes (packed E2M1, 128B
// swizzle, TMA) and the scale factors of the stage in the 512-byte "32 x 16" atoms
// tcgen05.cp.32x128b.warpx4 expects (rows r, r+32, r+64, r+96 share a 16-byte line; four scales
// per row per atom), fetched with contiguous bulk copies and copied to tensor memory by the
// UMMA-issuing thread ahead of the four K=64 UMMAs of the stage.
//
// 192 threads: warp 0 TMA producer, warp 1 TMEM allocation + UMMA issue, warps 2-5 epilogue.
#include "dq_common.h"
#include "dq_ptx.cuh"
#include "gemm_fp4.cuh"

#include <cuda_bf16.h>

namespace dq {

constexpr int kFp4DecodeTokens = 32;  // library's choice of the 32-token tile: M up to this
constexpr int kFThreads = 256;  // producer, UMMA issuer, 4 epilogue warps, 2 scale-factor copiers

// NT = token blocks of 128 per CTA; NT = 0 is the decode tile of 32 tokens.
//   NT = 0: 128 weight rows x 32 tokens (UMMA N = 32): a stage is 24 KB instead of 36 KB, of which
//           only the 16 KB weight tile comes from HBM, so four stages fit where three did and more
//           weight bytes are in flight per SM.  Two CTAs per SM, split-K over a cluster.
//   NT = 1: 3 stages of 36 KB and 256 tensor-memory columns, so two CTAs share an SM and one's
//           epilogue overlaps the other's K loop.
//   NT = 2: 128 weight rows x 256 tokens.  The weight tile of a stage is fetched once for two
//           token blocks (24 KB of operands per 128x128x256 block product instead of 32 KB): the
//           shape for long K loops, where the stream of operand tiles out of L2 is what bounds
//           the 128x128 tile.  4 stages of 54 KB, one CTA per SM, two fp32 accumulators.
template <int NT>
struct FCfg {
  static constexpr int kTok = (NT == 0) ? 32 : NT * kFTN;   // tokens per CTA
  static constexpr int kSfBlocks = (NT == 0) ? 1 : NT;      // blocks of 128 token rows whose scale factors a stage holds
  static constexpr int kBTileBytes = kTok * 128;            // activation tile of a stage
  static constexpr int kStages = (NT == 1) ? 3 : 4;
  static constexpr int kOffA = 0;
  static constexpr int kOffB = kOffA + kStages * kFTileBytes;
  static constexpr int kOffSFA = kOffB + kStages * kBTileBytes;       // up to 2 KB per stage
  static constexpr int kOffSFB = kOffSFA + kStages * 2048;            // up to 2 KB per block and stage
  static constexpr int kOffBar = kOffSFB + kStages * kSfBlocks * 2048;
  static constexpr int kSmemBytes = kOffBar + (3 * kStages + 1) * 8 + 16 + 1024;
  static_assert(((kTok < kFTN) ? kTok : kFTN) * kFBN * 4 <= kOffSFA, "split-K exchange tile must fit in the operand stages");
  static_assert(kSmemBytes <= 227 * 1024, "stages exceed the shared memory of an SM");
  static constexpr int kAccCols = (NT == 0) ? 32 : NT * kFTN;  // fp32 accumulator columns
  static constexpr int kSfColsStage = 16 + kSfBlocks * 16;  // scale-factor columns per stage: A, then B per block
  static constexpr int kSfColBase = kAccCols;
  static constexpr int kTmemCols = (NT == 2) ? 512 : 256;
  static_assert(kSfColBase + kStages * kSfColsStage <= kTmemCols, "tensor memory columns");
  static constexpr int kMinCtas = (NT == 2) ? 1 : 2;
};

enum { FSITE_TMA = 31, FSITE_MMA = 32, FSITE_EPI = 33, FSITE_SF = 34 };

template <int NVFP4, int NT>
__global__ void __launch_bounds__(kFThreads, FCfg<NT>::kMinCtas)
gemm_fp4_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                const __grid_constant__ CUtensorMap tm_y, int bulk_store,
                const uint8_t* __restrict__ sfw, const uint8_t* __restrict__ sfx,
                const float* __restrict__ r, const float* __restrict__ w_scale,
                const float* __restrict__ x_scale, void* __restrict__ y, int y_bf16, int M, int N,
                int K, int stages_per_split, int split_k, int tok_fast, int row_tile0, int* status) {
  using C = FCfg<NT>;
  constexpr int kFStages = C::kStages;
  constexpr int kAtoms = NVFP4 ? 4 : 2;           // scale-factor atoms per operand per stage
  constexpr uint32_t kSfBytes = kAtoms * 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint64_t* empty = full + kFStages;
  uint64_t* sf_ready = empty + kFStages;
  uint64_t* acc_full = sf_ready + kFStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // tok_fast: grid x walks the token tiles (CTAs that run together share one weight tile and the
  // whole, smaller, activation matrix stays in L2); otherwise grid x walks the row tiles
  const int n0 = (static_cast<int>(tok_fast ? blockIdx.y : blockIdx.x) + row_tile0) * kFBN;  // row_tile0: first row tile of this launch
  const int t0 = (tok_fast ? blockIdx.x : blockIdx.y) * C::kTok;
  // token blocks of this CTA that hold tokens (the last CTA of a ragged M may own only one)
  const int nblk = (NT == 2 && M - t0 > kFTN) ? 2 : 1;
  const int total_st = K / kFKStage;
  const int st_begin = blockIdx.z * stages_per_split;
  int st_end = st_begin + stages_per_split;
  if (st_end > total_st) st_end = total_st;
  const int nst = (st_end > st_begin) ? (st_end - st_begin) : 0;

  if (tid == 0) {
    for (int i = 0; i < kFStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
      mbar_init(&sf_ready[i], 2);  // one tcgen05.commit from each scale-factor copier
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
    if (bulk_store) tma_prefetch_desc(&tm_y);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    const uint64_t pol = l2_policy_evict_last();
    const uint8_t* sfw_tile = sfw + (static_cast<size_t>(n0 / kFBN) * total_st + st_begin) * kSfBytes;
    const uint8_t* sfx_tile = sfx + (static_cast<size_t>(t0 / kFTN) * total_st + st_begin) * kSfBytes;
    const size_t sfx_block = static_cast<size_t>(total_st) * kSfBytes;  // next token block of 128
    // Only lane 0 works; the other lanes go straight to the end of the role (32 lanes polling a
    // barrier cost issue slots and barrier-unit bandwidth that the other warps need).
    if (lane == 0) {
      for (int i = 0; i < nst; ++i) {
        const int s = i % kFStages;
        if (!mbar_wait(&empty[s], ((i / kFStages) & 1) ^ 1, abort_flag, FSITE_TMA)) break;
        // the activation box is the CTA's whole token tile (rows past M arrive as zeros and count)
        mbar_expect_tx(&full[s], kFTileBytes + C::kBTileBytes + (1 + nblk) * kSfBytes);
        tma_load_2d(smem + C::kOffA + s * kFTileBytes, &tm_w, (st_begin + i) * 128, n0, &full[s], pol);
        tma_load_2d(smem + C::kOffB + s * C::kBTileBytes, &tm_x, (st_begin + i) * 128, t0, &full[s], pol);
        bulk_load_1d(smem + C::kOffSFA + s * 2048, sfw_tile + static_cast<size_t>(i) * kSfBytes,
                     kSfBytes, &full[s], pol);
        for (int b = 0; b < nblk; ++b)
          bulk_load_1d(smem + C::kOffSFB + (s * C::kSfBlocks + b) * 2048,
                       sfx_tile + b * sfx_block + static_cast<size_t>(i) * kSfBytes, kSfBytes, &full[s], pol);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer
    if (lane == 0) {  // only lane 0 works (see the producer)
      for (int i = 0; i < nst; ++i) {
        const int s = i % kFStages;
        // operands landed (full) and their scale factors copied into tensor memory (sf_ready)
        if (!mbar_wait(&full[s], (i / kFStages) & 1, abort_flag, FSITE_MMA)) break;
        if (!mbar_wait(&sf_ready[s], (i / kFStages) & 1, abort_flag, FSITE_MMA)) break;
        tc_fence_after();
        const uint32_t sfa_t = tmem_base + C::kSfColBase + s * C::kSfColsStage;
        const uint64_t da = umma_desc_k_sw128(smem_u32(smem + C::kOffA + s * kFTileBytes));
        // One instruction per K = 64 step covers every token block of the CTA (UMMA N = 128 or
        // 256): the weight slice is read from shared memory once per step.  Scale factors of the
        // token rows: 4 columns per block of 128 rows, blocks side by side (rows 128..255 follow
        // rows 0..127), 4 * NT columns per atom.
        {
          // (the 32-token tile is only launched for M <= 32: its rows are rows 0..31 of the first
          // scale-factor block, the first column of each atom)
          const uint32_t sfb_t = sfa_t + 16;
          const uint64_t db = umma_desc_k_sw128(smem_u32(smem + C::kOffB + s * C::kBTileBytes));
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // four K=64 UMMAs: +32 bytes along K each
            const int atom = NVFP4 ? j : (j >> 1);
            const uint32_t sf_id = NVFP4 ? 0u : static_cast<uint32_t>((j & 1) * 2);
            const uint32_t idesc = umma_idesc_fp4(kFBN, (NT == 0) ? 32 : nblk * kFTN, NVFP4 ? 0 : 1, sf_id);
            umma_fp4<NVFP4>(tmem_base, da + 2 * j, db + 2 * j, idesc, sfa_t + 4 * atom,
                            sfb_t + 4 * C::kSfBlocks * atom, (i > 0 || j > 0) ? 1u : 0u);
          }
        }
        umma_commit(&empty[s]);
        if (i == nst - 1) umma_commit(acc_full);
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ scale-factor copiers
    // Warp 6 moves the weight scale factors of each stage from shared to tensor memory
    // (tcgen05.cp, one per 512-byte atom), warp 7 the activation scale factors.  They used to be
    // issued by the UMMA thread: 4-8 copies + 4 UMMAs + commits per stage, at ~70 cycles of issue
    // latency each, took that one thread several times the 271 cycles the UMMAs need to execute.
    // The stage's columns are free again once its previous UMMAs have finished, which the
    // producer has already waited for before refilling the stage (full implies it).
    if (lane == 0) {
      const bool is_b = (warp == 7);
      const int sf_off = is_b ? C::kOffSFB : C::kOffSFA;
      for (int i = 0; i < nst; ++i) {
        const int s = i % kFStages;
        if (!mbar_wait(&full[s], (i / kFStages) & 1, abort_flag, FSITE_SF)) break;
        tc_fence_after();
        const uint32_t sf_t = tmem_base + C::kSfColBase + s * C::kSfColsStage + (is_b ? 16 : 0);
        const int blocks = is_b ? nblk : 1;
        for (int b = 0; b < blocks; ++b) {
          const uint32_t src = smem_u32(smem + sf_off + (s * (is_b ? C::kSfBlocks : 1) + b) * 2048);
#pragma unroll
          for (int at = 0; at < kAtoms; ++at)
            tmem_cp_32x128b_warpx4(sf_t + (is_b ? 4 * C::kSfBlocks * at + 4 * b : 4 * at),
                                   sf_atom_desc(src + at * 512));
        }
        umma_commit(&sf_ready[s]);
      }
    }
  }
  __syncwarp();  // the role warps' lane 0 rejoins its warp
  // -------------------------------------------------------------------- epilogue
  // Two teams of four warps, one warp per TMEM lane quarter in each: warps 2-5, which have no
  // other role, and - when the output goes through bulk stores - the producer, issuer and copier
  // warps once their loops are over (four warps alone are too few to hide the latency of their own
  // instruction chains).  The teams take alternate 32-token chunks.
  const int team = (warp >= 2 && warp < 6) ? 0 : 1;
  const int nteams = (split_k == 1 && bulk_store) ? 2 : 1;
  if (team < nteams) {
    const int q = warp & 3;  // TMEM lane quarter of this warp
    const int n = n0 + q * 32 + lane;
    // token columns that exist in this tile, rounded up to the 32-column granularity of tcgen05.ld
    int tok_cols = M - t0;
    if (tok_cols > C::kTok) tok_cols = C::kTok;
    const int col_end = (tok_cols + 31) & ~31;
    const bool have_acc = (nst > 0) && mbar_wait_relaxed(acc_full, 0, abort_flag, FSITE_EPI);
    if (have_acc) tc_fence_after();
    float rn = 0.f;
    if (n < N) {
      rn = (r != nullptr) ? r[n] : 1.f;
      if (w_scale != nullptr) rn *= *w_scale;
    }
#pragma unroll 1
    for (int c0 = team * 32; c0 < col_end; c0 += 32 * nteams) {
      uint32_t v[32];
      if (have_acc) {
        tmem_ld_x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c0, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0u;
      }
      if (split_k == 1 && bulk_store) {
        // Through shared memory and out with one tiled bulk store per 32 tokens: the chunk is
        // laid out [token][128 weight rows] (a lane writes its row's column: conflict-free), the
        // copy engine writes 512-byte (fp32) runs per token and skips rows / tokens that do not
        // exist.  The operand stages are idle by now; every chunk has its own 16 KB of them, so no
        // chunk waits for an earlier store to have been read.
        uint8_t* buf = smem + (c0 >> 5) * (32 * kFBN * 4);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int m = t0 + c0 + j;
          const float tx = (x_scale != nullptr && m < M) ? x_scale[m] : 1.f;
          const float val = __uint_as_float(v[j]) * (rn * tx);
          if (y_bf16)
            reinterpret_cast<__nv_bfloat16*>(buf)[j * kFBN + q * 32 + lane] = __float2bfloat16_rn(val);
          else
            reinterpret_cast<float*>(buf)[j * kFBN + q * 32 + lane] = val;
        }
        fence_proxy_async_smem();  // generic-proxy writes before the async-proxy read of the store
        if (team == 0)  // the four warps of the team
          asm volatile("bar.sync 1, 128;" ::: "memory");
        else
          asm volatile("bar.sync 2, 128;" ::: "memory");
        if ((warp == 2 || warp == 0) && lane == 0) {
          tma_store_2d(&tm_y, buf, n0, t0 + c0);
          bulk_commit_group();
        }
      } else if (split_k == 1) {
        if (n < N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int m = t0 + c0 + j;
            if (m < M) {
              const float tx = (x_scale != nullptr) ? x_scale[m] : 1.f;
              const float val = __uint_as_float(v[j]) * (rn * tx);
              if (y_bf16)
                reinterpret_cast<__nv_bfloat16*>(y)[static_cast<size_t>(m) * N + n] = __float2bfloat16_rn(val);
              else
                reinterpret_cast<float*>(y)[static_cast<size_t>(m) * N + n] = val;
            }
          }
        }
      } else {
        // partial sums -> exchange tile red[token][row] over the (now idle) stage buffers
        float* red = reinterpret_cast<float*>(smem);
#pragma unroll
        for (int j = 0; j < 32; ++j) red[(c0 + j) * kFBN + q * 32 + lane] = __uint_as_float(v[j]);
      }
    }
    // shared memory must outlive the copy engine's reads of the staged chunks
    if (split_k == 1 && bulk_store && (warp == 2 || warp == 0) && lane == 0) bulk_wait_group_read0();
  }

  // -------------------------------------------------------------------- split-K reduction
  if (split_k > 1) {
    __syncwarp();
    cluster_sync_all();
    if (warp >= 2 && warp < 6) {
      int tok_cols = M - t0;
      if (tok_cols > C::kTok) tok_cols = C::kTok;
      const uint32_t rank = cluster_ctarank();
      const int e = tid - 64;   // 0..127
      const int c4 = e & 31;    // float4 column (4 weight rows)
      const uint32_t red_base = smem_u32(smem);
      for (int tl = static_cast<int>(rank) + split_k * (e >> 5); tl < tok_cols; tl += split_k * 4) {
        const int m = t0 + tl;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const uint32_t off = static_cast<uint32_t>((tl * kFBN + c4 * 4) * 4);
        for (int p = 0; p < split_k; ++p) {
          const float4 v = dsmem_ld_f4(dsmem_map(red_base + off, static_cast<uint32_t>(p)));
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        const float tx = (x_scale != nullptr) ? x_scale[m] : 1.f;
        const float ws = (w_scale != nullptr) ? *w_scale : 1.f;
        const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int nn = n0 + c4 * 4 + u;
          if (nn < N) {
            const float rr = ((r != nullptr) ? r[nn] : 1.f) * ws;
            const float val = vals[u] * (rr * tx);
            if (y_bf16)
              reinterpret_cast<__nv_bfloat16*>(y)[static_cast<size_t>(m) * N + nn] = __float2bfloat16_rn(val);
            else
              reinterpret_cast<float*>(y)[static_cast<size_t>(m) * N + nn] = val;
          }
        }
      }
    }
    __syncwarp();
    cluster_sync_all();  // peers may still be reading this CTA's exchange tile until here
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
  if (tid == 0 && *abort_flag != 0) atomicCAS(status, 0, *abort_flag);
}

// Scale factors from row-major [rows, nsf] bytes to the atom order the GEMM streams:
// [row tile of 128][k stage][atom][ (r % 32) * 16 + (r / 32) * 4 + (k % 4) ], rows past `rows` zero.
__global__ void fp4_sf_to_atoms_kernel(const uint8_t* __restrict__ sf, int rows, int nsf,
                                       uint8_t* __restrict__ out, int64_t total) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int within = static_cast<int>(i & 511);
  const int64_t atom = i >> 9;             // global atom index = tile * atoms_per_row_tile + a
  const int atoms_per_tile = nsf / 4;
  const int64_t tile = atom / atoms_per_tile;
  const int a = static_cast<int>(atom % atoms_per_tile);
  const int r = (within >> 4) + 32 * ((within >> 2) & 3);
  const int k = a * 4 + (within & 3);
  const int64_t row = tile * 128 + r;
  out[i] = (row < rows) ? sf[row * nsf + k] : static_cast<uint8_t>(0);
}

int init_gemm_fp4_kernels() {
  cudaError_t e = cudaFuncSetAttribute(gemm_fp4_kernel<0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       FCfg<1>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(gemm_fp4_kernel<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             FCfg<1>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(gemm_fp4_kernel<0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             FCfg<0>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(gemm_fp4_kernel<1, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             FCfg<0>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(gemm_fp4_kernel<0, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             FCfg<2>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(gemm_fp4_kernel<1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             FCfg<2>::kSmemBytes);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "cudaFuncSetAttribute(gemm_fp4) failed: %s", cudaGetErrorString(e));
  return DQ_OK;
}

}  // namespace dq

using namespace dq;

extern "C" size_t dq_fp4_sf_atoms_bytes(int rows, int K, int fmt) {
  const int blk = (fmt == DQ_FP4_MXFP4) ? 32 : 16;
  if (rows <= 0 || K <= 0) return 0;
  return (static_cast<size_t>(rows) + 127) / 128 * 128 * static_cast<size_t>(K / blk);
}

extern "C" int dq_fp4_sf_to_atoms(const uint8_t* sf, int rows, int K, int fmt, uint8_t* out,
                                  void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  DQ_REQUIRE(fmt == DQ_FP4_MXFP4 || fmt == DQ_FP4_NVFP4, DQ_ERR_UNSUPPORTED, "unknown FP4 format %d", fmt);
  DQ_REQUIRE(sf != nullptr && out != nullptr, DQ_ERR_NULL, "null pointer");
  DQ_REQUIRE(rows >= 1 && K % kFKStage == 0, DQ_ERR_SHAPE, "K=%d must be a multiple of %d", K, kFKStage);
  const int nsf = K / ((fmt == DQ_FP4_MXFP4) ? 32 : 16);
  const int64_t total = static_cast<int64_t>(dq_fp4_sf_atoms_bytes(rows, K, fmt));
  fp4_sf_to_atoms_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0,
                           static_cast<cudaStream_t>(stream)>>>(sf, rows, nsf, out, total);
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}

extern "C" int dq_gemm_w4a4_fp4(const uint8_t* x_codes, const uint8_t* x_sf_atoms,
                                const float* x_scale, const uint8_t* w_codes,
                                const uint8_t* w_sf_atoms, const float* w_scale, const float* r,
                                int M, int N, int K, int fmt, void* y, int y_dtype, void* stream) {
  return dq_gemm_w4a4_fp4_tiled(x_codes, x_sf_atoms, x_scale, w_codes, w_sf_atoms, w_scale, r, M, N, K,
                                fmt, y, y_dtype, 0, stream);  // 0: the library picks the token tile
}

extern "C" int dq_gemm_w4a4_fp4_tiled(const uint8_t* x_codes, const uint8_t* x_sf_atoms,
                                      const float* x_scale, const uint8_t* w_codes,
                                      const uint8_t* w_sf_atoms, const float* w_scale,
                                      const float* r, int M, int N, int K, int fmt, void* y,
                                      int y_dtype, int token_tile, void* stream) {
  DeviceState* st = current_state();
  if (st == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(fmt == DQ_FP4_MXFP4 || fmt == DQ_FP4_NVFP4, DQ_ERR_UNSUPPORTED, "unknown FP4 format %d", fmt);
  DQ_REQUIRE(x_codes && x_sf_atoms && w_codes && w_sf_atoms && y, DQ_ERR_NULL, "null operand pointer");
  DQ_REQUIRE(M >= 1 && N >= 1 && K >= kFKStage && K % kFKStage == 0, DQ_ERR_SHAPE,
             "bad shape M=%d N=%d K=%d (K must be a multiple of %d)", M, N, K, kFKStage);
  DQ_REQUIRE(aligned(x_codes, 16) && aligned(w_codes, 16) && aligned(x_sf_atoms, 16) &&
                 aligned(w_sf_atoms, 16),
             DQ_ERR_ALIGN, "operands must be 16-byte aligned");
  DQ_REQUIRE(y_dtype == DQ_DTYPE_F32 || y_dtype == DQ_DTYPE_BF16, DQ_ERR_UNSUPPORTED, "unknown y_dtype %d", y_dtype);
  DQ_REQUIRE(token_tile == 0 || token_tile == 32 || token_tile == 128 || token_tile == 256, DQ_ERR_SHAPE,
             "token_tile must be 0 (library's choice), 32, 128 or 256, got %d", token_tile);
  const int total_st = K / kFKStage;
  // Prefill-size batches (library's choice of tile, output addressable by the copy engine): the
  // persistent kernel on as many row tiles as fill whole rounds of one 256-token tile per SM, the
  // one-tile kernel (with split-K) on the row tiles that are left.  A last round with few tiles
  // would cost a full tile time: down of the Qwen2.5-7B shapes at M = 4096 is 448 tiles on 148 SMs
  // - 27 of its 28 row tiles go to the persistent kernel, the last to 256 split-K CTAs (measured
  // 163 -> 147 us; the same split on o, K = 3584, does not pay for its second launch).
  int row_tile0 = 0;  // first row tile of the one-tile launch below
  {
    const int esz0 = (y_dtype == DQ_DTYPE_BF16) ? 2 : 4;
    const int rt_all = (N + kFBN - 1) / kFBN, tok256 = (M + 255) / 256;
    if (token_tile == 0 && M >= 512 && (static_cast<size_t>(N) * esz0) % 16 == 0 && aligned(y, 16)) {
      const int64_t tiles256 = static_cast<int64_t>(rt_all) * tok256;
      const int64_t rounds = (tiles256 + st->sm_count - 1) / st->sm_count;
      int rt_p = 0;
      if (tiles256 * 100 >= rounds * st->sm_count * 85) rt_p = rt_all;                      // fills its rounds
      else if (tiles256 >= st->sm_count && K >= 8192)  // long K loops only: a second launch costs ~10 us
        rt_p = static_cast<int>((tiles256 / st->sm_count) * st->sm_count / tok256);
      if (rt_p > 0) {
        int rc0 = launch_gemm_fp4_persist(x_codes, x_sf_atoms, x_scale, w_codes, w_sf_atoms, w_scale, r, M, N, K,
                                          fmt == DQ_FP4_NVFP4 ? 1 : 0, y, y_dtype, rt_p,
                                          static_cast<cudaStream_t>(stream), st);
        if (rc0 != DQ_OK || rt_p == rt_all) return rc0;
        row_tile0 = rt_p;
      }
    }
  }
  // The library's own choice otherwise: 32-token tiles for decode batches, else 128.  The 256-token tile is
  // not chosen: measured on the Qwen2.5-7B-architecture linears at M = 4096 it is 3 % faster on the
  // longest K loop and 2-15 % slower elsewhere (one CTA and one UMMA-issuing thread per SM).
  const int tile_tok = token_tile ? token_tile : (M <= kFp4DecodeTokens ? 32 : kFTN);
  const int nt = tile_tok == 32 ? 0 : tile_tok / kFTN;
  // split K across a cluster when the output tiles alone leave most SMs idle (decode batches)
  int split = 1;
  {
    const int split_tok = (tile_tok == 32) ? 32 : kFTN;  // the 256-token tile never splits: judged as 128
    const int tiles1 = ((N + kFBN - 1) / kFBN - row_tile0) * ((M + split_tok - 1) / split_tok);
    while (split < 8 && tiles1 * split * 6 < st->sm_count * 2 * 5 && total_st / (2 * split) >= 2) split *= 2;
  }
  DQ_REQUIRE(nt != 0 || M <= 32, DQ_ERR_UNSUPPORTED, "the 32-token tile covers batches of up to 32 tokens, got M=%d", M);
  DQ_REQUIRE(nt != 2 || split == 1, DQ_ERR_UNSUPPORTED,
             "256-token tiles have no split-K path (M=%d N=%d K=%d would split %d ways)", M, N, K, split);
  CUtensorMap tm_w, tm_x;
  int rc = make_tmap_2d_u8(&tm_w, w_codes, static_cast<uint64_t>(K) / 2, N, static_cast<uint64_t>(K) / 2,
                           128, kFBN, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != DQ_OK) return rc;
  rc = make_tmap_2d_u8(&tm_x, x_codes, static_cast<uint64_t>(K) / 2, M, static_cast<uint64_t>(K) / 2, 128,
                       tile_tok, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != DQ_OK) return rc;
  // Output through tiled bulk stores when the copy engine can address it (16-byte pitch and
  // base); the split-K path reduces through distributed shared memory and stores directly.
  const int esz = (y_dtype == DQ_DTYPE_BF16) ? 2 : 4;
  const int bulk_store = (split == 1 && (static_cast<size_t>(N) * esz) % 16 == 0 && aligned(y, 16)) ? 1 : 0;
  CUtensorMap tm_y = tm_w;  // a valid map is passed either way; unused without bulk_store
  if (bulk_store) {
    rc = make_tmap_2d_out(&tm_y, y, esz, static_cast<uint64_t>(N), static_cast<uint64_t>(M), kFBN, 32);
    if (rc != DQ_OK) return rc;
  }
  const int sps = (total_st + split - 1) / split;
  cudaLaunchConfig_t cfg = {};
  const int row_tiles = (N + kFBN - 1) / kFBN - row_tile0, tok_tiles = (M + tile_tok - 1) / tile_tok;
  // the smaller operand is the one every CTA wave re-reads; it stays in L2 when grid x walks its tiles
  const int tok_fast = (tok_tiles > 1 && M < N && row_tiles <= 65535) ? 1 : 0;
  cfg.gridDim = tok_fast ? dim3(tok_tiles, row_tiles, split) : dim3(row_tiles, tok_tiles, split);
  cfg.blockDim = dim3(kFThreads, 1, 1);
  cfg.dynamicSmemBytes = (nt == 2) ? FCfg<2>::kSmemBytes : (nt == 1) ? FCfg<1>::kSmemBytes : FCfg<0>::kSmemBytes;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = split;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int bf = y_dtype == DQ_DTYPE_BF16 ? 1 : 0;
  cudaError_t e;
  auto kern = (fmt == DQ_FP4_NVFP4)
                  ? (nt == 2 ? gemm_fp4_kernel<1, 2> : nt == 1 ? gemm_fp4_kernel<1, 1> : gemm_fp4_kernel<1, 0>)
                  : (nt == 2 ? gemm_fp4_kernel<0, 2> : nt == 1 ? gemm_fp4_kernel<0, 1> : gemm_fp4_kernel<0, 0>);
  e = cudaLaunchKernelEx(&cfg, kern, tm_w, tm_x, tm_y, bulk_store, w_sf_atoms, x_sf_atoms, r, w_scale, x_scale, y, bf, M, N,
                         K, sps, split, tok_fast, row_tile0, st->status_dev);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "gemm_fp4 launch failed (split=%d): %s", split, cudaGetErrorString(e));
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}
