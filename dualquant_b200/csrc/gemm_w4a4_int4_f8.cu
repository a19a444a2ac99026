// W4A4 int4 dual-scale GEMM for large token counts (prefill) on the FP8 tensor-core path.
//
//   Y[m,n] = r[n] * sx[m] * sum_g sw[n,g] * ( sum_{k in group g} qx[m,k] * qw[n,k] )
//
// Same result, bit for bit, as the kind::i8 kernel (gemm_w4a4_int4.cu); what changes is how the
// per-group integer sums are formed.  Every int4 code (-8 .. 7) is an exact E4M3 number, products
// and 128-term sums of such codes are integers below 2^24, so tcgen05.mma kind::f8f6f4 with an
// fp32 accumulator delivers each group sum exactly - as a float.  That removes the two things that
// bound the integer kernel on the CUDA cores: the int32 -> fp32 conversion of every accumulator
// element (a quarter-rate instruction) and the nibble unpacking (the operands arrive as bytes,
// straight from TMA).  The epilogue is one packed FMA per two accumulator elements.
//
// Operands: weights and activation codes as E4M3 bytes, row-major [N, K] and [M, K]
// (dq_expand_w_int4_e4m3 makes the former from the packed int4 artefact, dq_codes_to_e4m3 the
// latter from the quantiser's int8 codes).  The 4-bit artefact stays the storage format; the byte
// form is a derived copy for token counts where the GEMM is compute-bound.
//
// Tile: 128 weight rows (UMMA M, TMEM lanes) x 256 tokens (UMMA N, TMEM columns), persistent CTAs,
// one per SM.  Per weight group (128 k = one 128-byte swizzle atom row): two tiled TMA copies
// (16 KB weights, 32 KB activations), four UMMAs of K = 32 into accumulator g & 1 (two accumulators
// of 256 columns fill the tensor memory), drained by eight epilogue warps (warp w: lanes
// 32 (w & 3) .., columns 128 (w >> 2) ..) while the next group's UMMAs run.  Three pipeline stages.
//   warps 0-7   epilogue: tcgen05.ld in batches of 2 x 32 columns, run += acc * sw[n,g]; at the end
//               of the tile Y = run * r[n] * sx[m]: bf16 tiles go to shared memory as [token][row]
//               and leave through one tiled bulk store, fp32 or residual-fused tiles are stored
//               directly
//   warp 8      TMA producer (one lane)
//   warp 9      UMMA issue (one lane), owns the TMEM allocation
//   warps 10-11 idle: registers are re-balanced per warpgroup (epilogue 232, the rest 40)
// Every barrier wait is bounded (the register re-balancing cannot block: its budgets are checked at
// compile time).
#include "dq_common.h"
#include "dq_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <string.h>

namespace dq {
namespace f8 {

constexpr int kBN = 128;    // weight rows per tile
constexpr int kTN = 256;    // tokens per tile
constexpr int kStages = 3;
constexpr int kABytes = kBN * kGroup;   // 16 KB
constexpr int kBBytes = kTN * kGroup;   // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
// EW epilogue warps (8 or 16), then the producer warp, the issuing warp and two idle warps that
// complete the last warpgroup (register re-balancing works on whole warpgroups).
template <int EW, int CH, int NB, bool REBAL>
struct Shape {
  static constexpr int kEpiWarps = EW;
  static constexpr int kProducerWarp = EW;
  static constexpr int kIssuerWarp = EW + 1;
  // with register re-balancing the CTA is padded to whole warpgroups (two idle warps)
  static constexpr int kThreads = (EW + (REBAL ? 4 : 2)) * 32;
  static constexpr int kCPW = kTN / (EW / 4);  // accumulator columns per epilogue warp
  static constexpr int kCH = CH;                // columns per tcgen05.ld
  static constexpr int kNB = NB;                // loads issued before one wait
  static_assert(kCPW % (CH * NB) == 0, "whole batches");
  // setmaxnreg.inc waits (without bound) until the CTA's pool holds the registers it asks for, and
  // the pool is what the launch granted (threads x registers per thread) minus what the other warps
  // keep: the two budgets below must fit into it or the kernel never starts.
  static constexpr int kLaunchRegs = (65536 / kThreads) / 8 * 8;
  static constexpr int kEpiRegs = (EW == 8) ? 232 : 104;
  static constexpr int kAuxRegs = 40;
  static_assert(!REBAL || EW * 32 * kEpiRegs + 128 * kAuxRegs <= kThreads * kLaunchRegs, "register pool of the CTA");
};

constexpr int kOffOut = kStages * kStageBytes;   // bf16 output tile [256 tokens][128 rows], source of the bulk store
constexpr int kOutBytes = kTN * kBN * 2;
constexpr int kOffSx = kOffOut + kOutBytes;      // token scales of the tile, double-buffered
constexpr int kOffBar = kOffSx + 2 * kTN * 4;
constexpr int kNumBars = 2 * kStages + 9;
constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16;
constexpr uint32_t kTmemCols = 512;
static_assert(kSmemBytes + 1024 <= 227 * 1024, "shared memory");

enum { FSITE_TMA = 61, FSITE_MMA_FULL = 62, FSITE_MMA_ACC = 63, FSITE_EPI = 64, FSITE_ALIGN = 65, FSITE_OUT = 66 };

// Instruction descriptor, kind::f8f6f4: E4M3 A and B (format code 0, both K-major), fp32 accumulator.
//   [4,6) D format (1 = F32)  [7,10) A format  [10,13) B format  [17,23) N >> 3  [24,29) M >> 4
__host__ __device__ constexpr uint32_t idesc_e4m3(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Four two's-complement nibbles (bits 0-15 of sel) -> four E4M3 bytes of the same integers.
// Non-negative codes 0..7: 00 38 40 44 48 4A 4C 4E; negative codes -8..-1: D0 CE CC CA C8 C4 C0 B8.
__device__ __forceinline__ uint32_t e4m3x4_of_nibbles(uint32_t sel) {
  const uint32_t s3 = sel & 0x7777u;
  const uint32_t pos = __byte_perm(0x44403800u, 0x4E4C4A48u, s3);
  const uint32_t neg = __byte_perm(0xCACCCED0u, 0xB8C0C4C8u, s3);
  const uint32_t m = sel & 0x8888u;
  const uint32_t msb = ((m & 0x8u) << 4) | ((m & 0x80u) << 8) | ((m & 0x800u) << 12) | ((m & 0x8000u) << 16);
  const uint32_t mask = (msb >> 7) * 0xFFu;  // 0xFF in the bytes of negative codes
  return (pos & ~mask) | (neg & mask);
}
// the low nibbles of the four bytes of v, packed into bits 0-15
__device__ __forceinline__ uint32_t low_nibbles(uint32_t v) {
  return (v & 0xFu) | ((v >> 4) & 0xF0u) | ((v >> 8) & 0xF00u) | ((v >> 12) & 0xF000u);
}

// packed int4 tiles -> E4M3 bytes, row-major [N, K]; one thread per 16-byte chunk (32 codes)
__global__ void __launch_bounds__(256) expand_w_e4m3_kernel(const uint8_t* __restrict__ w_packed, int N, int K,
                                                            uint8_t* __restrict__ w8) {
  grid_dep_launch_dependents();
  grid_dep_wait();
  const int64_t chunk = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int groups = K / kGroup;
  const int64_t tiles = (N + 127) / 128;
  if (chunk >= tiles * groups * 512) return;
  const int r = static_cast<int>((chunk >> 2) & 127);
  const int ch = static_cast<int>(chunk & 3) ^ ((r >> 1) & 3);
  const int64_t tg = chunk >> 9;
  const int g = static_cast<int>(tg % groups);
  const int64_t row = (tg / groups) * 128 + r;
  if (row >= N) return;
  const uint4 raw = *reinterpret_cast<const uint4*>(w_packed + tg * kTileBytes + (chunk & 511) * 16);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t lo[4], hi[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    lo[j] = e4m3x4_of_nibbles(low_nibbles(w[j]));       // k = 4j .. 4j+3 of the chunk
    hi[j] = e4m3x4_of_nibbles(low_nibbles(w[j] >> 4));  // k = 16 + 4j ..
  }
  uint8_t* dst = w8 + row * K + (g * 4 + ch) * 32;
  *reinterpret_cast<uint4*>(dst) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  *reinterpret_cast<uint4*>(dst + 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
}

// int8 codes (-8..7) [M, K] with row stride ld -> E4M3 bytes [M, K]; one thread per 16 codes
__global__ void __launch_bounds__(256) codes_to_e4m3_kernel(const int8_t* __restrict__ codes, int64_t ld, int M,
                                                            int K, uint8_t* __restrict__ x8) {
  grid_dep_launch_dependents();
  grid_dep_wait();
  const int vec = K / 16;
  const int64_t total = static_cast<int64_t>(M) * vec;
  for (int64_t u = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; u < total;
       u += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t m = u / vec;
    const int kv = static_cast<int>(u - m * vec);
    const uint4 raw = *reinterpret_cast<const uint4*>(codes + m * ld + kv * 16);
    uint4 o;
    o.x = e4m3x4_of_nibbles(low_nibbles(raw.x));
    o.y = e4m3x4_of_nibbles(low_nibbles(raw.y));
    o.z = e4m3x4_of_nibbles(low_nibbles(raw.z));
    o.w = e4m3x4_of_nibbles(low_nibbles(raw.w));
    *reinterpret_cast<uint4*>(x8 + m * K + kv * 16) = o;
  }
}

template <int CH>
__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, uint32_t* v) {
  if constexpr (CH == 8) tmem_ld_x8(taddr, v);
  else if constexpr (CH == 16) tmem_ld_x16(taddr, v);
  else tmem_ld_x32(taddr, v);
}

// Destinations of the scatter output mode (OUT = 4): the partial-output buffer of every rank,
// [world][tq][N] bf16, where slot `rank` of the owner of a tile's tokens receives the tile.
struct ScatterDst {
  unsigned short* part[8];
  int rank, tq, rot;  // rot: token tiles are visited starting at tile `rot`, so that the ranks start on different owners
};

// OUT: how the output tile leaves - 0 direct stores (any shape, fp32 or bf16, optional residual),
// 1 bf16 through shared memory and one tiled bulk store, 3 the same with the residual added, 2 fp32
// through shared memory in two halves, 4 bf16 through shared memory and then 16-byte stores into the partial
// buffer of the rank that owns the tile's tokens (peer memory; tensor-parallel prompt pass).  A template
// parameter: with all three epilogues in one kernel the K loop's code ran 20-25 % slower.
template <int EW, int CH, int NB, bool REBAL, int OUT>
__global__ void __launch_bounds__(Shape<EW, CH, NB, REBAL>::kThreads, 1)
gemm_w4a4_e4m3_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                      const __grid_constant__ CUtensorMap tm_y, const __grid_constant__ CUtensorMap tm_res,
                      const __half* __restrict__ sw_t, const float* __restrict__ r,
                      const float* __restrict__ sx, void* __restrict__ y, int y_bf16,
                      const void* __restrict__ residual, int M, int N, int K, int row_tiles, int tok_tiles,
                      int tok_block, int* status, const __grid_constant__ ScatterDst sc) {
  using S = Shape<EW, CH, NB, REBAL>;
  constexpr int bulk_out = (OUT == 3) ? 1 : OUT;  // non-zero: the tile is staged in shared memory
  constexpr int kEpiWarps = S::kEpiWarps, kProducerWarp = S::kProducerWarp, kIssuerWarp = S::kIssuerWarp;
  constexpr int kCPW = S::kCPW, kCH = S::kCH, kNB = S::kNB;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(status, 0, FSITE_ALIGN);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint64_t* full = bars;
  uint64_t* empty = full + kStages;
  uint64_t* acc_full = empty + kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* out_free = acc_empty + 2;   // the output tile may be overwritten and the token scales are in place
  uint64_t* out_ready = out_free + 1;   // the output tile is written
  uint64_t* res_full = out_ready + 1;   // the residual tile has landed in the output buffer (bf16 output);
                                        // fp32 output: the first half's store has left the buffer
  uint64_t* half_ready = res_full + 1;  // [2]: fp32 output, tokens 0-127 / 128-255 of the tile are written
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(half_ready + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int ng = K / kGroup;
  const int total_tiles = row_tiles * tok_tiles;
  const int my_tiles = (total_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                       static_cast<int>(gridDim.x);
  // Tile order: token tiles in blocks of tok_block; inside a block all row tiles, tokens fastest.  The
  // CTAs running at one time then share a few weight tiles, and a block's activations (sized by the
  // host to fit in L2 next to them) are read from HBM once.
  const int full_block = tok_block * row_tiles;
  auto tile_of = [&](int it, int& row, int& tok) {
    const int t = static_cast<int>(blockIdx.x) + it * static_cast<int>(gridDim.x);
    const int b = t / full_block, rem = t - b * full_block;
    const int width = (tok_tiles - b * tok_block < tok_block) ? (tok_tiles - b * tok_block) : tok_block;
    row = rem / width;
    tok = b * tok_block + (rem - row * width);
    if constexpr (OUT == 4) {
      tok += sc.rot;
      if (tok >= tok_tiles) tok -= tok_tiles;
    }
  };
  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], kEpiWarps); }
    mbar_init(out_free, kEpiWarps);
    mbar_init(out_ready, kEpiWarps);
    mbar_init(res_full, 1);
    mbar_init(&half_ready[0], kEpiWarps / 2);
    mbar_init(&half_ready[1], kEpiWarps / 2);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kIssuerWarp) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
    if (bulk_out && OUT != 4) tma_prefetch_desc(&tm_y);
    if (OUT == 3) tma_prefetch_desc(&tm_res);
  }
  grid_dep_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < kEpiWarps) {
    // ------------------------------------------------------------------ epilogue
    if constexpr (REBAL) setmaxnreg_inc<S::kEpiRegs>();
    const int q = warp & 3, h = warp >> 2;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(h * kCPW);
    float run[kCPW];
    uint32_t v[kNB * kCH];
    constexpr int kScaleAhead = 4;
    unsigned short sq[kScaleAhead];
    const unsigned short* sw_row = nullptr;
    auto consume = [&](const uint32_t* v, int c0, float s) {
#pragma unroll
      for (int j = 0; j < kCH; j += 2) {
        const float2 f = make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
        const float2 acc2 = __ffma2_rn(f, make_float2(s, s), make_float2(run[c0 + j], run[c0 + j + 1]));
        run[c0 + j] = acc2.x;
        run[c0 + j + 1] = acc2.y;
      }
    };
    auto group_step = [&](int i, int gi, unsigned short& sreg) -> bool {
      const int b = gi & 1;
      const float s = __half2float(__ushort_as_half(sreg));
      if (i + kScaleAhead < ng) sreg = __ldg(sw_row + static_cast<size_t>(i + kScaleAhead) * kBN);
      if (!mbar_wait(&acc_full[b], (gi >> 1) & 1, abort_flag, FSITE_EPI)) return false;
      tc_fence_after();
      const uint32_t t0a = t_lane + static_cast<uint32_t>(b * kTN);
      // batches of kNB loads under one wait: every wait costs a full tensor-memory round trip, so
      // the fewer per group the sooner the accumulator goes back to the tensor core
#pragma unroll
      for (int c0 = 0; c0 < kCPW; c0 += kNB * kCH) {
#pragma unroll
        for (int u = 0; u < kNB; ++u) tmem_ld_chunk<CH>(t0a + static_cast<uint32_t>(c0 + u * kCH), v + u * kCH);
        tmem_ld_wait();
        if (c0 + kNB * kCH >= kCPW) {  // accumulator b is free once its last column has been read
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[b]);
        }
#pragma unroll
        for (int u = 0; u < kNB; ++u) consume(v + u * kCH, c0 + u * kCH, s);
      }
      return true;
    };
    bool ok = true;
    unsigned short* out_sm = reinterpret_cast<unsigned short*>(smem + kOffOut);
    float* sx_sm = reinterpret_cast<float*>(smem + kOffSx);
    constexpr bool bulk_res = (OUT == 3);
    grid_dep_wait();  // the token scales come from the kernel before this one
    for (int it = 0; it < my_tiles && ok; ++it) {
      int row_tile, tok_tile;
      tile_of(it, row_tile, tok_tile);
      const int n = row_tile * kBN + q * 32 + lane;
      const int t0 = tok_tile * kTN;
      if (bulk_out && tid < kTN) sx_sm[(it & 1) * kTN + tid] = (t0 + tid < M) ? __ldg(sx + t0 + tid) : 0.f;
#pragma unroll
      for (int j = 0; j < kCPW; ++j) run[j] = 0.f;
      sw_row = reinterpret_cast<const unsigned short*>(sw_t) + static_cast<size_t>(row_tile) * ng * kBN + q * 32 + lane;
#pragma unroll
      for (int d = 0; d < kScaleAhead; ++d) sq[d] = (d < ng) ? __ldg(sw_row + static_cast<size_t>(d) * kBN) : 0;
      const int res_at = (ng / 2) / kScaleAhead * kScaleAhead;  // a group well after the previous tile's store
      for (int i0 = 0; i0 < ng && ok; i0 += kScaleAhead) {
        if (bulk_res && i0 == res_at && tid == 0) {
          // residual tile -> the output buffer (the previous tile's store has left it long ago)
          bulk_wait_group_read0();
          mbar_expect_tx(res_full, kOutBytes);
          tma_load_2d(out_sm, &tm_res, row_tile * kBN, t0, res_full, l2_policy_evict_first());
        }
#pragma unroll
        for (int u = 0; u < kScaleAhead; ++u) {
          if (ok && i0 + u < ng) ok = group_step(i0 + u, it * ng + i0 + u, sq[u]);
        }
      }
      if (!ok) break;
      if constexpr (OUT == 4) {
        // Y tile -> shared memory as [token][row] bf16, then every warp sends 32 tokens: 256 bytes per
        // token (16 lanes x 16 bytes) into slot sc.rank of the owner's partial buffer.  The host
        // guarantees whole tiles (N % 128 == 0, M % 256 == 0) and tiles that do not straddle owners.
        __syncwarp();
        if (lane == 0) mbar_arrive(out_free);  // this warp has read its share of the previous tile
        if (!mbar_wait(out_free, it & 1, abort_flag, FSITE_OUT)) break;
        const float rn = (r != nullptr) ? r[n] : 1.f;
        const float4* sx4 = reinterpret_cast<const float4*>(sx_sm + (it & 1) * kTN + h * kCPW);
        unsigned short* dst = out_sm + (h * kCPW) * kBN + q * 32 + lane;
#pragma unroll
        for (int j = 0; j < kCPW; j += 4) {
          const float4 sv = sx4[j >> 2];
          dst[(j + 0) * kBN] = __bfloat16_as_ushort(__float2bfloat16_rn(run[j + 0] * (rn * sv.x)));
          dst[(j + 1) * kBN] = __bfloat16_as_ushort(__float2bfloat16_rn(run[j + 1] * (rn * sv.y)));
          dst[(j + 2) * kBN] = __bfloat16_as_ushort(__float2bfloat16_rn(run[j + 2] * (rn * sv.z)));
          dst[(j + 3) * kBN] = __bfloat16_as_ushort(__float2bfloat16_rn(run[j + 3] * (rn * sv.w)));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(out_ready);
        if (!mbar_wait(out_ready, it & 1, abort_flag, FSITE_OUT)) break;
        const int owner = t0 / sc.tq;
        unsigned short* base = sc.part[owner] +
                               (static_cast<size_t>(sc.rank) * sc.tq + (t0 - owner * sc.tq)) * static_cast<size_t>(N) +
                               row_tile * kBN;
        constexpr int kTokPerWarp = kTN / kEpiWarps;
#pragma unroll 4
        for (int u = 0; u < kTokPerWarp / 2; ++u) {
          const int tok = warp * kTokPerWarp + 2 * u + (lane >> 4);
          const uint4 v16 = *reinterpret_cast<const uint4*>(out_sm + tok * kBN + (lane & 15) * 8);
          *reinterpret_cast<uint4*>(base + static_cast<size_t>(tok) * N + (lane & 15) * 8) = v16;
        }
      } else if constexpr (OUT == 1 || OUT == 3) {
        // Y tile -> shared memory as [token][row] bf16 (a warp's 32 rows of one token are 64
        // contiguous bytes), then one tiled bulk store; rows past N and tokens past M are clipped
        // by the copy.  With a residual, its tile was copied into the same buffer during the K loop.  Two-byte global stores from here would cost more than two groups' UMMAs.
        if (tid == 0) bulk_wait_group_read0();  // the previous tile's store has left the buffer
        __syncwarp();
        if (lane == 0) mbar_arrive(out_free);
        if (!mbar_wait(out_free, it & 1, abort_flag, FSITE_OUT)) break;
        if (bulk_res && !mbar_wait(res_full, it & 1, abort_flag, FSITE_OUT)) break;
        const float rn = (r != nullptr && n < N) ? r[n] : 1.f;
        const float4* sx4 = reinterpret_cast<const float4*>(sx_sm + (it & 1) * kTN + h * kCPW);
        unsigned short* dst = out_sm + (h * kCPW) * kBN + q * 32 + lane;
        // bf16(linear) [+ residual, rounded again]: what a bf16 "x = x + linear(h)" computes
        auto put = [&](int j, float val) {
          unsigned short bits = __bfloat16_as_ushort(__float2bfloat16_rn(val));
          if (bulk_res) {
            const float lin = __uint_as_float(static_cast<uint32_t>(bits) << 16);
            const float res = __uint_as_float(static_cast<uint32_t>(dst[j * kBN]) << 16);
            bits = __bfloat16_as_ushort(__float2bfloat16_rn(__fadd_rn(lin, res)));
          }
          dst[j * kBN] = bits;
        };
#pragma unroll
        for (int j = 0; j < kCPW; j += 4) {
          const float4 sv = sx4[j >> 2];
          put(j + 0, run[j + 0] * (rn * sv.x));
          put(j + 1, run[j + 1] * (rn * sv.y));
          put(j + 2, run[j + 2] * (rn * sv.z));
          put(j + 3, run[j + 3] * (rn * sv.w));
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(out_ready);
        bool stored = true;
        if (tid == 0) {
          stored = mbar_wait(out_ready, it & 1, abort_flag, FSITE_OUT);
          if (stored) {
            tma_store_2d(&tm_y, out_sm, row_tile * kBN, t0);
            bulk_commit_group();
          }
        }
        ok = __all_sync(0xffffffffu, stored ? 1 : 0) != 0;  // the warp leaves the loop together
      } else if constexpr (OUT == 2) {
        // fp32 output: the buffer holds half a tile, [128 tokens][128 rows] of fp32.  The four warps
        // with tokens 0-127 stage and store first; the other four follow once that store has been
        // read.  Each half is stored by a thread of its own team, which also waits for its copy
        // before the buffer is reused.
        static_assert(kCPW == 128 && kEpiWarps == 8, "one half of the tile per warp");
        if (lane == 0 && (warp == 0 || warp == 4)) bulk_wait_group_read0();
        __syncwarp();
        if (lane == 0) mbar_arrive(out_free);
        if (!mbar_wait(out_free, it & 1, abort_flag, FSITE_OUT)) break;
        if (h == 1 && !mbar_wait(res_full, it & 1, abort_flag, FSITE_OUT)) break;
        const float rn = (r != nullptr && n < N) ? r[n] : 1.f;
        const float4* sx4 = reinterpret_cast<const float4*>(sx_sm + (it & 1) * kTN + h * kCPW);
        float* dst = reinterpret_cast<float*>(out_sm) + q * 32 + lane;
#pragma unroll
        for (int j = 0; j < kCPW; j += 4) {
          const float4 sv = sx4[j >> 2];
          dst[(j + 0) * kBN] = run[j + 0] * (rn * sv.x);
          dst[(j + 1) * kBN] = run[j + 1] * (rn * sv.y);
          dst[(j + 2) * kBN] = run[j + 2] * (rn * sv.z);
          dst[(j + 3) * kBN] = run[j + 3] * (rn * sv.w);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&half_ready[h]);
        bool stored = true;
        if (lane == 0 && (warp == 0 || warp == 4)) {
          stored = mbar_wait(&half_ready[h], it & 1, abort_flag, FSITE_OUT);
          if (stored) {
            tma_store_2d(&tm_y, out_sm, row_tile * kBN, t0 + h * kCPW);
            bulk_commit_group();
            if (h == 0) {
              bulk_wait_group_read0();
              mbar_arrive(res_full);  // the second half may overwrite the buffer
            }
          }
        }
        ok = __all_sync(0xffffffffu, stored ? 1 : 0) != 0;
      } else if (n < N) {  // OUT == 0
        const float rn = (r != nullptr) ? r[n] : 1.f;
        const int m0 = t0 + h * kCPW;
        const int cnt = (M - m0 < kCPW) ? (M - m0) : kCPW;
        const float* sxp = sx + m0;
        if (residual != nullptr) {
          size_t idx = static_cast<size_t>(m0) * N + n;
#pragma unroll
          for (int j = 0; j < kCPW; ++j) {
            if (j < cnt) store_y(y, residual, y_bf16, idx, run[j] * (rn * __ldg(sxp + j)));
            idx += N;
          }
        } else if (y_bf16) {
          __nv_bfloat16* yp = reinterpret_cast<__nv_bfloat16*>(y) + static_cast<size_t>(m0) * N + n;
#pragma unroll
          for (int j = 0; j < kCPW; ++j) {
            if (j < cnt) *yp = __float2bfloat16_rn(run[j] * (rn * __ldg(sxp + j)));
            yp += N;
          }
        } else {
          float* yp = reinterpret_cast<float*>(y) + static_cast<size_t>(m0) * N + n;
#pragma unroll
          for (int j = 0; j < kCPW; ++j) {
            if (j < cnt) *yp = run[j] * (rn * __ldg(sxp + j));
            yp += N;
          }
        }
      }
    }
    if constexpr (OUT == 4) __threadfence_system();  // this thread's stores to peers are performed before the kernel ends
    if (bulk_out && OUT != 4 && lane == 0 && (warp == 0 || warp == 4)) bulk_wait_group_read0();
  } else {
    if constexpr (REBAL) setmaxnreg_dec<S::kAuxRegs>();
    if (warp == kProducerWarp) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0) {
        const uint64_t pol = l2_policy_evict_last();
        grid_dep_wait();  // operands may come from the kernels just before this one
        bool ok = true;
        int gi = 0;
        for (int it = 0; it < my_tiles && ok; ++it) {
          int row_tile, tok_tile;
          tile_of(it, row_tile, tok_tile);
          const int n0 = row_tile * kBN, t0 = tok_tile * kTN;
          for (int i = 0; i < ng; ++i, ++gi) {
            const int s = gi % kStages;
            if (!mbar_wait(&empty[s], ((gi / kStages) & 1) ^ 1, abort_flag, FSITE_TMA)) { ok = false; break; }
            mbar_expect_tx(&full[s], kStageBytes);
            uint8_t* st = smem + s * kStageBytes;
            tma_load_2d(st, &tm_w, i * kGroup, n0, &full[s], pol);
            tma_load_2d(st + kABytes, &tm_x, i * kGroup, t0, &full[s], pol);
          }
        }
      }
    } else if (warp == kIssuerWarp) {
      // ---------------------------------------------------------------- UMMA issue
      if (lane == 0) {
        constexpr uint32_t idesc = idesc_e4m3(kBN, kTN);
        const int my_groups = my_tiles * ng;
        for (int gi = 0; gi < my_groups; ++gi) {
          const int s = gi % kStages, b = gi & 1;
          if (!mbar_wait(&acc_empty[b], ((gi >> 1) & 1) ^ 1, abort_flag, FSITE_MMA_ACC)) break;
          if (!mbar_wait(&full[s], (gi / kStages) & 1, abort_flag, FSITE_MMA_FULL)) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * kStageBytes);
          const uint64_t da = umma_desc_k_sw128(a_addr);
          const uint64_t db = umma_desc_k_sw128(a_addr + kABytes);
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(b * kTN);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_f8(d_tmem, da + 2 * kk, db + 2 * kk, idesc, kk > 0 ? 1u : 0u);
          umma_commit(&empty[s]);
          umma_commit(&acc_full[b]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kIssuerWarp) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tid == 0 && *abort_flag != 0) atomicCAS(status, 0, *abort_flag);
}

// Eight epilogue warps, two batches of 2 x 32 columns per group.  Measured on B200 against sixteen
// warps with 16- or 32-column loads (rolling or one at a time): 3-7 % faster; the steady state
// (0.46 us per group) sits at what the shared-memory port moves - 48 KB written by the copy engine
// and 48 KB read by the tensor core per group.
using KernelShape = Shape<8, 32, 2, true>;
template <int OUT>
constexpr auto Kernel = gemm_w4a4_e4m3_kernel<8, 32, 2, true, OUT>;

}  // namespace f8

int init_gemm_int4_f8_kernels() {
  cudaError_t e = cudaFuncSetAttribute(f8::Kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, f8::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(f8::Kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, f8::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(f8::Kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, f8::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(f8::Kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, f8::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(f8::Kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, f8::kSmemBytes);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "cudaFuncSetAttribute(gemm_w4a4_e4m3) failed: %s", cudaGetErrorString(e));
  return DQ_OK;
}

// w8 / x8: E4M3 bytes, row-major [N, K] / [M, K]
static int launch_gemm_int4_e4m3_impl(const uint8_t* x8, const float* sx, const uint8_t* w8, const void* sw_t,
                                      const float* r, int M, int N, int K, void* y, int y_dtype, const void* residual,
                                      cudaStream_t stream, DeviceState* st, const f8::ScatterDst* scatter) {
  CUtensorMap tm_w, tm_x;
  int rc = make_tmap_2d_u8(&tm_w, w8, static_cast<uint64_t>(K), static_cast<uint64_t>(N), static_cast<uint64_t>(K),
                           128, f8::kBN, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != DQ_OK) return rc;
  rc = make_tmap_2d_u8(&tm_x, x8, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K), 128,
                       f8::kTN, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != DQ_OK) return rc;
  const int row_tiles = (N + f8::kBN - 1) / f8::kBN, tok_tiles = (M + f8::kTN - 1) / f8::kTN;
  const int64_t tiles = static_cast<int64_t>(row_tiles) * tok_tiles;
  const int grid = static_cast<int>(tiles < st->sm_count ? tiles : st->sm_count);
  // activations of one block of token tiles: about 40 MB, so that they stay in L2 (126 MB) beside
  // the weight tiles in use while every row tile passes over them
  int tok_block = static_cast<int>((40ll << 20) / (static_cast<int64_t>(f8::kTN) * K));
  if (tok_block < 1) tok_block = 1;
  if (tok_block > tok_tiles) tok_block = tok_tiles;
  const __half* sw = static_cast<const __half*>(sw_t);
  const int yb = y_dtype == DQ_DTYPE_BF16 ? 1 : 0;
  // bf16 output without a residual leaves through a tiled bulk store (needs 16-byte aligned rows)
  // bf16 output (optionally with a residual) and fp32 output without one leave through tiled bulk
  // stores (16-byte aligned rows); anything else is stored directly
  int bulk_out = 0;
  f8::ScatterDst sc;
  memset(&sc, 0, sizeof(sc));
  if (scatter != nullptr) sc = *scatter;
  if (scatter != nullptr) bulk_out = 4;
  else if (yb && N % 8 == 0 && aligned(y, 16) && (residual == nullptr || aligned(residual, 16))) bulk_out = 1;
  else if (!yb && residual == nullptr && N % 4 == 0 && aligned(y, 16)) bulk_out = 2;
  CUtensorMap tm_y, tm_res;
  memset(&tm_y, 0, sizeof(tm_y));
  memset(&tm_res, 0, sizeof(tm_res));
  if (bulk_out == 1) {
    rc = make_tmap_2d_out(&tm_y, y, 2, static_cast<uint64_t>(N), static_cast<uint64_t>(M), f8::kBN, f8::kTN);
    if (rc != DQ_OK) return rc;
    if (residual != nullptr) {
      rc = make_tmap_2d_out(&tm_res, residual, 2, static_cast<uint64_t>(N), static_cast<uint64_t>(M), f8::kBN, f8::kTN);
      if (rc != DQ_OK) return rc;
    }
  } else if (bulk_out == 2) {
    rc = make_tmap_2d_out(&tm_y, y, 4, static_cast<uint64_t>(N), static_cast<uint64_t>(M), f8::kBN, f8::kTN / 2);
    if (rc != DQ_OK) return rc;
  }
  cudaError_t e;
#define DQ_F8_LAUNCH(OUTV)                                                                                          \
  e = launch_pdl(f8::Kernel<OUTV>, dim3(grid), dim3(f8::KernelShape::kThreads), f8::kSmemBytes, stream, tm_w, tm_x, \
                 tm_y, tm_res, sw, r, sx, y, yb, residual, M, N, K, row_tiles, tok_tiles, tok_block, st->status_dev, sc)
  if (bulk_out == 4) DQ_F8_LAUNCH(4);
  else if (bulk_out == 1 && residual != nullptr) DQ_F8_LAUNCH(3);
  else if (bulk_out == 1) DQ_F8_LAUNCH(1);
  else if (bulk_out == 2) DQ_F8_LAUNCH(2);
  else DQ_F8_LAUNCH(0);
#undef DQ_F8_LAUNCH
  if (e != cudaSuccess) return set_error(DQ_ERR_CUDA, "gemm_w4a4_e4m3 launch failed: %s", cudaGetErrorString(e));
  return DQ_OK;
}

int launch_gemm_int4_e4m3(const uint8_t* x8, const float* sx, const uint8_t* w8, const void* sw_t, const float* r,
                          int M, int N, int K, void* y, int y_dtype, const void* residual, cudaStream_t stream,
                          DeviceState* st) {
  return launch_gemm_int4_e4m3_impl(x8, sx, w8, sw_t, r, M, N, K, y, y_dtype, residual, stream, st, nullptr);
}

}  // namespace dq

using namespace dq;

extern "C" int dq_gemm_w4a4_int4_e4m3_scatter(const uint8_t* x8, const float* sx, const uint8_t* w8, const void* sw_t,
                                              const float* r, int M, int N, int K, int G, const dq_exchange_ctx* ctx,
                                              void* stream) {
  DeviceState* st = current_state();
  if (st == nullptr) return DQ_ERR_NOT_INIT;
  DQ_REQUIRE(x8 != nullptr && sx != nullptr && w8 != nullptr && sw_t != nullptr && ctx != nullptr, DQ_ERR_NULL,
             "null x8 / sx / w8 / sw_t / ctx");
  DQ_REQUIRE(G == kGroup, DQ_ERR_UNSUPPORTED, "weight group size must be %d (got %d)", kGroup, G);
  DQ_REQUIRE(ctx->world >= 1 && ctx->world <= 8 && ctx->rank >= 0 && ctx->rank < ctx->world, DQ_ERR_SHAPE,
             "bad exchange context (world %d, rank %d)", ctx->world, ctx->rank);
  DQ_REQUIRE(K >= kGroup && K % kGroup == 0 && N == ctx->hidden && N % f8::kBN == 0 &&
                 ctx->tokens_per_rank % f8::kTN == 0 && static_cast<int64_t>(M) == ctx->world * ctx->tokens_per_rank,
             DQ_ERR_SHAPE, "scatter GEMM needs N == hidden (%d), N %% 128 == 0, tokens_per_rank %% 256 == 0 and "
             "M == world * tokens_per_rank (M=%d N=%d K=%d tokens_per_rank=%lld)", ctx->hidden, M, N, K,
             static_cast<long long>(ctx->tokens_per_rank));
  DQ_REQUIRE(aligned(x8, 16) && aligned(w8, 16), DQ_ERR_ALIGN, "x8 and w8 must be 16-byte aligned");
  f8::ScatterDst sc;
  memset(&sc, 0, sizeof(sc));
  for (int p = 0; p < ctx->world; ++p) {
    DQ_REQUIRE(ctx->part_ptrs[p] != nullptr && aligned(ctx->part_ptrs[p], 16), DQ_ERR_ALIGN,
               "partial buffer of rank %d is null or not 16-byte aligned", p);
    sc.part[p] = static_cast<unsigned short*>(ctx->part_ptrs[p]);
  }
  sc.rank = ctx->rank;
  sc.tq = static_cast<int>(ctx->tokens_per_rank);
  sc.rot = static_cast<int>(((ctx->rank + 1) % ctx->world) * (ctx->tokens_per_rank / f8::kTN));
  return launch_gemm_int4_e4m3_impl(x8, sx, w8, sw_t, r, M, N, K, nullptr, DQ_DTYPE_BF16, nullptr,
                                    static_cast<cudaStream_t>(stream), st, &sc);
}

extern "C" int dq_expand_w_int4_e4m3(const uint8_t* w_packed, int N, int K, int G, uint8_t* w8, void* stream) {
  DeviceState* st = current_state();
  if (st == nullptr) return DQ_ERR_NOT_INIT;
  DQ_REQUIRE(w_packed != nullptr && w8 != nullptr, DQ_ERR_NULL, "null w_packed / w8");
  DQ_REQUIRE(G == kGroup, DQ_ERR_UNSUPPORTED, "weight group size must be %d (got %d)", kGroup, G);
  DQ_REQUIRE(N >= 1 && K >= kGroup && K % kGroup == 0, DQ_ERR_SHAPE, "bad shape N=%d K=%d", N, K);
  DQ_REQUIRE(aligned(w_packed, 16) && aligned(w8, 16), DQ_ERR_ALIGN, "w_packed and w8 must be 16-byte aligned");
  const int64_t chunks = static_cast<int64_t>((N + 127) / 128) * (K / kGroup) * 512;
  DQ_CHECK_CUDA(launch_pdl(f8::expand_w_e4m3_kernel, dim3(static_cast<unsigned>((chunks + 255) / 256)), dim3(256), 0,
                           static_cast<cudaStream_t>(stream), w_packed, N, K, w8));
  return DQ_OK;
}

extern "C" int dq_codes_to_e4m3(const int8_t* codes, int64_t ld, int M, int K, uint8_t* x8, void* stream) {
  DeviceState* st = current_state();
  if (st == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(codes != nullptr && x8 != nullptr, DQ_ERR_NULL, "null codes / x8");
  DQ_REQUIRE(M >= 1 && K >= 16 && K % 16 == 0 && ld >= K && ld % 16 == 0, DQ_ERR_SHAPE, "bad shape M=%d K=%d ld=%lld", M,
             K, static_cast<long long>(ld));
  DQ_REQUIRE(aligned(codes, 16) && aligned(x8, 16), DQ_ERR_ALIGN, "codes and x8 must be 16-byte aligned");
  const int64_t vecs = static_cast<int64_t>(M) * (K / 16);
  int64_t blocks = (vecs + 255) / 256;
  if (blocks > st->sm_count * 16) blocks = st->sm_count * 16;
  DQ_CHECK_CUDA(launch_pdl(f8::codes_to_e4m3_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0,
                           static_cast<cudaStream_t>(stream), codes, ld, M, K, x8));
  return DQ_OK;
}

extern "C" int dq_gemm_w4a4_int4_e4m3(const uint8_t* x8, const float* sx, const uint8_t* w8, const void* sw_t,
                                      const float* r, int M, int N, int K, int G, void* y, int y_dtype,
                                      const void* residual, void* stream) {
  DeviceState* st = current_state();
  if (st == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(x8 != nullptr && sx != nullptr && w8 != nullptr && sw_t != nullptr && y != nullptr, DQ_ERR_NULL,
             "null x8 / sx / w8 / sw_t / y");
  DQ_REQUIRE(G == kGroup, DQ_ERR_UNSUPPORTED, "weight group size must be %d (got %d)", kGroup, G);
  DQ_REQUIRE(M >= 1 && N >= 1 && K >= kGroup && K % kGroup == 0, DQ_ERR_SHAPE, "bad shape M=%d N=%d K=%d", M, N, K);
  DQ_REQUIRE(y_dtype == DQ_DTYPE_F32 || y_dtype == DQ_DTYPE_BF16, DQ_ERR_UNSUPPORTED, "unknown y_dtype %d", y_dtype);
  DQ_REQUIRE(aligned(x8, 16) && aligned(w8, 16), DQ_ERR_ALIGN, "x8 and w8 must be 16-byte aligned");
  return launch_gemm_int4_e4m3(x8, sx, w8, sw_t, r, M, N, K, y, y_dtype, residual,
                               static_cast<cudaStream_t>(stream), st);
}
