// W4A4 int4 dual-scale GEMM for sm_100a, weights fed to the tensor core from tensor memory.
//
//   Y[m,n] = r[n] * sx[m] * sum_g sw[n,g] * ( sum_{k in group g} qx[m,k] * qw[n,k] )
//
// Orientation ("swap-AB"): the 128 weight rows of a CTA tile are the UMMA M dimension (TMEM
// lanes), the token tile TN is the UMMA N dimension (TMEM columns).  Per weight group (128 k):
// four tcgen05.mma kind::i8 (K = 32) into an int32 TMEM accumulator that is drained once per
// group, so the per-group partial sums are exact.
//
// The A operand (weights) never exists as int8 in shared memory.  The packed int4 tile arrives by
// one bulk copy per pair of groups; each of four unpack warps owns one TMEM lane quarter
// (32 weight rows), reads its rows from the packed stage (one row of 64 bytes per lane; the chunk
// positions inside a row are swizzled in the artefact so that these loads are conflict-free), expands
// nibbles to int8 (two's complement: (w << 4) & 0xF0.. / w & 0xF0.. = 16 * code, the 1/16 folded
// into the group scale) and writes them with tcgen05.st into the operand region of tensor memory:
// lane = row, 32-bit column j of a group's 32 columns = codes k = 4j .. 4j+3, lowest k in the low
// byte.  Against staging int8 tiles in shared memory this removes 32 KB of shared-memory traffic
// per group and the generic->async proxy hand-off, and leaves the shared memory to the rings.
//
// The pipeline advances in steps of two groups (one weight copy, one activation copy, one
// barrier round trip per role per step): every mbarrier / tcgen05 / TMA instruction costs the
// issuing thread 70-100 cycles, and those serial chains, not bandwidth, bound this kernel.
//
// Warp roles (E = 4 epilogue warps, 16 for the 128-token tile):
//   warps 0-3      unpack (lane quarter = warp index)
//   warps 4..3+E   epilogue: chunked tcgen05.ld of the group accumulator, run += float(acc) * sw;
//                  final scale by r[n] * sx[m], store / split-K reduction over the cluster
//   warp 4+E       TMA producer (packed weight steps, activation steps)
//   warp 5+E       UMMA issue, TMEM allocation
//
// Split-K (decode shapes): the CTAs that share an output tile form a thread-block cluster along
// grid z; partial tiles are exchanged through distributed shared memory and summed in rank
// order, so the result is deterministic and needs no global scratch and no second launch.
#include "dq_common.h"
#include "dq_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace dq {

namespace tm {

constexpr int kBN = 128;                     // weight rows per CTA tile (UMMA M)
constexpr int kStepGroups = 2;               // groups per pipeline step
constexpr int kWStepBytes = kStepGroups * kTileBytes;  // 2 x (8192 B codes + 256 B scales)
constexpr int kACols = 32;                   // TMEM columns of one unpacked group (128 int8 / 4)
constexpr int kUnpackWarps = 4;

// {SP, SX, NB, NA} for token tiles 16 / 32 / 64 / 128: packed-weight steps and activation steps
// in shared memory, accumulators and operand steps in tensor memory
constexpr int kCfgTab[4][4] = {{5, 4, 4, 2}, {4, 4, 4, 2}, {3, 3, 2, 2}, {5, 4, 3, 2}};

template <int TN>
struct Cfg {
  static constexpr int kRow = (TN == 16) ? 0 : (TN == 32) ? 1 : (TN == 64) ? 2 : 3;
  static constexpr int SP = kCfgTab[kRow][0];
  static constexpr int SX = kCfgTab[kRow][1];
  static constexpr int NB = kCfgTab[kRow][2];
  static constexpr int NA = kCfgTab[kRow][3];
  // epilogue warps: few warps with more columns each for the small tiles (every waiting warp
  // polls its barrier and costs issue slots)
  static constexpr int EW = (TN == 128) ? 16 : 4;
  static constexpr int kProducerWarp = kUnpackWarps + EW;
  static constexpr int kIssuerWarp = kProducerWarp + 1;
  // The 128-token tile runs one CTA per SM and re-balances registers between warpgroups, which
  // needs whole warpgroups: the CTA is padded to 24 warps, the last two idle.
  static constexpr bool kRebalance = (TN == 128);
  static constexpr int kThreads = kRebalance ? 768 : 32 * (kIssuerWarp + 1);
  static constexpr int kMinCtas = (TN <= 64) ? 2 : 1;
  static constexpr int kXBytes = TN * kGroup;            // one group of activation codes
  static constexpr int kXStepBytes = kStepGroups * kXBytes;
  static constexpr int kOffX = 0;
  static constexpr int kOffW = kOffX + SX * kXStepBytes;
  static constexpr int kOffBar = kOffW + SP * kWStepBytes;
  static constexpr int kNumBars = 2 * SP + 2 * SX + 2 * NA + 2 * NB;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16;
  static constexpr int kAOff = NB * TN;                  // first operand column
  static constexpr int kUsedCols = kAOff + NA * kStepGroups * kACols;
  static constexpr int kTmemCols = kUsedCols <= 32 ? 32 : kUsedCols <= 64 ? 64 : kUsedCols <= 128 ? 128
                                   : kUsedCols <= 256 ? 256 : 512;
  static_assert(kUsedCols <= 512 && kTmemCols * kMinCtas <= 512, "TMEM columns per SM");
  static_assert((kSmemBytes + 1024) * kMinCtas <= 233472, "shared memory per SM");
  static_assert(kOffW % 16 == 0 && kXBytes % 1024 == 0, "operand alignment");
  static constexpr int CPW = TN / (EW / 4);              // accumulator columns per epilogue warp
  static constexpr int CH = 8;                           // columns per tcgen05.ld
  static constexpr int NCH = CPW / CH;
  static_assert(TN * kBN * 4 <= kOffBar, "split-K exchange tile must fit in the stage buffers");
};

// site codes stored in the status word when a bounded wait expires
enum { SITE_TMA = 11, SITE_UNPACK_FULL, SITE_UNPACK_FREE, SITE_MMA_A, SITE_MMA_X, SITE_MMA_ACC,
       SITE_EPI, SITE_SMEM_ALIGN };

__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
      "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]),
      "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
      "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; one thread issues.
__device__ __forceinline__ void umma_i8_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

}  // namespace tm

namespace tm {

// Barriers (s = step, g = group, ring indices by modulo, phases by parity of the use count):
//   full_w / empty_w [SP]   packed weight steps   producer -> 4 unpack warps -> producer
//   full_x / empty_x [SX]   activation steps      producer -> UMMA issuer (tcgen05.commit)
//   a_full / a_free  [NA]   operand steps in TMEM 4 unpack warps -> issuer (tcgen05.commit)
//   acc_done / acc_free [NB] accumulators         issuer (tcgen05.commit) -> EW epilogue warps
// Every barrier is waited on by one role whose warps all pass every phase in order, so a waiter
// is never a whole phase ahead of the barrier (waits are by phase parity).
template <int TN, int MODE>
__global__ void __launch_bounds__(Cfg<TN>::kThreads, Cfg<TN>::kMinCtas)
gemm_w4a4_int4_tm_kernel(const uint8_t* __restrict__ w_packed,
                         const __grid_constant__ CUtensorMap tm_x,
                         const __half* __restrict__ sw_t, const float* __restrict__ r,
                         const float* __restrict__ sx, void* __restrict__ y, int y_bf16,
                         const void* __restrict__ residual,
                         int32_t* __restrict__ acc_dump, int M, int N, int K,
                         int groups_per_split, int split_k, int w_stream_once, int* status) {
  using C = Cfg<TN>;
  // MODE 0: Y with one activation scale per token; 1: dump the raw int32 group sums; 2: Y with one
  // activation scale per (token, weight group): sx is then [K / 128][M], group-major
  constexpr bool DUMP = (MODE == 1);
  constexpr bool GS = (MODE == 2);
  // The 128-byte swizzle of the activation tiles needs them on 1 KB boundaries.  The kernel has
  // no static shared memory, so the dynamic window starts on one; if it ever does not, every CTA
  // reports that and leaves before touching a barrier.
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(status, 0, SITE_SMEM_ALIGN);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint64_t* full_w = bars;
  uint64_t* empty_w = full_w + C::SP;
  uint64_t* full_x = empty_w + C::SP;
  uint64_t* empty_x = full_x + C::SX;
  uint64_t* a_full = empty_x + C::SX;
  uint64_t* a_free = a_full + C::NA;
  uint64_t* acc_done = a_free + C::NA;
  uint64_t* acc_free = acc_done + C::NB;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + C::NB);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n0 = blockIdx.x * kBN;
  const int t0 = blockIdx.y * TN;
  const int total_groups = K / kGroup;
  const int g_begin = blockIdx.z * groups_per_split;
  int g_end = g_begin + groups_per_split;
  if (g_end > total_groups) g_end = total_groups;
  const int ng = (g_end > g_begin) ? (g_end - g_begin) : 0;
  const int ns = (ng + kStepGroups - 1) / kStepGroups;  // steps; the last one may hold one group

  if (tid == 0) {
    for (int i = 0; i < C::SP; ++i) { mbar_init(&full_w[i], 1); mbar_init(&empty_w[i], kUnpackWarps); }
    for (int i = 0; i < C::SX; ++i) { mbar_init(&full_x[i], 1); mbar_init(&empty_x[i], 1); }
    for (int i = 0; i < C::NA; ++i) { mbar_init(&a_full[i], kUnpackWarps); mbar_init(&a_free[i], 1); }
    for (int i = 0; i < C::NB; ++i) { mbar_init(&acc_done[i], 1); mbar_init(&acc_free[i], C::EW); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == C::kIssuerWarp) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  if (warp == C::kProducerWarp && lane == 0) tma_prefetch_desc(&tm_x);
  grid_dep_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tiles of this CTA's 128 rows are contiguous along K: [row tile][group][8 KB codes + scales]
  const uint8_t* w_tile =
      w_packed + static_cast<size_t>(blockIdx.x) * static_cast<size_t>(total_groups) * kTileBytes;

  float run[C::CPW];  // epilogue running sums (only epilogue warps use them)
#pragma unroll
  for (int j = 0; j < C::CPW; ++j) run[j] = 0.f;

  if constexpr (C::kRebalance) {
    if (warp < kUnpackWarps) {
      setmaxnreg_dec<64>();
    } else if (warp < C::kProducerWarp) {
      setmaxnreg_inc<88>();
    } else {
      setmaxnreg_dec<40>();
    }
  }

  if (warp < kUnpackWarps) {
    // ------------------------------------------------------------------ unpack warps
    // Lane l of warp w owns weight row 32 w + l = TMEM lane 32 w + l.
    const uint32_t lane_field = static_cast<uint32_t>(warp * 32) << 16;
    const int row = warp * 32 + lane;
    for (int s = 0; s < ns; ++s) {
      const int sp = s % C::SP, ab = s % C::NA;
      const int cnt = (ng - s * kStepGroups >= kStepGroups) ? kStepGroups : 1;
      if (!mbar_wait(&full_w[sp], (s / C::SP) & 1, abort_flag, SITE_UNPACK_FULL)) break;
      const uint8_t* stage = smem + C::kOffW + sp * kWStepBytes;
      // both groups' packed rows first (8 loads in flight), then the wait for the operand
      // buffer, then expansion and the TMEM stores
      uint4 raw[kStepGroups][4];
#pragma unroll
      for (int h = 0; h < kStepGroups; ++h) {
        if (h < cnt) {
          const uint4* src = reinterpret_cast<const uint4*>(stage + h * kTileBytes + row * 64);
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) raw[h][ch] = src[ch ^ ((row >> 1) & 3)];  // swizzled position
        }
      }
      if (!mbar_wait(&a_free[ab], ((s / C::NA) & 1) ^ 1, abort_flag, SITE_UNPACK_FREE)) break;
      tc_fence_after();
#pragma unroll
      for (int h = 0; h < kStepGroups; ++h) {
        if (h < cnt) {
          uint32_t v[32];
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            // chunk ch, byte b = code[32 ch + b] | code[32 ch + 16 + b] << 4
            const uint4 w = raw[h][ch];
            v[8 * ch + 0] = (w.x << 4) & 0xF0F0F0F0u; v[8 * ch + 4] = w.x & 0xF0F0F0F0u;
            v[8 * ch + 1] = (w.y << 4) & 0xF0F0F0F0u; v[8 * ch + 5] = w.y & 0xF0F0F0F0u;
            v[8 * ch + 2] = (w.z << 4) & 0xF0F0F0F0u; v[8 * ch + 6] = w.z & 0xF0F0F0F0u;
            v[8 * ch + 3] = (w.w << 4) & 0xF0F0F0F0u; v[8 * ch + 7] = w.w & 0xF0F0F0F0u;
          }
          tmem_st_x32(tmem_base + lane_field +
                          static_cast<uint32_t>(C::kAOff + (ab * kStepGroups + h) * kACols),
                      v);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();  // every lane has consumed its loads from the packed stage
      if (lane == 0) {
        mbar_arrive(&a_full[ab]);
        mbar_arrive(&empty_w[sp]);
      }
    }
  } else if (warp < C::kProducerWarp) {
    // ------------------------------------------------------------------ epilogue warps
    const int q = warp & 3;                    // TMEM lane quarter this warp may read
    const int h = (warp - kUnpackWarps) >> 2;  // which slice of the token columns
    const int n = n0 + q * 32 + lane;
    const bool n_ok = n < N;
    if (lane == 0) {  // every accumulator starts out free
#pragma unroll
      for (int b = 0; b < C::NB; ++b) mbar_arrive(&acc_free[b]);
    }
    // Group scales of this thread's weight row, [row tile][group][128] in memory.  A new 256-byte
    // run is touched every group, so loads are issued kScaleAhead groups early.  The ring holds
    // the raw fp16 bits: converting at load time would make the warp wait for the load at once.
    constexpr int kScaleAhead = 4;
    const unsigned short* sw_row = nullptr;
    unsigned short sq[kScaleAhead];
#pragma unroll
    for (int d = 0; d < kScaleAhead; ++d) sq[d] = 0;
    if constexpr (!DUMP) {
      sw_row = reinterpret_cast<const unsigned short*>(sw_t) +
               (static_cast<size_t>(blockIdx.x) * total_groups + g_begin) * kBN + q * 32 + lane;
#pragma unroll
      for (int d = 0; d < kScaleAhead; ++d)
        if (d < ng) sq[d] = __ldg(sw_row + static_cast<size_t>(d) * kBN);
    }
    auto ld_chunk = [&](int b, int c0, uint32_t* v) {
      tmem_ld_x8(tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                     static_cast<uint32_t>(b * TN + h * C::CPW + c0),
                 v);
    };
    auto consume = [&](const uint32_t* v, int c0, int i, float s) {
      if constexpr (DUMP) {
        if (n_ok) {
#pragma unroll
          for (int j = 0; j < C::CH; ++j) {
            const int m = t0 + h * C::CPW + c0 + j;
            if (m < M)
              acc_dump[(static_cast<size_t>(m) * N + n) * total_groups + (g_begin + i)] =
                  static_cast<int32_t>(v[j]) >> 4;
          }
        }
      } else {
        // two columns per instruction: packed fp32 FMA (each half rounds like a scalar fmaf)
        const float* sg = nullptr;
        if constexpr (GS) sg = sx + static_cast<size_t>(g_begin + i) * M;  // this group's token scales
#pragma unroll
        for (int j = 0; j < C::CH; j += 2) {
          const float2 f = make_float2(static_cast<float>(static_cast<int32_t>(v[j])),
                                       static_cast<float>(static_cast<int32_t>(v[j + 1])));
          float2 p = make_float2(s, s);
          if constexpr (GS) {
            // warp-uniform addresses (every lane of a warp holds the same token columns)
            const int m0 = t0 + h * C::CPW + c0 + j;
            p.x = __fmul_rn(s, __ldg(sg + (m0 < M ? m0 : M - 1)));
            p.y = __fmul_rn(s, __ldg(sg + (m0 + 1 < M ? m0 + 1 : M - 1)));
          }
          const float2 acc2 = __ffma2_rn(f, p, make_float2(run[c0 + j], run[c0 + j + 1]));
          run[c0 + j] = acc2.x;
          run[c0 + j + 1] = acc2.y;
        }
      }
    };
    // The accumulator of a group is read in chunks of 8 columns.  tcgen05.ld is asynchronous, so
    // chunk c + 1 is in flight while chunk c is scaled and added, and as soon as the accumulator
    // is drained the first chunk of the next group is requested (if its UMMAs have finished)
    // before the last chunk of this one is consumed.
    uint32_t va[C::CH], vb[C::CH];
    bool prefetched = false;
    auto group_step = [&](int i, unsigned short& sreg) -> bool {
      const int b = i % C::NB;
      const float s = __half2float(__ushort_as_half(sreg)) * 0.0625f;
      if constexpr (!DUMP) {
        if (i + kScaleAhead < ng) sreg = __ldg(sw_row + static_cast<size_t>(i + kScaleAhead) * kBN);
      }
      if (!prefetched) {
        if (!mbar_wait(&acc_done[b], (i / C::NB) & 1, abort_flag, SITE_EPI)) return false;
        tc_fence_after();
        ld_chunk(b, 0, va);
      }
#pragma unroll
      for (int c = 0; c < C::NCH; ++c) {  // chunk c lives in va (c even) or vb (c odd)
        uint32_t* cur = (c & 1) ? vb : va;
        uint32_t* nxt = (c & 1) ? va : vb;
        tmem_ld_wait();  // chunk c has landed
        if (c + 1 < C::NCH) {
          ld_chunk(b, (c + 1) * C::CH, nxt);
        } else {
          // accumulator b is free once its last column has been read
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_free[b]);
          if constexpr (C::NCH > 1) {  // NCH is even: the next group's first chunk goes to va
            prefetched = false;
            if (i + 1 < ng) {
              const int b1 = (i + 1) % C::NB;
              // tcgen05.ld is warp-collective: take the early path only if every lane saw the phase
              if (__all_sync(0xffffffffu,
                             mbar_test_wait(&acc_done[b1], ((i + 1) / C::NB) & 1) ? 1 : 0)) {
                tc_fence_after();
                ld_chunk(b1, 0, nxt);
                prefetched = true;
              }
            }
          }
        }
        consume(cur, c * C::CH, i, s);
      }
      return true;
    };
    bool ok = true;
    for (int i0 = 0; i0 < ng && ok; i0 += kScaleAhead) {
#pragma unroll
      for (int u = 0; u < kScaleAhead; ++u) {
        if (ok && i0 + u < ng) ok = group_step(i0 + u, sq[u]);
      }
    }
    if constexpr (!DUMP) {
      if (split_k == 1) {
        if (n_ok) {
          // one running pointer per thread instead of a multiply and two tests per element
          const float rn = (r != nullptr) ? r[n] : 1.f;
          const int m0 = t0 + h * C::CPW;
          const int cnt = (M - m0 < C::CPW) ? (M - m0) : C::CPW;  // tokens of this slice that exist
          const float* sxp = sx + m0;
          auto tok_scale = [&](int j) -> float {  // per-token scale; already applied per group in GS mode
            if constexpr (GS) return 1.f;
            return __ldg(sxp + j);
          };
          if (residual != nullptr) {
            size_t idx = static_cast<size_t>(m0) * N + n;
#pragma unroll
            for (int j = 0; j < C::CPW; ++j) {
              if (j < cnt) store_y(y, residual, y_bf16, idx, run[j] * (rn * tok_scale(j)));
              idx += N;
            }
          } else if (y_bf16) {
            __nv_bfloat16* yp = reinterpret_cast<__nv_bfloat16*>(y) + static_cast<size_t>(m0) * N + n;
#pragma unroll
            for (int j = 0; j < C::CPW; ++j) {
              if (j < cnt) *yp = __float2bfloat16_rn(run[j] * (rn * tok_scale(j)));
              yp += N;
            }
          } else {
            float* yp = reinterpret_cast<float*>(y) + static_cast<size_t>(m0) * N + n;
#pragma unroll
            for (int j = 0; j < C::CPW; ++j) {
              if (j < cnt) *yp = run[j] * (rn * tok_scale(j));
              yp += N;
            }
          }
        }
      } else {
        // Partial tile -> this CTA's exchange buffer red[token][row] (aliases the stage buffers:
        // the last acc_done wait above implies every UMMA, hence every operand read, is over,
        // and the producer has no copy in flight once the last step has been consumed).
        float* red = reinterpret_cast<float*>(smem);
#pragma unroll
        for (int j = 0; j < C::CPW; ++j) red[(h * C::CPW + j) * kBN + q * 32 + lane] = run[j];
      }
    }
  } else if (warp == C::kProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    // Weights run up to SP steps ahead of the unpack warps, activations up to SX steps ahead of
    // the UMMAs.  Weights do not depend on the preceding kernel of the stream, the activation
    // codes do: the weight ring is filled before the wait for the prerequisite grid
    // (programmatic dependent launch).
    const uint64_t pol_w = w_stream_once ? l2_policy_evict_first() : l2_policy_evict_last();
    const uint64_t pol_x = l2_policy_evict_last();
    auto issue_w = [&](int s) {
      const int sp = s % C::SP;
      const int cnt = (ng - s * kStepGroups >= kStepGroups) ? kStepGroups : 1;
      const uint32_t bytes = static_cast<uint32_t>(cnt) * kTileBytes;
      mbar_expect_tx(&full_w[sp], bytes);
      bulk_load_1d(smem + C::kOffW + sp * kWStepBytes,
                   w_tile + static_cast<size_t>(g_begin + s * kStepGroups) * kTileBytes, bytes,
                   &full_w[sp], pol_w);
    };
    // Only lane 0 works; the other lanes go straight to the end of the role (a waiting warp of
    // 32 polling lanes costs the SM issue slots and barrier-unit bandwidth the other roles need).
    if (lane == 0) {
      const int pre = (ns < C::SP) ? ns : C::SP;
      for (int s = 0; s < pre; ++s) issue_w(s);
      grid_dep_wait();
      // Step s: its activation box (needed by the UMMAs of step s), then the weight step SP
      // ahead.  Both waits are on consumers of strictly earlier copies, so the order cannot
      // dead-lock.
      for (int s = 0; s < ns; ++s) {
        const int sxi = s % C::SX;
        if (!mbar_wait(&empty_x[sxi], ((s / C::SX) & 1) ^ 1, abort_flag, SITE_TMA)) break;
        // one box = 2 groups x TN tokens; a group past the end of K is zero-filled and still
        // counted, so the byte count is always that of the full box
        mbar_expect_tx(&full_x[sxi], C::kXStepBytes);
        tma_load_3d(smem + C::kOffX + sxi * C::kXStepBytes, &tm_x, 0, t0,
                    g_begin + s * kStepGroups, &full_x[sxi], pol_x);
        const int sw_next = s + C::SP;
        if (sw_next < ns) {
          if (!mbar_wait(&empty_w[sw_next % C::SP], ((sw_next / C::SP) & 1) ^ 1, abort_flag, SITE_TMA))
            break;
          issue_w(sw_next);
        }
      }
    }
  } else if (warp == C::kIssuerWarp) {
    // ------------------------------------------------------------------ UMMA issuer
    // Whole warp waits (uniform control flow); lane 0 issues tcgen05.mma / tcgen05.commit.
    constexpr uint32_t idesc = umma_idesc_i8(kBN, TN);
    const uint32_t x_base = smem_u32(smem + C::kOffX);
    // Only lane 0 works (see the producer).
    if (lane == 0) {
      bool ok = true;
      for (int s = 0; s < ns && ok; ++s) {
        const int ab = s % C::NA, sxi = s % C::SX;
        const int cnt = (ng - s * kStepGroups >= kStepGroups) ? kStepGroups : 1;
        if (!mbar_wait(&a_full[ab], (s / C::NA) & 1, abort_flag, SITE_MMA_A)) break;
        if (!mbar_wait(&full_x[sxi], (s / C::SX) & 1, abort_flag, SITE_MMA_X)) break;
#pragma unroll
        for (int h = 0; h < kStepGroups; ++h) {
          if (h < cnt && ok) {
            const int g = s * kStepGroups + h;
            const int b = g % C::NB;
            if (!mbar_wait(&acc_free[b], (g / C::NB) & 1, abort_flag, SITE_MMA_ACC)) {
              ok = false;
            } else {
              tc_fence_after();
              const uint64_t db = umma_desc_k_sw128(x_base + sxi * C::kXStepBytes + h * C::kXBytes);
              const uint32_t a_tmem =
                  tmem_base + static_cast<uint32_t>(C::kAOff + (ab * kStepGroups + h) * kACols);
              const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(b * TN);
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)  // 32 k = 8 operand columns = 32 bytes of an X row
                umma_i8_ta(d_tmem, a_tmem + 8 * kk, db + 2 * kk, idesc, kk > 0 ? 1u : 0u);
              umma_commit(&acc_done[b]);
            }
          }
        }
        if (ok) {
          umma_commit(&a_free[ab]);
          umma_commit(&empty_x[sxi]);
        }
      }
    }
  }

  // -------------------------------------------------------------------- split-K reduction
  if (!DUMP && split_k > 1) {
    __syncwarp();
    cluster_sync_all();
    if (warp < 8) {  // 256 threads (unpack warps and the first epilogue warps; all roles are done)
      const uint32_t rank = cluster_ctarank();
      const int rows = TN / split_k;  // token rows of the tile this CTA finishes
      const int e = tid;              // 0..255
      const int c4 = e & 31;                  // float4 column
      const uint32_t red_base = smem_u32(smem);
      for (int rr = e >> 5; rr < rows; rr += 8) {
        const int tl = static_cast<int>(rank) * rows + rr;
        const int m = t0 + tl;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const uint32_t off = static_cast<uint32_t>((tl * kBN + c4 * 4) * 4);
        for (int p = 0; p < split_k; ++p) {
          const float4 v = dsmem_ld_f4(dsmem_map(red_base + off, static_cast<uint32_t>(p)));
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if (m < M) {
          const float sm = GS ? 1.f : sx[m];
          const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int n = n0 + c4 * 4 + u;
            if (n < N) {
              const float rn = (r != nullptr) ? r[n] : 1.f;
              store_y(y, residual, y_bf16, static_cast<size_t>(m) * N + n, vals[u] * (rn * sm));
            }
          }
        }
      }
    }
    __syncwarp();
    cluster_sync_all();  // peers may still be reading this CTA's exchange buffer until here
  }

  // -------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == C::kIssuerWarp) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
  if (tid == 0 && *abort_flag != 0) atomicCAS(status, 0, *abort_flag);
}

template <int TN, int MODE>
static int set_attr() {
  cudaError_t e = cudaFuncSetAttribute(gemm_w4a4_int4_tm_kernel<TN, MODE>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg<TN>::kSmemBytes);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "cudaFuncSetAttribute(gemm tm TN=%d) failed: %s", TN,
                     cudaGetErrorString(e));
  return DQ_OK;
}

template <int TN, int MODE>
static int launch(const int8_t* codes, const float* sx, const uint8_t* w_packed, const __half* sw_t,
                  const float* r, int M, int N, int K, void* y, int y_dtype, int32_t* acc_dump,
                  int split, cudaStream_t stream, DeviceState* st, const void* residual) {
  CUtensorMap tm_x;
  int rc = make_tmap_x_groups(&tm_x, codes, K, M, TN, kStepGroups);
  if (rc != DQ_OK) return rc;
  const int total_groups = K / kGroup;
  const int gps = (total_groups + split - 1) / split;
  const int tok_tiles = (M + TN - 1) / TN;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((N + kBN - 1) / kBN, tok_tiles, split);
  cfg.blockDim = dim3(Cfg<TN>::kThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg<TN>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = split;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const int w_stream_once = (tok_tiles == 1) ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_w4a4_int4_tm_kernel<TN, MODE>, w_packed, tm_x, sw_t,
                                     r, sx, y, y_dtype == DQ_DTYPE_BF16 ? 1 : 0, residual, acc_dump, M, N, K,
                                     gps, split, w_stream_once, st->status_dev);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "gemm_w4a4_int4 (tm) launch failed (TN=%d split=%d): %s", TN,
                     split, cudaGetErrorString(e));
  return DQ_OK;
}

}  // namespace tm

int init_gemm_int4_tm_kernels() {
  int rc;
  if ((rc = tm::set_attr<16, 0>()) != DQ_OK) return rc;
  if ((rc = tm::set_attr<32, 0>()) != DQ_OK) return rc;
  if ((rc = tm::set_attr<64, 0>()) != DQ_OK) return rc;
  if ((rc = tm::set_attr<128, 0>()) != DQ_OK) return rc;
  if ((rc = tm::set_attr<16, 1>()) != DQ_OK) return rc;
  if ((rc = tm::set_attr<128, 1>()) != DQ_OK) return rc;
  if ((rc = tm::set_attr<16, 2>()) != DQ_OK) return rc;
  if ((rc = tm::set_attr<32, 2>()) != DQ_OK) return rc;
  if ((rc = tm::set_attr<64, 2>()) != DQ_OK) return rc;
  if ((rc = tm::set_attr<128, 2>()) != DQ_OK) return rc;
  return DQ_OK;
}

// tn: 16 / 32 / 64 / 128; acc_dump != nullptr selects the accumulator-dump variant (tn 16 or 128).
int launch_gemm_int4_tm(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                        const void* sw_t, const float* r, int M, int N, int K, void* y, int y_dtype,
                        int32_t* acc_dump, int tn, int split, cudaStream_t s, DeviceState* st,
                        const void* residual, bool grouped_sx) {
  const __half* swp = static_cast<const __half*>(sw_t);
  if (grouped_sx && acc_dump == nullptr) {
    switch (tn) {
      case 16: return tm::launch<16, 2>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, nullptr, split, s, st, residual);
      case 32: return tm::launch<32, 2>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, nullptr, split, s, st, residual);
      case 64: return tm::launch<64, 2>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, nullptr, split, s, st, residual);
      default: return tm::launch<128, 2>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, nullptr, split, s, st, residual);
    }
  }
  if (acc_dump != nullptr) {
    if (tn == 16)
      return tm::launch<16, 1>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, acc_dump, 1, s, st, residual);
    return tm::launch<128, 1>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, acc_dump, 1, s, st, residual);
  }
  switch (tn) {
    case 16: return tm::launch<16, 0>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, nullptr, split, s, st, residual);
    case 32: return tm::launch<32, 0>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, nullptr, split, s, st, residual);
    case 64: return tm::launch<64, 0>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, nullptr, split, s, st, residual);
    default: return tm::launch<128, 0>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, nullptr, split, s, st, residual);
  }
}

}  // namespace dq
