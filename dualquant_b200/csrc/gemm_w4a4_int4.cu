// W4A4 int4 dual-scale GEMM for sm_100a.
//
//   Y[m,n] = r[n] * sx[m] * sum_g sw[n,g] * ( sum_{k in group g} qx[m,k] * qw[n,k] )
//
// Orientation ("swap-AB"): the 128 weight rows of a CTA tile are the UMMA M dimension (TMEM
// lanes), the token tile TN is the UMMA N dimension (TMEM columns).  One pipeline stage is one
// weight group (128 k): four tcgen05.mma kind::i8 (K=32) into an int32 TMEM accumulator that is
// drained once per group, so the per-group partial sums are exact.  Each epilogue thread owns
// one weight row and therefore one scalar group scale per stage.
//
// Warp roles (E = 8 epilogue warps, 16 for the 128-token tile):
//   warps 0-3        unpack: packed int4 tile (TMA-staged, 8 KB) -> int8 tile in the 128B-swizzled
//                    K-major layout UMMA reads (16 KB).  Nibbles are two's complement; a byte is
//                    expanded as (w << 4) & 0xF0.. / w & 0xF0.., i.e. 16 * code, and the 1/16 is
//                    folded into the group scale (exact: power of two).  One warp expands a whole
//                    group, so four consecutive groups are in work at once.
//   warps 4..3+E     epilogue: tcgen05.ld of the group accumulator in two column chunks, the load
//                    of a chunk overlapping the arithmetic of the one before (also across groups);
//                    run += float(acc) * sw; final scale by r[n]*sx[m], store / split-K reduction.
//   warp 4+E         TMA producer: packed weight tiles (contiguous 8 KB bulk copies) and int8
//                    activation tiles (tiled, 128B swizzle).
//   warps 5+E(,6+E)  UMMA issue (two warps, even / odd groups, for the 128-token tile; one
//                    otherwise); warp 5+E also owns the TMEM allocation.
//                    Every tcgen05 / mbarrier instruction costs tens of cycles of issue latency on
//                    the thread that executes it; one wait pair, four UMMAs and two commits per
//                    group come to ~400 cycles, more than the UMMAs of a group take to execute,
//                    hence two issuing threads.
//
// Split-K (decode shapes): the CTAs that share an output tile form a thread-block cluster along
// grid z; partial tiles are exchanged through distributed shared memory and summed in rank
// order, so the result is deterministic and needs no global scratch and no second launch.
#include "dq_common.h"
#include "dq_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace dq {

constexpr int kBN = 128;           // weight rows per CTA tile (UMMA M)

constexpr int kWpBytes = kBN * kGroup / 2;  // packed stage: 8 KB
constexpr int kWaBytes = kBN * kGroup;      // unpacked stage: 16 KB

// {SP, SX, XC} for token tiles 16 / 32 / 64 / 128
constexpr int kCfgTab[4][3] = {{4, 2, 4}, {4, 2, 2}, {4, 2, 1}, {12, 4, 1}};
constexpr int kUnpackWarps = 4;

template <int TN>
struct Cfg {
  // NB unpacked weight buffers = TMEM accumulators in flight (buffer b and accumulator b of a
  // group travel together through the ready/done barriers), SP packed-weight stages, SX
  // activation stages of XC groups each (one 3-D TMA copy per stage: every instruction the
  // producer thread issues costs it ~100 cycles).  Two CTAs per SM for TN <= 64.
  static constexpr int kRow = (TN == 16) ? 0 : (TN == 32) ? 1 : (TN == 64) ? 2 : 3;
  static constexpr int NB = 4;
  static constexpr int SP = kCfgTab[kRow][0];
  static constexpr int SX = kCfgTab[kRow][1];
  static constexpr int XC = kCfgTab[kRow][2];
  // A role that is split over several warps by group index must find every barrier it waits on
  // owned by one warp: waits are by phase parity, so a warp may never be a whole phase ahead of
  // the barrier's previous user.
  static_assert(NB % kUnpackWarps == 0 && SP % kUnpackWarps == 0, "stage and buffer rings: multiples of 4");
  // UMMA-issuing warps: two for the 128-token tile (the issue cost of a group exceeds its UMMA
  // time there); one otherwise, which keeps two 448-thread CTAs per SM at 72 registers.
  static constexpr int kIssuers = (TN == 128) ? 2 : 1;
  static_assert(NB % kIssuers == 0 && SX % kIssuers == 0, "buffer and activation rings: even");
  static_assert(kIssuers == 1 || XC == 1, "two issuing warps: one group per activation stage");
  static constexpr int EW = (TN == 128) ? 16 : 8;       // epilogue warps
  static constexpr int kProducerWarp = kUnpackWarps + EW;
  static constexpr int kIssuerWarp0 = kProducerWarp + 1;
  // The 128-token tile runs one CTA per SM and re-balances registers between warpgroups
  // (unpack 56, epilogue 96, producer/issuers 40 of the 80 the launch grants each thread), which
  // needs whole warpgroups: the CTA is padded to 24 warps, the last one idle.
  static constexpr bool kRebalance = (TN == 128);
  static constexpr int kThreads = kRebalance ? 768 : 32 * (kIssuerWarp0 + kIssuers);
  static_assert(!kRebalance || (kIssuerWarp0 + kIssuers <= 24 && kProducerWarp % 4 == 0), "warpgroup layout");
  static constexpr int kReadyCount = EW + 1;            // epilogue warps + the unpacking warp
  static constexpr int kXBytes = TN * kGroup;           // one group of activation codes
  static constexpr int kMinCtas = (TN <= 64) ? 2 : 1;
  static constexpr int kOffA = 0;                       // NB unpacked weight buffers
  static constexpr int kOffX = kOffA + NB * kWaBytes;
  static constexpr int kXStageBytes = XC * kXBytes;
  static constexpr int kOffP = kOffX + SX * kXStageBytes;
  static constexpr int kOffBar = kOffP + SP * kWpBytes;
  static constexpr int kNumBars = SP + 2 * SX + 2 * NB;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16;
  static constexpr int kAccCols = NB * TN;
  static constexpr int kTmemCols = kAccCols <= 32 ? 32 : kAccCols <= 64 ? 64 : kAccCols <= 128 ? 128
                                   : kAccCols <= 256 ? 256 : 512;
  static_assert(kTmemCols * kMinCtas <= 512, "TMEM columns per SM");
  static_assert((kSmemBytes + 1024) * kMinCtas <= 233472, "shared memory per SM");
  static constexpr int CPW = TN / (EW / 4);             // accumulator columns per epilogue warp
  static constexpr int CH = 8;  // columns per tcgen05.ld (16 measured 7-10 % slower at TN = 128)
  static constexpr int NCH = CPW / CH;                  // chunks per group: 1, 2 or 4
  static_assert(TN * kBN * 4 <= kOffBar, "split-K exchange tile must fit in the stage buffers");
};

// site codes stored in the status word when a bounded wait expires
enum { SITE_TMA = 1, SITE_UNPACK_FULL, SITE_UNPACK_FREE, SITE_MMA_READY, SITE_MMA_X, SITE_EPI,
       SITE_SMEM_ALIGN };

// Barrier protocol (b = i % NB selects the unpacked-weight buffer and the TMEM accumulator):
//   full_p [SP]            packed weight ring   TMA -> the unpacking warp that owns the stage
//                          (it re-arms the barrier and refills the stage itself)
//   full_x / empty_x [SX]  activation ring      producer -> UMMA issuer  (tcgen05.commit)
//   ready[b]               buffer b written by its unpacking warp AND accumulator b drained by
//                          all epilogue warps (EW + 1 arrivals; the epilogue pre-arrives once)
//   done[b]                UMMAs of the group finished (tcgen05.commit): the epilogue may read
//                          accumulator b, the unpack warp may overwrite buffer b
template <int TN>
__global__ void __launch_bounds__(Cfg<TN>::kThreads, Cfg<TN>::kMinCtas)
gemm_w4a4_int4_kernel(const uint8_t* __restrict__ w_packed,
                      const __grid_constant__ CUtensorMap tm_x,
                      const __half* __restrict__ sw_t, const float* __restrict__ r,
                      const float* __restrict__ sx, void* __restrict__ y, int y_bf16,
                      const void* __restrict__ residual, int M, int N, int K, int groups_per_split,
                      int split_k, int w_stream_once, int* status) {
  using C = Cfg<TN>;
  // The 128-byte swizzle of the UMMA operands needs the buffers on 1 KB boundaries.  The kernel has
  // no static shared memory, so the dynamic window starts on one; if it ever does not, every CTA
  // reports that and leaves before touching a barrier.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(status, 0, SITE_SMEM_ALIGN);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint64_t* full_p = bars;
  uint64_t* full_x = full_p + C::SP;
  uint64_t* empty_x = full_x + C::SX;
  uint64_t* ready = empty_x + C::SX;
  uint64_t* done = ready + C::NB;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + C::NB);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int total_groups = K / kGroup;
  const int g_begin = blockIdx.z * groups_per_split;
  int g_end = g_begin + groups_per_split;
  if (g_end > total_groups) g_end = total_groups;
  const int ng = (g_end > g_begin) ? (g_end - g_begin) : 0;
  // Tile walk.  Without split-K the grid is persistent: CTA c takes the output tiles c,
  // c + gridDim.x, ... of the list ordered token tile fastest (CTAs that run together share a
  // few weight tiles and the activations through L2), and its pipeline runs on from one tile
  // into the next: the global group counter gi = (tile iteration) * ng + i indexes every ring and
  // barrier phase.  With split-K every CTA owns one tile (grid x = row tile, y = token tile).
  const int tok_tiles = (M + TN - 1) / TN;
  const int n_tiles = ((N + kBN - 1) / kBN) * tok_tiles;
  const bool persistent = (split_k == 1);
  const int tile0 = persistent ? static_cast<int>(blockIdx.x)
                               : static_cast<int>(blockIdx.x) * tok_tiles + static_cast<int>(blockIdx.y);
  const int tile_step = persistent ? static_cast<int>(gridDim.x) : n_tiles;
  const int my_tiles = (tile0 < n_tiles) ? (n_tiles - tile0 + tile_step - 1) / tile_step : 0;
  const int my_groups = my_tiles * ng;
  const int nxs = (ng + C::XC - 1) / C::XC;  // activation stages per tile
  auto tile_row = [&](int it) { return (tile0 + it * tile_step) / tok_tiles; };  // 128-row tile index
  auto tile_tok = [&](int it) { return (tile0 + it * tile_step) % tok_tiles; };  // token tile index
  // packed tile of global group gi: tiles of a row tile are contiguous along K
  auto w_group = [&](int gi) {
    return w_packed + (static_cast<size_t>(tile_row(gi / ng)) * static_cast<size_t>(total_groups) +
                       static_cast<size_t>(g_begin + gi % ng)) * kTileBytes;
  };

  if (tid == 0) {
    for (int i = 0; i < C::SP; ++i) mbar_init(&full_p[i], 1);
    for (int i = 0; i < C::SX; ++i) { mbar_init(&full_x[i], 1); mbar_init(&empty_x[i], 1); }
    for (int i = 0; i < C::NB; ++i) { mbar_init(&ready[i], C::kReadyCount); mbar_init(&done[i], 1); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == C::kIssuerWarp0) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  if (warp == C::kProducerWarp && lane == 0) tma_prefetch_desc(&tm_x);
  grid_dep_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  float run[C::CPW];  // epilogue running sums (only epilogue warps use them)
#pragma unroll
  for (int j = 0; j < C::CPW; ++j) run[j] = 0.f;

  if constexpr (C::kRebalance) {
    if (warp < kUnpackWarps) {
      setmaxnreg_dec<56>();
    } else if (warp < C::kProducerWarp) {
      setmaxnreg_inc<96>();
    } else {
      setmaxnreg_dec<40>();
    }
  }

  if (warp < kUnpackWarps) {
    // ------------------------------------------------------------------ unpack warps
    // One warp expands a whole group (groups warp, warp + 4, ...): the four warps work on four
    // consecutive groups at once, so the wait / expand / proxy-fence / arrive chain of a group,
    // which is latency and not throughput, overlaps with that of its neighbours.
    const uint64_t pol_w = w_stream_once ? l2_policy_evict_first() : l2_policy_evict_last();
    for (int i = warp; i < my_groups; i += kUnpackWarps) {  // i: global group index
      const int sp = i % C::SP, b = i % C::NB;
      if (!mbar_wait(&full_p[sp], (i / C::SP) & 1, abort_flag, SITE_UNPACK_FULL)) break;
      if (!mbar_wait(&done[b], ((i / C::NB) & 1) ^ 1, abort_flag, SITE_UNPACK_FREE)) break;
      const uint8_t* src = smem + C::kOffP + sp * kWpBytes;
      uint8_t* dst = smem + C::kOffA + b * kWaBytes;
#pragma unroll
      for (int c8 = 0; c8 < 16; c8 += 8) {
        uint4 wv[8];
#pragma unroll
        for (int c = 0; c < 8; ++c)
          wv[c] = *reinterpret_cast<const uint4*>(src + (lane + (c8 + c) * 32) * 16);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int id = lane + (c8 + c) * 32;  // 16-byte chunk of the packed tile
          const int row = id >> 2;
          const int ch = (id & 3) ^ ((row >> 1) & 3);  // position in the row -> k chunk
          const uint4 w = wv[c];
          uint4 lo, hi;
          lo.x = (w.x << 4) & 0xF0F0F0F0u; hi.x = w.x & 0xF0F0F0F0u;
          lo.y = (w.y << 4) & 0xF0F0F0F0u; hi.y = w.y & 0xF0F0F0F0u;
          lo.z = (w.z << 4) & 0xF0F0F0F0u; hi.z = w.z & 0xF0F0F0F0u;
          lo.w = (w.w << 4) & 0xF0F0F0F0u; hi.w = w.w & 0xF0F0F0F0u;
          uint8_t* rowp = dst + row * 128;
          const int sw = row & 7;
          *reinterpret_cast<uint4*>(rowp + (((2 * ch) ^ sw) << 4)) = lo;
          *reinterpret_cast<uint4*>(rowp + (((2 * ch + 1) ^ sw) << 4)) = hi;
        }
      }
      fence_proxy_async_smem();  // each writer orders its own stores before the UMMA reads
      __syncwarp();               // every lane has consumed its loads from the packed stage
      if (lane == 0) {
        mbar_arrive(&ready[b]);
        // The stage belongs to this warp (SP is a multiple of the unpack warp count): refill it
        // for group i + SP right away instead of handing it back to the producer warp.
        if (i + C::SP < my_groups) {
          mbar_expect_tx(&full_p[sp], kWpBytes);
          bulk_load_1d(smem + C::kOffP + sp * kWpBytes, w_group(i + C::SP), kWpBytes,
                       &full_p[sp], pol_w);
        }
      }
    }
  } else if (warp < C::kProducerWarp) {
    // ------------------------------------------------------------------ epilogue warps
    const int q = warp & 3;          // TMEM lane quarter this warp may read
    const int h = (warp - kUnpackWarps) >> 2;  // which slice of the token columns
    if (lane == 0) {  // every accumulator starts out free
#pragma unroll
      for (int b = 0; b < C::NB; ++b) mbar_arrive(&ready[b]);
    }
    auto ld_chunk = [&](int b, int c0, uint32_t* v) {
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                             static_cast<uint32_t>(b * TN + h * C::CPW + c0);
      tmem_ld_x8(taddr, v);
    };
    auto consume = [&](const uint32_t* v, int c0, float s) {
      // two columns per instruction: packed fp32 FMA (each half rounds like a scalar fmaf)
#pragma unroll
      for (int j = 0; j < C::CH; j += 2) {
        const float2 f = make_float2(static_cast<float>(static_cast<int32_t>(v[j])),
                                     static_cast<float>(static_cast<int32_t>(v[j + 1])));
        const float2 acc2 = __ffma2_rn(f, make_float2(s, s), make_float2(run[c0 + j], run[c0 + j + 1]));
        run[c0 + j] = acc2.x;
        run[c0 + j + 1] = acc2.y;
      }
    };
    // Group scales of this thread's weight row, [row tile][group][128] in memory.  A new 256-byte
    // run is touched every group, so loads are issued kScaleAhead groups early.  The ring holds
    // the raw fp16 bits: converting at load time would make the warp wait for the load at once;
    // the conversion happens when the group comes up.
    constexpr int kScaleAhead = 4;
    const unsigned short* sw_row = nullptr;
    unsigned short sq[kScaleAhead];
    // The accumulator of a group is read in chunks of 8 columns.  tcgen05.ld is asynchronous, so
    // chunk c + 1 is in flight while chunk c is scaled and added, and as soon as the accumulator
    // is drained the first chunk of the next group (of this tile or the next) is requested, if its
    // UMMAs have finished, before the last chunk of this one is consumed.
    uint32_t va[C::CH], vb[C::CH];
    bool prefetched = false;
    // One group; i = index inside the tile, gi = global index (rings and phases).  `sreg` is this
    // group's slot of the scale ring, refilled for group i + kScaleAhead right after it is read
    // (the loop below is unrolled by the ring size, so slots are registers with static indices).
    auto group_step = [&](int i, int gi, unsigned short& sreg) -> bool {
      const int b = gi % C::NB;
      const float s = __half2float(__ushort_as_half(sreg)) * 0.0625f;
      if (i + kScaleAhead < ng) sreg = __ldg(sw_row + static_cast<size_t>(i + kScaleAhead) * kBN);
      if (!prefetched) {
        if (!mbar_wait(&done[b], (gi / C::NB) & 1, abort_flag, SITE_EPI)) return false;
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
          if (lane == 0) mbar_arrive(&ready[b]);
          if constexpr (C::NCH > 1) {  // NCH is even: the next group's first chunk goes to va
            prefetched = false;
            if (gi + 1 < my_groups) {
              const int b1 = (gi + 1) % C::NB;
              // tcgen05.ld is warp-collective: take the early path only if every lane saw the phase
              if (__all_sync(0xffffffffu, mbar_test_wait(&done[b1], ((gi + 1) / C::NB) & 1) ? 1 : 0)) {
                tc_fence_after();
                ld_chunk(b1, 0, nxt);
                prefetched = true;
              }
            }
          }
        }
        consume(cur, c * C::CH, s);
      }
      return true;
    };
    bool ok = true;
    for (int it = 0; it < my_tiles && ok; ++it) {
      const int row_tile = tile_row(it);
      const int n = row_tile * kBN + q * 32 + lane;
      const int t0 = tile_tok(it) * TN;
#pragma unroll
      for (int j = 0; j < C::CPW; ++j) run[j] = 0.f;
      sw_row = reinterpret_cast<const unsigned short*>(sw_t) +
               (static_cast<size_t>(row_tile) * total_groups + g_begin) * kBN + q * 32 + lane;
#pragma unroll
      for (int d = 0; d < kScaleAhead; ++d) sq[d] = (d < ng) ? __ldg(sw_row + static_cast<size_t>(d) * kBN) : 0;
      for (int i0 = 0; i0 < ng && ok; i0 += kScaleAhead) {
#pragma unroll
        for (int u = 0; u < kScaleAhead; ++u) {
          if (ok && i0 + u < ng) ok = group_step(i0 + u, it * ng + i0 + u, sq[u]);
        }
      }
      if (!ok) break;
      if (split_k == 1) {
        if (n < N) {
          // One running pointer per thread (a 64-bit add per token instead of a multiply and the
          // m < M / dtype tests per element): these stores are on the epilogue warps' own chain.
          const float rn = (r != nullptr) ? r[n] : 1.f;
          const int m0 = t0 + h * C::CPW;
          const int cnt = (M - m0 < C::CPW) ? (M - m0) : C::CPW;  // tokens of this slice that exist
          const float* sxp = sx + m0;
          if (residual != nullptr) {
            size_t idx = static_cast<size_t>(m0) * N + n;
#pragma unroll
            for (int j = 0; j < C::CPW; ++j) {
              if (j < cnt) store_y(y, residual, y_bf16, idx, run[j] * (rn * __ldg(sxp + j)));
              idx += N;
            }
          } else if (y_bf16) {
            __nv_bfloat16* yp = reinterpret_cast<__nv_bfloat16*>(y) + static_cast<size_t>(m0) * N + n;
#pragma unroll
            for (int j = 0; j < C::CPW; ++j) {
              if (j < cnt) *yp = __float2bfloat16_rn(run[j] * (rn * __ldg(sxp + j)));
              yp += N;
            }
          } else {
            float* yp = reinterpret_cast<float*>(y) + static_cast<size_t>(m0) * N + n;
#pragma unroll
            for (int j = 0; j < C::CPW; ++j) {
              if (j < cnt) *yp = run[j] * (rn * __ldg(sxp + j));
              yp += N;
            }
          }
        }
      } else {
        // Partial tile -> this CTA's exchange buffer red[token][row] (aliases the stage buffers:
        // the last done[] wait above implies every UMMA, hence every smem operand read, is over).
        float* red = reinterpret_cast<float*>(smem);
#pragma unroll
        for (int j = 0; j < C::CPW; ++j) red[(h * C::CPW + j) * kBN + q * 32 + lane] = run[j];
      }
    }
  } else if (warp == C::kProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    // Weights do not depend on the preceding kernel of the stream; the activation codes do.
    // Fill the weight ring first (the unpack warps refill their stages themselves afterwards),
    // then wait for the prerequisite grid (programmatic dependent launch), then stream the
    // activation stages, up to SX stages of XC groups ahead of the UMMAs.
    const uint64_t pol_w = w_stream_once ? l2_policy_evict_first() : l2_policy_evict_last();
    const uint64_t pol_x = l2_policy_evict_last();
    // Only lane 0 works; the other lanes go straight to the end of the role (a waiting warp of
    // 32 polling lanes costs the SM issue slots and barrier-unit bandwidth the other roles need).
    if (lane == 0) {
      const int pre = (my_groups < C::SP) ? my_groups : C::SP;
      for (int gi = 0; gi < pre; ++gi) {
        mbar_expect_tx(&full_p[gi], kWpBytes);
        bulk_load_1d(smem + C::kOffP + gi * kWpBytes, w_group(gi), kWpBytes, &full_p[gi], pol_w);
      }
      grid_dep_wait();
      bool ok = true;
      for (int it = 0; it < my_tiles && ok; ++it) {
        const int t0 = tile_tok(it) * TN;
        for (int ix = 0; ix < nxs; ++ix) {
          const int xs = it * nxs + ix;  // global activation-stage index
          const int sxi = xs % C::SX;
          if (!mbar_wait(&empty_x[sxi], ((xs / C::SX) & 1) ^ 1, abort_flag, SITE_TMA)) { ok = false; break; }
          // one box = XC groups x TN tokens; groups past the end of K are zero-filled and still
          // counted, so the byte count is always that of the full box
          mbar_expect_tx(&full_x[sxi], C::kXStageBytes);
          tma_load_3d(smem + C::kOffX + sxi * C::kXStageBytes, &tm_x, 0, t0, g_begin + ix * C::XC,
                      &full_x[sxi], pol_x);
        }
      }
    }
  } else if (warp < C::kIssuerWarp0 + C::kIssuers) {
    // ------------------------------------------------------------------ UMMA issuer
    constexpr uint32_t idesc = umma_idesc_i8(kBN, TN);
    const uint32_t a_base = smem_u32(smem + C::kOffA);
    const uint32_t x_base = smem_u32(smem + C::kOffX);
    // The (global) groups alternate between the two issuing warps; accumulator b, buffer b and
    // the activation stage of a group are always waited for and released by the same warp.
    if (lane == 0) {  // only lane 0 works (see the producer)
      for (int gi = warp - C::kIssuerWarp0; gi < my_groups; gi += C::kIssuers) {
        const int it = gi / ng, i = gi % ng;  // tile iteration, group inside the tile
        const int b = gi % C::NB;
        const int xs = it * nxs + i / C::XC, xj = i % C::XC, sxi = xs % C::SX;
        if (!mbar_wait(&ready[b], (gi / C::NB) & 1, abort_flag, SITE_MMA_READY)) break;
        if (xj == 0 || C::kIssuers > 1) {
          if (!mbar_wait(&full_x[sxi], (xs / C::SX) & 1, abort_flag, SITE_MMA_X)) break;
        }
        tc_fence_after();
        const uint64_t da = umma_desc_k_sw128(a_base + b * kWaBytes);
        const uint64_t db = umma_desc_k_sw128(x_base + sxi * C::kXStageBytes + xj * C::kXBytes);
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(b * TN);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)  // +32 bytes along K inside the swizzle atom = +2 (>>4)
          umma_i8(d_tmem, da + 2 * kk, db + 2 * kk, idesc, kk > 0 ? 1u : 0u);
        umma_commit(&done[b]);
        if (xj == C::XC - 1 || i == ng - 1) umma_commit(&empty_x[sxi]);
      }
    }
  }

  // -------------------------------------------------------------------- split-K reduction
  if (split_k > 1) {
    __syncwarp();
    cluster_sync_all();
    if (warp >= kUnpackWarps && warp < kUnpackWarps + 8) {
      const int n0 = tile_row(0) * kBN, t0 = tile_tok(0) * TN;  // split-K: one tile per CTA
      const uint32_t rank = cluster_ctarank();
      const int rows = TN / split_k;  // token rows of the tile this CTA finishes
      const int e = tid - 4 * 32;     // 0..255
      const int c4 = e & 31;          // float4 column
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
          const float sm = sx[m];
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
  if (warp == C::kIssuerWarp0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
  if (tid == 0 && *abort_flag != 0) atomicCAS(status, 0, *abort_flag);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template <int TN>
static int set_attr() {
  cudaError_t e = cudaFuncSetAttribute(gemm_w4a4_int4_kernel<TN>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg<TN>::kSmemBytes);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "cudaFuncSetAttribute(gemm TN=%d) failed: %s", TN,
                     cudaGetErrorString(e));
  return DQ_OK;
}

int init_gemm_int4_kernels() {
  int rc;
  if ((rc = set_attr<16>()) != DQ_OK) return rc;
  if ((rc = set_attr<32>()) != DQ_OK) return rc;
  if ((rc = set_attr<64>()) != DQ_OK) return rc;
  if ((rc = set_attr<128>()) != DQ_OK) return rc;
  return DQ_OK;
}

static int pick_token_tile(int M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  return 128;
}

// Smallest power-of-two split (<= 8, <= TN so every rank finishes at least one token row, and
// leaving at least two groups per CTA) that fills roughly 60% of the CTA slots of the machine;
// beyond that the cluster reduction costs more than the extra CTAs bring (measured on the
// Llama-3.1-8B shapes).
static int pick_split(int tiles, int total_groups, int tn, int sm_count) {
  const int target = (sm_count * ((tn <= 64) ? 2 : 1) * 6) / 10;
  int s = 1;
  while (s < 8 && tiles * s < target && total_groups / (2 * s) >= 2 && 2 * s <= tn) s *= 2;
  return s;
}

template <int TN>
static int launch(const int8_t* codes, const float* sx, const uint8_t* w_packed, const __half* sw_t,
                  const float* r, int M, int N, int K, void* y, int y_dtype, int split,
                  cudaStream_t stream, DeviceState* st, const void* residual) {
  CUtensorMap tm_x;
  int rc = make_tmap_x_groups(&tm_x, codes, K, M, TN, Cfg<TN>::XC);
  if (rc != DQ_OK) return rc;

  const int total_groups = K / kGroup;
  const int gps = (total_groups + split - 1) / split;
  const int tok_tiles = (M + TN - 1) / TN;
  cudaLaunchConfig_t cfg = {};
  const int row_tiles = (N + kBN - 1) / kBN;
  if (split == 1) {
    // persistent: one CTA per slot of the machine, each walks the tile list with that stride
    const int slots = st->sm_count * Cfg<TN>::kMinCtas;
    const int tiles = row_tiles * tok_tiles;
    cfg.gridDim = dim3(tiles < slots ? tiles : slots, 1, 1);
  } else {
    cfg.gridDim = dim3(row_tiles, tok_tiles, split);
  }
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
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_w4a4_int4_kernel<TN>, w_packed, tm_x, sw_t, r, sx,
                                     y, y_dtype == DQ_DTYPE_BF16 ? 1 : 0, residual, M, N, K, gps,
                                     split, w_stream_once, st->status_dev);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "gemm_w4a4_int4 launch failed (TN=%d split=%d): %s", TN, split,
                     cudaGetErrorString(e));
  return DQ_OK;
}

static int check_gemm_args(const void* codes, const void* w_packed, int M, int N, int K, int G) {
  DQ_REQUIRE(codes != nullptr && w_packed != nullptr, DQ_ERR_NULL, "null operand pointer");
  DQ_REQUIRE(G == kGroup, DQ_ERR_UNSUPPORTED, "weight group size must be %d (got %d)", kGroup, G);
  DQ_REQUIRE(M >= 1 && N >= 1 && K >= kGroup, DQ_ERR_SHAPE, "bad shape M=%d N=%d K=%d", M, N, K);
  DQ_REQUIRE(K % kGroup == 0, DQ_ERR_SHAPE, "K=%d must be a multiple of %d", K, kGroup);
  DQ_REQUIRE(aligned(codes, 16) && aligned(w_packed, 16), DQ_ERR_ALIGN,
             "codes and w_packed must be 16-byte aligned");
  return DQ_OK;
}

}  // namespace dq

using namespace dq;

extern "C" size_t dq_gemm_w4a4_int4_workspace_bytes(int, int, int) { return 0; }

static int gemm_int4_dispatch(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                              const void* sw_t, const float* r, const void* residual, int M, int N,
                              int K, int G, void* y, int y_dtype, void* stream, int token_tile,
                              int split_k, bool grouped_sx = false) {
  DeviceState* st = current_state();
  if (st == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  int rc = check_gemm_args(codes, w_packed, M, N, K, G);
  if (rc != DQ_OK) return rc;
  DQ_REQUIRE(sx != nullptr && sw_t != nullptr && y != nullptr, DQ_ERR_NULL, "null sx / sw_t / y");
  DQ_REQUIRE(y_dtype == DQ_DTYPE_F32 || y_dtype == DQ_DTYPE_BF16, DQ_ERR_UNSUPPORTED,
             "unknown y_dtype %d", y_dtype);
  DQ_REQUIRE(aligned(sw_t, 16), DQ_ERR_ALIGN, "sw_t must be 16-byte aligned");
  const int total_groups = K / kGroup;
  // token_tile: 0 = choose; 16/32/64/128 = tensor-memory kernel with that token tile;
  // -8/-16/-32 = register-path decode kernel with that token capacity.
  const bool decode_path = token_tile < 0 || (token_tile == 0 && M <= 16);
  if (decode_path) {
    const int tok = token_tile < 0 ? -token_tile : (M <= 8 ? 8 : 16);
    DQ_REQUIRE((tok == 8 || tok == 16 || tok == 32) && M <= tok, DQ_ERR_SHAPE,
               "decode kernel token capacity %d does not cover M=%d", tok, M);
    const int tiles_n = (N + kBN - 1) / kBN;
    int split = split_k ? split_k : gemv_pick_split(tiles_n, total_groups, tok, st->sm_count);
    DQ_REQUIRE(split == 1 || split == 2 || split == 4 || split == 8, DQ_ERR_SHAPE,
               "split_k must be 1/2/4/8 (got %d)", split);
    DQ_REQUIRE(split <= tok && split <= total_groups, DQ_ERR_SHAPE,
               "split_k=%d too large for %d tokens / %d groups", split, tok, total_groups);
    return launch_gemv_int4(codes, sx, w_packed, sw_t, r, M, N, K, y, y_dtype, tok, split,
                            static_cast<cudaStream_t>(stream), st, nullptr, residual, grouped_sx);
  }
  // 1000 + tile / 2000 + tile force the shared-memory-operand / tensor-memory-operand kernel
  int forced = 0;
  if (token_tile >= 2000) { forced = 2; token_tile -= 2000; }
  else if (token_tile >= 1000) { forced = 1; token_tile -= 1000; }
  const int tn = token_tile ? token_tile : pick_token_tile(M);
  DQ_REQUIRE(tn == 16 || tn == 32 || tn == 64 || tn == 128, DQ_ERR_SHAPE,
             "token tile must be 16/32/64/128 (got %d)", tn);
  const int tiles = ((N + kBN - 1) / kBN) * ((M + tn - 1) / tn);
  int split = split_k ? split_k : pick_split(tiles, total_groups, tn, st->sm_count);
  DQ_REQUIRE(split == 1 || split == 2 || split == 4 || split == 8, DQ_ERR_SHAPE,
             "split_k must be 1/2/4/8 (got %d)", split);
  DQ_REQUIRE(split <= tn && split <= total_groups, DQ_ERR_SHAPE,
             "split_k=%d too large for token tile %d / %d groups", split, tn, total_groups);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __half* swp = static_cast<const __half*>(sw_t);
  // Two tcgen05 kernels.  Token tiles up to 64 (weight-streaming regime, two CTAs per SM): the
  // kernel that feeds the weights to the tensor core from tensor memory, which leaves all shared
  // memory to the copy rings.  Token tile 128 (prefill): the kernel with int8 weight tiles in
  // shared memory, four accumulators and two issuing warps, measured 10-15 % faster there.
  // (the per-group activation-scale variant exists in the tensor-memory-operand kernel only)
  const bool use_tm = grouped_sx || (forced ? (forced == 2) : (tn <= 64));
  if (use_tm)
    return launch_gemm_int4_tm(codes, sx, w_packed, sw_t, r, M, N, K, y, y_dtype, nullptr, tn, split, s, st,
                               residual, grouped_sx);
  switch (tn) {
    case 16: return launch<16>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, split, s, st, residual);
    case 32: return launch<32>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, split, s, st, residual);
    case 64: return launch<64>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, split, s, st, residual);
    default: return launch<128>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, split, s, st, residual);
  }
}

extern "C" int dq_gemm_w4a4_int4_ex(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                                    const void* sw_t, const float* r, int M, int N, int K, int G,
                                    void* y, int y_dtype, void* /*workspace*/,
                                    size_t /*workspace_bytes*/, void* stream, int token_tile,
                                    int split_k) {
  return gemm_int4_dispatch(codes, sx, w_packed, sw_t, r, nullptr, M, N, K, G, y, y_dtype, stream,
                            token_tile, split_k);
}

extern "C" int dq_gemm_w4a4_int4_residual(const int8_t* codes, const float* sx,
                                          const uint8_t* w_packed, const void* sw_t, const float* r,
                                          const void* residual, int M, int N, int K, int G, void* y,
                                          int y_dtype, void* stream) {
  DQ_REQUIRE(residual != nullptr, DQ_ERR_NULL, "null residual");
  DQ_REQUIRE(aligned(residual, y_dtype == DQ_DTYPE_BF16 ? 2 : 4), DQ_ERR_ALIGN, "misaligned residual");
  return gemm_int4_dispatch(codes, sx, w_packed, sw_t, r, residual, M, N, K, G, y, y_dtype, stream, 0, 0);
}

extern "C" int dq_gemm_w4a4_int4_grouped(const int8_t* codes, const float* sx_groups,
                                         const uint8_t* w_packed, const void* sw_t, const float* r,
                                         int M, int N, int K, int G, void* y, int y_dtype,
                                         void* stream) {
  return gemm_int4_dispatch(codes, sx_groups, w_packed, sw_t, r, nullptr, M, N, K, G, y, y_dtype, stream,
                            0, 0, true);
}

extern "C" int dq_gemm_w4a4_int4(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                                 const void* sw_t, const float* r, int M, int N, int K, int G,
                                 void* y, int y_dtype, void* workspace, size_t workspace_bytes,
                                 void* stream) {
  return dq_gemm_w4a4_int4_ex(codes, sx, w_packed, sw_t, r, M, N, K, G, y, y_dtype, workspace,
                              workspace_bytes, stream, 0, 0);
}

extern "C" int dq_gemm_w4a4_int4_acc(const int8_t* codes, const uint8_t* w_packed, int M, int N,
                                     int K, int G, int32_t* acc, void* stream) {
  DeviceState* st = current_state();
  if (st == nullptr) return DQ_ERR_NOT_INIT;
  int rc = check_gemm_args(codes, w_packed, M, N, K, G);
  if (rc != DQ_OK) return rc;
  DQ_REQUIRE(acc != nullptr, DQ_ERR_NULL, "null acc");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return launch_gemm_int4_tm(codes, nullptr, w_packed, nullptr, nullptr, M, N, K, nullptr, DQ_DTYPE_F32,
                             acc, M <= 16 ? 16 : 128, 1, s, st);
}

extern "C" int dq_gemm_w4a4_int4_ar_residual(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                                             const void* sw_t, const float* r, const void* residual, int M, int N,
                                             int K, int G, void* y, int y_dtype, void* stream,
                                             const dq_allreduce_ctx* ctx);

extern "C" int dq_gemm_w4a4_int4_ar(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                                    const void* sw_t, const float* r, int M, int N, int K, int G,
                                    void* y, int y_dtype, void* stream,
                                    const dq_allreduce_ctx* ctx) {
  return dq_gemm_w4a4_int4_ar_residual(codes, sx, w_packed, sw_t, r, nullptr, M, N, K, G, y, y_dtype, stream, ctx);
}

extern "C" int dq_gemm_w4a4_int4_ar_residual(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                                             const void* sw_t, const float* r, const void* residual, int M, int N,
                                             int K, int G, void* y, int y_dtype, void* stream,
                                             const dq_allreduce_ctx* ctx) {
  DeviceState* st = current_state();
  if (st == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  int rc = check_gemm_args(codes, w_packed, M, N, K, G);
  if (rc != DQ_OK) return rc;
  DQ_REQUIRE(sx != nullptr && sw_t != nullptr && y != nullptr, DQ_ERR_NULL, "null sx / sw_t / y");
  DQ_REQUIRE(M <= 16, DQ_ERR_UNSUPPORTED, "the fused all-reduce covers decode batches (M <= 16), got M=%d", M);
  const int tok = (M <= 8) ? 8 : 16;
  const int total_groups = K / kGroup;
  const int split = gemv_pick_split((N + kBN - 1) / kBN, total_groups, tok, st->sm_count);
  return launch_gemv_int4(codes, sx, w_packed, sw_t, r, M, N, K, y, y_dtype, tok, split,
                          static_cast<cudaStream_t>(stream), st, ctx, residual);
}
