// W4A4 int4 dual-scale linear for decode batches (M <= 32 tokens) on sm_100a.
//
// Same arithmetic and the same weight artefact as gemm_w4a4_int4.cu, different machine mapping.
// With a handful of tokens the job is to stream the packed weights out of HBM once, so this
// kernel is built around bytes in flight rather than around the tensor memory pipeline:
//
//   * one producer warp keeps a ring of stages full; a stage is two consecutive weight groups of
//     the CTA's 128 rows - 2 x (8 KB of packed int4 + 256 B of fp16 group scales), contiguous in
//     memory and fetched by ONE bulk copy - plus the int8 activation codes of those groups
//     (one tiled copy);
//     the ring depth is chosen at launch so that the CTAs sharing an SM together keep
//     well over 100 KB of weights in flight (throughput = bytes in flight / HBM latency);
//   * eight compute warps, each owning 16 weight rows.  A lane reads its packed nibbles straight
//     from the stage (two 16-byte loads), splits them in registers ((w << 4) & 0xF0.. and
//     w & 0xF0.., i.e. 16 * code, the 1/16 folded into the group scale) and feeds
//     mma.sync.m16n8k32.s8 with int32 accumulation per group - no second shared-memory pass,
//     no cross-warp hand-off on the critical path.  The k order inside a group is permuted
//     identically for weights and activations (a dot product does not care);
//   * per group: acc -> fp32, times the group scale, added to a running fp32 sum; at the end
//     times r[n] * sx[m].  Split-K partial tiles are reduced across the thread-block cluster
//     through distributed shared memory in rank order (deterministic, no global scratch).
#include "dq_common.h"
#include "dq_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace dq {

constexpr int kVBN = 128;       // weight rows per CTA
constexpr int kVSets = 1;  // warp sets that split the groups of a stage between them (1 or 2)
constexpr int kVComputeWarps = 8 * kVSets;
constexpr int kVThreads = (kVComputeWarps + 1) * 32;  // + 1 producer warp
constexpr int kVGS = 2;         // weight groups per pipeline stage

template <int NT>  // NT = number of 8-token blocks (tokens handled: 8 * NT)
struct VCfg {
  static constexpr int TOK = 8 * NT;
  static constexpr int kXRows = (TOK < 16) ? 16 : TOK;       // rows of the activation tile box
  // Activation codes of a stage: [group][token row][128 B], 128-byte swizzle (one 3-D TMA box).
  // Swizzled because token rows 128 bytes apart would otherwise put the 16-byte fragment loads
  // of lanes with different token index on the same banks.
  static constexpr int kXGroupBytes = kXRows * kGroup;
  static constexpr int kXBytes = kVGS * kXGroupBytes;
  static constexpr int kOffX = 0;
  static constexpr int kOffW = kXBytes;                       // kVGS tiles of kTileBytes
  static constexpr int kStage = (kOffW + kVGS * kTileBytes + 1023) / 1024 * 1024;  // swizzle atoms: 1 KB
  // The ring depth is a launch parameter: the host gives each CTA as many stages as fit next to
  // the other CTAs expected on its SM, because throughput here is (bytes in flight) / (HBM latency).
  static constexpr int kMinStages = 2;
  static constexpr int kMaxStages = 10;
  static constexpr int kMinCtas = (kVSets == 1) ? ((NT == 1) ? 4 : (NT == 2) ? 3 : 2) : ((NT <= 2) ? 2 : 1);
  static constexpr int kBarBytes = 2 * kMaxStages * 8 + 16;
  static_assert(TOK * kVBN * 4 <= kMinStages * kStage, "split-K exchange tile must fit in the ring");
  static constexpr int smem_bytes(int stages) { return stages * kStage + kBarBytes + 1024; }
};

enum { VSITE_PRODUCER = 21, VSITE_COMPUTE = 22, VSITE_ALLREDUCE = 23 };

// Cross-GPU all-reduce fused into the epilogue (row-parallel linears under tensor parallelism).
// Every rank runs the same launch on its K slice.  A CTA that has finished its rows of an output
// tile writes them (already scaled by r[n] * sx[m]) to its rank's exchange buffer, raises a flag
// on every peer, waits - bounded - for the peers' flags of the same (tile, split) unit, then sums
// the ranks' contributions in rank order through plain peer loads and stores the final rows.
// Buffers alternate with the parity of a per-rank call counter that a one-thread kernel bumps
// after each launch, so a rank that is already in the next call never overwrites data a slower
// peer is still reading.  No NCCL, no multicast; the waits give up after about half a second.
struct ArDev {
  float* bufs[8];        // exchange buffer of every rank (2 * cap floats each), peer-mapped
  uint32_t* flags[8];    // flag array of every rank: [unit][8]
  const uint32_t* seq;   // this rank's call counter
  int rank, world;
  uint32_t cap;          // floats per parity half
  long long wait_cycles; // how long a peer's flag is waited for before the kernel gives up
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_relaxed_sys_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__global__ void ar_bump_kernel(uint32_t* seq) { *seq = *seq + 1u; }

__device__ __forceinline__ void mma_s8_16x8x32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// GS: one activation scale per (token, weight group) - sx is then [K / 128][M], group-major - instead
// of one per token.
template <int NT, bool GS>
__global__ void __launch_bounds__(kVThreads, VCfg<NT>::kMinCtas)
gemv_w4a4_int4_kernel(const uint8_t* __restrict__ w_packed,
                      const __grid_constant__ CUtensorMap tm_x,
                      const float* __restrict__ r, const float* __restrict__ sx,
                      void* __restrict__ y, int y_bf16, const void* __restrict__ residual, int M, int N,
                      int K, int groups_per_split, int split_k, int stages, int* status, const ArDev ar) {
  using C = VCfg<NT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + stages * C::kStage);
  uint64_t* empty = full + C::kMaxStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + C::kMaxStages);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n0 = blockIdx.x * kVBN;
  const int total_groups = K / kGroup;
  const int g_begin = blockIdx.z * groups_per_split;
  int g_end = g_begin + groups_per_split;
  if (g_end > total_groups) g_end = total_groups;
  const int ng = (g_end > g_begin) ? (g_end - g_begin) : 0;
  const int nst = (ng + kVGS - 1) / kVGS;  // pipeline stages this CTA walks through

  if (tid == 0) {
    for (int i = 0; i < stages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], kVComputeWarps); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kVComputeWarps && lane == 0) tma_prefetch_desc(&tm_x);
  grid_dep_launch_dependents();
  __syncthreads();

  if (warp == kVComputeWarps) {
    // ------------------------------------------------------------------ producer warp
    // Per stage: one bulk copy (codes + scales of up to kVGS consecutive groups, contiguous in
    // memory) and one tiled copy of the activation codes.  Every asynchronous-copy instruction
    // costs this warp tens of cycles of issue latency, so a stage is made as large as practical.
    const uint64_t pol_w = l2_policy_evict_first();
    const uint64_t pol_x = l2_policy_evict_last();
    const uint8_t* w_src =
        w_packed + (static_cast<size_t>(blockIdx.x) * total_groups + g_begin) * kTileBytes;
    // The weights do not depend on the preceding kernel of the stream, the activation codes do
    // (they come from the quantiser): fill the ring with weights first, then wait for the
    // prerequisite grid, then fetch the activation tiles of those stages.
    const int prefill = (nst < stages) ? nst : stages;
    // Only lane 0 works; the other lanes go straight to the end of the role (32 lanes polling a
    // barrier cost issue slots and barrier-unit bandwidth that the compute warps need).
    if (lane == 0) {
      for (int i = 0; i < prefill; ++i) {
        uint8_t* st = smem + i * C::kStage;
        int cnt = ng - i * kVGS;
        if (cnt > kVGS) cnt = kVGS;
        const uint32_t wbytes = static_cast<uint32_t>(cnt) * kTileBytes;
        mbar_expect_tx(&full[i], wbytes + C::kXBytes);
        bulk_load_1d(st + C::kOffW, w_src + static_cast<size_t>(i) * kVGS * kTileBytes, wbytes,
                     &full[i], pol_w);
      }
      grid_dep_wait();
      for (int i = 0; i < prefill; ++i)
        tma_load_3d(smem + i * C::kStage + C::kOffX, &tm_x, 0, 0, g_begin + i * kVGS, &full[i], pol_x);
      int s = (prefill == stages) ? 0 : prefill;
      uint32_t ph = (prefill == stages) ? 0u : 1u;  // parity of the "stage is free" phase waited for
      for (int i = prefill; i < nst; ++i) {
        if (!mbar_wait(&empty[s], ph, abort_flag, VSITE_PRODUCER)) break;
        uint8_t* st = smem + s * C::kStage;
        int cnt = ng - i * kVGS;
        if (cnt > kVGS) cnt = kVGS;
        const uint32_t wbytes = static_cast<uint32_t>(cnt) * kTileBytes;
        mbar_expect_tx(&full[s], wbytes + C::kXBytes);
        bulk_load_1d(st + C::kOffW, w_src + static_cast<size_t>(i) * kVGS * kTileBytes, wbytes,
                     &full[s], pol_w);
        tma_load_3d(st + C::kOffX, &tm_x, 0, 0, g_begin + i * kVGS, &full[s], pol_x);
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    const int g = lane >> 2;  // fragment row / token index inside an 8-block
    const int t = lane & 3;
    const int set = warp >> 3;      // which group of each stage this warp works on
    const int row = (warp & 7) * 16 + g;  // local weight row (and row + 8)
    float run[NT][4];
#pragma unroll
    for (int nb = 0; nb < NT; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) run[nb][e] = 0.f;

    int s = 0;
    uint32_t ph = 0;
    for (int i = 0; i < nst; ++i) {
      if (!mbar_wait(&full[s], ph, abort_flag, VSITE_COMPUTE)) break;
      const uint8_t* st = smem + s * C::kStage;
      int cnt = ng - i * kVGS;
      if (cnt > kVGS) cnt = kVGS;
      // with two warp sets, warps 0-7 take the first group of the stage and warps 8-15 the second
#pragma unroll
      for (int gi = set; gi < kVGS; gi += kVSets) {
        if (gi >= cnt) break;
        const uint8_t* tile = st + C::kOffW + gi * kTileBytes;
        // k chunk t of rows `row` and `row + 8` (chunk positions are swizzled by (row >> 1) & 3,
        // the same value for both rows)
        const int tp = t ^ ((g >> 1) & 3);
        const uint4 wa = *reinterpret_cast<const uint4*>(tile + row * 64 + tp * 16);
        const uint4 wb = *reinterpret_cast<const uint4*>(tile + (row + 8) * 64 + tp * 16);
        const __half* sc = reinterpret_cast<const __half*>(tile + kTileCodeBytes);
        const float s0 = __half2float(sc[row]) * 0.0625f;
        const float s1 = __half2float(sc[row + 8]) * 0.0625f;
        uint4 xlo[NT], xhi[NT];
#pragma unroll
        for (int nb = 0; nb < NT; ++nb) {
          // activation codes: [group][token][128 B]; 16-byte chunk c of token row m sits at
          // chunk position c ^ (m & 7) (128-byte swizzle); this lane needs chunks 2t and 2t + 1
          const uint8_t* xr = st + C::kOffX + gi * C::kXGroupBytes + (nb * 8 + g) * kGroup;
          xlo[nb] = *reinterpret_cast<const uint4*>(xr + (((2 * t) ^ g) << 4));
          xhi[nb] = *reinterpret_cast<const uint4*>(xr + (((2 * t + 1) ^ g) << 4));
        }
        // Word j of a lane's 16-byte chunk feeds MMA step j: low nibbles are
        // k = 32t + 4j + {0..3} of the group (fragment slots a0/a1), high nibbles
        // k = 32t + 16 + 4j + {0..3} (a2/a3).
        const uint32_t wav[4] = {wa.x, wa.y, wa.z, wa.w};
        const uint32_t wbv[4] = {wb.x, wb.y, wb.z, wb.w};
        int c[NT][2][4];  // two partial accumulators per token block: dependent chains of 2 MMAs
#pragma unroll
        for (int nb = 0; nb < NT; ++nb)
#pragma unroll
          for (int e = 0; e < 4; ++e) { c[nb][0][e] = 0; c[nb][1][e] = 0; }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t a0 = (wav[j] << 4) & 0xF0F0F0F0u;
          const uint32_t a2 = wav[j] & 0xF0F0F0F0u;
          const uint32_t a1 = (wbv[j] << 4) & 0xF0F0F0F0u;
          const uint32_t a3 = wbv[j] & 0xF0F0F0F0u;
#pragma unroll
          for (int nb = 0; nb < NT; ++nb) {
            const uint32_t b0 = (j == 0) ? xlo[nb].x : (j == 1) ? xlo[nb].y : (j == 2) ? xlo[nb].z : xlo[nb].w;
            const uint32_t b1 = (j == 0) ? xhi[nb].x : (j == 1) ? xhi[nb].y : (j == 2) ? xhi[nb].z : xhi[nb].w;
            mma_s8_16x8x32(c[nb][j & 1], a0, a1, a2, a3, b0, b1);
          }
        }
#pragma unroll
        for (int nb = 0; nb < NT; ++nb) {
          float xa = 1.f, xb = 1.f;  // activation scales of tokens 2t, 2t + 1 of this block
          if constexpr (GS) {
            const float* sg = sx + static_cast<size_t>(g_begin + i * kVGS + gi) * M;
            const int m = nb * 8 + 2 * t;
            xa = __ldg(sg + (m < M ? m : M - 1));
            xb = __ldg(sg + (m + 1 < M ? m + 1 : M - 1));
          }
          run[nb][0] = fmaf(static_cast<float>(c[nb][0][0] + c[nb][1][0]), GS ? __fmul_rn(s0, xa) : s0, run[nb][0]);
          run[nb][1] = fmaf(static_cast<float>(c[nb][0][1] + c[nb][1][1]), GS ? __fmul_rn(s0, xb) : s0, run[nb][1]);
          run[nb][2] = fmaf(static_cast<float>(c[nb][0][2] + c[nb][1][2]), GS ? __fmul_rn(s1, xa) : s1, run[nb][2]);
          run[nb][3] = fmaf(static_cast<float>(c[nb][0][3] + c[nb][1][3]), GS ? __fmul_rn(s1, xb) : s1, run[nb][3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
      if (++s == stages) { s = 0; ph ^= 1u; }
    }

    // Fold the second warp set's partial sums into the first through shared memory.  All compute
    // warps are past their last stage at the first barrier, so the ring can be reused.
    if constexpr (kVSets == 2) {
      float* red = reinterpret_cast<float*>(smem);
      asm volatile("bar.sync 1, 512;" ::: "memory");
      if (set == 1) {
#pragma unroll
        for (int nb = 0; nb < NT; ++nb)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int m = nb * 8 + 2 * t + e;
            red[m * kVBN + row] = run[nb][e];
            red[m * kVBN + row + 8] = run[nb][2 + e];
          }
      }
      asm volatile("bar.sync 1, 512;" ::: "memory");
      if (set == 0) {
#pragma unroll
        for (int nb = 0; nb < NT; ++nb)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int m = nb * 8 + 2 * t + e;
            run[nb][e] += red[m * kVBN + row];
            run[nb][2 + e] += red[m * kVBN + row + 8];
          }
      }
    }
    // accumulator fragment: c0/c1 = (row, tokens 2t, 2t+1), c2/c3 = (row + 8, same tokens)
    if constexpr (kVSets == 1) {
      if (split_k > 1 || ar.world > 1) asm volatile("bar.sync 1, 256;" ::: "memory");  // ring reused as exchange tile
    }
    if (set == 1) {
      // nothing left to do for the second set
    } else if (split_k == 1 && ar.world <= 1) {
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        const int n = n0 + row + 8 * hrow;
        if (n < N) {
          const float rn = (r != nullptr) ? r[n] : 1.f;
#pragma unroll
          for (int nb = 0; nb < NT; ++nb)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int m = nb * 8 + 2 * t + e;
              if (m < M) {
                store_y(y, residual, y_bf16, static_cast<size_t>(m) * N + n, run[nb][2 * hrow + e] * (GS ? rn : rn * sx[m]));
              }
            }
        }
      }
    } else {
      // each thread overwrites exactly the exchange-tile entries it has just read
      float* red = reinterpret_cast<float*>(smem);
#pragma unroll
      for (int nb = 0; nb < NT; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int m = nb * 8 + 2 * t + e;
          red[m * kVBN + row] = run[nb][e];
          red[m * kVBN + row + 8] = run[nb][2 + e];
        }
    }
  }

  // -------------------------------------------------------------------- split-K / cross-GPU reduction
  if (split_k > 1 || ar.world > 1) {
    __syncwarp();
    cluster_sync_all();
    if (warp < 8) {  // 256 threads finish this CTA's share of the tile
      const uint32_t crank = cluster_ctarank();
      const int rows = C::TOK / split_k;  // token rows of the tile this CTA finishes
      const int c4 = tid & 31;            // float4 column
      const uint32_t red_base = smem_u32(smem);
      uint32_t seq = 0;
      float* my_buf = nullptr;
      if (ar.world > 1) {
        grid_dep_wait();  // the call counter is bumped by the kernel before this one's prerequisites
        seq = *ar.seq;
        my_buf = ar.bufs[ar.rank] + static_cast<size_t>(seq & 1u) * ar.cap;
      }
      for (int rr = tid >> 5; rr < rows; rr += 8) {
        const int m = static_cast<int>(crank) * rows + rr;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const uint32_t off = static_cast<uint32_t>((m * kVBN + c4 * 4) * 4);
        for (int p = 0; p < split_k; ++p) {
          const float4 v = dsmem_ld_f4(dsmem_map(red_base + off, static_cast<uint32_t>(p)));
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if (m < M) {
          const float sm = GS ? 1.f : sx[m];
          float vals[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int n = n0 + c4 * 4 + u;
            const float rn = (n < N && r != nullptr) ? r[n] : 1.f;
            vals[u] = (n < N) ? vals[u] * (rn * sm) : 0.f;
          }
          if (ar.world > 1) {
            // N is a multiple of 4 in this mode (checked on the host): aligned float4 store
            if (n0 + c4 * 4 < N)
              *reinterpret_cast<float4*>(my_buf + static_cast<size_t>(m) * N + n0 + c4 * 4) =
                  make_float4(vals[0], vals[1], vals[2], vals[3]);
          } else {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int n = n0 + c4 * 4 + u;
              if (n < N) store_y(y, residual, y_bf16, static_cast<size_t>(m) * N + n, vals[u]);
            }
          }
        }
      }
      if (ar.world > 1) {
        const uint32_t epoch = seq + 1u;
        const uint32_t unit = blockIdx.x * static_cast<uint32_t>(split_k) + crank;
        asm volatile("bar.sync 1, 256;" ::: "memory");  // all rows of this CTA are in the buffer
        if (tid == 0) {
          __threadfence_system();
          for (int p = 0; p < ar.world; ++p)
            if (p != ar.rank) st_release_sys(ar.flags[p] + unit * 8u + ar.rank, epoch);
        }
        if (tid < ar.world && tid != ar.rank) {
          const uint32_t* f = ar.flags[ar.rank] + unit * 8u + tid;
          const long long t_start = clock64();
          while (static_cast<int32_t>(ld_acquire_sys(f) - epoch) < 0) {
            if (clock64() - t_start > ar.wait_cycles || *abort_flag != 0) {
              *abort_flag = VSITE_ALLREDUCE;
              break;
            }
          }
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (*abort_flag == 0) {
          for (int rr = tid >> 5; rr < rows; rr += 8) {
            const int m = static_cast<int>(crank) * rows + rr;
            const int nb = n0 + c4 * 4;
            if (m < M && nb < N) {
              float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
              for (int p = 0; p < ar.world; ++p) {  // rank order: every rank forms the same sum
                const float* src = ar.bufs[p] + static_cast<size_t>(seq & 1u) * ar.cap +
                                   static_cast<size_t>(m) * N + nb;
                const float4 v = ld_relaxed_sys_f4(src);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
              }
              const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
              for (int u = 0; u < 4; ++u) store_y(y, residual, y_bf16, static_cast<size_t>(m) * N + nb + u, vals[u]);
            }
          }
        }
      }
    }
    __syncwarp();
    cluster_sync_all();  // peers may still be reading this CTA's exchange tile until here
  }
  __syncthreads();
  if (tid == 0 && *abort_flag != 0) atomicCAS(status, 0, *abort_flag);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template <int NT>
static int set_gemv_attr() {
  cudaError_t e = cudaFuncSetAttribute(gemv_w4a4_int4_kernel<NT, false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(gemv_w4a4_int4_kernel<NT, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "cudaFuncSetAttribute(gemv NT=%d) failed: %s", NT,
                     cudaGetErrorString(e));
  return DQ_OK;
}

int init_gemv_int4_kernels() {
  int rc;
  if ((rc = set_gemv_attr<1>()) != DQ_OK) return rc;
  if ((rc = set_gemv_attr<2>()) != DQ_OK) return rc;
  if ((rc = set_gemv_attr<4>()) != DQ_OK) return rc;
  return DQ_OK;
}

// Smallest power-of-two split that gives roughly one CTA per SM (measured optimum on the
// Llama-3.1-8B decode shapes: more splits cost more in cluster exchange than they win).
int gemv_pick_split(int tiles, int total_groups, int tok, int sm_count) {
  int s = 1;
  while (s < 8 && tiles * s * 6 < sm_count * 5 && total_groups / (2 * s) >= 2 && 2 * s <= tok) s *= 2;
  return s;
}

template <int NT, bool GS>
static int launch_gemv_t(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                         const __half* sw_t, const float* r, int M, int N, int K, void* y,
                         int y_dtype, int split, cudaStream_t stream, DeviceState* st,
                         const ArDev& ar, const void* residual) {
  using C = VCfg<NT>;
  CUtensorMap tm_x;
  int rc = make_tmap_x_groups(&tm_x, codes, K, M, C::kXRows, kVGS);
  if (rc != DQ_OK) return rc;
  const int total_groups = K / kGroup;
  const int gps = (total_groups + split - 1) / split;
  const int tiles_n = (N + kVBN - 1) / kVBN;
  // stages: share the SM's shared memory between the CTAs expected to be co-resident
  int per_sm = (tiles_n * split + st->sm_count - 1) / st->sm_count;
  if (per_sm > C::kMinCtas) per_sm = C::kMinCtas;
  if (per_sm < 1) per_sm = 1;
  const int avail = (227 * 1024) / per_sm - 1024 - C::kBarBytes - 1024;
  int stages = avail / C::kStage;
  if (stages > C::kMaxStages) stages = C::kMaxStages;
  if (stages > (gps + kVGS - 1) / kVGS) stages = (gps + kVGS - 1) / kVGS;
  if (stages < C::kMinStages) stages = C::kMinStages;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles_n, 1, split);
  cfg.blockDim = dim3(kVThreads, 1, 1);
  cfg.dynamicSmemBytes = C::smem_bytes(stages);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = split;
  // programmatic dependent launch: the kernel may start (and stream weights) while the kernel
  // before it in the stream is still running; it executes griddepcontrol.wait before it reads
  // anything that kernel could have produced
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_w4a4_int4_kernel<NT, GS>, w_packed, tm_x, r, sx, y,
                                     y_dtype == DQ_DTYPE_BF16 ? 1 : 0, residual, M, N, K, gps, split,
                                     stages, st->status_dev, ar);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "gemv_w4a4_int4 launch failed (tokens=%d split=%d): %s", C::TOK,
                     split, cudaGetErrorString(e));
  return DQ_OK;
}

// tok: token capacity of the variant (8, 16 or 32) >= M.
int launch_gemv_int4(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                     const void* sw_t, const float* r, int M, int N, int K, void* y, int y_dtype,
                     int tok, int split, cudaStream_t stream, DeviceState* st,
                     const dq_allreduce_ctx* ctx, const void* residual, bool grouped_sx) {
  const __half* swp = static_cast<const __half*>(sw_t);
  ArDev ar = {};
  ar.world = 1;
  if (ctx != nullptr && ctx->world > 1) {
    DQ_REQUIRE(ctx->world <= 8 && ctx->rank >= 0 && ctx->rank < ctx->world, DQ_ERR_SHAPE,
               "bad all-reduce context: rank %d of %d", ctx->rank, ctx->world);
    DQ_REQUIRE(N % 4 == 0, DQ_ERR_SHAPE, "fused all-reduce needs N %% 4 == 0 (N=%d)", N);
    DQ_REQUIRE(static_cast<uint64_t>(M) * N <= ctx->buf_capacity_floats, DQ_ERR_WORKSPACE,
               "M*N=%lld exceeds the exchange buffer capacity %llu", (long long)M * N,
               (unsigned long long)ctx->buf_capacity_floats);
    DQ_REQUIRE(static_cast<uint64_t>((N + kVBN - 1) / kVBN) * split <= ctx->flag_units, DQ_ERR_WORKSPACE,
               "too many (tile, split) units for the flag array");
    for (int p = 0; p < ctx->world; ++p) {
      DQ_REQUIRE(ctx->buf_ptrs[p] != nullptr && ctx->flag_ptrs[p] != nullptr, DQ_ERR_NULL,
                 "null peer pointer for rank %d", p);
      ar.bufs[p] = static_cast<float*>(ctx->buf_ptrs[p]);
      ar.flags[p] = static_cast<uint32_t*>(ctx->flag_ptrs[p]);
    }
    DQ_REQUIRE(ctx->seq != nullptr, DQ_ERR_NULL, "null call counter");
    ar.seq = static_cast<const uint32_t*>(ctx->seq);
    ar.rank = ctx->rank;
    ar.world = ctx->world;
    ar.cap = static_cast<uint32_t>(ctx->buf_capacity_floats);
    const int wl = tuning(DQ_TUNE_AR_WAIT_LOG2);
    ar.wait_cycles = 1ll << ((wl >= 10 && wl <= 40) ? wl : 30);  // default: about half a second
  }
  int rc;
  if (tok != 8 && tok != 16 && tok != 32)
    return set_error(DQ_ERR_SHAPE, "register-path token capacity must be 8/16/32 (got %d)", tok);
  if (grouped_sx) {
    rc = (tok == 8) ? launch_gemv_t<1, true>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, split, stream, st, ar, residual)
       : (tok == 16) ? launch_gemv_t<2, true>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, split, stream, st, ar, residual)
                     : launch_gemv_t<4, true>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, split, stream, st, ar, residual);
  } else {
    rc = (tok == 8) ? launch_gemv_t<1, false>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, split, stream, st, ar, residual)
       : (tok == 16) ? launch_gemv_t<2, false>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, split, stream, st, ar, residual)
                     : launch_gemv_t<4, false>(codes, sx, w_packed, swp, r, M, N, K, y, y_dtype, split, stream, st, ar, residual);
  }
  if (rc == DQ_OK && ar.world > 1) {
    ar_bump_kernel<<<1, 1, 0, stream>>>(static_cast<uint32_t*>(ctx->seq));
    DQ_CHECK_CUDA(cudaGetLastError());
  }
  return rc;
}

}  // namespace dq
