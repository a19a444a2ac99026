// One-launch W4A4 int4 dual-scale linear for decode batches (M <= 16 tokens) on sm_100a:
// the per-token activation quantiser of PermLinear and the dual-scale GEMM in ONE kernel.
//
// The stand-alone path is two launches (quantiser -> codes/scales in global scratch -> GEMM).  At
// decode sizes both are latency chains, and the hand-over through global memory plus the kernel
// boundary cost as much as the weight stream itself.  Here the CTAs of a thread-block cluster
// quantise the <= 16 token rows TOGETHER and hand each other the codes through distributed
// shared memory, so that no CTA repeats another's work and nothing goes through global memory:
//
//   * a cluster is cx row tiles x split K-slices (cx * split <= 8 CTAs).  The K axis is cut into
//     cx * split chunks; CTA (ix, iz) owns the chunk ix of K-slice iz;
//   * pass 1: the eight compute warps load their chunk of X (bf16, 64-byte units kept in
//     registers), multiply by the column scale a[k] in fp32 and take the per-row absmax; the
//     partial maxima go to every CTA of the cluster (st.shared::cluster), cluster barrier;
//   * every CTA now knows the full-row absmax -> token scale (same arithmetic as the stand-alone
//     quantiser: absmax / 7, optional fp16 rounding, bit-identical codes);
//   * pass 2: each CTA quantises its chunk from the registers and writes the codes - packed two
//     per byte in the weight artefact's own nibble order - into the code region of the cx CTAs
//     that work on the same K-slice; cluster barrier;
//   * meanwhile the producer warp has been streaming the CTA's packed weights into its ring
//     (weights do not depend on the previous kernel of the stream, activations do: the compute
//     warps execute griddepcontrol.wait before they touch X, the producer does not);
//   * main loop as in the stand-alone decode kernel: packed nibbles straight from shared memory
//     into mma.sync.m16n8k32.s8 fragments, exact int32 sums per weight group, fp32 running sums.
//     Both operands are expanded as 16 * code, the 1/256 is folded into the group scale (exact);
//   * epilogue: r[n] * sx[m]; split-K partial tiles are reduced across the cluster through
//     distributed shared memory in rank order (deterministic, no global scratch).
//
// Results are bit-identical to dq_quant_act_int4 followed by dq_gemm_w4a4_int4.
#include "dq_common.h"
#include "dq_ptx.cuh"
#include "dq_quant.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace dq {
namespace fused {

constexpr int kBN = 128;            // weight rows per CTA
constexpr int kComputeWarps = 8;
constexpr int kThreads = (kComputeWarps + 1) * 32;  // + 1 producer warp
constexpr int kComputeThreads = kComputeWarps * 32;
constexpr int kGS = 2;              // weight groups per pipeline stage
constexpr int kStage = kGS * kTileBytes;  // 16896 B, a multiple of 16
constexpr int kMaxStages = 12;
constexpr int kMaxCluster = 8;
constexpr int kCodeRowBytes = 64;   // one token's codes of one weight group, two per byte

enum { FSITE_PRODUCER = 31, FSITE_COMPUTE = 32 };

template <int NT>
struct FCfg {
  static constexpr int TOK = 8 * NT;
  static constexpr int kThreadsPerRow = kComputeThreads / TOK;  // 32 or 16 lanes share a token row
  static constexpr int kPmaxBytes = kMaxCluster * TOK * 4;
  static constexpr int kSxBytes = TOK * 4;
  static constexpr int kBarBytes = 2 * kMaxStages * 8 + 16;
  static_assert(TOK * kBN * 4 <= 2 * kStage, "split-K exchange tile must fit in two ring stages");
  // bytes in front of the ring: code region (groups of the K-slice) + exchange slots + barriers
  __host__ __device__ static constexpr int head_bytes(int groups_per_split) {
    return (groups_per_split * TOK * kCodeRowBytes + kPmaxBytes + kSxBytes + kBarBytes + 127) / 128 * 128;
  }
  __host__ __device__ static constexpr int smem_bytes(int groups_per_split, int stages) {
    return head_bytes(groups_per_split) + stages * kStage + 128;
  }
};

__device__ __forceinline__ void mma_s8_16x8x32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void dsmem_st_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void dsmem_st_u4(uint32_t addr, uint4 v) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctaid_x() {
  uint32_t v;
  asm volatile("mov.u32 %0, %%cluster_ctaid.x;" : "=r"(v));
  return v;
}
__device__ __forceinline__ uint32_t cluster_ctaid_z() {
  uint32_t v;
  asm volatile("mov.u32 %0, %%cluster_ctaid.z;" : "=r"(v));
  return v;
}

// 8 bf16 (one 16-byte vector) -> 8 floats, times 8 entries of the column scale (or 1)
__device__ __forceinline__ void expand_scale8(const uint4& raw, const float* __restrict__ a_ptr,
                                              float* v) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
  if (a_ptr != nullptr) {
    const float4 a0 = __ldg(reinterpret_cast<const float4*>(a_ptr));
    const float4 a1 = __ldg(reinterpret_cast<const float4*>(a_ptr + 4));
    v[0] = __fmul_rn(v[0], a0.x); v[1] = __fmul_rn(v[1], a0.y);
    v[2] = __fmul_rn(v[2], a0.z); v[3] = __fmul_rn(v[3], a0.w);
    v[4] = __fmul_rn(v[4], a1.x); v[5] = __fmul_rn(v[5], a1.y);
    v[6] = __fmul_rn(v[6], a1.z); v[7] = __fmul_rn(v[7], a1.w);
  }
}

// NT: 8-token blocks (tokens handled: 8 * NT).  U: 64-byte units of X a thread keeps in
// registers between the absmax pass and the code pass.
template <int NT, int U>
__global__ void __launch_bounds__(kThreads, (U <= 2) ? 3 : 2)
gemv_fused_kernel(const uint8_t* __restrict__ w_packed, const __nv_bfloat16* __restrict__ x,
                  int64_t ldx, const float* __restrict__ a, const float* __restrict__ r,
                  void* __restrict__ y, int y_bf16, const void* __restrict__ residual, int M, int N,
                  int K, int groups_per_split, int split_k, int cx, int stages, int scale_fp16,
                  int* status) {
  using C = FCfg<NT>;
  constexpr int TOK = C::TOK;
  constexpr int TPR = C::kThreadsPerRow;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) &
                                             ~static_cast<uintptr_t>(127));
  // layout: [codes: groups_per_split x TOK x 64 B][pmax: 8 x TOK fp32][sx: TOK fp32][barriers][ring]
  uint8_t* codes_sm = smem;
  float* pmax = reinterpret_cast<float*>(smem + groups_per_split * TOK * kCodeRowBytes);
  float* sxs = pmax + kMaxCluster * TOK;
  uint64_t* full = reinterpret_cast<uint64_t*>(sxs + TOK);
  uint64_t* empty = full + kMaxStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kMaxStages);
  uint8_t* ring = smem + C::head_bytes(groups_per_split);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int ix = static_cast<int>(cluster_ctaid_x());   // row tile inside the cluster
  const int iz = static_cast<int>(cluster_ctaid_z());   // K-slice (== blockIdx.z)
  const int csize = cx * split_k;                        // CTAs in the cluster
  const int my_rank = ix + cx * iz;                      // == %cluster_ctarank (x fastest)
  const int n0 = blockIdx.x * kBN;
  const bool has_rows = n0 < N;                          // false for a padding tile of the cluster
  const int total_groups = K / kGroup;
  const int g_begin = iz * groups_per_split;
  int g_end = g_begin + groups_per_split;
  if (g_end > total_groups) g_end = total_groups;
  const int ng = (g_end > g_begin) ? (g_end - g_begin) : 0;
  const int nst = has_rows ? (ng + kGS - 1) / kGS : 0;   // pipeline stages this CTA walks through

  if (tid == 0) {
    for (int i = 0; i < stages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], kComputeWarps); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  grid_dep_launch_dependents();
  __syncthreads();

  if (warp == kComputeWarps) {
    // ------------------------------------------------------------------ producer warp
    const uint64_t pol_w = l2_policy_evict_first();
    const uint8_t* w_src =
        w_packed + (static_cast<size_t>(blockIdx.x) * total_groups + g_begin) * kTileBytes;
    const int prefill = (nst < stages) ? nst : stages;
    if (lane == 0) {
      for (int i = 0; i < prefill; ++i) {
        int cnt = ng - i * kGS;
        if (cnt > kGS) cnt = kGS;
        const uint32_t wbytes = static_cast<uint32_t>(cnt) * kTileBytes;
        mbar_expect_tx(&full[i], wbytes);
        bulk_load_1d(ring + i * kStage, w_src + static_cast<size_t>(i) * kGS * kTileBytes, wbytes,
                     &full[i], pol_w);
      }
    }
    __syncwarp();
    // the two cluster barriers of the quantisation phase (every thread of the cluster arrives)
    cluster_sync_all();
    cluster_sync_all();
    if (lane == 0) {
      int s = (prefill == stages) ? 0 : prefill;
      uint32_t ph = (prefill == stages) ? 0u : 1u;
      for (int i = prefill; i < nst; ++i) {
        if (!mbar_wait(&empty[s], ph, abort_flag, FSITE_PRODUCER)) break;
        int cnt = ng - i * kGS;
        if (cnt > kGS) cnt = kGS;
        const uint32_t wbytes = static_cast<uint32_t>(cnt) * kTileBytes;
        mbar_expect_tx(&full[s], wbytes);
        bulk_load_1d(ring + s * kStage, w_src + static_cast<size_t>(i) * kGS * kTileBytes, wbytes,
                     &full[s], pol_w);
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ cooperative quantiser
    grid_dep_wait();  // X may be the output of the kernel before this one
    {
      // this CTA's chunk of the K-slice: groups [q_begin, q_end)
      const int gpc = (ng + cx - 1) / cx;
      int q_begin = g_begin + ix * gpc;
      int q_end = q_begin + gpc;
      if (q_end > g_end) q_end = g_end;
      const int nq = (q_end > q_begin) ? (q_end - q_begin) : 0;
      const int units_per_row = nq * 4;     // 64-byte units (32 elements, one k chunk of a group)
      const int row = tid / TPR;
      const int lr = tid % TPR;
      const bool live = row < M;
      const __nv_bfloat16* xrow = x + static_cast<int64_t>(row) * ldx + static_cast<int64_t>(q_begin) * kGroup;
      const float* arow = (a != nullptr) ? a + static_cast<int64_t>(q_begin) * kGroup : nullptr;
      uint4 raw[U][4];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int unit = lr + u * TPR;
        if (live && unit < units_per_row) {
          const uint4* p = reinterpret_cast<const uint4*>(xrow + unit * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) raw[u][q] = __ldg(p + q);
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q) raw[u][q] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      float amax = 0.f;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int unit = lr + u * TPR;
        if (live && unit < units_per_row) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float v[8];
            expand_scale8(raw[u][q], arow != nullptr ? arow + unit * 32 + q * 8 : nullptr, v);
#pragma unroll
            for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
          }
        }
      }
      // the TPR lanes of a row are consecutive lanes of one warp
#pragma unroll
      for (int o = TPR / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      // partial maximum of (this CTA, row) -> slot [my_rank][row] of every CTA of the cluster
      if (lr < csize) {
        const uint32_t slot = smem_u32(pmax + my_rank * TOK + row);
        dsmem_st_f32(dsmem_map(slot, static_cast<uint32_t>(lr)), amax);
      }
      cluster_sync_all();   // barrier 1: all partial maxima have landed
      float full_max = 0.f;
      for (int j = 0; j < csize; ++j) full_max = fmaxf(full_max, pmax[j * TOK + row]);
      const float s = token_scale(full_max, scale_fp16);
      const float inv_s = __fdiv_rn(1.0f, s);
      if (lr == 0) sxs[row] = s;
      // pass 2: codes of this chunk, two per byte: byte b of a 16-byte k chunk holds code[b] in the
      // low nibble and code[16 + b] in the high nibble (the weight artefact's order)
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int unit = lr + u * TPR;
        if (live && unit < units_per_row) {
          uint32_t bytes[8];  // 32 codes as int8, four per word
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float v[8], c8[8];
            expand_scale8(raw[u][q], arow != nullptr ? arow + unit * 32 + q * 8 : nullptr, v);
            quant_codes8(v, s, inv_s, c8);
            bytes[2 * q] = pack_codes4(c8[0], c8[1], c8[2], c8[3]);
            bytes[2 * q + 1] = pack_codes4(c8[4], c8[5], c8[6], c8[7]);
          }
          uint4 packed;
          packed.x = (bytes[0] & 0x0F0F0F0Fu) | ((bytes[4] & 0x0F0F0F0Fu) << 4);
          packed.y = (bytes[1] & 0x0F0F0F0Fu) | ((bytes[5] & 0x0F0F0F0Fu) << 4);
          packed.z = (bytes[2] & 0x0F0F0F0Fu) | ((bytes[6] & 0x0F0F0F0Fu) << 4);
          packed.w = (bytes[3] & 0x0F0F0F0Fu) | ((bytes[7] & 0x0F0F0F0Fu) << 4);
          const int gl = (q_begin - g_begin) + (unit >> 2);  // group index inside the K-slice
          const uint32_t dst = smem_u32(codes_sm + (gl * TOK + row) * kCodeRowBytes + (unit & 3) * 16);
          for (int p = 0; p < cx; ++p)  // every row tile of the cluster that works on this K-slice
            dsmem_st_u4(dsmem_map(dst, static_cast<uint32_t>(p + cx * iz)), packed);
        }
      }
      cluster_sync_all();   // barrier 2: the code region of this CTA is complete
    }

    // ------------------------------------------------------------------ main loop
    const int g = lane >> 2;  // fragment row / token index inside an 8-block
    const int t = lane & 3;
    const int row = warp * 16 + g;  // local weight row (and row + 8)
    float run[NT][4];
#pragma unroll
    for (int nb = 0; nb < NT; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) run[nb][e] = 0.f;

    int s = 0;
    uint32_t ph = 0;
    for (int i = 0; i < nst; ++i) {
      if (!mbar_wait(&full[s], ph, abort_flag, FSITE_COMPUTE)) break;
      const uint8_t* st = ring + s * kStage;
      int cnt = ng - i * kGS;
      if (cnt > kGS) cnt = kGS;
#pragma unroll
      for (int gi = 0; gi < kGS; ++gi) {
        if (gi >= cnt) break;
        const uint8_t* tile = st + gi * kTileBytes;
        const int tp = t ^ ((g >> 1) & 3);  // chunk positions are swizzled by (row >> 1) & 3
        const uint4 wa = *reinterpret_cast<const uint4*>(tile + row * 64 + tp * 16);
        const uint4 wb = *reinterpret_cast<const uint4*>(tile + (row + 8) * 64 + tp * 16);
        const __half* sc = reinterpret_cast<const __half*>(tile + kTileCodeBytes);
        const float s0 = __half2float(sc[row]) * 0.00390625f;      // both operands carry a factor 16
        const float s1 = __half2float(sc[row + 8]) * 0.00390625f;
        uint4 xq[NT];
        const uint8_t* xg = codes_sm + ((i * kGS + gi) * TOK) * kCodeRowBytes;
#pragma unroll
        for (int nb = 0; nb < NT; ++nb)
          xq[nb] = *reinterpret_cast<const uint4*>(xg + (nb * 8 + g) * kCodeRowBytes + t * 16);
        const uint32_t wav[4] = {wa.x, wa.y, wa.z, wa.w};
        const uint32_t wbv[4] = {wb.x, wb.y, wb.z, wb.w};
        int c[NT][2][4];
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
            const uint32_t xw = (j == 0) ? xq[nb].x : (j == 1) ? xq[nb].y : (j == 2) ? xq[nb].z : xq[nb].w;
            const uint32_t b0 = (xw << 4) & 0xF0F0F0F0u;
            const uint32_t b1 = xw & 0xF0F0F0F0u;
            mma_s8_16x8x32(c[nb][j & 1], a0, a1, a2, a3, b0, b1);
          }
        }
#pragma unroll
        for (int nb = 0; nb < NT; ++nb) {
          run[nb][0] = fmaf(static_cast<float>(c[nb][0][0] + c[nb][1][0]), s0, run[nb][0]);
          run[nb][1] = fmaf(static_cast<float>(c[nb][0][1] + c[nb][1][1]), s0, run[nb][1]);
          run[nb][2] = fmaf(static_cast<float>(c[nb][0][2] + c[nb][1][2]), s1, run[nb][2]);
          run[nb][3] = fmaf(static_cast<float>(c[nb][0][3] + c[nb][1][3]), s1, run[nb][3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
      if (++s == stages) { s = 0; ph ^= 1u; }
    }

    // accumulator fragment: c0/c1 = (row, tokens 2t, 2t+1), c2/c3 = (row + 8, same tokens)
    if (split_k == 1) {
      if (has_rows) {
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
                  store_y(y, residual, y_bf16, static_cast<size_t>(m) * N + n, run[nb][2 * hrow + e] * (rn * sxs[m]));
                }
              }
          }
        }
      }
    } else {
      // the ring is no longer read by any compute warp of this CTA: reuse it as the exchange tile
      asm volatile("bar.sync 1, 256;" ::: "memory");
      float* red = reinterpret_cast<float*>(ring);
#pragma unroll
      for (int nb = 0; nb < NT; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int m = nb * 8 + 2 * t + e;
          red[m * kBN + row] = run[nb][e];
          red[m * kBN + row + 8] = run[nb][2 + e];
        }
    }
  }

  // -------------------------------------------------------------------- split-K reduction
  if (split_k > 1) {
    __syncwarp();
    cluster_sync_all();
    if (warp < kComputeWarps && has_rows) {
      const int rows = TOK / split_k;  // token rows of the tile this CTA finishes
      const int c4 = tid & 31;         // float4 column
      const uint32_t red_base = smem_u32(ring);
      for (int rr = tid >> 5; rr < rows; rr += kComputeWarps) {
        const int m = iz * rows + rr;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const uint32_t off = static_cast<uint32_t>((m * kBN + c4 * 4) * 4);
        for (int p = 0; p < split_k; ++p) {  // K-slice p of the same row tile: rank ix + cx * p
          const float4 v = dsmem_ld_f4(dsmem_map(red_base + off, static_cast<uint32_t>(ix + cx * p)));
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if (m < M) {
          const float sm = sxs[m];
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
    cluster_sync_all();  // peers may still be reading this CTA's exchange tile until here
  }
  __syncthreads();
  if (tid == 0 && *abort_flag != 0) atomicCAS(status, 0, *abort_flag);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template <int NT, int U>
static cudaError_t set_attr() {
  return cudaFuncSetAttribute(gemv_fused_kernel<NT, U>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              227 * 1024);
}

}  // namespace fused

int init_gemv_fused_kernels() {
  cudaError_t e = fused::set_attr<1, 1>();
  if (e == cudaSuccess) e = fused::set_attr<1, 2>();
  if (e == cudaSuccess) e = fused::set_attr<1, 4>();
  if (e == cudaSuccess) e = fused::set_attr<2, 1>();
  if (e == cudaSuccess) e = fused::set_attr<2, 2>();
  if (e == cudaSuccess) e = fused::set_attr<2, 4>();
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "cudaFuncSetAttribute(gemv_fused) failed: %s", cudaGetErrorString(e));
  return DQ_OK;
}

// Launch geometry of the one-launch decode linear for (M, N, K); ok = false when the shape is
// outside what the kernel covers (the caller then takes the two-launch path).
struct FusedPlan {
  bool ok;
  int nt, units, split, cx, gps, stages, tiles_x;
  size_t smem;
};

static FusedPlan plan_fused(int M, int N, int K, int sm_count) {
  FusedPlan p = {};
  if (M < 1 || M > 16 || K % kGroup != 0 || K < kGroup) return p;
  p.nt = (M <= 8) ? 1 : 2;
  const int tok = 8 * p.nt;
  const int total_groups = K / kGroup;
  const int tiles_n = (N + fused::kBN - 1) / fused::kBN;
  int split = tuning(DQ_TUNE_FUSED_SPLIT);
  if (split <= 0) split = gemv_pick_split(tiles_n, total_groups, tok, sm_count);
  if (!(split == 1 || split == 2 || split == 4 || split == 8) || split > tok || split > total_groups)
    return p;
  p.split = split;
  p.gps = (total_groups + split - 1) / split;
  if ((split - 1) * p.gps >= total_groups) return p;  // an empty K-slice
  // row tiles per cluster: fill the cluster to 8 CTAs without padding tiles
  int cx = fused::kMaxCluster / split;
  while (cx > 1 && tiles_n % cx != 0) cx >>= 1;
  p.cx = cx;
  p.tiles_x = tiles_n;
  // 64-byte units of X a thread must hold: ceil(groups of its chunk * 4 / lanes per row)
  const int gpc = (p.gps + cx - 1) / cx;
  const int tpr = fused::kComputeThreads / tok;
  const int need = (gpc * 4 + tpr - 1) / tpr;
  p.units = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 0;
  if (p.units == 0) return p;
  // ring depth: what is left of an SM's shared memory when it is shared by the CTAs expected on
  // it plus one more, so that the first CTAs of the next launch of the stream can start streaming
  // their weights while this one drains (programmatic dependent launch)
  const int head = (p.nt == 1) ? fused::FCfg<1>::head_bytes(p.gps) : fused::FCfg<2>::head_bytes(p.gps);
  const int ctas = tiles_n * split;
  int per_sm = (ctas + sm_count - 1) / sm_count;
  const int max_ctas = (p.units <= 2) ? 3 : 2;
  if (per_sm > max_ctas) per_sm = max_ctas;
  int share = per_sm + tuning(DQ_TUNE_FUSED_EXTRA_CTA);
  if (share < 1) share = 1;
  int avail = (227 * 1024) / share - 1024 - head - 128;
  int stages = tuning(DQ_TUNE_FUSED_STAGES) > 0 ? tuning(DQ_TUNE_FUSED_STAGES) : avail / fused::kStage;
  const int walk = (p.gps + fused::kGS - 1) / fused::kGS;
  if (stages > walk) stages = walk;
  if (stages > fused::kMaxStages) stages = fused::kMaxStages;
  if (stages < 2) stages = 2;
  p.stages = stages;
  p.smem = static_cast<size_t>(head) + static_cast<size_t>(stages) * fused::kStage + 128;
  if (p.smem > 227 * 1024) return p;
  p.ok = true;
  return p;
}

bool gemv_fused_covers(int M, int N, int K, const DeviceState* st) {
  return plan_fused(M, N, K, st->sm_count).ok;
}

template <int NT, int U>
static int launch_fused_t(const FusedPlan& p, const void* x, int64_t ldx, const float* a,
                          const uint8_t* w_packed, const float* r, int M, int N, int K, void* y,
                          int y_dtype, int scale_fp16, cudaStream_t stream, DeviceState* st,
                          const void* residual) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.tiles_x, 1, p.split);
  cfg.blockDim = dim3(fused::kThreads, 1, 1);
  cfg.dynamicSmemBytes = p.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.cx;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = p.split;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, fused::gemv_fused_kernel<NT, U>, w_packed,
                                     static_cast<const __nv_bfloat16*>(x), ldx, a, r, y,
                                     y_dtype == DQ_DTYPE_BF16 ? 1 : 0, residual, M, N, K, p.gps, p.split, p.cx,
                                     p.stages, scale_fp16, st->status_dev);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "gemv_fused launch failed (tokens=%d split=%d cx=%d stages=%d): %s",
                     8 * NT, p.split, p.cx, p.stages, cudaGetErrorString(e));
  return DQ_OK;
}

int launch_gemv_fused(const void* x_bf16, int64_t ldx, const float* a, const uint8_t* w_packed,
                      const float* r, int M, int N, int K, void* y, int y_dtype, int scale_fp16,
                      cudaStream_t stream, DeviceState* st, const void* residual) {
  const FusedPlan p = plan_fused(M, N, K, st->sm_count);
  DQ_REQUIRE(p.ok, DQ_ERR_UNSUPPORTED, "one-launch decode linear does not cover M=%d N=%d K=%d", M, N, K);
  DQ_REQUIRE(x_bf16 != nullptr && w_packed != nullptr && y != nullptr, DQ_ERR_NULL, "null x / w_packed / y");
  DQ_REQUIRE(aligned(x_bf16, 16) && ldx % 8 == 0 && ldx >= K, DQ_ERR_ALIGN,
             "x must be 16-byte aligned with ldx a multiple of 8 and >= K");
  DQ_REQUIRE(a == nullptr || aligned(a, 16), DQ_ERR_ALIGN, "a must be 16-byte aligned");
  DQ_REQUIRE(aligned(w_packed, 16), DQ_ERR_ALIGN, "w_packed must be 16-byte aligned");
#define DQ_FUSED_CASE(NTV, UV)                                                                     \
  if (p.nt == NTV && p.units == UV)                                                                \
    return launch_fused_t<NTV, UV>(p, x_bf16, ldx, a, w_packed, r, M, N, K, y, y_dtype, scale_fp16, \
                                   stream, st, residual)
  DQ_FUSED_CASE(1, 1);
  DQ_FUSED_CASE(1, 2);
  DQ_FUSED_CASE(1, 4);
  DQ_FUSED_CASE(2, 1);
  DQ_FUSED_CASE(2, 2);
  DQ_FUSED_CASE(2, 4);
#undef DQ_FUSED_CASE
  return set_error(DQ_ERR_UNSUPPORTED, "no one-launch decode kernel for nt=%d units=%d", p.nt, p.units);
}

}  // namespace dq
