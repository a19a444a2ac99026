// The fast online-Hadamard quantiser kernels and their dispatch, as templates over the input type.
// Included by one translation unit per input type (act_quant_had_bf16.cu, act_quant_had_f32.cu):
// every unit has its own copy of the constant-bank factor table and of the upload cache, and only
// launches its own kernels, so the copies never have to agree.
#pragma once
#include "act_quant_common.cuh"

namespace dq {
namespace {

constexpr int kHadFastMaxSmem = 200 * 1024;

// ---------------------------------------------------------------------------------------------
// fast online Hadamard: warp-shuffle butterflies inside segments, one thread per column across
// ---------------------------------------------------------------------------------------------
// The row is viewed as S segments of P contiguous elements (S <= 32, P = 32 * R).
//   phase A (wht_inner): Walsh-Hadamard of length P inside every segment; a warp owns a segment,
//            lane l holds elements l + 32 r: stages h < 32 exchange registers with lane ^ h, stages
//            h >= 32 are register butterflies.  Same stage order and operand order as
//            the reference loop (h = 1, 2, 4, ...; (a, b) -> (a + b, a - b)), so bit-identical.
//   phase B: per column c (0..P-1) across the S segments:
//            matrix mode   out[i] = sum_j H[i][j] * (v[j] * scale), j ascending  (had_K @ x)
//            butterfly mode  remaining Walsh-Hadamard stages over the segment index, then * scale
// Full transform of size 28 * 512: A + matrix.  Full power-of-two size: A + butterflies.
// Partial (across heads) transform: butterflies only, segments = heads.
template <int R>
__device__ __forceinline__ void wht_segment_warp(float* seg, int lane, float post = 1.0f) {
  // lane l holds elements l + 32 r (r < R): conflict-free shared-memory access; stages h < 32
  // pair lanes (shuffle), stages h >= 32 pair registers r and r + h/32.  Stage order h = 1, 2, ...
  float v[R];
#pragma unroll
  for (int r = 0; r < R; ++r) v[r] = seg[lane + 32 * r];
  // the lane with bit m clear keeps a + b, its partner a - b: other + sign * own, one FMA either
  // way (the product with +-1 is exact, so the FMA rounds exactly like the addition / subtraction)
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    const float sign = (lane & m) != 0 ? -1.0f : 1.0f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float other = __shfl_xor_sync(0xffffffffu, v[r], m);
      v[r] = __fmaf_rn(v[r], sign, other);
    }
  }
#pragma unroll
  for (int h = 1; h < R; h <<= 1) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if ((r & h) == 0) {
        const float u = v[r], w = v[r + h];
        v[r] = __fadd_rn(u, w);
        v[r + h] = __fsub_rn(u, w);
      }
    }
  }
  // `post`: the transform's scale when a matrix stage follows (it multiplies every value once, here,
  // instead of once per thread that reads the value there); 1 otherwise, an exact identity
#pragma unroll
  for (int r = 0; r < R; ++r) seg[lane + 32 * r] = __fmul_rn(v[r], post);
}

// The K x K +-1 matrix of the "full" transform, in constant memory so that an FMA takes its
// coefficient as an immediate constant-bank operand (one instruction per term instead of a
// shared-memory load plus an FMA).  Every entry is stored twice, (h, h): the matrix stage works on
// two columns at a time with packed fp32 FMAs, each half of which rounds like the scalar fmaf.
// Refreshed by the host when a call brings a different matrix.
__constant__ float2 c_had_mat2[32 * 32];
__device__ float2 g_had_stage[32 * 32];  // the table is assembled here, then copied to the constant bank

__global__ void __launch_bounds__(1024) had_table_kernel(const float* __restrict__ had_mat, int S) {
  const int t = threadIdx.x, i = t >> 5, j = t & 31;
  const float h = (i < S && j < S) ? had_mat[i * S + j] : 0.f;  // rows and columns padded to 32 with zeros
  g_had_stage[t] = make_float2(h, h);
}

// Output rows QI, QI + G, ... of the matrix stage for one column pair, fully unrolled (see the
// call site); matrix_rows_dispatch selects the copy for a run-time qi in [0, G).
template <int HN, int G, int QI>
__device__ __forceinline__ void matrix_rows_static(const float2* v, float* row, int P, int c, int S, float& amax) {
#pragma unroll
  for (int i = QI; i < HN; i += G) {
    if (i < S) {  // (kept as a run-time test also for a known order: without it the short-row shapes ran 10-25 % slower)
      float2 acc = make_float2(0.f, 0.f);
#pragma unroll
      for (int j = 0; j < HN; ++j) acc = __ffma2_rn(c_had_mat2[i * 32 + j], v[j], acc);
      *reinterpret_cast<float2*>(row + i * P + c) = acc;
      amax = fmaxf(amax, fmaxf(fabsf(acc.x), fabsf(acc.y)));
    }
  }
}
template <int HN, int G, int QI = 0>
__device__ __forceinline__ void matrix_rows_dispatch(int qi, const float2* v, float* row, int P, int c, int S,
                                                     float& amax) {
  if constexpr (QI < G) {
    if (qi == QI) matrix_rows_static<HN, G, QI>(v, row, P, c, S, amax);
    else matrix_rows_dispatch<HN, G, QI + 1>(qi, v, row, P, c, S, amax);
  }
}

// THREADS = 512: one CTA per SM, the shortest time per row (decode batches, one row per SM at most).
// THREADS = 256: three CTAs per SM; with many rows one row's load, barrier and store phases overlap
// another row's arithmetic (two CTAs per SM with more registers each measured 30 % slower).
// HS: order of the +-1 factor when it is one of the common ones (28: 14336 = 28 * 512 and
// 28672 = 28 * 1024), so that the matrix stage has no padded terms; 0 = any order up to 32.
template <int R, typename XT, int THREADS, int HS = 0>
__global__ void __launch_bounds__(THREADS, THREADS == 256 ? 3 : 1)
act_quant_had_fast_kernel(const XT* __restrict__ x, const XT* __restrict__ up, int64_t ldx,
                          const float* __restrict__ a, int K,
                          int S, int inner, int matrix, float had_scale,
                          const float* __restrict__ had_mat, int8_t* __restrict__ codes,
                          float* __restrict__ sx, float* __restrict__ out, int mode, int scale_fp16) {
  extern __shared__ float sm_row[];
  __shared__ float red[THREADS / 32];
  float* row = sm_row;
  float* hm = sm_row + K;
  grid_dep_launch_dependents();
  grid_dep_wait();
  const int P = K / S;
  const int rr = blockIdx.x;
  const XT* xr = x + static_cast<int64_t>(rr) * ldx;
  const XT* ur = (up != nullptr) ? up + static_cast<int64_t>(rr) * ldx : nullptr;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int idx = threadIdx.x * 8; idx < K; idx += THREADS * 8) {
    float v[8];
    load8(xr + idx, v);
    apply_gate(ur != nullptr ? ur + idx : nullptr, v);
    if (a != nullptr) {
      float av[8];
      load8(a + idx, av);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(v[e], av[e]);
    }
    *reinterpret_cast<float4*>(row + idx) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(row + idx + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
  (void)hm;
  (void)had_mat;
  __syncthreads();

  if (inner) {
    for (int sgm = warp; sgm < S; sgm += THREADS / 32)
      wht_segment_warp<R>(row + sgm * P, lane, matrix ? had_scale : 1.0f);
    __syncthreads();
  }
  const bool scale_here = !inner;  // no Walsh-Hadamard phase: the matrix stage scales its own inputs

  float amax = 0.f;
  if (matrix) {
    // two adjacent columns per thread (P is even): packed loads, packed FMAs
    constexpr int HN = (HS > 0) ? HS : 32;  // factor order known at compile time, or padded to 32
    constexpr int pairs = 16 * R;  // P = 32 R
    if constexpr (pairs < THREADS) {
      // Short segments (rows of 28 * 64 ... 28 * 256 values, the shards of a row-parallel linear):
      // fewer column pairs than threads.  G = THREADS / pairs threads share one pair, each holding
      // its S inputs in registers and forming the output rows i = qi, qi + G, ...; every sum is the
      // same j-ascending chain as below.  (pairs is a power of two, so G is whole; qi is the same for
      // all lanes of a warp once a segment has 64 values, which keeps the coefficient loads uniform.)
      constexpr int G = THREADS / pairs;
      const int c = 2 * (static_cast<int>(threadIdx.x) & (pairs - 1)), qi = static_cast<int>(threadIdx.x) / pairs;
      float2 v[HN];
#pragma unroll
      for (int j = 0; j < HN; ++j)
        v[j] = (j < S) ? *reinterpret_cast<const float2*>(row + j * P + c) : make_float2(0.f, 0.f);
      if (scale_here) {
#pragma unroll
        for (int j = 0; j < HN; ++j) {
          v[j].x = __fmul_rn(v[j].x, had_scale);
          v[j].y = __fmul_rn(v[j].y, had_scale);
        }
      }
      __syncthreads();  // every thread holds its inputs before the first output row replaces them
      if constexpr (G <= 8) {
        // the thread's output rows are known once qi is: one fully unrolled copy per value of qi, so
        // that every coefficient is a constant-bank operand of its FMA (HN x HN FMAs of code in all)
        matrix_rows_dispatch<HN, G>(qi, v, row, P, c, S, amax);
      } else
      for (int i = qi; i < S; i += 2 * G) {  // two independent chains in flight
        const int i2 = i + G;
        const bool second = i2 < S;
        const float2* h0 = c_had_mat2 + i * 32;
        const float2* h1 = c_had_mat2 + (second ? i2 : i) * 32;
        float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < HN; ++j) {
          acc0 = __ffma2_rn(h0[j], v[j], acc0);
          acc1 = __ffma2_rn(h1[j], v[j], acc1);
        }
        *reinterpret_cast<float2*>(row + i * P + c) = acc0;
        amax = fmaxf(amax, fmaxf(fabsf(acc0.x), fabsf(acc0.y)));
        if (second) {
          *reinterpret_cast<float2*>(row + i2 * P + c) = acc1;
          amax = fmaxf(amax, fmaxf(fabsf(acc1.x), fabsf(acc1.y)));
        }
      }
    } else
    for (int c = 2 * threadIdx.x; c < P; c += 2 * THREADS) {
      float2 v[HN];
#pragma unroll
      for (int j = 0; j < HN; ++j)
        v[j] = (HS > 0 || j < S) ? *reinterpret_cast<const float2*>(row + j * P + c) : make_float2(0.f, 0.f);
      if (scale_here) {
#pragma unroll
        for (int j = 0; j < HN; ++j) {
          v[j].x = __fmul_rn(v[j].x, had_scale);
          v[j].y = __fmul_rn(v[j].y, had_scale);
        }
      }
      // the known order is fully unrolled, so that every coefficient is a constant-bank operand of
      // its FMA and the independent accumulation chains can be interleaved; the generic form keeps
      // two output rows in flight (a fully unrolled 32 x 32 stage in every instantiation is most of
      // this file's compile time)
      constexpr int kUnrollRows = (HS > 0) ? HN : 2;
#pragma unroll kUnrollRows
      for (int i = 0; i < HN; ++i) {
        if (HS > 0 || i < S) {  // a known order is the factor's order: no padded rows
          float2 acc = make_float2(0.f, 0.f);
#pragma unroll
          for (int j = 0; j < HN; ++j)  // H entries are +-1 (0 in the padding): same as acc + H*v, j ascending
            acc = __ffma2_rn(c_had_mat2[i * 32 + j], v[j], acc);
          *reinterpret_cast<float2*>(row + i * P + c) = acc;
          amax = fmaxf(amax, fmaxf(fabsf(acc.x), fabsf(acc.y)));
        }
      }
    }
  } else {
  for (int c = threadIdx.x; c < P; c += THREADS) {
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = (j < S) ? row[j * P + c] : 0.f;
    {
#pragma unroll
      for (int hb = 0; hb < 5; ++hb) {
        constexpr int kOne = 1;
        const int h = kOne << hb;
        if (h < S) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if ((j & h) == 0) {
              const float u = v[j], w = v[j + h];
              v[j] = __fadd_rn(u, w);
              v[j + h] = __fsub_rn(u, w);
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < S) {
          const float o = __fmul_rn(v[j], had_scale);
          row[j * P + c] = o;
          amax = fmaxf(amax, fabsf(o));
        }
      }
    }
  }
  }
  float s = 1.f;
  if (mode != MODE_RAW) {
    amax = block_max(amax, red, THREADS / 32);
    s = token_scale(amax, scale_fp16);
    if (threadIdx.x == 0 && sx != nullptr) sx[rr] = s;
  } else {
    __syncthreads();
  }
  int8_t* crow = (codes != nullptr) ? codes + static_cast<int64_t>(rr) * K : nullptr;
  float* orow = out_row_ptr(out, rr, K, mode);
  for (int idx = threadIdx.x * 8; idx < K; idx += THREADS * 8) {
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = row[idx + e];
    emit8(v, s, mode, crow, orow, idx, scale_fp16);
  }
}

// ---------------------------------------------------------------------------------------------
// the same transform for a handful of rows: one thread-block cluster per row
// ---------------------------------------------------------------------------------------------
// At decode sizes (a few token rows) the fast kernel is one CTA per row on a few SMs and its phases
// - load (+ SiLU * up), Walsh-Hadamard inside the segments, the S x S stage across them, absmax,
// codes - are a serial chain.  Here four CTAs share a row: CTA c loads and transforms segments
// [c S/4, (c+1) S/4), then computes the matrix stage for columns [c P/4, (c+1) P/4) of every
// segment, reading the other CTAs' segments through distributed shared memory; the row absmax is
// exchanged the same way.  Every sum is formed exactly as in the fast kernel (same Walsh-Hadamard
// routine, j ascending fp32 FMAs with the factor's entry as coefficient), so scales and codes are
// bit-identical.  Needs S % 4 == 0 and the factor in c_had_mat2.
constexpr int kHadClusterCtas = 4;
constexpr int kHadClusterThreads = 512;
constexpr int kHadClusterMaxRows = 64;

template <int R, typename XT>
__global__ void __launch_bounds__(kHadClusterThreads, 1)
act_quant_had_cluster_kernel(const XT* __restrict__ x, const XT* __restrict__ up, int64_t ldx,
                             const float* __restrict__ a, int S, float had_scale, int8_t* __restrict__ codes,
                             float* __restrict__ sx, float* __restrict__ out, int mode, int scale_fp16) {
  constexpr int P = 32 * R;                   // segment length
  constexpr int PC = P / kHadClusterCtas;     // columns of the matrix stage per CTA
  constexpr int G = kHadClusterThreads / PC;  // threads per column: output rows i = qi, qi + G, ...
  extern __shared__ float sm_row[];
  __shared__ float red[kHadClusterThreads / 32];
  __shared__ float pmax[kHadClusterCtas];
  const int SQ = S / kHadClusterCtas;         // segments per CTA
  const int K = S * P;
  float* seg = sm_row;                        // [SQ][P]: this CTA's segments (read by its peers)
  float* outv = sm_row + SQ * P;              // [S][PC]: this CTA's slice of the transformed row
  grid_dep_launch_dependents();
  grid_dep_wait();
  const int rank = static_cast<int>(cluster_ctarank());
  const int rr = blockIdx.x / kHadClusterCtas;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t base = static_cast<int64_t>(rr) * ldx + static_cast<int64_t>(rank) * SQ * P;
  const XT* xr = x + base;
  const XT* ur = (up != nullptr) ? up + base : nullptr;
  const float* ar = (a != nullptr) ? a + static_cast<int64_t>(rank) * SQ * P : nullptr;
  for (int idx = tid * 8; idx < SQ * P; idx += kHadClusterThreads * 8) {
    float v[8];
    load8(xr + idx, v);
    apply_gate(ur != nullptr ? ur + idx : nullptr, v);
    if (ar != nullptr) {
      float av[8];
      load8(ar + idx, av);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(v[e], av[e]);
    }
    *reinterpret_cast<float4*>(seg + idx) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(seg + idx + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
  __syncthreads();
  for (int sgm = warp; sgm < SQ; sgm += kHadClusterThreads / 32) wht_segment_warp<R>(seg + sgm * P, lane);
  cluster_sync_all();  // every CTA's segments are transformed and visible to its peers

  const int col = tid % PC, qi = tid / PC;
  float v[32];
  {
    const uint32_t seg_addr = smem_u32(seg);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      v[j] = 0.f;
      if (j < S) {
        const int owner = j / SQ, local = j - owner * SQ;
        const uint32_t addr = dsmem_map(seg_addr + static_cast<uint32_t>((local * P + rank * PC + col) * 4),
                                        static_cast<uint32_t>(owner));
        v[j] = __fmul_rn(dsmem_ld_f32(addr), had_scale);
      }
    }
  }
  float amax = 0.f;
  for (int i = qi; i < S; i += G) {  // i is the same for every lane of a warp
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) acc = fmaf(c_had_mat2[i * 32 + j].x, v[j], acc);  // padding entries are zero
    outv[i * PC + col] = acc;
    amax = fmaxf(amax, fabsf(acc));
  }
  float s = 1.f;
  amax = block_max(amax, red, kHadClusterThreads / 32);  // (also orders the outv writes before their reads below)
  if (tid < kHadClusterCtas)
    dsmem_store_f32(dsmem_map(smem_u32(&pmax[rank]), static_cast<uint32_t>(tid)), amax);
  cluster_sync_all();  // the four partial maxima have landed everywhere; no remote access after this point
  if (mode != MODE_RAW) {
    float full = pmax[0];
#pragma unroll
    for (int c = 1; c < kHadClusterCtas; ++c) full = fmaxf(full, pmax[c]);
    s = token_scale(full, scale_fp16);
    if (rank == 0 && tid == 0 && sx != nullptr) sx[rr] = s;
  }
  int8_t* crow = (codes != nullptr) ? codes + static_cast<int64_t>(rr) * K : nullptr;
  float* orow = out_row_ptr(out, rr, K, mode);
  for (int u = tid; u < S * (PC / 8); u += kHadClusterThreads) {
    const int i = u / (PC / 8), piece = u - i * (PC / 8);
    float e8[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) e8[e] = outv[i * PC + piece * 8 + e];
    emit8(e8, s, mode, crow, orow, i * P + rank * PC + piece * 8, scale_fp16);
  }
}

// ---------------------------------------------------------------------------------------------
// the across-heads transform (o_proj input) for many rows: registers only
// ---------------------------------------------------------------------------------------------
// Row = S heads of 128 values, Walsh-Hadamard over the head index for each of the 128 lanes of a
// head.  The one-CTA-per-row kernel above spends its time waiting (load, barrier, 128 busy threads,
// barrier, store); here a lane owns eight adjacent columns of min(S, 16) heads and keeps them in
// registers from the load to the codes: 16 lanes cover a row (32 for S = 32, where the halves of
// the warp hold heads 0-15 and 16-31 and the last stage is one shuffle per value), nothing goes
// through shared memory and no barrier is needed.  Same stage order and operand order as above.
// Codes only (int8 or E4M3, fp32 or fp16 scale), no gate: everything is unrolled over the heads, and
// with the other output modes and the SiLU gate expanded sixteen times the code outgrew the
// instruction cache (measured: 2.4x slower than the kernel above at 32 heads).
constexpr int kHeadsKernelThreads = 128;
constexpr int kHeadsKernelMinRows = 64;

template <int S, typename XT, bool E4M3>
__global__ void __launch_bounds__(kHeadsKernelThreads)
act_quant_had_heads_kernel(const XT* __restrict__ x, int64_t ldx, const float* __restrict__ a, int M,
                           float had_scale, int8_t* __restrict__ codes, float* __restrict__ sx, int scale_fp16) {
  constexpr int HL = (S < 16) ? S : 16;   // heads per lane
  constexpr int L = (S == 32) ? 32 : 16;  // lanes per row
  constexpr int K = S * 128;
  grid_dep_launch_dependents();
  grid_dep_wait();
  const int lane = threadIdx.x & 31;
  const int sub = lane & (L - 1);
  const int64_t rr = (static_cast<int64_t>(blockIdx.x) * (kHeadsKernelThreads / 32) + (threadIdx.x >> 5)) * (32 / L) +
                     lane / L;
  const bool live = rr < M;  // lanes of a row past the end keep running (shuffles), but touch no memory
  const int col = 8 * (sub & 15);
  const int head0 = (S == 32 && sub >= 16) ? 16 : 0;
  const XT* xr = x + (live ? rr : 0) * ldx;
  float v[HL][8];
#pragma unroll
  for (int j = 0; j < HL; ++j) {
    const int idx = (head0 + j) * 128 + col;
    if (live) {
      load8(xr + idx, v[j]);
      if (a != nullptr) {
        float av[8];
        load8(a + idx, av);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[j][e] = __fmul_rn(v[j][e], av[e]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[j][e] = 0.f;
    }
  }
#pragma unroll
  for (int h = 1; h < HL; h <<= 1) {
#pragma unroll
    for (int j = 0; j < HL; ++j) {
      if ((j & h) == 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float u = v[j][e], w = v[j + h][e];
          v[j][e] = __fadd_rn(u, w);
          v[j + h][e] = __fsub_rn(u, w);
        }
      }
    }
  }
  if constexpr (S == 32) {  // heads j and j + 16 sit in lanes l and l + 16
    const float sign = sub >= 16 ? -1.0f : 1.0f;  // a + b below, a - b above: other + sign * own, rounded once
#pragma unroll
    for (int j = 0; j < HL; ++j) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float other = __shfl_xor_sync(0xffffffffu, v[j][e], 16);
        v[j][e] = __fmaf_rn(v[j][e], sign, other);
      }
    }
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < HL; ++j) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      v[j][e] = __fmul_rn(v[j][e], had_scale);
      amax = fmaxf(amax, fabsf(v[j][e]));
    }
  }
#pragma unroll
  for (int o = L / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (!live) return;
  const float s = token_scale(amax, scale_fp16);
  if (sub == 0 && sx != nullptr) sx[rr] = s;
  const float inv_s = __fdiv_rn(1.0f, s);
  int8_t* crow = codes + rr * K;
#pragma unroll
  for (int j = 0; j < HL; ++j) {
    float q[8];
    quant_codes8(v[j], s, inv_s, q);
    const uint32_t lo = E4M3 ? pack_codes4_e4m3(q[0], q[1], q[2], q[3]) : pack_codes4(q[0], q[1], q[2], q[3]);
    const uint32_t hi = E4M3 ? pack_codes4_e4m3(q[4], q[5], q[6], q[7]) : pack_codes4(q[4], q[5], q[6], q[7]);
    *reinterpret_cast<uint2*>(crow + (head0 + j) * 128 + col) = make_uint2(lo, hi);
  }
}

// Copies a device-resident S x S matrix into c_had_mat2 (rows padded to 32) when it is not the
// one already there.  The matrix behind a given pointer is assumed immutable (it is the constant
// Hadamard factor of a layer); the copy is a stream-ordered device-to-device memcpy.
static int upload_had_matrix(const float* had_mat, int S, cudaStream_t stream) {
  static const float* cached[kMaxDevices] = {nullptr};
  static int cached_s[kMaxDevices] = {0};
  int dev = 0;
  DQ_CHECK_CUDA(cudaGetDevice(&dev));
  // While the stream is being captured the copy is always recorded, so that a replayed graph
  // carries its own matrix whatever was uploaded between capture and replay.  Outside capture
  // the copy is skipped when the same pointer was uploaded last; the upload is ordered on the
  // caller's stream only, so calls that bring a Hadamard matrix must share one stream per
  // device (or be ordered by the caller).
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  DQ_CHECK_CUDA(cudaStreamIsCapturing(stream, &cap));
  const bool capturing = cap != cudaStreamCaptureStatusNone;
  // Once an upload sits inside a graph, a replay can rewrite the table at any time behind the
  // back of this cache: from then on every call uploads.
  static bool seen_capture[kMaxDevices] = {false};
  if (capturing) seen_capture[dev] = true;
  if (!seen_capture[dev] && cached[dev] == had_mat && cached_s[dev] == S) return DQ_OK;
  void* sym = nullptr;
  void* stage = nullptr;
  DQ_CHECK_CUDA(cudaGetSymbolAddress(&sym, c_had_mat2));
  DQ_CHECK_CUDA(cudaGetSymbolAddress(&stage, g_had_stage));
  had_table_kernel<<<1, 1024, 0, stream>>>(had_mat, S);
  DQ_CHECK_CUDA(cudaGetLastError());
  DQ_CHECK_CUDA(cudaMemcpyAsync(sym, stage, sizeof(float2) * 32 * 32, cudaMemcpyDeviceToDevice, stream));
  // a captured copy has not run yet: whatever is cached no longer describes the table
  cached[dev] = capturing ? nullptr : had_mat;
  cached_s[dev] = capturing ? 0 : S;
  return DQ_OK;
}

// Picks the segmentation for the fast kernel; returns false when the shape is outside its range.
struct HadPlan {
  int S, R, inner, matrix;
};
static bool plan_fast_hadamard(const dq_hadamard_desc* had, int K, HadPlan* plan) {
  auto pow2 = [](int v) { return v > 0 && (v & (v - 1)) == 0; };
  if (had->kind == DQ_HAD_FULL && had->had_k > 1) {
    const int P = K / had->had_k;
    if (had->had_k > 32 || !pow2(P) || P < 32 || P > 1024) return false;
    *plan = {had->had_k, P / 32, 1, 1};
    return true;
  }
  if (had->kind == DQ_HAD_FULL) {  // pure Walsh-Hadamard of length K
    if (!pow2(K) || K < 64) return false;
    int P = K / 32 < 32 ? 32 : K / 32;   // S = K / P <= 32
    if (P > 1024) return false;
    *plan = {K / P, P / 32, 1, 0};
    return true;
  }
  if (had->kind == DQ_HAD_PARTIAL) {
    const int H = K / had->had_dim;
    if (H > 32 || !pow2(H)) return false;
    *plan = {H, 1, 0, 0};
    return true;
  }
  return false;
}

template <typename XT>
int init_had_fast_t() {
  constexpr int kHadMaxSmem = kHadFastMaxSmem;
  cudaError_t e = cudaSuccess;
#define DQ_HAD_ATTR(R)                                                                        \
  if (e == cudaSuccess)                                                                       \
    e = cudaFuncSetAttribute(act_quant_had_fast_kernel<R, XT, 512>,                             \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);        \
  if (e == cudaSuccess)                                                                       \
    e = cudaFuncSetAttribute(act_quant_had_fast_kernel<R, XT, 256>,                             \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);
  DQ_HAD_ATTR(1) DQ_HAD_ATTR(2) DQ_HAD_ATTR(4) DQ_HAD_ATTR(8) DQ_HAD_ATTR(16) DQ_HAD_ATTR(32)
#undef DQ_HAD_ATTR
#define DQ_HAD_ATTR28(R)                                                                      \
  if (e == cudaSuccess)                                                                       \
    e = cudaFuncSetAttribute(act_quant_had_fast_kernel<R, XT, 512, 28>,                         \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);        \
  if (e == cudaSuccess)                                                                       \
    e = cudaFuncSetAttribute(act_quant_had_fast_kernel<R, XT, 256, 28>,                         \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);
  DQ_HAD_ATTR28(2) DQ_HAD_ATTR28(4) DQ_HAD_ATTR28(8) DQ_HAD_ATTR28(16) DQ_HAD_ATTR28(32)
#undef DQ_HAD_ATTR28
#define DQ_HAD_ATTRC(R)                                                                       \
  if (e == cudaSuccess)                                                                       \
    e = cudaFuncSetAttribute(act_quant_had_cluster_kernel<R, XT>,                               \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
  DQ_HAD_ATTRC(4) DQ_HAD_ATTRC(8) DQ_HAD_ATTRC(16) DQ_HAD_ATTRC(32)
#undef DQ_HAD_ATTRC
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "cudaFuncSetAttribute(act_quant_had fast) failed: %s", cudaGetErrorString(e));
  return DQ_OK;
}

// Runs the fast (or, for a handful of rows, the cluster) kernel when the transform is one they cover;
// *taken tells the caller whether a launch was made.
template <typename XT>
int launch_had_fast_t(const XT* x, const XT* up, int64_t ldx, const float* a, const dq_hadamard_desc* had, int M, int K,
                      size_t smem, int8_t* codes, float* sx, float* out, int mode, int scale_fp16,
                      cudaStream_t stream, bool* taken) {
  *taken = false;
    HadPlan plan;
    if (plan_fast_hadamard(had, K, &plan)) {
      *taken = true;
      if (plan.matrix) {
        int rc2 = upload_had_matrix(had->had_mat, plan.S, stream);
        if (rc2 != DQ_OK) return rc2;
      }
      // across 2 ... 32 heads of 128 values, many rows: the register-only kernel
      if (had->kind == DQ_HAD_PARTIAL && had->had_dim == 128 && plan.S >= 2 && M >= kHeadsKernelMinRows &&
          up == nullptr && mode == MODE_CODES && codes != nullptr && (scale_fp16 & 0xFF) != 2) {
        const int rows_per_cta = (kHeadsKernelThreads / 32) * (plan.S == 32 ? 1 : 2);
        const dim3 grid((M + rows_per_cta - 1) / rows_per_cta);
#define DQ_HAD_HEADS(SS)                                                                                            \
  if ((scale_fp16 & kCodesE4M3) != 0)                                                                               \
    DQ_CHECK_CUDA(launch_pdl(act_quant_had_heads_kernel<SS, XT, true>, grid, dim3(kHeadsKernelThreads), 0, stream, x, \
                             ldx, a, M, had->scale, codes, sx, scale_fp16));                                        \
  else                                                                                                              \
    DQ_CHECK_CUDA(launch_pdl(act_quant_had_heads_kernel<SS, XT, false>, grid, dim3(kHeadsKernelThreads), 0, stream, x, \
                             ldx, a, M, had->scale, codes, sx, scale_fp16))
        switch (plan.S) {
          case 2: DQ_HAD_HEADS(2); break;
          case 4: DQ_HAD_HEADS(4); break;
          case 8: DQ_HAD_HEADS(8); break;
          case 16: DQ_HAD_HEADS(16); break;
          default: DQ_HAD_HEADS(32); break;
        }
#undef DQ_HAD_HEADS
        return DQ_OK;
      }
      // a handful of rows (decode): four CTAs per row
      if (plan.matrix && plan.inner && plan.S % kHadClusterCtas == 0 && M <= kHadClusterMaxRows && plan.R >= 4) {
        const int P = 32 * plan.R;
        const size_t csmem = static_cast<size_t>(plan.S / kHadClusterCtas * P + plan.S * (P / kHadClusterCtas)) * 4;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(kHadClusterCtas * M, 1, 1);
        cfg.blockDim = dim3(kHadClusterThreads, 1, 1);
        cfg.dynamicSmemBytes = csmem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = kHadClusterCtas;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
#define DQ_HAD_CLUSTER(RR)                                                                                  \
  DQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, act_quant_had_cluster_kernel<RR, XT>, x, up, ldx, a, plan.S, had->scale, \
                                   codes, sx, out, mode, scale_fp16))
        switch (plan.R) {
          case 4: DQ_HAD_CLUSTER(4); break;
          case 8: DQ_HAD_CLUSTER(8); break;
          case 16: DQ_HAD_CLUSTER(16); break;
          default: DQ_HAD_CLUSTER(32); break;
        }
#undef DQ_HAD_CLUSTER
        return DQ_OK;
      }
      // many rows: smaller CTAs, several per SM (the row must leave room for three of them)
      const DeviceState* dst = current_state();
      const bool small_cta = dst != nullptr && M > 2 * dst->sm_count && smem <= 72 * 1024;
#define DQ_HAD_FAST_T(RR, TT, HH)                                                                      \
  DQ_CHECK_CUDA(launch_pdl(act_quant_had_fast_kernel<RR, XT, TT, HH>, dim3(M), dim3(TT), smem, stream, x, up, \
                           ldx, a, K, plan.S, plan.inner, plan.matrix, had->scale, had->had_mat, codes, sx,   \
                           out, mode, scale_fp16))
#define DQ_HAD_FAST(RR)                                            \
  if (plan.matrix && plan.S == 28 && RR >= 2) {                    \
    if (small_cta) DQ_HAD_FAST_T(RR, 256, 28);                     \
    else DQ_HAD_FAST_T(RR, 512, 28);                               \
  } else if (small_cta) {                                          \
    DQ_HAD_FAST_T(RR, 256, 0);                                     \
  } else {                                                         \
    DQ_HAD_FAST_T(RR, 512, 0);                                     \
  }
      switch (plan.R) {
        case 1: DQ_HAD_FAST(1); break;
        case 2: DQ_HAD_FAST(2); break;
        case 4: DQ_HAD_FAST(4); break;
        case 8: DQ_HAD_FAST(8); break;
        case 16: DQ_HAD_FAST(16); break;
        default: DQ_HAD_FAST(32); break;
      }
#undef DQ_HAD_FAST
#undef DQ_HAD_FAST_T
      return DQ_OK;
    }
  return DQ_OK;
}

}  // namespace
}  // namespace dq
