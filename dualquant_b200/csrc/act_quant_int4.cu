// Per-token int4 activation quantiser (the runtime half of PermLinear) for sm_100a.
//
//   x32 = float(x) * a[k]            fp32 multiply, no contraction
//   x32 = online Hadamard(x32)       optional (QuaRot R4 "full" / R2 "partial")
//   s   = absmax(x32) / 7            IEEE division; 1 when the row is all zero; optional fp16 round
//   q   = clamp(rint(x32 / s), -8, 7)   IEEE division, round-half-even
//
// Two kernels, one CTA per token row:
//   * rows_kernel: row held in registers (no Hadamard) - one global read, one write.
//   * had_kernel : row staged in shared memory as fp32, butterflies in place, then the same tail.
// Both are HBM-bound streaming kernels (2 bytes in, 1 byte out per element).
#include "dq_common.h"
#include "dq_ptx.cuh"
#include "dq_quant.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace dq {

enum { MODE_CODES = 0, MODE_FAKE = 1, MODE_RAW = 2, MODE_FAKE_BF16 = 3 };

// Row `row` of the de-quantised output: fp32 elements, or bf16 elements for MODE_FAKE_BF16 (the
// pointer type stays float*; emit8 casts it back).
__device__ __forceinline__ float* out_row_ptr(float* out, int64_t row, int K, int mode) {
  if (out == nullptr) return nullptr;
  if (mode == MODE_FAKE_BF16)
    return reinterpret_cast<float*>(reinterpret_cast<__nv_bfloat16*>(out) + row * K);
  return out + row * K;
}

__device__ __forceinline__ float block_max(float v, float* red, int nwarps) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // red may still be read from a previous use
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float m = red[0];
  for (int i = 1; i < nwarps; ++i) m = fmaxf(m, red[i]);
  return m;
}

__device__ __forceinline__ float block_sum(float v, float* red, int nwarps) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // red may still be read from a previous use
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float m = red[0];
  for (int i = 1; i < nwarps; ++i) m += red[i];
  return m;
}

__device__ __forceinline__ float bf16_round(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void load8(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// SiLU(gate) * up the way a bf16 decoder computes it: SiLU evaluated in fp32 and rounded to
// bf16, the product rounded to bf16 again.
__device__ __forceinline__ float silu_mul_bf16(float g, float u) {
  const float sg = __fdiv_rn(g, 1.0f + expf(-g));
  const float sgb = __bfloat162float(__float2bfloat16_rn(sg));
  return __bfloat162float(__float2bfloat16_rn(__fmul_rn(sgb, u)));
}
template <typename XT>
__device__ __forceinline__ void apply_gate(const XT* up_ptr, float* v) {
  if (up_ptr != nullptr) {
    float u[8];
    load8(up_ptr, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = silu_mul_bf16(v[e], u[e]);
  }
}

// Eight input elements as loaded (bf16: one 16-byte vector; fp32: two).
template <typename XT>
struct Raw8;
template <>
struct Raw8<__nv_bfloat16> {
  uint4 r;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { r = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void expand(float* v) const {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
};
template <>
struct Raw8<float> {
  float4 lo, hi;
  __device__ __forceinline__ void load(const float* p) {
    lo = *reinterpret_cast<const float4*>(p);
    hi = *reinterpret_cast<const float4*>(p + 4);
  }
  __device__ __forceinline__ void expand(float* v) const {
    v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
    v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
  }
};

__device__ __forceinline__ void emit8(const float* v, float s, int mode, int8_t* codes_row,
                                      float* out_row, int idx, int smode = 0) {
  const float inv_s = __fdiv_rn(1.0f, s);
  const bool e4m3 = (smode & kCodesE4M3) != 0;
  smode &= 0xFF;
  if (smode == 2 && mode != MODE_RAW) {
    // bf16 arithmetic (see token_scale): codes, or the de-quantised value q * s as fp32 / bf16
    float q[8];
    quant_codes8_bf16(v, s, q);
    if (mode == MODE_CODES) {
      *reinterpret_cast<uint2*>(codes_row + idx) =
          e4m3 ? make_uint2(pack_codes4_e4m3(q[0], q[1], q[2], q[3]), pack_codes4_e4m3(q[4], q[5], q[6], q[7]))
               : make_uint2(pack_codes4(q[0], q[1], q[2], q[3]), pack_codes4(q[4], q[5], q[6], q[7]));
    } else if (mode == MODE_FAKE_BF16) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const __nv_bfloat162 pr = __floats2bfloat162_rn(__fmul_rn(q[2 * e], s), __fmul_rn(q[2 * e + 1], s));
        w[e] = *reinterpret_cast<const uint32_t*>(&pr);
      }
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out_row) + idx) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = round_to_bf16(__fmul_rn(q[e], s));
      *reinterpret_cast<float4*>(out_row + idx) = make_float4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<float4*>(out_row + idx + 4) = make_float4(o[4], o[5], o[6], o[7]);
    }
    return;
  }
  if (mode == MODE_CODES) {
    float q[8];
    quant_codes8(v, s, inv_s, q);
    const uint32_t lo = e4m3 ? pack_codes4_e4m3(q[0], q[1], q[2], q[3]) : pack_codes4(q[0], q[1], q[2], q[3]);
    const uint32_t hi = e4m3 ? pack_codes4_e4m3(q[4], q[5], q[6], q[7]) : pack_codes4(q[4], q[5], q[6], q[7]);
    *reinterpret_cast<uint2*>(codes_row + idx) = make_uint2(lo, hi);
  } else if (mode == MODE_FAKE_BF16) {
    float o[8];
    quant_codes8(v, s, inv_s, o);
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat162 pr = __floats2bfloat162_rn(__fmul_rn(o[2 * e], s), __fmul_rn(o[2 * e + 1], s));
      w[e] = *reinterpret_cast<const uint32_t*>(&pr);
    }
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out_row) + idx) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    float o[8];
    if (mode == MODE_FAKE) {
      quant_codes8(v, s, inv_s, o);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = __fmul_rn(o[e], s);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = v[e];
    }
    *reinterpret_cast<float4*>(out_row + idx) = make_float4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<float4*>(out_row + idx + 4) = make_float4(o[4], o[5], o[6], o[7]);
  }
}

// ---------------------------------------------------------------------------------------------
// register-resident rows (no Hadamard)
// ---------------------------------------------------------------------------------------------
// norm_eps >= 0 puts an RMSNorm in front (the reference's _RMSNbf16Safe, quarot/llama_quarot.py:
// 135-141, and HF's LlamaRMSNorm): v = bf16(x * rsqrt(mean(x^2) + eps)), times the bf16 weight
// (rounded to bf16 again) when norm_w is given - exactly the bf16 tensor the separate norm would
// have written and the quantiser read back.
// KEEP: the scaled values of the absmax pass stay in registers for the code pass (many-rows launch
// shape, where the kernel is bound by instruction issue and registers are plentiful) instead of
// being re-expanded from the raw row (few-rows shape, where occupancy hides latency).
template <int THREADS, int VPT, typename XT, bool KEEP = false>
__global__ void __launch_bounds__(THREADS, (THREADS >= 512 && VPT <= 2) ? 2048 / THREADS : 1)
act_quant_rows_kernel(const XT* __restrict__ x, int64_t ldx, const float* __restrict__ a, int K,
                      int8_t* __restrict__ codes, float* __restrict__ sx, float* __restrict__ out,
                      int mode, int scale_fp16, const __nv_bfloat16* __restrict__ norm_w,
                      float norm_eps) {
  __shared__ float red[THREADS / 32];
  // the GEMM that consumes the codes may be launched programmatically: let it start streaming
  // its weights now; it waits for this grid before it touches codes / sx
  grid_dep_launch_dependents();
  grid_dep_wait();  // x may come from the kernel before this one; codes / sx may still be read by it
  const int row = blockIdx.x;
  const XT* xr = x + static_cast<int64_t>(row) * ldx;
  // The row is held in registers in its input width (bf16: 4 registers per 8 elements) and
  // expanded once per pass - sum of squares (with a norm), absmax, codes - with identical
  // arithmetic, so that twice as many rows fit in the register file and more loads are in
  // flight per SM.
  Raw8<XT> raw[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = (i * THREADS + threadIdx.x) * 8;
    if (idx < K) raw[i].load(xr + idx);
  }
  const bool norm = norm_eps >= 0.f;
  float inv_rms = 1.f;
  if (norm) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = (i * THREADS + threadIdx.x) * 8;
      if (idx < K) {
        float v[8];
        raw[i].expand(v);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
      }
    }
    ss = block_sum(ss, red, THREADS / 32);
    inv_rms = rsqrtf(__fadd_rn(__fdiv_rn(ss, static_cast<float>(K)), norm_eps));
  }
  auto prologue = [&](float* v, int idx) {
    if (norm) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = bf16_round(__fmul_rn(v[e], inv_rms));
      if (norm_w != nullptr) {
        Raw8<__nv_bfloat16> wr;
        wr.load(norm_w + idx);
        float wv[8];
        wr.expand(wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = bf16_round(__fmul_rn(wv[e], v[e]));
      }
    }
    if (a != nullptr) {
      float av[8];
      load8(a + idx, av);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(v[e], av[e]);
    }
  };
  float amax = 0.f;
  float kept[KEEP ? VPT : 1][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = (i * THREADS + threadIdx.x) * 8;
    if (idx < K) {
      float v[8];
      raw[i].expand(v);
      prologue(v, idx);
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
      if constexpr (KEEP) {
#pragma unroll
        for (int e = 0; e < 8; ++e) kept[i][e] = v[e];
      }
    }
  }
  amax = block_max(amax, red, THREADS / 32);
  const float s = token_scale(amax, scale_fp16);
  if (threadIdx.x == 0 && sx != nullptr) sx[row] = s;
  int8_t* crow = (codes != nullptr) ? codes + static_cast<int64_t>(row) * K : nullptr;
  float* orow = out_row_ptr(out, row, K, mode);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = (i * THREADS + threadIdx.x) * 8;
    if (idx < K) {
      if constexpr (KEEP) {
        emit8(kept[i], s, mode, crow, orow, idx, scale_fp16);
      } else {
        float v[8];
        raw[i].expand(v);
        prologue(v, idx);
        emit8(v, s, mode, crow, orow, idx, scale_fp16);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// shared-memory rows with the online Hadamard
// ---------------------------------------------------------------------------------------------
// One radix-2 stage over the whole row: element index = (hi*2h + lo)*stride + c pairs with
// + h*stride; (a, b) -> (a + b, a - b).  stride = 1 for the "full" transform (independent
// contiguous segments whose length is a multiple of 2h), stride = head_dim for the "partial"
// one (butterflies across the head index).  Stages run in the order h = 1, 2, 4, ... so every
// sum is formed exactly as in the reference's butterfly loop.
template <int THREADS>
__device__ __forceinline__ void wht_stage(float* row, int K, int h, int stride) {
  for (int b = threadIdx.x; b < K / 2; b += THREADS) {
    const int c = b % stride;
    const int hb = b / stride;
    const int i = ((hb / h) * 2 * h + (hb % h)) * stride + c;
    const int j = i + h * stride;
    const float u = row[i], w = row[j];
    row[i] = __fadd_rn(u, w);
    row[j] = __fsub_rn(u, w);
  }
}

constexpr int kMaxHadK = 32;

template <int THREADS, typename XT>
__global__ void __launch_bounds__(THREADS)
act_quant_had_kernel(const XT* __restrict__ x, const XT* __restrict__ up, int64_t ldx,
                     const float* __restrict__ a, int K,
                     int had_kind, int had_k, int had_dim, float had_scale,
                     const float* __restrict__ had_mat, int8_t* __restrict__ codes,
                     float* __restrict__ sx, float* __restrict__ out, int mode, int scale_fp16) {
  extern __shared__ float sm_row[];
  __shared__ float red[THREADS / 32];
  float* row = sm_row;
  float* hm = sm_row + K;  // [had_k, had_k] when had_k > 1
  grid_dep_launch_dependents();
  grid_dep_wait();
  const int r = blockIdx.x;
  const XT* xr = x + static_cast<int64_t>(r) * ldx;
  const XT* ur = (up != nullptr) ? up + static_cast<int64_t>(r) * ldx : nullptr;

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
#pragma unroll
    for (int e = 0; e < 8; ++e) row[idx + e] = v[e];
  }
  if (had_kind == DQ_HAD_FULL && had_k > 1)
    for (int i = threadIdx.x; i < had_k * had_k; i += THREADS) hm[i] = had_mat[i];
  __syncthreads();

  if (had_kind == DQ_HAD_FULL) {
    const int P = K / had_k;  // Walsh-Hadamard length of each contiguous segment
    for (int h = 1; h < P; h <<= 1) {
      wht_stage<THREADS>(row, K, h, 1);
      __syncthreads();
    }
    if (had_k > 1) {
      // out[i][c] = sum_j H[i][j] * (v[j][c] * scale), j ascending, fp32
      for (int c = threadIdx.x; c < P; c += THREADS) {
        float v[kMaxHadK];
#pragma unroll
        for (int j = 0; j < kMaxHadK; ++j)
          v[j] = (j < had_k) ? __fmul_rn(row[j * P + c], had_scale) : 0.f;
        for (int i = 0; i < had_k; ++i) {
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < kMaxHadK; ++j)
            if (j < had_k) acc = __fadd_rn(acc, __fmul_rn(hm[i * had_k + j], v[j]));
          row[i * P + c] = acc;
        }
      }
    } else {
      for (int i = threadIdx.x; i < K; i += THREADS) row[i] = __fmul_rn(row[i], had_scale);
    }
    __syncthreads();
  } else if (had_kind == DQ_HAD_PARTIAL) {
    const int H = K / had_dim;
    for (int h = 1; h < H; h <<= 1) {
      wht_stage<THREADS>(row, K, h, had_dim);
      __syncthreads();
    }
    for (int i = threadIdx.x; i < K; i += THREADS) row[i] = __fmul_rn(row[i], had_scale);
    __syncthreads();
  }

  float s = 1.f;
  if (mode != MODE_RAW) {
    float amax = 0.f;
    for (int i = threadIdx.x; i < K; i += THREADS) amax = fmaxf(amax, fabsf(row[i]));
    amax = block_max(amax, red, THREADS / 32);
    s = token_scale(amax, scale_fp16);
    if (threadIdx.x == 0 && sx != nullptr) sx[r] = s;
  }
  int8_t* crow = (codes != nullptr) ? codes + static_cast<int64_t>(r) * K : nullptr;
  float* orow = out_row_ptr(out, r, K, mode);
  for (int idx = threadIdx.x * 8; idx < K; idx += THREADS * 8) {
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = row[idx + e];
    emit8(v, s, mode, crow, orow, idx, scale_fp16);
  }
}

// ---------------------------------------------------------------------------------------------
// full online Hadamard with a large +-1 factor (orders 36 ... 172 of the reference's table)
// ---------------------------------------------------------------------------------------------
// Same arithmetic as act_quant_had_kernel for had_k up to kMaxHadKBig: the row (as fp32) and a
// second buffer of the same size sit in shared memory next to the factor stored as one byte per
// entry.  Walsh-Hadamard stages over the contiguous segments in place, then one thread per output
// element: out[i][c] = sum_j H[i][j] * (v[j][c] * scale), j ascending, fp32 - the order of the
// stand-alone restatement, so codes stay bit-identical.  Used for decode-size batches of models
// whose intermediate size is not 28 * 2^k (e.g. 11008 = 172 * 64); not a tuned path.
constexpr int kMaxHadKBig = 172;

template <int THREADS, typename XT>
__global__ void __launch_bounds__(THREADS)
act_quant_had_big_kernel(const XT* __restrict__ x, const XT* __restrict__ up, int64_t ldx,
                         const float* __restrict__ a, int K, int had_k, float had_scale,
                         const float* __restrict__ had_mat, int8_t* __restrict__ codes,
                         float* __restrict__ sx, float* __restrict__ out, int mode, int scale_fp16) {
  extern __shared__ float sm_row[];
  __shared__ float red[THREADS / 32];
  float* row = sm_row;
  float* res = sm_row + K;
  signed char* hm = reinterpret_cast<signed char*>(sm_row + 2 * K);
  grid_dep_launch_dependents();
  grid_dep_wait();
  const int r = blockIdx.x;
  const XT* xr = x + static_cast<int64_t>(r) * ldx;
  const XT* ur = (up != nullptr) ? up + static_cast<int64_t>(r) * ldx : nullptr;
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
#pragma unroll
    for (int e = 0; e < 8; ++e) row[idx + e] = v[e];
  }
  for (int i = threadIdx.x; i < had_k * had_k; i += THREADS) hm[i] = had_mat[i] > 0.f ? 1 : -1;
  __syncthreads();
  const int P = K / had_k;
  for (int h = 1; h < P; h <<= 1) {
    wht_stage<THREADS>(row, K, h, 1);
    __syncthreads();
  }
  for (int i = threadIdx.x; i < K; i += THREADS) row[i] = __fmul_rn(row[i], had_scale);
  __syncthreads();
  for (int o = threadIdx.x; o < K; o += THREADS) {
    const int i = o / P, c = o - i * P;
    const signed char* hrow = hm + i * had_k;
    float acc = 0.f;
    for (int j = 0; j < had_k; ++j) {
      const float v = row[j * P + c];
      acc = __fadd_rn(acc, hrow[j] > 0 ? v : -v);
    }
    res[o] = acc;
  }
  __syncthreads();
  float s = 1.f;
  if (mode != MODE_RAW) {
    float amax = 0.f;
    for (int i = threadIdx.x; i < K; i += THREADS) amax = fmaxf(amax, fabsf(res[i]));
    amax = block_max(amax, red, THREADS / 32);
    s = token_scale(amax, scale_fp16);
    if (threadIdx.x == 0 && sx != nullptr) sx[r] = s;
  }
  int8_t* crow = (codes != nullptr) ? codes + static_cast<int64_t>(r) * K : nullptr;
  float* orow = out_row_ptr(out, r, K, mode);
  for (int idx = threadIdx.x * 8; idx < K; idx += THREADS * 8) {
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = res[idx + e];
    emit8(v, s, mode, crow, orow, idx, scale_fp16);
  }
}

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
__device__ __forceinline__ void wht_segment_warp(float* seg, int lane) {
  // lane l holds elements l + 32 r (r < R): conflict-free shared-memory access; stages h < 32
  // pair lanes (shuffle), stages h >= 32 pair registers r and r + h/32.  Stage order h = 1, 2, ...
  float v[R];
#pragma unroll
  for (int r = 0; r < R; ++r) v[r] = seg[lane + 32 * r];
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    const bool upper = (lane & m) != 0;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float other = __shfl_xor_sync(0xffffffffu, v[r], m);
      v[r] = upper ? __fsub_rn(other, v[r]) : __fadd_rn(v[r], other);
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
#pragma unroll
  for (int r = 0; r < R; ++r) seg[lane + 32 * r] = v[r];
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
    for (int sgm = warp; sgm < S; sgm += THREADS / 32) wht_segment_warp<R>(row + sgm * P, lane);
    __syncthreads();
  }

  float amax = 0.f;
  if (matrix) {
    // two adjacent columns per thread (P is even): packed loads, packed FMAs
    constexpr int HN = (HS > 0) ? HS : 32;  // factor order known at compile time, or padded to 32
    for (int c = 2 * threadIdx.x; c < P; c += 2 * THREADS) {
      float2 v[HN];
#pragma unroll
      for (int j = 0; j < HN; ++j) {
        v[j] = (j < S) ? *reinterpret_cast<const float2*>(row + j * P + c) : make_float2(0.f, 0.f);
        v[j].x = __fmul_rn(v[j].x, had_scale);
        v[j].y = __fmul_rn(v[j].y, had_scale);
      }
      // fully unrolled so that every coefficient is a constant-bank operand of its FMA and the
      // independent accumulation chains can be interleaved
#pragma unroll
      for (int i = 0; i < HN; ++i) {
        if (i < S) {
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

constexpr int kHadThreads = 512;
constexpr int kHadMaxSmem = 200 * 1024;

int init_act_quant_kernels() {
  cudaError_t e = cudaFuncSetAttribute(act_quant_had_kernel<kHadThreads, __nv_bfloat16>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(act_quant_had_big_kernel<kHadThreads, __nv_bfloat16>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(act_quant_had_big_kernel<kHadThreads, float>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(act_quant_had_kernel<kHadThreads, float>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);
#define DQ_HAD_ATTR(R, T)                                                                     \
  if (e == cudaSuccess)                                                                       \
    e = cudaFuncSetAttribute(act_quant_had_fast_kernel<R, T, 512>,                              \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);        \
  if (e == cudaSuccess)                                                                       \
    e = cudaFuncSetAttribute(act_quant_had_fast_kernel<R, T, 256>,                              \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);
  DQ_HAD_ATTR(1, __nv_bfloat16) DQ_HAD_ATTR(2, __nv_bfloat16) DQ_HAD_ATTR(4, __nv_bfloat16)
  DQ_HAD_ATTR(8, __nv_bfloat16) DQ_HAD_ATTR(16, __nv_bfloat16) DQ_HAD_ATTR(32, __nv_bfloat16)
  DQ_HAD_ATTR(1, float) DQ_HAD_ATTR(2, float) DQ_HAD_ATTR(4, float)
  DQ_HAD_ATTR(8, float) DQ_HAD_ATTR(16, float) DQ_HAD_ATTR(32, float)
#undef DQ_HAD_ATTR
#define DQ_HAD_ATTR28(R, T)                                                                   \
  if (e == cudaSuccess)                                                                       \
    e = cudaFuncSetAttribute(act_quant_had_fast_kernel<R, T, 512, 28>,                          \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);        \
  if (e == cudaSuccess)                                                                       \
    e = cudaFuncSetAttribute(act_quant_had_fast_kernel<R, T, 256, 28>,                          \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);
  DQ_HAD_ATTR28(16, __nv_bfloat16) DQ_HAD_ATTR28(32, __nv_bfloat16) DQ_HAD_ATTR28(16, float) DQ_HAD_ATTR28(32, float)
#undef DQ_HAD_ATTR28
#define DQ_HAD_ATTRC(R, T)                                                                    \
  if (e == cudaSuccess)                                                                       \
    e = cudaFuncSetAttribute(act_quant_had_cluster_kernel<R, T>,                                \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
  DQ_HAD_ATTRC(4, __nv_bfloat16) DQ_HAD_ATTRC(8, __nv_bfloat16) DQ_HAD_ATTRC(16, __nv_bfloat16)
  DQ_HAD_ATTRC(32, __nv_bfloat16) DQ_HAD_ATTRC(4, float) DQ_HAD_ATTRC(8, float) DQ_HAD_ATTRC(16, float)
  DQ_HAD_ATTRC(32, float)
#undef DQ_HAD_ATTRC
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "cudaFuncSetAttribute(act_quant_had) failed: %s",
                     cudaGetErrorString(e));
  return DQ_OK;
}

static bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

static int check_had(const dq_hadamard_desc* had, int K) {
  if (had == nullptr || had->kind == DQ_HAD_NONE) return DQ_OK;
  if (had->kind == DQ_HAD_FULL) {
    DQ_REQUIRE(had->had_k >= 1 && had->had_k <= kMaxHadKBig, DQ_ERR_UNSUPPORTED,
               "had_k=%d outside [1,%d]", had->had_k, kMaxHadKBig);
    DQ_REQUIRE(K % had->had_k == 0 && is_pow2(K / had->had_k), DQ_ERR_SHAPE,
               "K=%d is not had_k=%d times a power of two", K, had->had_k);
    DQ_REQUIRE(had->had_k == 1 || had->had_mat != nullptr, DQ_ERR_NULL, "had_mat is null");
    return DQ_OK;
  }
  if (had->kind == DQ_HAD_PARTIAL) {
    DQ_REQUIRE(had->had_k == 1, DQ_ERR_UNSUPPORTED,
               "partial Hadamard with a non-power-of-two head count is not implemented");
    DQ_REQUIRE(had->had_dim >= 1 && K % had->had_dim == 0 && is_pow2(K / had->had_dim),
               DQ_ERR_SHAPE, "K=%d / had_dim=%d must be a power of two", K, had->had_dim);
    return DQ_OK;
  }
  return set_error(DQ_ERR_UNSUPPORTED, "unknown Hadamard kind %d", had->kind);
}

template <typename XT>
static int launch_act(const XT* x, int64_t ldx, const float* a, const dq_hadamard_desc* had, int M,
                      int K, int8_t* codes, float* sx, float* out, int mode, int scale_fp16,
                      cudaStream_t stream, const XT* up = nullptr,
                      const __nv_bfloat16* norm_w = nullptr, float norm_eps = -1.f) {
  DQ_REQUIRE(x != nullptr, DQ_ERR_NULL, "x is null");
  DQ_REQUIRE(M >= 0 && K >= 8 && K % 8 == 0, DQ_ERR_SHAPE, "bad shape M=%d K=%d (K %% 8 != 0)", M, K);
  DQ_REQUIRE(ldx >= K && ldx % 8 == 0, DQ_ERR_ALIGN, "ldx=%lld must be >= K and a multiple of 8",
             (long long)ldx);
  DQ_REQUIRE(aligned(x, 16) && (a == nullptr || aligned(a, 16)), DQ_ERR_ALIGN,
             "x and a must be 16-byte aligned");
  DQ_REQUIRE((codes == nullptr || aligned(codes, 8)) && (out == nullptr || aligned(out, 16)),
             DQ_ERR_ALIGN, "outputs must be aligned (codes 8 B, out 16 B)");
  DQ_REQUIRE(K <= 65536, DQ_ERR_UNSUPPORTED, "K=%d exceeds 65536", K);
  int rc = check_had(had, K);
  if (rc != DQ_OK) return rc;
  if (M == 0) return DQ_OK;
  const bool use_had = had != nullptr && had->kind != DQ_HAD_NONE;
  DQ_REQUIRE(norm_eps < 0.f || (!use_had && up == nullptr && mode != MODE_RAW && K <= 32768),
             DQ_ERR_UNSUPPORTED, "the fused RMSNorm covers plain rows of K <= 32768 without a Hadamard");
  if (use_had || mode == MODE_RAW || K > 32768 || up != nullptr) {  // longer rows than the register path holds
    const int hk = use_had ? had->had_k : 1;
    if (use_had && had->kind == DQ_HAD_FULL && hk > kMaxHadK) {
      // large +-1 factor: row + result buffer + the factor as bytes
      const size_t big = static_cast<size_t>(K) * 8 + (static_cast<size_t>(hk) * hk + 15) / 16 * 16;
      DQ_REQUIRE(big <= static_cast<size_t>(kHadMaxSmem), DQ_ERR_UNSUPPORTED,
                 "row of K=%d with a Hadamard factor of order %d does not fit in shared memory", K, hk);
      DQ_CHECK_CUDA(launch_pdl(act_quant_had_big_kernel<kHadThreads, XT>, dim3(M), dim3(kHadThreads), big,
                               stream, x, up, ldx, a, K, hk, had->scale, had->had_mat, codes, sx, out, mode,
                               scale_fp16));
      DQ_CHECK_CUDA(cudaGetLastError());
      return DQ_OK;
    }
    const size_t smem = static_cast<size_t>(K) * 4 + (hk > 1 ? static_cast<size_t>(hk) * hk * 4 : 0);
    DQ_REQUIRE(smem <= static_cast<size_t>(kHadMaxSmem), DQ_ERR_UNSUPPORTED,
               "row of K=%d does not fit in shared memory", K);
    HadPlan plan;
    if (use_had && plan_fast_hadamard(had, K, &plan)) {
      if (plan.matrix) {
        int rc2 = upload_had_matrix(had->had_mat, plan.S, stream);
        if (rc2 != DQ_OK) return rc2;
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
  if (plan.matrix && plan.S == 28 && (RR == 16 || RR == 32)) {     \
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
    DQ_CHECK_CUDA(launch_pdl(act_quant_had_kernel<kHadThreads, XT>, dim3(M), dim3(kHadThreads), smem,
                             stream, x, up, ldx, a, K, use_had ? had->kind : DQ_HAD_NONE, hk,
                             use_had ? had->had_dim : 0, use_had ? had->scale : 1.f,
                             use_had ? had->had_mat : nullptr, codes, sx, out, mode, scale_fp16));
  } else {
    // one CTA per row; as many threads as the row has 16-byte vectors (up to 1024) so that each
    // thread holds few elements and many warps are resident to hide the load -> reduce -> store
    // latency chain
    const int vec = K / 8;
#define DQ_ROWS_LAUNCH_K(T, V, KP)                                                                \
  DQ_CHECK_CUDA(launch_pdl(act_quant_rows_kernel<T, V, XT, KP>, dim3(M), dim3(T), 0, stream, x, ldx, a, K, \
                           codes, sx, out, mode, scale_fp16, norm_w, norm_eps))
#define DQ_ROWS_LAUNCH(T, V) DQ_ROWS_LAUNCH_K(T, V, false)
    constexpr int kBigM = 1024;
    // Many rows (prefill): fewer threads per row, each with four 16-byte loads in flight - the
    // kernel is then bound by bytes in flight per SM, not by the per-row latency chain.
    if (M >= kBigM && vec > 128 && vec <= 512) DQ_ROWS_LAUNCH_K(128, 4, true);
    else if (M >= kBigM && vec > 512 && vec <= 1024) DQ_ROWS_LAUNCH_K(256, 4, true);
    else if (M >= kBigM && vec > 1024 && vec <= 2048) DQ_ROWS_LAUNCH_K(512, 4, true);
    else if (vec <= 128) DQ_ROWS_LAUNCH(128, 1);
    else if (vec <= 256) DQ_ROWS_LAUNCH(256, 1);
    else if (vec <= 512) DQ_ROWS_LAUNCH(512, 1);
    else if (vec <= 1024) DQ_ROWS_LAUNCH(1024, 1);
    else if (vec <= 2048) DQ_ROWS_LAUNCH(1024, 2);
    else DQ_ROWS_LAUNCH(1024, 4);
#undef DQ_ROWS_LAUNCH
#undef DQ_ROWS_LAUNCH_K
  }
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}

// ---------------------------------------------------------------------------------------------
// one activation scale per (token, group of 128): the quantiser of the reference's fused W4A4
// Triton kernel (per row and K tile) as a stand-alone pass
// ---------------------------------------------------------------------------------------------
// One warp per (token, group); a lane holds four consecutive elements.  IEEE divisions (this
// variant is not on the measured path).  round_away = 1 rounds halves away from zero like the
// Triton kernel's libdevice.round, 0 rounds them to even like torch.round.
__global__ void __launch_bounds__(256)
act_quant_grouped_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const float* __restrict__ a,
                         int M, int K, int8_t* __restrict__ codes, float* __restrict__ sxg,
                         int scale_fp16, int round_away) {
  grid_dep_launch_dependents();
  grid_dep_wait();
  const int groups = K / kGroup;
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // (token, group)
  if (unit >= M * groups) return;
  const int m = unit / groups, g = unit % groups;
  const int lane = threadIdx.x & 31;
  const int k0 = g * kGroup + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(x + static_cast<int64_t>(m) * ldx + k0);
  float v[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u),
                __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000u)};
  if (a != nullptr) {
    const float4 av = *reinterpret_cast<const float4*>(a + k0);
    v[0] = __fmul_rn(v[0], av.x); v[1] = __fmul_rn(v[1], av.y);
    v[2] = __fmul_rn(v[2], av.z); v[3] = __fmul_rn(v[3], av.w);
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = token_scale(amax, scale_fp16);
  if (lane == 0) sxg[static_cast<size_t>(g) * M + m] = s;
  int q[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float t = __fdiv_rn(v[e], s);
    const float rq = round_away ? roundf(t) : rintf(t);
    q[e] = static_cast<int>(fminf(fmaxf(rq, -8.0f), 7.0f));
  }
  const uint32_t packed = (static_cast<uint32_t>(q[0]) & 0xFFu) | ((static_cast<uint32_t>(q[1]) & 0xFFu) << 8) |
                          ((static_cast<uint32_t>(q[2]) & 0xFFu) << 16) | ((static_cast<uint32_t>(q[3]) & 0xFFu) << 24);
  *reinterpret_cast<uint32_t*>(codes + static_cast<int64_t>(m) * K + k0) = packed;
}

}  // namespace dq

using namespace dq;

extern "C" int dq_quant_act_int4_grouped(const void* x_bf16, int64_t ldx, const float* a, int M, int K,
                                         int G, int8_t* codes, float* sx_groups, int scale_fp16,
                                         int round_away, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(x_bf16 != nullptr && codes != nullptr && sx_groups != nullptr, DQ_ERR_NULL, "null x / codes / sx_groups");
  DQ_REQUIRE(G == kGroup, DQ_ERR_UNSUPPORTED, "activation group size must be %d (got %d)", kGroup, G);
  DQ_REQUIRE(M >= 0 && K >= kGroup && K % kGroup == 0, DQ_ERR_SHAPE, "bad shape M=%d K=%d", M, K);
  DQ_REQUIRE(ldx >= K && ldx % 4 == 0, DQ_ERR_ALIGN, "ldx=%lld must be >= K and a multiple of 4", (long long)ldx);
  DQ_REQUIRE(aligned(x_bf16, 8) && (a == nullptr || aligned(a, 16)) && aligned(codes, 4), DQ_ERR_ALIGN,
             "x (8 B), a (16 B) and codes (4 B) must be aligned");
  const int64_t units = static_cast<int64_t>(M) * (K / kGroup);
  DQ_REQUIRE(units < (1ll << 31), DQ_ERR_SHAPE, "too many (token, group) units");
  const int per_cta = 8;
  DQ_CHECK_CUDA(launch_pdl(act_quant_grouped_kernel, dim3(static_cast<unsigned>((units + per_cta - 1) / per_cta)),
                           dim3(per_cta * 32), 0, static_cast<cudaStream_t>(stream),
                           static_cast<const __nv_bfloat16*>(x_bf16), ldx, a, M, K, codes, sx_groups,
                           scale_fp16, round_away));
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}

extern "C" int dq_quant_act_int4(const void* x_bf16, int64_t ldx, const float* a,
                                 const dq_hadamard_desc* had, int M, int K, int8_t* codes,
                                 float* sx, int scale_fp16, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(codes != nullptr && sx != nullptr, DQ_ERR_NULL, "codes / sx is null");
  return launch_act(static_cast<const __nv_bfloat16*>(x_bf16), ldx, a, had, M, K, codes, sx,
                    nullptr, MODE_CODES, scale_fp16, static_cast<cudaStream_t>(stream));
}

extern "C" int dq_quant_act_int4_f32(const float* x_f32, int64_t ldx, const float* a,
                                     const dq_hadamard_desc* had, int M, int K, int8_t* codes,
                                     float* sx, int scale_fp16, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(codes != nullptr && sx != nullptr, DQ_ERR_NULL, "codes / sx is null");
  return launch_act(x_f32, ldx, a, had, M, K, codes, sx, nullptr, MODE_CODES, scale_fp16,
                    static_cast<cudaStream_t>(stream));
}

extern "C" int dq_quant_act_int4_rmsnorm(const void* x_bf16, int64_t ldx, const void* norm_weight_bf16,
                                         float eps, const float* a, int M, int K, int8_t* codes,
                                         float* sx, int scale_fp16, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(codes != nullptr && sx != nullptr, DQ_ERR_NULL, "codes / sx is null");
  DQ_REQUIRE(eps >= 0.f, DQ_ERR_SHAPE, "eps must be >= 0 (got %g)", (double)eps);
  DQ_REQUIRE(norm_weight_bf16 == nullptr || aligned(norm_weight_bf16, 16), DQ_ERR_ALIGN,
             "norm weight must be 16-byte aligned");
  return launch_act(static_cast<const __nv_bfloat16*>(x_bf16), ldx, a, nullptr, M, K, codes, sx,
                    nullptr, MODE_CODES, scale_fp16, static_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(nullptr),
                    static_cast<const __nv_bfloat16*>(norm_weight_bf16), eps);
}

extern "C" int dq_fakequant_act_int4(const void* x, int x_is_f32, int64_t ldx, const float* a,
                                     const dq_hadamard_desc* had, int M, int K, float* out,
                                     int scale_fp16, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(out != nullptr, DQ_ERR_NULL, "out is null");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (x_is_f32)
    return launch_act(static_cast<const float*>(x), ldx, a, had, M, K, nullptr, nullptr, out,
                      MODE_FAKE, scale_fp16, s);
  return launch_act(static_cast<const __nv_bfloat16*>(x), ldx, a, had, M, K, nullptr, nullptr, out,
                    MODE_FAKE, scale_fp16, s);
}

extern "C" int dq_fakequant_act_int4_bf16(const void* x_bf16, int64_t ldx, int M, int K,
                                          void* out_bf16, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(out_bf16 != nullptr, DQ_ERR_NULL, "out is null");
  return launch_act(static_cast<const __nv_bfloat16*>(x_bf16), ldx, nullptr, nullptr, M, K, nullptr,
                    nullptr, static_cast<float*>(out_bf16), MODE_FAKE_BF16, 0,
                    static_cast<cudaStream_t>(stream));
}

extern "C" int dq_hadamard_f32(const float* x, float* out, int M, int K,
                               const dq_hadamard_desc* had, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  DQ_REQUIRE(out != nullptr, DQ_ERR_NULL, "out is null");
  DQ_REQUIRE(had != nullptr && had->kind != DQ_HAD_NONE, DQ_ERR_NULL, "no Hadamard described");
  return launch_act(x, static_cast<int64_t>(K), nullptr, had, M, K, nullptr, nullptr, out, MODE_RAW,
                    0, static_cast<cudaStream_t>(stream));
}

extern "C" int dq_quant_act_int4_gated(const void* gate_bf16, const void* up_bf16, int64_t ld,
                                       const float* a, const dq_hadamard_desc* had, int M, int K,
                                       int8_t* codes, float* sx, int scale_fp16, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(codes != nullptr && sx != nullptr && up_bf16 != nullptr, DQ_ERR_NULL, "codes / sx / up is null");
  DQ_REQUIRE(aligned(up_bf16, 16), DQ_ERR_ALIGN, "up must be 16-byte aligned");
  return launch_act(static_cast<const __nv_bfloat16*>(gate_bf16), ld, a, had, M, K, codes, sx, nullptr,
                    MODE_CODES, scale_fp16, static_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(up_bf16));
}
