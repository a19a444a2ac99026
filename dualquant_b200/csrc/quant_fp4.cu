// Block-scaled FP4 quantisers for sm_100a: MXFP4 (E2M1 elements, blocks of 32, E8M0 scale) and
// NVFP4 (E2M1 elements, blocks of 16, E4M3 block scale over a second-level fp32 scale).
//
//   x32 = float(x) * a[k]                       (a optional)
//   MXFP4: e = floor(log2(absmax_block)) - 2 clamped to [-127, 127] (-127 for a zero block);
//          q = e2m1(x32 * 2^-e)                 scale byte = e + 127
//   NVFP4: ts = absmax_row / (6 * 448) (1 for a zero row), or a given per-tensor value;
//          bs = e4m3(clamp(absmax_block / 6 / ts, 2^-6, 448));    q = e2m1(x32 / (ts * bs))
// Element and scale conversions use the hardware converters (cvt.rn.satfinite.e2m1x2.f32 /
// .e4m3x2.f32: round to nearest even, saturating), divisions are IEEE.  One CTA per row, the row
// in registers, 8 consecutive elements per thread; a block spans 2 (NVFP4) or 4 (MXFP4) lanes.
// HBM-bound: 2 bytes in, 0.5 byte + scale out per element.
#include "dq_common.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace dq {

enum { FP4_MODE_CODES = 0, FP4_MODE_FAKE = 1 };
// the streaming kernel (several small CTAs per SM) takes over from the row-in-registers kernel
constexpr int kFp4StreamMinRows = 512;  // rows: enough CTAs to fill the SMs several times
constexpr int kFp4StreamMinVec = 1024;  // MXFP4: vectors of 8 per row (K >= 8192); shorter rows are as fast in registers
constexpr int kFp4StreamMinVecNv = 256;  // NVFP4 (two phases per row): from K = 2048 (6-10 % at K = 3584-4096)

__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
  uint16_t out;
  asm("{\n"
      ".reg .b8 t;\n"
      "cvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n"
      "cvt.u16.u8 %0, t;\n"
      "}\n"
      : "=h"(out)
      : "f"(hi), "f"(lo));
  return out;  // high nibble = hi, low nibble = lo
}

__device__ __forceinline__ float e2m1_value(uint32_t code) {
  // 1 sign, 2 exponent, 1 mantissa bit: 0, 0.5, then (1 + m/2) * 2^(e-1)
  const uint32_t e = (code >> 1) & 3u, m = code & 1u;
  const float frac = 1.0f + 0.5f * static_cast<float>(m);
  const float v = (e == 0) ? 0.5f * static_cast<float>(m) : frac * __uint_as_float((126u + e) << 23);
  return (code & 8u) ? -v : v;
}

__device__ __forceinline__ uint32_t e4m3_byte_of(float v) {
  uint16_t out;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(out) : "f"(0.f), "f"(v));
  return out & 0xFFu;  // second operand lands in the low byte
}

__device__ __forceinline__ float e4m3_value(uint32_t byte) {
  // unsigned use only (scales are non-negative): 4 exponent bits (bias 7), 3 mantissa bits
  const uint32_t e = (byte >> 3) & 0xF, m = byte & 7;
  if (e == 0) return static_cast<float>(m) * 0.001953125f;  // m * 2^-9
  return __uint_as_float(((e + 120u) << 23) | (m << 20));
}

__device__ __forceinline__ void fp4_load8(const __nv_bfloat16* p, float* v) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void fp4_load8(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// One vector of 8 consecutive elements (already scaled by the column scale) whose block absmax is
// known: block scale, element codes, stores.  sf_off = where this vector's block scale byte goes
// (used by the first vector of a block only).
__device__ __forceinline__ void fp4_emit_vector(const float* v, float bmax, float ts, int fmt, int mode,
                                                int row, int K, int idx, int blk, int64_t sf_off,
                                                uint8_t* __restrict__ codes, uint8_t* __restrict__ sf,
                                                float* __restrict__ out) {
    float q[8];
    float deq_scale;
    uint32_t sf_byte;
    if (fmt == DQ_FP4_MXFP4) {
      int e = -127;
      if (bmax != 0.f) {
        e = static_cast<int>((__float_as_uint(bmax) >> 23) & 0xFFu) - 127 - 2;
        e = max(-127, min(127, e));
      }
      sf_byte = static_cast<uint32_t>(e + 127);
      // 2^-e is representable (as a subnormal at the far end), so one multiplication rounds
      // exactly like scalbnf(v, -e) would
      const float down = scalbnf(1.0f, -e);
#pragma unroll
      for (int k = 0; k < 8; ++k) q[k] = __fmul_rn(v[k], down);
      deq_scale = scalbnf(1.0f, e);
    } else {
      const float want = __fdiv_rn(__fdiv_rn(bmax, 6.0f), ts);
      // clamped to the normal range of E4M3 [2^-6, 448] before the cast, as the reference's scale
      // quantiser does (scale_formats.py:39-45): an all-zero or tiny block gets the scale 2^-6
      sf_byte = e4m3_byte_of(fmaxf(fminf(want, 448.0f), 0.015625f));
      const float bs = e4m3_value(sf_byte);
      const float denom = __fmul_rn(ts, bs);
      deq_scale = denom;
      if (mode == FP4_MODE_FAKE) deq_scale = bs;  // applied as (q * bs) * ts below
      if (denom == 0.f) {
#pragma unroll
        for (int k = 0; k < 8; ++k) q[k] = 0.f;
      } else {
        // v / denom rounded to E2M1 without eight IEEE divisions: t = v * (1 / denom) is within
        // 2^-22 |t| of the quotient; if t (1 - 2^-21) and t (1 + 2^-21) convert to the same codes,
        // so does everything between them, the correctly rounded quotient included.  Otherwise
        // (an element sits on a rounding boundary, or t is not finite) the thread takes the exact
        // divisions, in a branch of its own.
        const float inv = __fdiv_rn(1.0f, denom);
        float lo[8], hi[8];
        bool exact = false;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float t = __fmul_rn(v[k], inv);
          exact |= !(fabsf(t) <= 1e30f);
          lo[k] = __fmul_rn(t, 0.99999952316284179688f);  // 1 - 2^-21
          hi[k] = __fmul_rn(t, 1.00000047683715820312f);  // 1 + 2^-21
        }
        uint32_t plo = 0, phi = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          plo |= e2m1x2(lo[2 * k], lo[2 * k + 1]) << (8 * k);
          phi |= e2m1x2(hi[2 * k], hi[2 * k + 1]) << (8 * k);
        }
        if (exact || plo != phi) {
#pragma unroll
          for (int k = 0; k < 8; ++k) q[k] = __fdiv_rn(v[k], denom);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) q[k] = lo[k];
        }
      }
    }
    uint32_t packed = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) packed |= e2m1x2(q[2 * k], q[2 * k + 1]) << (8 * k);
    if (mode == FP4_MODE_CODES) {
      *reinterpret_cast<uint32_t*>(codes + static_cast<int64_t>(row) * (K / 2) + idx / 2) = packed;
      if ((idx % blk) == 0) sf[sf_off] = static_cast<uint8_t>(sf_byte);
    } else {
      float o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float qv = e2m1_value((packed >> (4 * k)) & 0xFu);
        o[k] = (fmt == DQ_FP4_MXFP4) ? __fmul_rn(qv, deq_scale) : __fmul_rn(__fmul_rn(qv, deq_scale), ts);
      }
      float* orow = out + static_cast<int64_t>(row) * K + idx;
      *reinterpret_cast<float4*>(orow) = make_float4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<float4*>(orow + 4) = make_float4(o[4], o[5], o[6], o[7]);
    }
}

template <int THREADS, int VPT, typename XT>
__global__ void __launch_bounds__(THREADS)
quant_fp4_kernel(const XT* __restrict__ x, int64_t ldx, const float* __restrict__ a, int K, int fmt,
                 const float* __restrict__ tensor_scale, uint8_t* __restrict__ codes,
                 uint8_t* __restrict__ sf, float* __restrict__ row_scale, float* __restrict__ out,
                 int mode, int M, int sf_atoms) {
  // THREADS bounds the launch; the CTA may be smaller (a multiple of 32): vectors are dealt out
  // with the launched size as the stride, so that a row of K/8 vectors leaves few idle slots.
  __shared__ float red[THREADS / 32];
  const int nthreads = static_cast<int>(blockDim.x);
  const int row = blockIdx.x;
  // sf_atoms: the scale bytes go straight into the order the GEMM streams,
  // [row tile of 128][k / (4 blocks)][(r % 32) * 16 + (r / 32) * 4 + block % 4]; the grid then
  // covers the rows up to the next multiple of 128 and the CTAs past M write zero scales.
  const int blk_sz = (fmt == DQ_FP4_MXFP4) ? 32 : 16;
  const int nsf = K / blk_sz;
  auto sf_offset = [&](int ksf) -> int64_t {
    if (!sf_atoms) return static_cast<int64_t>(row) * nsf + ksf;
    const int rr = row & 127;
    return (static_cast<int64_t>(row >> 7) * (nsf >> 2) + (ksf >> 2)) * 512 + (rr & 31) * 16 +
           (rr >> 5) * 4 + (ksf & 3);
  };
  if (row >= M) {
    for (int ksf = threadIdx.x; ksf < nsf; ksf += nthreads) sf[sf_offset(ksf)] = 0;
    return;
  }
  const XT* xr = x + static_cast<int64_t>(row) * ldx;
  float v[VPT][8];
  float bmax[VPT];
  float rmax = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = (i * nthreads + threadIdx.x) * 8;
    bmax[i] = 0.f;
    if (idx < K) {
      fp4_load8(xr + idx, v[i]);
      if (a != nullptr) {
        float av[8];
        fp4_load8(a + idx, av);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = __fmul_rn(v[i][e], av[e]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) bmax[i] = fmaxf(bmax[i], fabsf(v[i][e]));
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[i][e] = 0.f;
    }
    // block absmax: 16 elements = 2 adjacent lanes, 32 elements = 4 adjacent lanes
    bmax[i] = fmaxf(bmax[i], __shfl_xor_sync(0xffffffffu, bmax[i], 1));
    if (fmt == DQ_FP4_MXFP4) bmax[i] = fmaxf(bmax[i], __shfl_xor_sync(0xffffffffu, bmax[i], 2));
    rmax = fmaxf(rmax, bmax[i]);
  }
  float ts = 1.f;
  if (fmt == DQ_FP4_NVFP4) {
    if (tensor_scale != nullptr) {
      ts = *tensor_scale;
    } else {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, o));
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = rmax;
      __syncthreads();
      float m = red[0];
      for (int i = 1; i < nthreads / 32; ++i) m = fmaxf(m, red[i]);
      ts = (m == 0.f) ? 1.f : __fdiv_rn(m, 2688.0f);
    }
    if (threadIdx.x == 0 && row_scale != nullptr) row_scale[row] = ts;
  }
  const int blk = (fmt == DQ_FP4_MXFP4) ? 32 : 16;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = (i * nthreads + threadIdx.x) * 8;
    if (idx >= K) continue;
    fp4_emit_vector(v[i], bmax[i], ts, fmt, mode, row, K, idx, blk, sf_offset(idx / blk), codes, sf, out);
  }
}

// The same quantiser for many long rows: a CTA of 256 threads walks its row in steps of 256
// vectors instead of holding it in registers, so that several CTAs share an SM and one row's loads
// overlap another row's arithmetic (the register version runs one 800-thread CTA per SM at
// K = 18944).  NVFP4 without a given tensor scale needs the row's absmax first: a first pass over
// the row, which the second pass then finds in L2.  Same per-vector arithmetic (fp4_emit_vector),
// same results.
template <typename XT>
__global__ void __launch_bounds__(256, 6)  // 39 registers: six CTAs per SM (four measured 12 % slower)
quant_fp4_stream_kernel(const XT* __restrict__ x, int64_t ldx, const float* __restrict__ a, int K, int fmt,
                        const float* __restrict__ tensor_scale, uint8_t* __restrict__ codes,
                        uint8_t* __restrict__ sf, float* __restrict__ row_scale, float* __restrict__ out,
                        int mode, int M, int sf_atoms) {
  constexpr int T = 256;
  __shared__ float red[T / 32];
  const int row = blockIdx.x;
  const int blk = (fmt == DQ_FP4_MXFP4) ? 32 : 16;
  const int nsf = K / blk;
  auto sf_offset = [&](int ksf) -> int64_t {
    if (!sf_atoms) return static_cast<int64_t>(row) * nsf + ksf;
    const int rr = row & 127;
    return (static_cast<int64_t>(row >> 7) * (nsf >> 2) + (ksf >> 2)) * 512 + (rr & 31) * 16 +
           (rr >> 5) * 4 + (ksf & 3);
  };
  if (row >= M) {
    for (int ksf = threadIdx.x; ksf < nsf; ksf += T) sf[sf_offset(ksf)] = 0;
    return;
  }
  const XT* xr = x + static_cast<int64_t>(row) * ldx;
  const int nvec = K / 8;
  const int iters = (nvec + T - 1) / T;
  auto load_scaled = [&](int idx, float* v) {
    fp4_load8(xr + idx, v);
    if (a != nullptr) {
      float av[8];
      fp4_load8(a + idx, av);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(v[e], av[e]);
    }
  };
  float ts = 1.f;
  if (fmt == DQ_FP4_NVFP4) {
    if (tensor_scale != nullptr) {
      ts = *tensor_scale;
    } else {
      float rmax = 0.f;
      for (int it = 0; it < iters; ++it) {
        const int idx = (it * T + threadIdx.x) * 8;
        if (idx < K) {
          float v[8];
          load_scaled(idx, v);
#pragma unroll
          for (int e = 0; e < 8; ++e) rmax = fmaxf(rmax, fabsf(v[e]));
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, o));
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = rmax;
      __syncthreads();
      float m = red[0];
#pragma unroll
      for (int i = 1; i < T / 32; ++i) m = fmaxf(m, red[i]);
      ts = (m == 0.f) ? 1.f : __fdiv_rn(m, 2688.0f);
    }
    if (threadIdx.x == 0 && row_scale != nullptr) row_scale[row] = ts;
  }
  for (int it = 0; it < iters; ++it) {  // every lane runs every iteration: the shuffles need the warp
    const int idx = (it * T + threadIdx.x) * 8;
    float v[8];
    float bmax = 0.f;
    if (idx < K) {
      load_scaled(idx, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) bmax = fmaxf(bmax, fabsf(v[e]));
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.f;
    }
    // block absmax: 16 elements = 2 adjacent lanes, 32 elements = 4 adjacent lanes
    bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 1));
    if (fmt == DQ_FP4_MXFP4) bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 2));
    if (idx < K)
      fp4_emit_vector(v, bmax, ts, fmt, mode, row, K, idx, blk, sf_offset(idx / blk), codes, sf, out);
  }
}

// Per-tensor second-level NVFP4 scale: absmax(x) / (6 * 448), 1 for an all-zero tensor.
template <typename XT>
__global__ void absmax_kernel(const XT* __restrict__ x, int64_t n, unsigned int* __restrict__ bits) {
  float m = 0.f;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    m = fmaxf(m, fabsf(static_cast<float>(x[i])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(bits, __float_as_uint(m));  // order-preserving for m >= 0
}
__global__ void nvfp4_scale_finalize_kernel(float* scale) {
  const float m = *scale;  // holds the absmax bit pattern
  *scale = (m == 0.f) ? 1.f : __fdiv_rn(m, 2688.0f);
}

template <typename XT>
static int launch_fp4(const XT* x, int64_t ldx, const float* a, int M, int K, int fmt,
                      const float* tensor_scale, uint8_t* codes, uint8_t* sf, float* row_scale,
                      float* out, int mode, cudaStream_t stream, int sf_atoms = 0) {
  DQ_REQUIRE(fmt == DQ_FP4_MXFP4 || fmt == DQ_FP4_NVFP4, DQ_ERR_UNSUPPORTED, "unknown FP4 format %d", fmt);
  DQ_REQUIRE(x != nullptr, DQ_ERR_NULL, "x is null");
  const int blk = (fmt == DQ_FP4_MXFP4) ? 32 : 16;
  DQ_REQUIRE(M >= 0 && K >= blk && K % blk == 0, DQ_ERR_SHAPE, "K=%d must be a multiple of the block size %d", K, blk);
  DQ_REQUIRE(K <= 32768, DQ_ERR_UNSUPPORTED, "K=%d exceeds 32768", K);
  DQ_REQUIRE(ldx >= K && ldx % 8 == 0, DQ_ERR_ALIGN, "ldx=%lld must be >= K and a multiple of 8", (long long)ldx);
  DQ_REQUIRE(aligned(x, 16) && (a == nullptr || aligned(a, 16)), DQ_ERR_ALIGN, "x and a must be 16-byte aligned");
  DQ_REQUIRE((codes == nullptr || aligned(codes, 4)) && (out == nullptr || aligned(out, 16)), DQ_ERR_ALIGN,
             "outputs misaligned");
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(!sf_atoms || (K / blk) % 4 == 0, DQ_ERR_SHAPE,
             "scale factors in GEMM order need K %% %d == 0 (K=%d)", 4 * blk, K);
  const int vec = K / 8;
  const int rows = sf_atoms ? (M + 127) / 128 * 128 : M;
  // T bounds the CTA, V = vectors of 8 per thread; the CTA launched is the smallest multiple of
  // 32 threads that covers the row with V vectors each.
#define DQ_FP4_LAUNCH(T, V)                                                                        \
  quant_fp4_kernel<T, V, XT><<<rows, ((vec + (V) - 1) / (V) + 31) / 32 * 32, 0, stream>>>(        \
      x, ldx, a, K, fmt, tensor_scale, codes, sf, row_scale, out, mode, M, sf_atoms)
  // (four vectors per thread in smaller CTAs for many rows measured no faster: 126 vs 107 us at
  // M = 4096, K = 18944)
  if (M >= kFp4StreamMinRows && vec >= (fmt == DQ_FP4_NVFP4 ? kFp4StreamMinVecNv : kFp4StreamMinVec)) {
    quant_fp4_stream_kernel<XT><<<rows, 256, 0, stream>>>(x, ldx, a, K, fmt, tensor_scale, codes, sf,
                                                          row_scale, out, mode, M, sf_atoms);
  } else if (vec <= 128) DQ_FP4_LAUNCH(128, 1);
  else if (vec <= 256) DQ_FP4_LAUNCH(256, 1);
  else if (vec <= 512) DQ_FP4_LAUNCH(512, 1);
  else if (vec <= 1024) DQ_FP4_LAUNCH(512, 2);
  else if (vec <= 1536) DQ_FP4_LAUNCH(512, 3);
  else if (vec <= 2048) DQ_FP4_LAUNCH(512, 4);
  else if (vec <= 3072) DQ_FP4_LAUNCH(1024, 3);
  else DQ_FP4_LAUNCH(1024, 4);
#undef DQ_FP4_LAUNCH
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}

}  // namespace dq

using namespace dq;

extern "C" int dq_quant_fp4(const void* x, int x_is_f32, int64_t ldx, const float* a, int M, int K,
                            int fmt, const float* tensor_scale, uint8_t* codes, uint8_t* sf,
                            float* row_scale, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(codes != nullptr && sf != nullptr, DQ_ERR_NULL, "codes / sf is null");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (x_is_f32)
    return launch_fp4(static_cast<const float*>(x), ldx, a, M, K, fmt, tensor_scale, codes, sf,
                      row_scale, nullptr, FP4_MODE_CODES, s);
  return launch_fp4(static_cast<const __nv_bfloat16*>(x), ldx, a, M, K, fmt, tensor_scale, codes, sf,
                    row_scale, nullptr, FP4_MODE_CODES, s);
}

extern "C" int dq_quant_fp4_atoms(const void* x, int x_is_f32, int64_t ldx, const float* a, int M,
                                  int K, int fmt, const float* tensor_scale, uint8_t* codes,
                                  uint8_t* sf_atoms, float* row_scale, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(codes != nullptr && sf_atoms != nullptr, DQ_ERR_NULL, "codes / sf_atoms is null");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (x_is_f32)
    return launch_fp4(static_cast<const float*>(x), ldx, a, M, K, fmt, tensor_scale, codes, sf_atoms,
                      row_scale, nullptr, FP4_MODE_CODES, s, 1);
  return launch_fp4(static_cast<const __nv_bfloat16*>(x), ldx, a, M, K, fmt, tensor_scale, codes,
                    sf_atoms, row_scale, nullptr, FP4_MODE_CODES, s, 1);
}

extern "C" int dq_fakequant_fp4(const void* x, int x_is_f32, int64_t ldx, const float* a, int M,
                                int K, int fmt, const float* tensor_scale, float* out,
                                void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(out != nullptr, DQ_ERR_NULL, "out is null");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (x_is_f32)
    return launch_fp4(static_cast<const float*>(x), ldx, a, M, K, fmt, tensor_scale, nullptr, nullptr,
                      nullptr, out, FP4_MODE_FAKE, s);
  return launch_fp4(static_cast<const __nv_bfloat16*>(x), ldx, a, M, K, fmt, tensor_scale, nullptr,
                    nullptr, nullptr, out, FP4_MODE_FAKE, s);
}

extern "C" int dq_nvfp4_tensor_scale(const void* x, int x_is_f32, int64_t numel, float* scale,
                                     void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  DQ_REQUIRE(x != nullptr && scale != nullptr && numel > 0, DQ_ERR_NULL, "null or empty input");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  DQ_CHECK_CUDA(cudaMemsetAsync(scale, 0, sizeof(float), s));
  const int blocks = static_cast<int>(numel / 4096 > 1184 ? 1184 : (numel + 4095) / 4096);
  if (x_is_f32)
    absmax_kernel<<<blocks, 256, 0, s>>>(static_cast<const float*>(x), numel,
                                         reinterpret_cast<unsigned int*>(scale));
  else
    absmax_kernel<<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), numel,
                                         reinterpret_cast<unsigned int*>(scale));
  nvfp4_scale_finalize_kernel<<<1, 1, 0, s>>>(scale);
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}
