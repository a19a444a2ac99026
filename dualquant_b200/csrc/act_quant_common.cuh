// Device helpers shared by the activation-quantiser translation units: output modes, block
// reductions, 8-element loads, the bf16 SiLU * up gate and the code / fake-quant emitter.
#pragma once
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

}  // namespace dq
