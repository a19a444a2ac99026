// Small bf16 kernels of the decode step around the W4A4 linears (end-to-end harness only; the
// reference leaves these steps to the HF decoder layer it wraps).
//
// rope_kv_append_kernel: rotary position embedding of the query and key heads of S tokens per
// sequence (S = 1 in decode, the prompt length in prefill) and the write of their key / value heads
// into the cache, in one launch instead of the
// dozen element-wise launches of `x * cos + rotate_half(x) * sin`, `index_copy_` and friends.
// The arithmetic is the bf16 tensor arithmetic of that expression: both products are rounded to
// bf16, then their sum is rounded to bf16.
#include "dq_common.h"
#include "dq_ptx.cuh"
#include "dq_quant.cuh"

#include <cuda_bf16.h>

namespace dq {

__device__ __forceinline__ float bf16_bits_to_float(unsigned short b) {
  return __uint_as_float(static_cast<uint32_t>(b) << 16);
}
__device__ __forceinline__ unsigned short float_to_bf16_bits(float v) {
  unsigned short bits;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(bits) : "f"(v));
  return bits;
}

// grid: (B * S, heads = hq + 2 * hkv); block: head_dim / 2 threads (thread i owns elements i, i + d/2).
// Token (b, s) sits in row b * S + s of qkv and goes to cache position pos0 + s, pos0 = *pos_ptr when
// a device pointer is given (decode inside a captured graph), else the host value.
__global__ void rope_kv_append_kernel(const unsigned short* __restrict__ qkv, int64_t ld_qkv,
                                      const unsigned short* __restrict__ cos_tab,
                                      const unsigned short* __restrict__ sin_tab,
                                      const long long* __restrict__ pos_ptr, long long pos_host, int S,
                                      int hq, int hkv, int hd, int max_len,
                                      unsigned short* __restrict__ q_out,
                                      unsigned short* __restrict__ k_cache,
                                      unsigned short* __restrict__ v_cache) {
  grid_dep_launch_dependents();
  grid_dep_wait();
  const int head = blockIdx.y, row = blockIdx.x, i = threadIdx.x, half = hd / 2;
  const int b = row / S, sidx = row - b * S;
  const long long pos = ((pos_ptr != nullptr) ? *pos_ptr : pos_host) + sidx;
  if (pos < 0 || pos >= max_len) return;  // out-of-range position: nothing is written
  const unsigned short* x = qkv + static_cast<int64_t>(row) * ld_qkv + static_cast<int64_t>(head) * hd;
  const unsigned short x1b = x[i], x2b = x[i + half];
  if (head >= hq + hkv) {  // value head: plain append
    unsigned short* dst = v_cache + ((static_cast<int64_t>(b) * hkv + (head - hq - hkv)) * max_len + pos) * hd;
    dst[i] = x1b;
    dst[i + half] = x2b;
    return;
  }
  const float x1 = bf16_bits_to_float(x1b), x2 = bf16_bits_to_float(x2b);
  const unsigned short* c = cos_tab + pos * hd;
  const unsigned short* s = sin_tab + pos * hd;
  // out[i] = x[i] * cos[i] + (-x[i + d/2]) * sin[i];  out[i + d/2] = x[i + d/2] * cos[i + d/2] + x[i] * sin[i + d/2]
  const float lo = __fadd_rn(round_to_bf16(__fmul_rn(x1, bf16_bits_to_float(c[i]))),
                             round_to_bf16(__fmul_rn(-x2, bf16_bits_to_float(s[i]))));
  const float hi = __fadd_rn(round_to_bf16(__fmul_rn(x2, bf16_bits_to_float(c[i + half]))),
                             round_to_bf16(__fmul_rn(x1, bf16_bits_to_float(s[i + half]))));
  unsigned short* dst;
  if (head < hq) {
    dst = q_out + (static_cast<int64_t>(row) * hq + head) * hd;  // [B, S, hq, d]
  } else {
    dst = k_cache + ((static_cast<int64_t>(b) * hkv + (head - hq)) * max_len + pos) * hd;
  }
  dst[i] = float_to_bf16_bits(lo);
  dst[i + half] = float_to_bf16_bits(hi);
}

// The same step, eight elements per access: thread = (head, chunk of 8 elements of the first half
// of the head); it also owns the matching chunk of the second half.  grid: (B * S, ceil(units /
// blockDim.x)), units = heads * head_dim / 16.  Needs head_dim % 16 == 0 and 16-byte aligned rows.
__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[2 * j] = __uint_as_float(w[j] << 16);
    f[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
  }
}

__global__ void __launch_bounds__(128)
rope_kv_append_vec_kernel(const unsigned short* __restrict__ qkv, int64_t ld_qkv,
                          const unsigned short* __restrict__ cos_tab,
                          const unsigned short* __restrict__ sin_tab,
                          const long long* __restrict__ pos_ptr, long long pos_host, int S, int hq,
                          int hkv, int hd, int max_len, unsigned short* __restrict__ q_out,
                          unsigned short* __restrict__ k_cache, unsigned short* __restrict__ v_cache) {
  grid_dep_launch_dependents();
  grid_dep_wait();
  const int half = hd / 2, chunks = half / 8;
  const int unit = blockIdx.y * blockDim.x + threadIdx.x;
  if (unit >= (hq + 2 * hkv) * chunks) return;
  const int head = unit / chunks, i = (unit - head * chunks) * 8;
  const int row = blockIdx.x;
  const int b = row / S, sidx = row - b * S;
  const long long pos = ((pos_ptr != nullptr) ? *pos_ptr : pos_host) + sidx;
  if (pos < 0 || pos >= max_len) return;
  const unsigned short* x = qkv + static_cast<int64_t>(row) * ld_qkv + static_cast<int64_t>(head) * hd;
  const uint4 lo_in = *reinterpret_cast<const uint4*>(x + i);
  const uint4 hi_in = *reinterpret_cast<const uint4*>(x + i + half);
  unsigned short* dst;
  if (head >= hq + hkv) {
    dst = v_cache + ((static_cast<int64_t>(b) * hkv + (head - hq - hkv)) * max_len + pos) * hd;
    *reinterpret_cast<uint4*>(dst + i) = lo_in;
    *reinterpret_cast<uint4*>(dst + i + half) = hi_in;
    return;
  }
  float x1[8], x2[8], c1[8], c2[8], s1[8], s2[8];
  unpack_bf16x8(lo_in, x1);
  unpack_bf16x8(hi_in, x2);
  const unsigned short* c = cos_tab + pos * hd;
  const unsigned short* s = sin_tab + pos * hd;
  unpack_bf16x8(*reinterpret_cast<const uint4*>(c + i), c1);
  unpack_bf16x8(*reinterpret_cast<const uint4*>(c + i + half), c2);
  unpack_bf16x8(*reinterpret_cast<const uint4*>(s + i), s1);
  unpack_bf16x8(*reinterpret_cast<const uint4*>(s + i + half), s2);
  uint32_t lo[4], hi[4];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float l = __fadd_rn(round_to_bf16(__fmul_rn(x1[j], c1[j])), round_to_bf16(__fmul_rn(-x2[j], s1[j])));
    const float h = __fadd_rn(round_to_bf16(__fmul_rn(x2[j], c2[j])), round_to_bf16(__fmul_rn(x1[j], s2[j])));
    const uint32_t lb = float_to_bf16_bits(l), hb = float_to_bf16_bits(h);
    if (j & 1) {
      lo[j >> 1] |= lb << 16;
      hi[j >> 1] |= hb << 16;
    } else {
      lo[j >> 1] = lb;
      hi[j >> 1] = hb;
    }
  }
  if (head < hq) {
    dst = q_out + (static_cast<int64_t>(row) * hq + head) * hd;
  } else {
    dst = k_cache + ((static_cast<int64_t>(b) * hkv + (head - hq)) * max_len + pos) * hd;
  }
  *reinterpret_cast<uint4*>(dst + i) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  *reinterpret_cast<uint4*>(dst + i + half) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
}

}  // namespace dq

using namespace dq;

extern "C" int dq_rope_kv_append(const void* qkv_bf16, int64_t ld_qkv, const void* cos_tab_bf16,
                                 const void* sin_tab_bf16, const int64_t* pos_dev, int64_t pos_host, int B,
                                 int S, int hq, int hkv, int head_dim, int max_len, void* q_out_bf16,
                                 void* k_cache_bf16, void* v_cache_bf16, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (B == 0 || S == 0) return DQ_OK;
  DQ_REQUIRE(qkv_bf16 != nullptr && cos_tab_bf16 != nullptr && sin_tab_bf16 != nullptr &&
                 q_out_bf16 != nullptr && k_cache_bf16 != nullptr && v_cache_bf16 != nullptr,
             DQ_ERR_NULL, "null pointer");
  DQ_REQUIRE(B >= 1 && S >= 1 && hq >= 1 && hkv >= 1 && head_dim >= 2 && head_dim % 2 == 0 && head_dim <= 2048 &&
                 max_len >= 1 && hq + 2 * hkv <= 65535 && static_cast<int64_t>(B) * S < (1ll << 31),
             DQ_ERR_SHAPE, "bad shape B=%d S=%d hq=%d hkv=%d head_dim=%d max_len=%d", B, S, hq, hkv, head_dim, max_len);
  DQ_REQUIRE(ld_qkv >= static_cast<int64_t>(hq + 2 * hkv) * head_dim, DQ_ERR_SHAPE, "ld_qkv too small");
  DQ_REQUIRE(pos_dev != nullptr || (pos_host >= 0 && pos_host + S <= max_len), DQ_ERR_SHAPE,
             "positions %lld..%lld outside the cache of %d", (long long)pos_host, (long long)(pos_host + S), max_len);
  const cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const auto* xq = static_cast<const unsigned short*>(qkv_bf16);
  const auto* ct = static_cast<const unsigned short*>(cos_tab_bf16);
  const auto* sn = static_cast<const unsigned short*>(sin_tab_bf16);
  const auto* pp = reinterpret_cast<const long long*>(pos_dev);
  auto* qo = static_cast<unsigned short*>(q_out_bf16);
  auto* kc = static_cast<unsigned short*>(k_cache_bf16);
  auto* vc = static_cast<unsigned short*>(v_cache_bf16);
  const auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (head_dim % 16 == 0 && ld_qkv % 8 == 0 && al16(xq) && al16(ct) && al16(sn) && al16(qo) && al16(kc) && al16(vc)) {
    const int units = (hq + 2 * hkv) * (head_dim / 16);
    DQ_CHECK_CUDA(launch_pdl(rope_kv_append_vec_kernel, dim3(B * S, (units + 127) / 128), dim3(128), 0, cs, xq,
                             ld_qkv, ct, sn, pp, static_cast<long long>(pos_host), S, hq, hkv, head_dim, max_len, qo,
                             kc, vc));
  } else {
    DQ_CHECK_CUDA(launch_pdl(rope_kv_append_kernel, dim3(B * S, hq + 2 * hkv), dim3(head_dim / 2), 0, cs, xq, ld_qkv,
                             ct, sn, pp, static_cast<long long>(pos_host), S, hq, hkv, head_dim, max_len, qo, kc, vc));
  }
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}
