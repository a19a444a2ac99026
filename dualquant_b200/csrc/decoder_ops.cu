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
  DQ_CHECK_CUDA(launch_pdl(rope_kv_append_kernel, dim3(B * S, hq + 2 * hkv), dim3(head_dim / 2), 0,
                           static_cast<cudaStream_t>(stream), static_cast<const unsigned short*>(qkv_bf16), ld_qkv,
                           static_cast<const unsigned short*>(cos_tab_bf16),
                           static_cast<const unsigned short*>(sin_tab_bf16),
                           reinterpret_cast<const long long*>(pos_dev), static_cast<long long>(pos_host), S, hq, hkv,
                           head_dim, max_len, static_cast<unsigned short*>(q_out_bf16),
                           static_cast<unsigned short*>(k_cache_bf16), static_cast<unsigned short*>(v_cache_bf16)));
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}
