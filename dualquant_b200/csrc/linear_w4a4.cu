// One-call PermLinear.forward on the real int4 path: activation quantiser + GEMM on the
// caller's stream, intermediates in caller-provided scratch.
#include "dq_common.h"

namespace {
inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
}  // namespace

extern "C" size_t dq_linear_w4a4_int4_scratch_bytes(int M, int N, int K) {
  (void)N;
  if (M < 0 || K < 0) return 0;
  return round_up(static_cast<size_t>(M) * static_cast<size_t>(K), 256) +
         round_up(static_cast<size_t>(M) * sizeof(float), 256);
}

extern "C" int dq_linear_w4a4_int4(const void* x_bf16, int64_t ldx, const float* a,
                                   const dq_hadamard_desc* had, const uint8_t* w_packed,
                                   const void* sw_t, const float* r, int M, int N, int K, int G,
                                   void* y, int y_dtype, int scale_fp16, void* scratch,
                                   size_t scratch_bytes, void* stream) {
  DQ_REQUIRE(scratch != nullptr, DQ_ERR_NULL, "scratch is null");
  DQ_REQUIRE(dq::aligned(scratch, 256), DQ_ERR_ALIGN, "scratch must be 256-byte aligned");
  DQ_REQUIRE(scratch_bytes >= dq_linear_w4a4_int4_scratch_bytes(M, N, K), DQ_ERR_WORKSPACE,
             "scratch of %zu bytes is smaller than the %zu required", scratch_bytes,
             dq_linear_w4a4_int4_scratch_bytes(M, N, K));
  if (M == 0) return DQ_OK;
  int8_t* codes = static_cast<int8_t*>(scratch);
  float* sx = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) +
                                       round_up(static_cast<size_t>(M) * K, 256));
  int rc = dq_quant_act_int4(x_bf16, ldx, a, had, M, K, codes, sx, scale_fp16, stream);
  if (rc != DQ_OK) return rc;
  return dq_gemm_w4a4_int4(codes, sx, w_packed, sw_t, r, M, N, K, G, y, y_dtype, nullptr, 0, stream);
}
