// Fast online-Hadamard quantiser kernels for bf16 rows (see act_quant_had.cuh).
#include "act_quant_had.cuh"

namespace dq {

int init_had_fast_bf16() { return init_had_fast_t<__nv_bfloat16>(); }

int launch_had_fast(const __nv_bfloat16* x, const __nv_bfloat16* up, int64_t ldx, const float* a,
                    const dq_hadamard_desc* had, int M, int K, size_t smem, int8_t* codes, float* sx, float* out,
                    int mode, int scale_fp16, cudaStream_t stream, bool* taken) {
  return launch_had_fast_t<__nv_bfloat16>(x, up, ldx, a, had, M, K, smem, codes, sx, out, mode, scale_fp16, stream,
                                          taken);
}

}  // namespace dq
