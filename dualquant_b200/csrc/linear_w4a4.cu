// One-call PermLinear.forward on the real int4 path.  Decode batches (M <= 16, no online Hadamard)
// may run as ONE kernel that quantises in its prologue; everything else is activation quantiser +
// GEMM on the caller's stream with the intermediates in caller-provided scratch.  Prefill batches
// (M >= kPrefillTokens) take the FP8 tensor-core path when the caller's scratch also has room for
// the byte form of the weight: quantiser (E4M3 codes) + weight expansion + GEMM.
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

// From this many tokens on the FP8-path GEMM wins even with the weight expanded on every call
// (the expansion moves 1.5 bytes per weight; measured on B200 it pays from about 1000 tokens).
static constexpr int kPrefillTokens = 1024;

extern "C" size_t dq_linear_w4a4_int4_prefill_scratch_bytes(int M, int N, int K) {
  const size_t base = dq_linear_w4a4_int4_scratch_bytes(M, N, K);
  if (M < kPrefillTokens || N < 1 || K < 1) return base;
  return base + round_up(static_cast<size_t>(N) * static_cast<size_t>(K), 256);
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
  // Decode batches without an online Hadamard: one launch, the quantiser runs inside the GEMM
  // kernel and the scratch stays untouched.  Same codes, scales and sums as the two launches below.
  if ((had == nullptr || had->kind == DQ_HAD_NONE) && G == dq::kGroup &&
      dq::tuning(dq::DQ_TUNE_LINEAR_FUSED) != 0) {
    dq::DeviceState* st = dq::current_state();
    if (st == nullptr) return DQ_ERR_NOT_INIT;
    if (dq::gemv_fused_covers(M, N, K, st)) {
      DQ_REQUIRE(y_dtype == DQ_DTYPE_F32 || y_dtype == DQ_DTYPE_BF16, DQ_ERR_UNSUPPORTED,
                 "unknown y_dtype %d", y_dtype);
      return dq::launch_gemv_fused(x_bf16, ldx, a, w_packed, r, M, N, K, y, y_dtype, scale_fp16,
                                   static_cast<cudaStream_t>(stream), st);
    }
  }
  int8_t* codes = static_cast<int8_t*>(scratch);
  float* sx = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) +
                                       round_up(static_cast<size_t>(M) * K, 256));
  if (M >= kPrefillTokens && G == dq::kGroup && (scale_fp16 & ~0xFF) == 0 &&
      scratch_bytes >= dq_linear_w4a4_int4_prefill_scratch_bytes(M, N, K)) {
    uint8_t* w8 = static_cast<uint8_t*>(scratch) + dq_linear_w4a4_int4_scratch_bytes(M, N, K);
    int rc = dq_expand_w_int4_e4m3(w_packed, N, K, G, w8, stream);
    if (rc != DQ_OK) return rc;
    rc = dq_quant_act_int4(x_bf16, ldx, a, had, M, K, codes, sx, scale_fp16 | DQ_CODES_E4M3, stream);
    if (rc != DQ_OK) return rc;
    return dq_gemm_w4a4_int4_e4m3(reinterpret_cast<const uint8_t*>(codes), sx, w8, sw_t, r, M, N, K, G, y, y_dtype,
                                  nullptr, stream);
  }
  int rc = dq_quant_act_int4(x_bf16, ldx, a, had, M, K, codes, sx, scale_fp16, stream);
  if (rc != DQ_OK) return rc;
  return dq_gemm_w4a4_int4(codes, sx, w_packed, sw_t, r, M, N, K, G, y, y_dtype, nullptr, 0, stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant
// ---------------------------------------------------------------------------------------------
// Scratch for dq_linear_w4a4_int4_static lives in the library image itself, so the caller never
// has to obtain device memory.  Every GPU that loads the library carries these bytes until the
// process exits.  The array name below is only a host-side handle: the device address that
// kernels can use is looked up once per device with cudaGetSymbolAddress.
#define DQ_STATIC_SCRATCH_BYTES (2u * 1024u * 1024u + 16u * 1024u)
static __device__ __align__(256) unsigned char g_static_scratch[DQ_STATIC_SCRATCH_BYTES];
static void* g_static_scratch_addr[dq::kMaxDevices] = {nullptr};

extern "C" size_t dq_linear_w4a4_int4_static_max_bytes(void) { return DQ_STATIC_SCRATCH_BYTES; }

extern "C" int dq_linear_w4a4_int4_static(const void* x_bf16, int64_t ldx, const float* a,
                                          const dq_hadamard_desc* had, const uint8_t* w_packed,
                                          const void* sw_t, const float* r, int M, int N, int K,
                                          int G, void* y, int y_dtype, int scale_fp16,
                                          void* stream) {
  DQ_REQUIRE(M >= 0 && N >= 1 && K >= 1, DQ_ERR_SHAPE, "bad shape M=%d N=%d K=%d", M, N, K);
  const size_t need = dq_linear_w4a4_int4_scratch_bytes(M, N, K);
  DQ_REQUIRE(need <= DQ_STATIC_SCRATCH_BYTES, DQ_ERR_WORKSPACE,
             "M=%d x K=%d needs %zu bytes of scratch; the built-in scratch holds %u "
             "(use dq_linear_w4a4_int4 with caller-provided scratch for larger batches)",
             M, K, need, DQ_STATIC_SCRATCH_BYTES);
  int dev = -1;
  DQ_CHECK_CUDA(cudaGetDevice(&dev));
  DQ_REQUIRE(dev >= 0 && dev < dq::kMaxDevices, DQ_ERR_SHAPE, "device index %d out of range", dev);
  if (g_static_scratch_addr[dev] == nullptr) {
    // one-time set-up for this device (it is the current one): symbol -> device address
    void* ptr = nullptr;
    DQ_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
    DQ_REQUIRE(ptr != nullptr, DQ_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_static_scratch_addr[dev] = ptr;
  }
  return dq_linear_w4a4_int4(x_bf16, ldx, a, had, w_packed, sw_t, r, M, N, K, G, y, y_dtype,
                             scale_fp16, g_static_scratch_addr[dev], DQ_STATIC_SCRATCH_BYTES,
                             stream);
}
