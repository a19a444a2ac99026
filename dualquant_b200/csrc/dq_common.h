// Host-side plumbing shared by the translation units of libdualquant_b200: error reporting,
// per-device state, argument checks.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/dualquant_b200.h"

namespace dq {

constexpr int kMaxDevices = 16;
constexpr int kGroup = 128;  // weight-group size = K extent of one pipeline stage
// One streamed weight tile: 128 rows x 128 k of packed int4 (8192 B) followed by the 128 fp16
// group scales of those rows (256 B).
constexpr int kTileCodeBytes = 8192;
constexpr int kTileBytes = kTileCodeBytes + 256;

// Per-device state created by dq_init.
struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int* status_dev = nullptr;  // device word written by kernels whose bounded waits expire
};

DeviceState* device_state(int device);
// State of the current device, or nullptr (and the error text set) if dq_init has not run.
DeviceState* current_state();

int set_error(int code, const char* fmt, ...);

// cuTensorMapEncodeTiled resolved through the runtime (no link-time libcuda dependency).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();

// 2-D row-major byte matrix [rows, row_bytes] (row pitch = pitch_bytes), box = box_rows x box_bytes.
int make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t row_bytes, uint64_t rows,
                    uint64_t pitch_bytes, uint32_t box_bytes, uint32_t box_rows,
                    CUtensorMapSwizzle swizzle);
// 2-D row-major fp32 / bf16 output matrix for tiled bulk stores (no swizzle).
int make_tmap_2d_out(CUtensorMap* out, const void* base, int elem_bytes, uint64_t cols, uint64_t rows,
                     uint32_t box_cols, uint32_t box_rows);
int make_tmap_x_groups(CUtensorMap* out, const void* base, uint64_t row_bytes, uint64_t rows,
                       uint32_t box_rows, uint32_t box_groups);

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

#define DQ_CHECK_CUDA(expr)                                                                 \
  do {                                                                                      \
    cudaError_t _e = (expr);                                                                \
    if (_e != cudaSuccess)                                                                  \
      return dq::set_error(DQ_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e));    \
  } while (0)

#define DQ_REQUIRE(cond, code, ...)                          \
  do {                                                       \
    if (!(cond)) return dq::set_error((code), __VA_ARGS__);  \
  } while (0)

// Launch with the programmatic-stream-serialization attribute: the kernel may begin while its
// predecessor in the stream is still running and must execute griddepcontrol.wait before it
// reads or writes anything the predecessor could touch.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Tuning knobs (dq_set_tuning): launch-shape overrides for measurement sweeps and tests.  0 means
// "the library's own choice" for every knob except DQ_TUNE_LINEAR_FUSED (1 = on, 0 = off, the default:
// measured on B200 the one-launch kernel is not faster than quantiser + GEMM chained by programmatic
// dependent launch, see the note at the top of gemv_w4a4_int4_fused.cu).
enum {
  DQ_TUNE_LINEAR_FUSED = 0,     // dq_linear_w4a4_int4 may take the one-launch decode kernel
  DQ_TUNE_FUSED_STAGES = 1,     // ring depth of the one-launch decode kernel
  DQ_TUNE_FUSED_SPLIT = 2,      // its split of K
  DQ_TUNE_FUSED_EXTRA_CTA = 3,  // CTAs' worth of shared memory left free per SM for the next launch
  DQ_TUNE_AR_WAIT_LOG2 = 4,     // fused all-reduce: a peer's flag is waited for 2^value SM cycles (0 = 30)
  DQ_TUNE_COUNT = 5
};
int tuning(int key);

// One-time kernel attribute set-up of each translation unit (called from dq_init).
int init_gemm_int4_kernels();
int init_gemv_int4_kernels();
int init_gemm_int4_tm_kernels();
int init_gemm_fp4_kernels();
int init_act_quant_kernels();
int init_gemv_fused_kernels();
int init_mma_peak_kernels();
int init_gemm_a16w4_kernels();
int init_gemm_int4_f8_kernels();
int init_gemm_fp4_persist_kernels();
int launch_gemm_fp4_persist(const uint8_t* x_codes, const uint8_t* x_sf_atoms, const float* x_scale,
                            const uint8_t* w_codes, const uint8_t* w_sf_atoms, const float* w_scale, const float* r,
                            int M, int N, int K, int nvfp4, void* y, int y_dtype, int row_tiles, cudaStream_t stream,
                            DeviceState* st);
int launch_gemm_int4_e4m3(const uint8_t* x8, const float* sx, const uint8_t* w8, const void* sw_t, const float* r,
                          int M, int N, int K, void* y, int y_dtype, const void* residual, cudaStream_t stream,
                          DeviceState* st);

// One-launch decode linear (quantiser inside the GEMM kernel), defined in gemv_w4a4_int4_fused.cu.
bool gemv_fused_covers(int M, int N, int K, const DeviceState* st);
int launch_gemv_fused(const void* x_bf16, int64_t ldx, const float* a, const uint8_t* w_packed,
                      const float* r, int M, int N, int K, void* y, int y_dtype, int scale_fp16,
                      cudaStream_t stream, DeviceState* st, const void* residual = nullptr);

// Decode-batch (register-path) variant of the int4 linear, defined in gemv_w4a4_int4.cu.
int launch_gemm_int4_tm(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                        const void* sw_t, const float* r, int M, int N, int K, void* y, int y_dtype,
                        int32_t* acc_dump, int tn, int split, cudaStream_t s, DeviceState* st,
                        const void* residual = nullptr, bool grouped_sx = false);
int gemv_pick_split(int tiles, int total_groups, int tok, int sm_count);
int launch_gemv_int4(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                     const void* sw_t, const float* r, int M, int N, int K, void* y, int y_dtype,
                     int tok, int split, cudaStream_t stream, DeviceState* st,
                     const dq_allreduce_ctx* ctx = nullptr, const void* residual = nullptr,
                     bool grouped_sx = false);

}  // namespace dq
