// Library state: per-device initialisation, error text, the device status word and the
// tensor-map encoder.  No kernel lives here.
#include <stdarg.h>
#include <string.h>

#include "dq_common.h"

namespace dq {

static DeviceState g_state[kMaxDevices];
static thread_local char g_err[512] = "";
static EncodeTiledFn g_encode = nullptr;

DeviceState* device_state(int device) {
  if (device < 0 || device >= kMaxDevices) return nullptr;
  return &g_state[device];
}

DeviceState* current_state() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    set_error(DQ_ERR_CUDA, "cudaGetDevice failed");
    return nullptr;
  }
  DeviceState* st = device_state(dev);
  if (st == nullptr || !st->ready) {
    set_error(DQ_ERR_NOT_INIT, "dq_init(%d) has not been called", dev);
    return nullptr;
  }
  return st;
}

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

EncodeTiledFn encode_tiled_fn() { return g_encode; }

static int g_tuning[DQ_TUNE_COUNT] = {0, 0, 0, 1, 0};
int tuning(int key) { return (key >= 0 && key < DQ_TUNE_COUNT) ? g_tuning[key] : 0; }

int make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t row_bytes, uint64_t rows,
                    uint64_t pitch_bytes, uint32_t box_bytes, uint32_t box_rows,
                    CUtensorMapSwizzle swizzle) {
  if (g_encode == nullptr) return set_error(DQ_ERR_NOT_INIT, "tensor-map encoder not resolved");
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(DQ_ERR_CUDA,
                     "cuTensorMapEncodeTiled failed (%d): base=%p row_bytes=%llu rows=%llu "
                     "pitch=%llu box=%ux%u",
                     (int)r, base, (unsigned long long)row_bytes, (unsigned long long)rows,
                     (unsigned long long)pitch_bytes, box_bytes, box_rows);
  return DQ_OK;
}

// 2-D row-major output matrix [rows, cols] of fp32 (elem_bytes 4) or bf16 (2), row pitch
// cols * elem_bytes, box = box_rows x box_cols elements, no swizzle: the map of a tiled bulk store.
int make_tmap_2d_out(CUtensorMap* out, const void* base, int elem_bytes, uint64_t cols, uint64_t rows,
                     uint32_t box_cols, uint32_t box_rows) {
  if (g_encode == nullptr) return set_error(DQ_ERR_NOT_INIT, "tensor-map encoder not resolved");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(out, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                        2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(DQ_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed (%d): base=%p cols=%llu rows=%llu box=%ux%u",
                     (int)r, base, (unsigned long long)cols, (unsigned long long)rows, box_cols, box_rows);
  return DQ_OK;
}

// Activation codes [rows][row_bytes] seen as (128-byte group chunk, row, group): one box is
// `box_groups` consecutive K groups of `box_rows` rows, laid out in shared memory as
// [group][row][128 B] (each group block is one 128B-swizzled UMMA operand tile).
int make_tmap_x_groups(CUtensorMap* out, const void* base, uint64_t row_bytes, uint64_t rows,
                       uint32_t box_rows, uint32_t box_groups) {
  if (g_encode == nullptr) return set_error(DQ_ERR_NOT_INIT, "tensor-map encoder not resolved");
  cuuint64_t dims[3] = {128, rows, row_bytes / 128};
  cuuint64_t strides[2] = {row_bytes, 128};
  cuuint32_t box[3] = {128, box_rows, box_groups};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(DQ_ERR_CUDA,
                     "cuTensorMapEncodeTiled (3-D) failed (%d): base=%p row_bytes=%llu rows=%llu "
                     "box=%ux%u",
                     (int)r, base, (unsigned long long)row_bytes, (unsigned long long)rows,
                     box_rows, box_groups);
  return DQ_OK;
}

}  // namespace dq

using namespace dq;

extern "C" int dq_abi_version(void) { return 2; }

extern "C" int dq_set_tuning(const char* name, int value) {
  static const char* const names[DQ_TUNE_COUNT] = {"linear_fused", "fused_stages", "fused_split",
                                                   "fused_extra_cta", "ar_wait_log2"};
  DQ_REQUIRE(name != nullptr, DQ_ERR_NULL, "null tuning name");
  for (int i = 0; i < DQ_TUNE_COUNT; ++i) {
    if (strcmp(name, names[i]) == 0) {
      g_tuning[i] = value;
      return DQ_OK;
    }
  }
  return set_error(DQ_ERR_UNSUPPORTED, "unknown tuning knob '%s'", name);
}

extern "C" const char* dq_last_error_string(void) { return g_err; }

extern "C" int dq_init(int device) {
  DeviceState* st = device_state(device);
  DQ_REQUIRE(st != nullptr, DQ_ERR_SHAPE, "device index %d out of range", device);
  if (st->ready) return DQ_OK;
  int cur = -1;
  DQ_CHECK_CUDA(cudaGetDevice(&cur));
  DQ_REQUIRE(cur == device, DQ_ERR_SHAPE, "dq_init(%d) called while device %d is current", device,
             cur);
  cudaDeviceProp prop;
  DQ_CHECK_CUDA(cudaGetDeviceProperties(&prop, device));
  DQ_REQUIRE(prop.major == 10, DQ_ERR_ARCH,
             "device %d is sm_%d%d; this library contains sm_100a code only", device, prop.major,
             prop.minor);
  st->sm_count = prop.multiProcessorCount;

  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    DQ_CHECK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    DQ_REQUIRE(fn != nullptr && qres == cudaDriverEntryPointSuccess, DQ_ERR_CUDA,
               "cuTensorMapEncodeTiled is not available from this driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  DQ_CHECK_CUDA(cudaMalloc(&st->status_dev, sizeof(int)));
  DQ_CHECK_CUDA(cudaMemset(st->status_dev, 0, sizeof(int)));

  int rc = init_gemm_int4_kernels();
  if (rc != DQ_OK) return rc;
  rc = init_gemm_int4_tm_kernels();
  if (rc != DQ_OK) return rc;
  rc = init_gemv_int4_kernels();
  if (rc != DQ_OK) return rc;
  rc = init_gemm_fp4_kernels();
  if (rc != DQ_OK) return rc;
  rc = init_act_quant_kernels();
  if (rc != DQ_OK) return rc;
  rc = init_gemv_fused_kernels();
  if (rc != DQ_OK) return rc;
  rc = init_mma_peak_kernels();
  if (rc != DQ_OK) return rc;
  rc = init_gemm_a16w4_kernels();
  if (rc != DQ_OK) return rc;
  rc = init_gemm_int4_f8_kernels();
  if (rc != DQ_OK) return rc;
  rc = init_gemm_fp4_persist_kernels();
  if (rc != DQ_OK) return rc;
  DQ_CHECK_CUDA(cudaDeviceSynchronize());
  st->ready = true;
  return DQ_OK;
}

extern "C" int dq_device_status(int device) {
  DeviceState* st = device_state(device);
  DQ_REQUIRE(st != nullptr && st->ready, DQ_ERR_NOT_INIT, "dq_init(%d) has not been called",
             device);
  int cur = -1;
  DQ_CHECK_CUDA(cudaGetDevice(&cur));
  DQ_REQUIRE(cur == device, DQ_ERR_SHAPE, "device %d is not current", device);
  DQ_CHECK_CUDA(cudaDeviceSynchronize());
  int word = 0;
  DQ_CHECK_CUDA(cudaMemcpy(&word, st->status_dev, sizeof(int), cudaMemcpyDeviceToHost));
  if (word != 0) {
    DQ_CHECK_CUDA(cudaMemset(st->status_dev, 0, sizeof(int)));
    set_error(DQ_ERR_TIMEOUT, "a bounded device-side wait expired (site %d)", word);
    return DQ_ERR_TIMEOUT | (word << 16);
  }
  return DQ_OK;
}
