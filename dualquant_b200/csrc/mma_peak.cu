// Tensor-pipe ceiling probe: tcgen05.mma issue loops on operands that never leave shared / tensor
// memory.  Gives the denominator "what the tensor cores sustain with nothing else going on" for
// kind::i8 and kind::f8f6f4 (the int4 paths) and kind::mxf4nvf4.block_scale (MXFP4 / NVFP4), measured on the
// GPU at hand instead of scaled from a bf16 figure.  One CTA per SM; one thread issues UMMAs of
// 128 x 256 x (32 bytes of K) back to back into one accumulator, commits once and waits (bounded).
#include "dq_common.h"
#include "dq_ptx.cuh"

namespace dq {
namespace peak {

constexpr int kThreads = 128;
constexpr int kATile = 128 * 128;   // 128 rows x 128 bytes, 128B swizzle layout
constexpr int kBTile = 256 * 128;
constexpr int kSmem = kATile + kBTile + 1024 + 64;
constexpr uint32_t kTmemCols = 512;
enum { PSITE_WAIT = 41 };

__device__ __forceinline__ uint32_t idesc_fp4(int m, int n, int e8m0, uint32_t sf_id) {
  return (sf_id << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(e8m0) << 23) | (static_cast<uint32_t>(m >> 4) << 24) | (sf_id << 29);
}

template <int NVFP4>
__device__ __forceinline__ void umma_fp4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  if constexpr (NVFP4) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}\n" ::
            "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n}\n" ::
            "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
  }
}

__device__ __forceinline__ void umma_e4m3(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// KIND: 0 = kind::i8, 1 = MXFP4 (E8M0, scale_vec::2X), 2 = NVFP4 (E4M3, scale_vec::4X),
//       3 = kind::f8f6f4 with E4M3 operands and an fp32 accumulator
template <int KIND>
__global__ void __launch_bounds__(kThreads, 1) mma_peak_kernel(int iters, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* a_tile = smem;
  uint8_t* b_tile = smem + kATile;
  uint64_t* done = reinterpret_cast<uint64_t*>(smem + kATile + kBTile);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x;
  // operand bytes: small non-zero codes (the rate does not depend on the values)
  for (int i = tid; i < (kATile + kBTile) / 4; i += kThreads)
    reinterpret_cast<uint32_t*>(smem)[i] = 0x01020301u * static_cast<uint32_t>((i % 3) + 1);
  if (tid == 0) {
    mbar_init(done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  fence_proxy_async_smem();
  __syncthreads();
  if (tid < 32) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (tid == 0) {
    const uint64_t da = umma_desc_k_sw128(smem_u32(a_tile));
    const uint64_t db = umma_desc_k_sw128(smem_u32(b_tile));
    if constexpr (KIND == 0) {
      const uint32_t idesc = umma_idesc_i8(128, 256);
      for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_i8(tmem_base, da + 2 * j, db + 2 * j, idesc, (i | j) ? 1u : 0u);
      }
    } else if constexpr (KIND == 3) {
      // E4M3 A and B (format code 0), fp32 accumulator (D format 1)
      const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(256 >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
      for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_e4m3(tmem_base, da + 2 * j, db + 2 * j, idesc, (i | j) ? 1u : 0u);
      }
    } else {
      constexpr int NV = (KIND == 2) ? 1 : 0;
      const uint32_t sfa = tmem_base + 256;
      const uint32_t sfb = sfa + 16;
      for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int atom = NV ? j : (j >> 1);
          const uint32_t sf_id = NV ? 0u : static_cast<uint32_t>((j & 1) * 2);
          umma_fp4<NV>(tmem_base, da + 2 * j, db + 2 * j, idesc_fp4(128, 256, NV ? 0 : 1, sf_id),
                       sfa + 4 * atom, sfb + 8 * atom, (i | j) ? 1u : 0u);
        }
      }
    }
    umma_commit(done);
    mbar_wait(done, 0, abort_flag, PSITE_WAIT);
  }
  __syncthreads();
  tc_fence_after();
  if (tid < 32) tmem_dealloc(tmem_base, kTmemCols);
  if (tid == 0 && *abort_flag != 0) atomicCAS(status, 0, *abort_flag);
}

// The same E4M3 issue loop with the operands REFILLED: a second thread streams a fresh 16 KB + 32 KB
// operand pair per four UMMAs from an L2-resident global buffer into a three-stage ring (bulk
// copies, mbarrier hand-off both ways), i.e. the K loop of the prefill GEMM without its epilogue.
// What is lost against the resident-operand loop is what the copy engine's writes and the tensor
// core's reads cost each other on the shared-memory port.
constexpr int kRefillStages = 3;
constexpr int kRefillStageBytes = kATile + kBTile;
constexpr int kRefillSmem = kRefillStages * kRefillStageBytes + 1024 + 128;
__device__ __align__(128) uint8_t g_refill_src[kRefillStageBytes];
enum { PSITE_REFILL_FULL = 42, PSITE_REFILL_FREE = 43 };

__global__ void __launch_bounds__(kThreads, 1) mma_refill_kernel(int iters, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kRefillStages * kRefillStageBytes);
  uint64_t* free_ = full + kRefillStages;
  uint64_t* done = free_ + kRefillStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x;
  if (tid == 0) {
    for (int i = 0; i < kRefillStages; ++i) { mbar_init(&full[i], 1); mbar_init(&free_[i], 1); }
    mbar_init(done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (tid < 32) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (tid == 32) {  // refill thread
    const uint64_t pol = l2_policy_evict_last();
    for (int i = 0; i < iters; ++i) {
      const int s = i % kRefillStages;
      if (!mbar_wait(&free_[s], ((i / kRefillStages) & 1) ^ 1, abort_flag, PSITE_REFILL_FREE)) break;
      mbar_expect_tx(&full[s], kRefillStageBytes);
      bulk_load_1d(smem + s * kRefillStageBytes, g_refill_src, kATile, &full[s], pol);
      bulk_load_1d(smem + s * kRefillStageBytes + kATile, g_refill_src + kATile, kBTile, &full[s], pol);
    }
  } else if (tid == 0) {
    const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(256 >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
    for (int i = 0; i < iters; ++i) {
      const int s = i % kRefillStages;
      if (!mbar_wait(&full[s], (i / kRefillStages) & 1, abort_flag, PSITE_REFILL_FULL)) break;
      tc_fence_after();
      const uint64_t da = umma_desc_k_sw128(smem_u32(smem + s * kRefillStageBytes));
      const uint64_t db = umma_desc_k_sw128(smem_u32(smem + s * kRefillStageBytes + kATile));
#pragma unroll
      for (int j = 0; j < 4; ++j) umma_e4m3(tmem_base, da + 2 * j, db + 2 * j, idesc, (i | j) ? 1u : 0u);
      umma_commit(&free_[s]);
    }
    umma_commit(done);
    mbar_wait(done, 0, abort_flag, PSITE_WAIT);
  }
  __syncthreads();
  tc_fence_after();
  if (tid < 32) tmem_dealloc(tmem_base, kTmemCols);
  if (tid == 0 && *abort_flag != 0) atomicCAS(status, 0, *abort_flag);
}

}  // namespace peak

int init_mma_peak_kernels() {
  cudaError_t e = cudaFuncSetAttribute(peak::mma_peak_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, peak::kSmem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(peak::mma_peak_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, peak::kSmem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(peak::mma_peak_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, peak::kSmem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(peak::mma_peak_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, peak::kSmem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(peak::mma_refill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, peak::kRefillSmem);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "cudaFuncSetAttribute(mma_peak) failed: %s", cudaGetErrorString(e));
  return DQ_OK;
}

}  // namespace dq

using namespace dq;

extern "C" int dq_mma_peak_probe(int kind, int iters, double* ops_out, void* stream) {
  DeviceState* st = current_state();
  if (st == nullptr) return DQ_ERR_NOT_INIT;
  DQ_REQUIRE(kind >= 0 && kind <= 4, DQ_ERR_SHAPE,
             "kind must be 0 (int8), 1 (MXFP4), 2 (NVFP4), 3 (E4M3) or 4 (E4M3 with operand refill)");
  DQ_REQUIRE(iters >= 1 && iters <= (1 << 20), DQ_ERR_SHAPE, "iters out of range");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(st->sm_count), block(peak::kThreads);
  if (kind == 0) peak::mma_peak_kernel<0><<<grid, block, peak::kSmem, s>>>(iters, st->status_dev);
  else if (kind == 1) peak::mma_peak_kernel<1><<<grid, block, peak::kSmem, s>>>(iters, st->status_dev);
  else if (kind == 2) peak::mma_peak_kernel<2><<<grid, block, peak::kSmem, s>>>(iters, st->status_dev);
  else if (kind == 3) peak::mma_peak_kernel<3><<<grid, block, peak::kSmem, s>>>(iters, st->status_dev);
  else peak::mma_refill_kernel<<<grid, block, peak::kRefillSmem, s>>>(iters, st->status_dev);
  DQ_CHECK_CUDA(cudaGetLastError());
  if (ops_out != nullptr) {
    const double k_elems = (kind == 0 || kind >= 3) ? 32.0 : 64.0;  // K per instruction
    *ops_out = static_cast<double>(st->sm_count) * iters * 4.0 * 2.0 * 128.0 * 256.0 * k_elems;
  }
  return DQ_OK;
}
