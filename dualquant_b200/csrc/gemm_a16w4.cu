// A16W4 dual-scale linear for sm_100a: 16-bit activations against the int4 weight artefact,
//
//   Y[m,n] = r[n] * sum_k fp16(x[m,k] * a[k]) * fp16(qw[n,k] * sw[n, k/128])
//
// the computation of the reference's fused-beta Triton kernel
// (vendor/dualscale_kernel_benchmark/fused_dual_scale_kernel.py:55-149: beta multiplied into the
// activation tile on its way in, nibbles de-quantised with the group scale, floating-point dot
// product) on the tensor cores of this GPU: tcgen05.mma kind::f16 with fp16 operands and ONE fp32
// accumulator in tensor memory over the whole K (the group scale is folded into the fp16 weight,
// so nothing has to be drained per group).  fp16 rather than bf16 operands: with 8-bit mantissas
// the reference's own acceptance check (mean relative error below 1 % against the fp32 formulation,
// fused_dual_scale_kernel.py:269-308) fails at 1.4-5.7 %, with 11-bit mantissas it passes at
// 0.25-0.4 %; the group scales are fp16 already, so code * scale is one exactly rounded product.
// Activations beyond the fp16 range saturate at +-65504.
//
// Orientation as in the int4 kernels: the CTA's 128 weight rows are the UMMA M dimension, the token
// tile TN is UMMA N.  Per weight group (128 k, one pipeline step):
//   producer warp   one bulk copy of the packed tile (8 KB codes + 256 B fp16 scales) and two tiled
//                   copies of the activation tile (TN x 64 fp16 each, 128-byte swizzle);
//   16 unpack warps thread (row, k chunk) expands 16 bytes of nibbles into 32 fp16 = code * scale and
//                   writes them as four 16-byte pieces into the 128B-swizzled K-major operand tile.
//                   A nibble pair becomes half2 by bit tricks: (w >> s) & 0x000F000F picks two
//                   two's-complement nibbles, ^ 0x64086408 turns them into the fp16 numbers
//                   1032 + code, a packed subtract gives code exactly and a packed multiply by the
//                   fp16 group scale the weight;
//   issuing warp    eight tcgen05.mma (K = 16) per group, tcgen05.commit frees the operand buffers.
// After the last group the first four unpack warps read the accumulator (one weight row per
// thread), multiply by r[n] and store bf16 or fp32.  Every wait is bounded.
//
// Bound (ncu at gate+up, M = 4096: tensor pipe 31 % active, issue slots 45 %): the shared-memory port.
// Per 128 x 128 x 128 block the tensor core reads 64 KB of operands (a 128 x 128 tile saturates the
// port on its own: 8 KB per 68-cycle UMMA), the unpack warps write 32 KB and read 8 KB, the copy
// engine writes 40 KB - 144 KB against the ~69 KB the port moves in the block's 542 UMMA cycles.  Tried
// and not kept: a second issuing warp with its own accumulator (slower: one activation stage less).
// The next step is the weight operand through tensor memory (tcgen05.st by the unpack warps, as
// the int4 kernel for small token tiles does), which takes 64 KB per block off the port.
//
// The activation scale and the conversion to fp16 run as a small separate pass
// (xs = fp16(x * a), caller scratch) so that the GEMM can stage activations with TMA.
#include "dq_common.h"
#include "dq_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace dq {
namespace a16 {

constexpr int kBN = 128;                 // weight rows per CTA (UMMA M)
constexpr int kUnpackWarps = 16;  // four threads per weight row: two resident warps per scheduler hid too little latency
constexpr int kProducerWarp = kUnpackWarps;
constexpr int kIssuerWarp = kUnpackWarps + 1;
constexpr int kThreads = (kUnpackWarps + 2) * 32;
constexpr int kWTile = kBN * kGroup * 2;  // fp16 weight tile of one group: 32 KB (two 16 KB atoms)
constexpr int kAtom = kBN * 128;          // 128 rows x 128 B

enum { ASITE_TMA = 51, ASITE_UNPACK = 52, ASITE_MMA = 53, ASITE_EPI = 54, ASITE_ALIGN = 55 };

template <int TN>
struct Cfg {
  static constexpr int NB = 2;                      // unpacked weight buffers
  static constexpr int SP = 4;                      // packed-tile stages
  static constexpr int SX = (TN <= 64) ? 4 : 3;     // activation stages
  static constexpr int kXStage = TN * kGroup * 2;   // TN x 128 fp16 = two atoms of TN x 128 B
  static constexpr int kXAtom = TN * 128;
  static constexpr int kOffW = 0;
  static constexpr int kOffX = kOffW + NB * kWTile;
  static constexpr int kOffP = kOffX + SX * kXStage;
  static constexpr int kPStage = (kTileBytes + 127) / 128 * 128;
  static constexpr int kOffBar = kOffP + SP * kPStage;
  static constexpr int kNumBars = 2 * SP + 2 * NB + 2 * SX + 1;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 32;
  static constexpr int kTmemCols = (TN <= 32) ? 32 : (TN <= 64) ? 64 : 128;
  static_assert(kSmemBytes + 1024 <= 227 * 1024, "shared memory");
  static_assert(kOffX % 1024 == 0 && kXStage % 1024 == 0 && kXAtom % 1024 == 0, "swizzle atoms on 1 KB boundaries");
};

// Instruction descriptor, kind::f16: fp16 A and B (both K-major), fp32 accumulator.
//   [4,6) D format (1 = F32)  [7,10) A format (0 = F16)  [10,13) B format (0 = F16)
//   [17,23) N >> 3  [24,29) M >> 4
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// two two's-complement nibbles (bits 0-3 and 16-19 of t) -> half2 (code * scale)
__device__ __forceinline__ uint32_t nib2_to_f16x2(uint32_t t, __half2 s2) {
  const uint32_t biased = (t & 0x000F000Fu) ^ 0x64086408u;  // fp16 numbers 1024 + 8 + code
  __half2 v = *reinterpret_cast<const __half2*>(&biased);
  const uint32_t k1032 = 0x64086408u;
  v = __hsub2(v, *reinterpret_cast<const __half2*>(&k1032));  // exact: small integers
  v = __hmul2(v, s2);                                          // one rounding: fp16(code * scale)
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Eight consecutive k of one row: the low (HI = 0) or high (HI = 1) nibbles of packed words wa, wb.
template <int HI>
__device__ __forceinline__ uint4 expand8(uint32_t wa, uint32_t wb, __half2 s2) {
  // byte b of a word: nibble of k = 4j + b (low) or 16 + 4j + b (high).  (w >> s) & 0x000F000F
  // picks bytes 0 and 2, (w >> (s + 8)) bytes 1 and 3.
  const uint32_t a02 = nib2_to_f16x2(wa >> (4 * HI), s2), a13 = nib2_to_f16x2(wa >> (4 * HI + 8), s2);
  const uint32_t b02 = nib2_to_f16x2(wb >> (4 * HI), s2), b13 = nib2_to_f16x2(wb >> (4 * HI + 8), s2);
  uint4 o;
  o.x = __byte_perm(a02, a13, 0x5410);  // (k0, k1)
  o.y = __byte_perm(a02, a13, 0x7632);  // (k2, k3)
  o.z = __byte_perm(b02, b13, 0x5410);
  o.w = __byte_perm(b02, b13, 0x7632);
  return o;
}

template <int TN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_a16w4_kernel(const uint8_t* __restrict__ w_packed, const __grid_constant__ CUtensorMap tm_x,
                  const float* __restrict__ r, void* __restrict__ y, int y_bf16, int M, int N, int K,
                  int* status) {
  using C = Cfg<TN>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(status, 0, ASITE_ALIGN);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint64_t* full_p = bars;
  uint64_t* empty_p = full_p + C::SP;
  uint64_t* w_ready = empty_p + C::SP;
  uint64_t* w_free = w_ready + C::NB;
  uint64_t* full_x = w_free + C::NB;
  uint64_t* empty_x = full_x + C::SX;
  uint64_t* acc_done = empty_x + C::SX;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int ng = K / kGroup;
  const int n0 = blockIdx.x * kBN;
  const int t0 = blockIdx.y * TN;

  if (tid == 0) {
    for (int i = 0; i < C::SP; ++i) { mbar_init(&full_p[i], 1); mbar_init(&empty_p[i], kUnpackWarps); }
    for (int i = 0; i < C::NB; ++i) { mbar_init(&w_ready[i], kUnpackWarps); mbar_init(&w_free[i], 1); }
    for (int i = 0; i < C::SX; ++i) { mbar_init(&full_x[i], 1); mbar_init(&empty_x[i], 1); }
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kIssuerWarp) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  if (warp == kProducerWarp && lane == 0) tma_prefetch_desc(&tm_x);
  grid_dep_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const uint64_t pol_w = (gridDim.y == 1) ? l2_policy_evict_first() : l2_policy_evict_last();
      const uint64_t pol_x = l2_policy_evict_last();
      const uint8_t* w_src = w_packed + static_cast<size_t>(blockIdx.x) * ng * kTileBytes;
      // The weights do not depend on the kernel before this one, the activations may: the first
      // weight tiles go out before the dependency wait.
      const int pre = (ng < C::SP) ? ng : C::SP;
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full_p[i], kTileBytes);
        bulk_load_1d(smem + C::kOffP + i * C::kPStage, w_src + static_cast<size_t>(i) * kTileBytes, kTileBytes,
                     &full_p[i], pol_w);
      }
      grid_dep_wait();
      for (int i = 0; i < ng; ++i) {
        const int sp = i % C::SP, sx = i % C::SX;
        if (i >= pre) {
          if (!mbar_wait(&empty_p[sp], ((i / C::SP) & 1) ^ 1, abort_flag, ASITE_TMA)) break;
          mbar_expect_tx(&full_p[sp], kTileBytes);
          bulk_load_1d(smem + C::kOffP + sp * C::kPStage, w_src + static_cast<size_t>(i) * kTileBytes,
                       kTileBytes, &full_p[sp], pol_w);
        }
        if (!mbar_wait(&empty_x[sx], ((i / C::SX) & 1) ^ 1, abort_flag, ASITE_TMA)) break;
        mbar_expect_tx(&full_x[sx], C::kXStage);
        uint8_t* xs = smem + C::kOffX + sx * C::kXStage;
        tma_load_2d(xs, &tm_x, i * 256, t0, &full_x[sx], pol_x);                    // k 0..63 of the group
        tma_load_2d(xs + C::kXAtom, &tm_x, i * 256 + 128, t0, &full_x[sx], pol_x);  // k 64..127
      }
    }
  } else if (warp == kIssuerWarp) {
    // ------------------------------------------------------------------ UMMA issue
    if (lane == 0) {
      const uint32_t idesc = idesc_f16(kBN, TN);
      for (int i = 0; i < ng; ++i) {
        const int b = i % C::NB, sx = i % C::SX;
        if (!mbar_wait(&w_ready[b], (i / C::NB) & 1, abort_flag, ASITE_MMA)) break;
        if (!mbar_wait(&full_x[sx], (i / C::SX) & 1, abort_flag, ASITE_MMA)) break;
        tc_fence_after();
        const uint32_t wbase = smem_u32(smem + C::kOffW + b * kWTile);
        const uint32_t xbase = smem_u32(smem + C::kOffX + sx * C::kXStage);
#pragma unroll
        for (int j = 0; j < 8; ++j) {  // eight K = 16 steps: 32 bytes along K inside an atom
          const uint64_t da = umma_desc_k_sw128(wbase + (j >> 2) * kAtom) + 2 * (j & 3);
          const uint64_t db = umma_desc_k_sw128(xbase + (j >> 2) * C::kXAtom) + 2 * (j & 3);
          umma_f16(tmem_base, da, db, idesc, (i | j) ? 1u : 0u);
        }
        umma_commit(&w_free[b]);
        umma_commit(&empty_x[sx]);
      }
      umma_commit(acc_done);
    }
  } else {
    // ------------------------------------------------------------------ unpack warps
    const int row = tid & 127;
    const int ch = tid >> 7;    // k chunk (32 k) of the group this thread expands: 0..3
    const int swz = row & 7;
    bool ok = true;
    for (int i = 0; i < ng && ok; ++i) {
      const int sp = i % C::SP, b = i % C::NB;
      if (!mbar_wait(&full_p[sp], (i / C::SP) & 1, abort_flag, ASITE_UNPACK)) { ok = false; break; }
      if (!mbar_wait(&w_free[b], ((i / C::NB) & 1) ^ 1, abort_flag, ASITE_UNPACK)) { ok = false; break; }
      const uint8_t* tile = smem + C::kOffP + sp * C::kPStage;
      const __half sc = reinterpret_cast<const __half*>(tile + kTileCodeBytes)[row];
      const __half2 s2 = __half2half2(sc);
      // chunks 0, 1 -> atom 0 (k 0..63), chunks 2, 3 -> atom 1; inside the atom 16-byte pieces c0..c0+3
      uint8_t* dst = smem + C::kOffW + b * kWTile + (ch >> 1) * kAtom + row * 128;
      const int c0 = (ch & 1) * 4;
      const int pos = ch ^ ((row >> 1) & 3);           // the chunk's position in the packed row
      const uint4 w = *reinterpret_cast<const uint4*>(tile + row * 64 + pos * 16);
      // the chunk's 32 k as four 16-byte pieces: k 0-7, 8-15 (low nibbles of words 0,1 / 2,3),
      // 16-23, 24-31 (high nibbles)
      *reinterpret_cast<uint4*>(dst + (((c0 + 0) ^ swz) << 4)) = expand8<0>(w.x, w.y, s2);
      *reinterpret_cast<uint4*>(dst + (((c0 + 1) ^ swz) << 4)) = expand8<0>(w.z, w.w, s2);
      *reinterpret_cast<uint4*>(dst + (((c0 + 2) ^ swz) << 4)) = expand8<1>(w.x, w.y, s2);
      *reinterpret_cast<uint4*>(dst + (((c0 + 3) ^ swz) << 4)) = expand8<1>(w.z, w.w, s2);
      fence_proxy_async_smem();  // generic-proxy stores before the tensor core's reads
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&w_ready[b]);
        mbar_arrive(&empty_p[sp]);
      }
    }
    // ------------------------------------------------------------------ epilogue (warps 0-3)
    if (warp < 4 && ok) {
      if (mbar_wait_relaxed(acc_done, 0, abort_flag, ASITE_EPI)) {
        tc_fence_after();
        const int n = n0 + warp * 32 + lane;  // warp w reads TMEM lanes 32 w .. 32 w + 31
        const float rn = (n < N && r != nullptr) ? r[n] : 1.f;
#pragma unroll 1
        for (int c0 = 0; c0 < TN; c0 += 16) {
          uint32_t v[16];
          tmem_ld_x16(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + static_cast<uint32_t>(c0), v);
          tmem_ld_wait();
          if (n < N) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = t0 + c0 + j;
              if (m < M) store_y(y, nullptr, y_bf16, static_cast<size_t>(m) * N + n, __uint_as_float(v[j]) * rn);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == kIssuerWarp) tmem_dealloc(tmem_base, C::kTmemCols);
  if (tid == 0 && *abort_flag != 0) atomicCAS(status, 0, *abort_flag);
}

// xs[m, k] = fp16(float(x[m, k]) * a[k]) (a may be null), saturating at the fp16 range
__global__ void __launch_bounds__(256) scale_cols_f16_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx,
                                                             const float* __restrict__ a, int M, int K,
                                                             __half* __restrict__ xs) {
  grid_dep_launch_dependents();
  grid_dep_wait();
  const int vec = K / 8;
  const int64_t total = static_cast<int64_t>(M) * vec;
  for (int64_t u = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; u < total;
       u += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(u / vec), kv = static_cast<int>(u % vec);
    const uint4 raw = *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(m) * ldx + kv * 8);
    float av[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
    if (a != nullptr) {
      const float4 a0 = *reinterpret_cast<const float4*>(a + kv * 8);
      const float4 a1 = *reinterpret_cast<const float4*>(a + kv * 8 + 4);
      av[0] = a0.x; av[1] = a0.y; av[2] = a0.z; av[3] = a0.w;
      av[4] = a1.x; av[5] = a1.y; av[6] = a1.z; av[7] = a1.w;
    }
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float lo = fminf(fmaxf(__fmul_rn(__uint_as_float(w[i] << 16), av[2 * i]), -65504.f), 65504.f);
      const float hi = fminf(fmaxf(__fmul_rn(__uint_as_float(w[i] & 0xFFFF0000u), av[2 * i + 1]), -65504.f), 65504.f);
      const __half2 p = __floats2half2_rn(lo, hi);
      o[i] = *reinterpret_cast<const uint32_t*>(&p);
    }
    *reinterpret_cast<uint4*>(xs + static_cast<int64_t>(m) * K + kv * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <int TN>
static int launch(const void* xs, int64_t ld_elems, const uint8_t* w_packed, const float* r, int M, int N,
                  int K, void* y, int y_dtype, cudaStream_t stream, DeviceState* st) {
  CUtensorMap tm_x;
  int rc = make_tmap_2d_u8(&tm_x, xs, static_cast<uint64_t>(K) * 2, M, static_cast<uint64_t>(ld_elems) * 2, 128, TN,
                           CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != DQ_OK) return rc;
  const dim3 grid((N + kBN - 1) / kBN, (M + TN - 1) / TN, 1);
  cudaError_t e = launch_pdl(gemm_a16w4_kernel<TN>, grid, dim3(kThreads), Cfg<TN>::kSmemBytes, stream, w_packed,
                             tm_x, r, y, y_dtype == DQ_DTYPE_BF16 ? 1 : 0, M, N, K, st->status_dev);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "gemm_a16w4 launch failed (TN=%d): %s", TN, cudaGetErrorString(e));
  return DQ_OK;
}

}  // namespace a16

int init_gemm_a16w4_kernels() {
  cudaError_t e = cudaFuncSetAttribute(a16::gemm_a16w4_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       a16::Cfg<32>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(a16::gemm_a16w4_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             a16::Cfg<128>::kSmemBytes);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "cudaFuncSetAttribute(gemm_a16w4) failed: %s", cudaGetErrorString(e));
  return DQ_OK;
}

}  // namespace dq

using namespace dq;

extern "C" size_t dq_linear_a16w4_scratch_bytes(int M, int N, int K) {
  (void)N;
  if (M < 0 || K < 0) return 0;
  return (static_cast<size_t>(M) * static_cast<size_t>(K) * 2 + 255) / 256 * 256;
}

extern "C" int dq_linear_a16w4(const void* x_bf16, int64_t ldx, const float* a, const uint8_t* w_packed,
                               const float* r, int M, int N, int K, int G, void* y, int y_dtype,
                               void* scratch, size_t scratch_bytes, void* stream) {
  DeviceState* st = current_state();
  if (st == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(x_bf16 != nullptr && w_packed != nullptr && y != nullptr, DQ_ERR_NULL, "null x / w_packed / y");
  DQ_REQUIRE(G == kGroup, DQ_ERR_UNSUPPORTED, "weight group size must be %d (got %d)", kGroup, G);
  DQ_REQUIRE(M >= 1 && N >= 1 && K >= kGroup && K % kGroup == 0, DQ_ERR_SHAPE, "bad shape M=%d N=%d K=%d", M, N, K);
  DQ_REQUIRE(y_dtype == DQ_DTYPE_F32 || y_dtype == DQ_DTYPE_BF16, DQ_ERR_UNSUPPORTED, "unknown y_dtype %d", y_dtype);
  DQ_REQUIRE(aligned(x_bf16, 16) && aligned(w_packed, 16) && ldx % 8 == 0 && ldx >= K, DQ_ERR_ALIGN,
             "x and w_packed must be 16-byte aligned, ldx a multiple of 8 and >= K");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  DQ_REQUIRE(a == nullptr || aligned(a, 16), DQ_ERR_ALIGN, "a must be 16-byte aligned");
  DQ_REQUIRE(scratch != nullptr && aligned(scratch, 256), DQ_ERR_ALIGN, "scratch must be non-null and 256-byte aligned");
  DQ_REQUIRE(scratch_bytes >= dq_linear_a16w4_scratch_bytes(M, N, K), DQ_ERR_WORKSPACE,
             "scratch of %zu bytes is smaller than the %zu required", scratch_bytes,
             dq_linear_a16w4_scratch_bytes(M, N, K));
  const int64_t vecs = static_cast<int64_t>(M) * (K / 8);
  int blocks = static_cast<int>((vecs + 255) / 256);
  if (blocks > st->sm_count * 8) blocks = st->sm_count * 8;
  DQ_CHECK_CUDA(launch_pdl(a16::scale_cols_f16_kernel, dim3(blocks), dim3(256), 0, s,
                           static_cast<const __nv_bfloat16*>(x_bf16), ldx, a, M, K,
                           static_cast<__half*>(scratch)));
  const void* xs = scratch;
  const int64_t ld = K;
  if (M <= 32) return a16::launch<32>(xs, ld, w_packed, r, M, N, K, y, y_dtype, s, st);
  return a16::launch<128>(xs, ld, w_packed, r, M, N, K, y, y_dtype, s, st);
}
