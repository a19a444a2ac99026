// Per-token int4 activation quantiser (the runtime half of PermLinear) for sm_100a.
//
//   x32 = float(x) * a[k]            fp32 multiply, no contraction
//   x32 = online Hadamard(x32)       optional (QuaRot R4 "full" / R2 "partial")
//   s   = absmax(x32) / 7            IEEE division; 1 when the row is all zero; optional fp16 round
//   q   = clamp(rint(x32 / s), -8, 7)   IEEE division, round-half-even
//
// Two kernels, one CTA per token row:
//   * rows_kernel: row held in registers (no Hadamard) - one global read, one write.
//   * had_kernel : row staged in shared memory as fp32, butterflies in place, then the same tail.
// Both are HBM-bound streaming kernels (2 bytes in, 1 byte out per element).
#include "act_quant_common.cuh"

namespace dq {

// ---------------------------------------------------------------------------------------------
// register-resident rows (no Hadamard)
// ---------------------------------------------------------------------------------------------
// norm_eps >= 0 puts an RMSNorm in front (the reference's _RMSNbf16Safe, quarot/llama_quarot.py:
// 135-141, and HF's LlamaRMSNorm): v = bf16(x * rsqrt(mean(x^2) + eps)), times the bf16 weight
// (rounded to bf16 again) when norm_w is given - exactly the bf16 tensor the separate norm would
// have written and the quantiser read back.
// KEEP: the scaled values of the absmax pass stay in registers for the code pass (many-rows launch
// shape, where the kernel is bound by instruction issue and registers are plentiful) instead of
// being re-expanded from the raw row (few-rows shape, where occupancy hides latency).
template <int THREADS, int VPT, typename XT, bool KEEP = false>
__global__ void __launch_bounds__(THREADS, (THREADS >= 512 && VPT <= 2) ? 2048 / THREADS : (VPT >= 4 && !KEEP) ? 1024 / THREADS : 1)
act_quant_rows_kernel(const XT* __restrict__ x, int64_t ldx, const float* __restrict__ a, int K,
                      int8_t* __restrict__ codes, float* __restrict__ sx, float* __restrict__ out,
                      int mode, int scale_fp16, const __nv_bfloat16* __restrict__ norm_w,
                      float norm_eps) {
  __shared__ float red[THREADS / 32];
  // the GEMM that consumes the codes may be launched programmatically: let it start streaming
  // its weights now; it waits for this grid before it touches codes / sx
  grid_dep_launch_dependents();
  grid_dep_wait();  // x may come from the kernel before this one; codes / sx may still be read by it
  const int row = blockIdx.x;
  const XT* xr = x + static_cast<int64_t>(row) * ldx;
  // The row is held in registers in its input width (bf16: 4 registers per 8 elements) and
  // expanded once per pass - sum of squares (with a norm), absmax, codes - with identical
  // arithmetic, so that twice as many rows fit in the register file and more loads are in
  // flight per SM.
  Raw8<XT> raw[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = (i * THREADS + threadIdx.x) * 8;
    if (idx < K) raw[i].load(xr + idx);
  }
  const bool norm = norm_eps >= 0.f;
  float inv_rms = 1.f;
  if (norm) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = (i * THREADS + threadIdx.x) * 8;
      if (idx < K) {
        float v[8];
        raw[i].expand(v);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
      }
    }
    ss = block_sum(ss, red, THREADS / 32);
    inv_rms = rsqrtf(__fadd_rn(__fdiv_rn(ss, static_cast<float>(K)), norm_eps));
  }
  auto prologue = [&](float* v, int idx) {
    if (norm) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = bf16_round(__fmul_rn(v[e], inv_rms));
      if (norm_w != nullptr) {
        Raw8<__nv_bfloat16> wr;
        wr.load(norm_w + idx);
        float wv[8];
        wr.expand(wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = bf16_round(__fmul_rn(wv[e], v[e]));
      }
    }
    if (a != nullptr) {
      float av[8];
      load8(a + idx, av);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(v[e], av[e]);
    }
  };
  float amax = 0.f;
  float kept[KEEP ? VPT : 1][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = (i * THREADS + threadIdx.x) * 8;
    if (idx < K) {
      float v[8];
      raw[i].expand(v);
      prologue(v, idx);
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
      if constexpr (KEEP) {
#pragma unroll
        for (int e = 0; e < 8; ++e) kept[i][e] = v[e];
      }
    }
  }
  amax = block_max(amax, red, THREADS / 32);
  const float s = token_scale(amax, scale_fp16);
  if (threadIdx.x == 0 && sx != nullptr) sx[row] = s;
  int8_t* crow = (codes != nullptr) ? codes + static_cast<int64_t>(row) * K : nullptr;
  float* orow = out_row_ptr(out, row, K, mode);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = (i * THREADS + threadIdx.x) * 8;
    if (idx < K) {
      if constexpr (KEEP) {
        emit8(kept[i], s, mode, crow, orow, idx, scale_fp16);
      } else {
        float v[8];
        raw[i].expand(v);
        prologue(v, idx);
        emit8(v, s, mode, crow, orow, idx, scale_fp16);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// shared-memory rows with the online Hadamard
// ---------------------------------------------------------------------------------------------
// One radix-2 stage over the whole row: element index = (hi*2h + lo)*stride + c pairs with
// + h*stride; (a, b) -> (a + b, a - b).  stride = 1 for the "full" transform (independent
// contiguous segments whose length is a multiple of 2h), stride = head_dim for the "partial"
// one (butterflies across the head index).  Stages run in the order h = 1, 2, 4, ... so every
// sum is formed exactly as in the reference's butterfly loop.
template <int THREADS>
__device__ __forceinline__ void wht_stage(float* row, int K, int h, int stride) {
  for (int b = threadIdx.x; b < K / 2; b += THREADS) {
    const int c = b % stride;
    const int hb = b / stride;
    const int i = ((hb / h) * 2 * h + (hb % h)) * stride + c;
    const int j = i + h * stride;
    const float u = row[i], w = row[j];
    row[i] = __fadd_rn(u, w);
    row[j] = __fsub_rn(u, w);
  }
}

constexpr int kMaxHadK = 32;

template <int THREADS, typename XT>
__global__ void __launch_bounds__(THREADS)
act_quant_had_kernel(const XT* __restrict__ x, const XT* __restrict__ up, int64_t ldx,
                     const float* __restrict__ a, int K,
                     int had_kind, int had_k, int had_dim, float had_scale,
                     const float* __restrict__ had_mat, int8_t* __restrict__ codes,
                     float* __restrict__ sx, float* __restrict__ out, int mode, int scale_fp16) {
  extern __shared__ float sm_row[];
  __shared__ float red[THREADS / 32];
  float* row = sm_row;
  float* hm = sm_row + K;  // [had_k, had_k] when had_k > 1
  grid_dep_launch_dependents();
  grid_dep_wait();
  const int r = blockIdx.x;
  const XT* xr = x + static_cast<int64_t>(r) * ldx;
  const XT* ur = (up != nullptr) ? up + static_cast<int64_t>(r) * ldx : nullptr;

  for (int idx = threadIdx.x * 8; idx < K; idx += THREADS * 8) {
    float v[8];
    load8(xr + idx, v);
    apply_gate(ur != nullptr ? ur + idx : nullptr, v);
    if (a != nullptr) {
      float av[8];
      load8(a + idx, av);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(v[e], av[e]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) row[idx + e] = v[e];
  }
  if (had_kind == DQ_HAD_FULL && had_k > 1)
    for (int i = threadIdx.x; i < had_k * had_k; i += THREADS) hm[i] = had_mat[i];
  __syncthreads();

  if (had_kind == DQ_HAD_FULL) {
    const int P = K / had_k;  // Walsh-Hadamard length of each contiguous segment
    for (int h = 1; h < P; h <<= 1) {
      wht_stage<THREADS>(row, K, h, 1);
      __syncthreads();
    }
    if (had_k > 1) {
      // out[i][c] = sum_j H[i][j] * (v[j][c] * scale), j ascending, fp32
      for (int c = threadIdx.x; c < P; c += THREADS) {
        float v[kMaxHadK];
#pragma unroll
        for (int j = 0; j < kMaxHadK; ++j)
          v[j] = (j < had_k) ? __fmul_rn(row[j * P + c], had_scale) : 0.f;
        for (int i = 0; i < had_k; ++i) {
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < kMaxHadK; ++j)
            if (j < had_k) acc = __fadd_rn(acc, __fmul_rn(hm[i * had_k + j], v[j]));
          row[i * P + c] = acc;
        }
      }
    } else {
      for (int i = threadIdx.x; i < K; i += THREADS) row[i] = __fmul_rn(row[i], had_scale);
    }
    __syncthreads();
  } else if (had_kind == DQ_HAD_PARTIAL) {
    const int H = K / had_dim;
    for (int h = 1; h < H; h <<= 1) {
      wht_stage<THREADS>(row, K, h, had_dim);
      __syncthreads();
    }
    for (int i = threadIdx.x; i < K; i += THREADS) row[i] = __fmul_rn(row[i], had_scale);
    __syncthreads();
  }

  float s = 1.f;
  if (mode != MODE_RAW) {
    float amax = 0.f;
    for (int i = threadIdx.x; i < K; i += THREADS) amax = fmaxf(amax, fabsf(row[i]));
    amax = block_max(amax, red, THREADS / 32);
    s = token_scale(amax, scale_fp16);
    if (threadIdx.x == 0 && sx != nullptr) sx[r] = s;
  }
  int8_t* crow = (codes != nullptr) ? codes + static_cast<int64_t>(r) * K : nullptr;
  float* orow = out_row_ptr(out, r, K, mode);
  for (int idx = threadIdx.x * 8; idx < K; idx += THREADS * 8) {
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = row[idx + e];
    emit8(v, s, mode, crow, orow, idx, scale_fp16);
  }
}

// ---------------------------------------------------------------------------------------------
// full online Hadamard with a large +-1 factor (orders 36 ... 172 of the reference's table)
// ---------------------------------------------------------------------------------------------
// Same arithmetic as act_quant_had_kernel for had_k up to kMaxHadKBig: the row (as fp32) and a
// second buffer of the same size sit in shared memory next to the factor stored as one byte per
// entry.  Walsh-Hadamard stages over the contiguous segments in place, then one thread per output
// element: out[i][c] = sum_j H[i][j] * (v[j][c] * scale), j ascending, fp32 - the order of the
// stand-alone restatement, so codes stay bit-identical.  Used for decode-size batches of models
// whose intermediate size is not 28 * 2^k (e.g. 11008 = 172 * 64); not a tuned path.
constexpr int kMaxHadKBig = 172;

template <int THREADS, typename XT>
__global__ void __launch_bounds__(THREADS)
act_quant_had_big_kernel(const XT* __restrict__ x, const XT* __restrict__ up, int64_t ldx,
                         const float* __restrict__ a, int K, int had_k, float had_scale,
                         const float* __restrict__ had_mat, int8_t* __restrict__ codes,
                         float* __restrict__ sx, float* __restrict__ out, int mode, int scale_fp16) {
  extern __shared__ float sm_row[];
  __shared__ float red[THREADS / 32];
  float* row = sm_row;
  float* res = sm_row + K;
  signed char* hm = reinterpret_cast<signed char*>(sm_row + 2 * K);
  grid_dep_launch_dependents();
  grid_dep_wait();
  const int r = blockIdx.x;
  const XT* xr = x + static_cast<int64_t>(r) * ldx;
  const XT* ur = (up != nullptr) ? up + static_cast<int64_t>(r) * ldx : nullptr;
  for (int idx = threadIdx.x * 8; idx < K; idx += THREADS * 8) {
    float v[8];
    load8(xr + idx, v);
    apply_gate(ur != nullptr ? ur + idx : nullptr, v);
    if (a != nullptr) {
      float av[8];
      load8(a + idx, av);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(v[e], av[e]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) row[idx + e] = v[e];
  }
  for (int i = threadIdx.x; i < had_k * had_k; i += THREADS) hm[i] = had_mat[i] > 0.f ? 1 : -1;
  __syncthreads();
  const int P = K / had_k;
  for (int h = 1; h < P; h <<= 1) {
    wht_stage<THREADS>(row, K, h, 1);
    __syncthreads();
  }
  for (int i = threadIdx.x; i < K; i += THREADS) row[i] = __fmul_rn(row[i], had_scale);
  __syncthreads();
  for (int o = threadIdx.x; o < K; o += THREADS) {
    const int i = o / P, c = o - i * P;
    const signed char* hrow = hm + i * had_k;
    float acc = 0.f;
    for (int j = 0; j < had_k; ++j) {
      const float v = row[j * P + c];
      acc = __fadd_rn(acc, hrow[j] > 0 ? v : -v);
    }
    res[o] = acc;
  }
  __syncthreads();
  float s = 1.f;
  if (mode != MODE_RAW) {
    float amax = 0.f;
    for (int i = threadIdx.x; i < K; i += THREADS) amax = fmaxf(amax, fabsf(res[i]));
    amax = block_max(amax, red, THREADS / 32);
    s = token_scale(amax, scale_fp16);
    if (threadIdx.x == 0 && sx != nullptr) sx[r] = s;
  }
  int8_t* crow = (codes != nullptr) ? codes + static_cast<int64_t>(r) * K : nullptr;
  float* orow = out_row_ptr(out, r, K, mode);
  for (int idx = threadIdx.x * 8; idx < K; idx += THREADS * 8) {
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = res[idx + e];
    emit8(v, s, mode, crow, orow, idx, scale_fp16);
  }
}

// The fast online-Hadamard kernels (warp-shuffle butterflies, constant-bank matrix stage, the four-CTA
// cluster form) are compiled in translation units of their own (act_quant_had.cuh, one .cu per input
// type): their unrolled matrix stages dominate the build time.
int launch_had_fast(const __nv_bfloat16* x, const __nv_bfloat16* up, int64_t ldx, const float* a,
                    const dq_hadamard_desc* had, int M, int K, size_t smem, int8_t* codes, float* sx, float* out,
                    int mode, int scale_fp16, cudaStream_t stream, bool* taken);
int launch_had_fast(const float* x, const float* up, int64_t ldx, const float* a, const dq_hadamard_desc* had,
                    int M, int K, size_t smem, int8_t* codes, float* sx, float* out, int mode, int scale_fp16,
                    cudaStream_t stream, bool* taken);
int init_had_fast_bf16();
int init_had_fast_f32();


constexpr int kHadThreads = 512;
constexpr int kHadMaxSmem = 200 * 1024;

int init_act_quant_kernels() {
  cudaError_t e = cudaFuncSetAttribute(act_quant_had_kernel<kHadThreads, __nv_bfloat16>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(act_quant_had_big_kernel<kHadThreads, __nv_bfloat16>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(act_quant_had_big_kernel<kHadThreads, float>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(act_quant_had_kernel<kHadThreads, float>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kHadMaxSmem);
  if (e != cudaSuccess)
    return set_error(DQ_ERR_CUDA, "cudaFuncSetAttribute(act_quant_had) failed: %s",
                     cudaGetErrorString(e));
  int rc = init_had_fast_bf16();
  if (rc != DQ_OK) return rc;
  return init_had_fast_f32();
}

static bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

static int check_had(const dq_hadamard_desc* had, int K) {
  if (had == nullptr || had->kind == DQ_HAD_NONE) return DQ_OK;
  if (had->kind == DQ_HAD_FULL) {
    DQ_REQUIRE(had->had_k >= 1 && had->had_k <= kMaxHadKBig, DQ_ERR_UNSUPPORTED,
               "had_k=%d outside [1,%d]", had->had_k, kMaxHadKBig);
    DQ_REQUIRE(K % had->had_k == 0 && is_pow2(K / had->had_k), DQ_ERR_SHAPE,
               "K=%d is not had_k=%d times a power of two", K, had->had_k);
    DQ_REQUIRE(had->had_k == 1 || had->had_mat != nullptr, DQ_ERR_NULL, "had_mat is null");
    return DQ_OK;
  }
  if (had->kind == DQ_HAD_PARTIAL) {
    DQ_REQUIRE(had->had_k == 1, DQ_ERR_UNSUPPORTED,
               "partial Hadamard with a non-power-of-two head count is not implemented");
    DQ_REQUIRE(had->had_dim >= 1 && K % had->had_dim == 0 && is_pow2(K / had->had_dim),
               DQ_ERR_SHAPE, "K=%d / had_dim=%d must be a power of two", K, had->had_dim);
    return DQ_OK;
  }
  return set_error(DQ_ERR_UNSUPPORTED, "unknown Hadamard kind %d", had->kind);
}

template <typename XT>
static int launch_act(const XT* x, int64_t ldx, const float* a, const dq_hadamard_desc* had, int M,
                      int K, int8_t* codes, float* sx, float* out, int mode, int scale_fp16,
                      cudaStream_t stream, const XT* up = nullptr,
                      const __nv_bfloat16* norm_w = nullptr, float norm_eps = -1.f) {
  DQ_REQUIRE(x != nullptr, DQ_ERR_NULL, "x is null");
  DQ_REQUIRE(M >= 0 && K >= 8 && K % 8 == 0, DQ_ERR_SHAPE, "bad shape M=%d K=%d (K %% 8 != 0)", M, K);
  DQ_REQUIRE(ldx >= K && ldx % 8 == 0, DQ_ERR_ALIGN, "ldx=%lld must be >= K and a multiple of 8",
             (long long)ldx);
  DQ_REQUIRE(aligned(x, 16) && (a == nullptr || aligned(a, 16)), DQ_ERR_ALIGN,
             "x and a must be 16-byte aligned");
  DQ_REQUIRE((codes == nullptr || aligned(codes, 8)) && (out == nullptr || aligned(out, 16)),
             DQ_ERR_ALIGN, "outputs must be aligned (codes 8 B, out 16 B)");
  DQ_REQUIRE(K <= 65536, DQ_ERR_UNSUPPORTED, "K=%d exceeds 65536", K);
  int rc = check_had(had, K);
  if (rc != DQ_OK) return rc;
  if (M == 0) return DQ_OK;
  const bool use_had = had != nullptr && had->kind != DQ_HAD_NONE;
  DQ_REQUIRE(norm_eps < 0.f || (!use_had && up == nullptr && mode != MODE_RAW && K <= 32768),
             DQ_ERR_UNSUPPORTED, "the fused RMSNorm covers plain rows of K <= 32768 without a Hadamard");
  if (use_had || mode == MODE_RAW || K > 32768 || up != nullptr) {  // longer rows than the register path holds
    const int hk = use_had ? had->had_k : 1;
    if (use_had && had->kind == DQ_HAD_FULL && hk > kMaxHadK) {
      // large +-1 factor: row + result buffer + the factor as bytes
      const size_t big = static_cast<size_t>(K) * 8 + (static_cast<size_t>(hk) * hk + 15) / 16 * 16;
      DQ_REQUIRE(big <= static_cast<size_t>(kHadMaxSmem), DQ_ERR_UNSUPPORTED,
                 "row of K=%d with a Hadamard factor of order %d does not fit in shared memory", K, hk);
      DQ_CHECK_CUDA(launch_pdl(act_quant_had_big_kernel<kHadThreads, XT>, dim3(M), dim3(kHadThreads), big,
                               stream, x, up, ldx, a, K, hk, had->scale, had->had_mat, codes, sx, out, mode,
                               scale_fp16));
      DQ_CHECK_CUDA(cudaGetLastError());
      return DQ_OK;
    }
    const size_t smem = static_cast<size_t>(K) * 4 + (hk > 1 ? static_cast<size_t>(hk) * hk * 4 : 0);
    DQ_REQUIRE(smem <= static_cast<size_t>(kHadMaxSmem), DQ_ERR_UNSUPPORTED,
               "row of K=%d does not fit in shared memory", K);
    if (use_had) {
      bool taken = false;
      const int rc2 = launch_had_fast(x, up, ldx, a, had, M, K, smem, codes, sx, out, mode, scale_fp16, stream, &taken);
      if (taken) return rc2;
    }
    DQ_CHECK_CUDA(launch_pdl(act_quant_had_kernel<kHadThreads, XT>, dim3(M), dim3(kHadThreads), smem,
                             stream, x, up, ldx, a, K, use_had ? had->kind : DQ_HAD_NONE, hk,
                             use_had ? had->had_dim : 0, use_had ? had->scale : 1.f,
                             use_had ? had->had_mat : nullptr, codes, sx, out, mode, scale_fp16));
  } else {
    // one CTA per row; as many threads as the row has 16-byte vectors (up to 1024) so that each
    // thread holds few elements and many warps are resident to hide the load -> reduce -> store
    // latency chain
    const int vec = K / 8;
#define DQ_ROWS_LAUNCH_K(T, V, KP)                                                                \
  DQ_CHECK_CUDA(launch_pdl(act_quant_rows_kernel<T, V, XT, KP>, dim3(M), dim3(T), 0, stream, x, ldx, a, K, \
                           codes, sx, out, mode, scale_fp16, norm_w, norm_eps))
#define DQ_ROWS_LAUNCH(T, V) DQ_ROWS_LAUNCH_K(T, V, false)
    constexpr int kBigM = 1024;
    // Many rows (prefill): fewer threads per row, each with four 16-byte loads in flight - the
    // kernel is then bound by bytes in flight per SM, not by the per-row latency chain.
    if (M >= kBigM && vec > 128 && vec <= 512) DQ_ROWS_LAUNCH_K(128, 4, true);
    else if (M >= kBigM && vec > 512 && vec <= 1024) DQ_ROWS_LAUNCH_K(256, 4, true);
    // long rows (e.g. 14336): 256 threads with eight vectors each, re-expanded in the code pass, so
    // that four CTAs (four rows) share an SM - 512 threads keeping their values held one row per SM
    // and ran at 1.85 TB/s where this shape reaches 2.7
    else if (M >= kBigM && vec > 1024 && vec <= 2048) DQ_ROWS_LAUNCH_K(256, 8, false);
    else if (vec <= 128) DQ_ROWS_LAUNCH(128, 1);
    else if (vec <= 256) DQ_ROWS_LAUNCH(256, 1);
    else if (vec <= 512) DQ_ROWS_LAUNCH(512, 1);
    else if (vec <= 1024) DQ_ROWS_LAUNCH(1024, 1);
    else if (vec <= 2048) DQ_ROWS_LAUNCH(1024, 2);
    else DQ_ROWS_LAUNCH(1024, 4);
#undef DQ_ROWS_LAUNCH
#undef DQ_ROWS_LAUNCH_K
  }
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}

// ---------------------------------------------------------------------------------------------
// one activation scale per (token, group of 128): the quantiser of the reference's fused W4A4
// Triton kernel (per row and K tile) as a stand-alone pass
// ---------------------------------------------------------------------------------------------
// One warp per (token, group); a lane holds four consecutive elements.  IEEE divisions (this
// variant is not on the measured path).  round_away = 1 rounds halves away from zero like the
// Triton kernel's libdevice.round, 0 rounds them to even like torch.round.
__global__ void __launch_bounds__(256)
act_quant_grouped_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const float* __restrict__ a,
                         int M, int K, int8_t* __restrict__ codes, float* __restrict__ sxg,
                         int scale_fp16, int round_away) {
  grid_dep_launch_dependents();
  grid_dep_wait();
  const int groups = K / kGroup;
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // (token, group)
  if (unit >= M * groups) return;
  const int m = unit / groups, g = unit % groups;
  const int lane = threadIdx.x & 31;
  const int k0 = g * kGroup + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(x + static_cast<int64_t>(m) * ldx + k0);
  float v[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u),
                __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000u)};
  if (a != nullptr) {
    const float4 av = *reinterpret_cast<const float4*>(a + k0);
    v[0] = __fmul_rn(v[0], av.x); v[1] = __fmul_rn(v[1], av.y);
    v[2] = __fmul_rn(v[2], av.z); v[3] = __fmul_rn(v[3], av.w);
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = token_scale(amax, scale_fp16);
  if (lane == 0) sxg[static_cast<size_t>(g) * M + m] = s;
  int q[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float t = __fdiv_rn(v[e], s);
    const float rq = round_away ? roundf(t) : rintf(t);
    q[e] = static_cast<int>(fminf(fmaxf(rq, -8.0f), 7.0f));
  }
  const uint32_t packed = (static_cast<uint32_t>(q[0]) & 0xFFu) | ((static_cast<uint32_t>(q[1]) & 0xFFu) << 8) |
                          ((static_cast<uint32_t>(q[2]) & 0xFFu) << 16) | ((static_cast<uint32_t>(q[3]) & 0xFFu) << 24);
  *reinterpret_cast<uint32_t*>(codes + static_cast<int64_t>(m) * K + k0) = packed;
}

}  // namespace dq

using namespace dq;

extern "C" int dq_quant_act_int4_grouped(const void* x_bf16, int64_t ldx, const float* a, int M, int K,
                                         int G, int8_t* codes, float* sx_groups, int scale_fp16,
                                         int round_away, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(x_bf16 != nullptr && codes != nullptr && sx_groups != nullptr, DQ_ERR_NULL, "null x / codes / sx_groups");
  DQ_REQUIRE(G == kGroup, DQ_ERR_UNSUPPORTED, "activation group size must be %d (got %d)", kGroup, G);
  DQ_REQUIRE(M >= 0 && K >= kGroup && K % kGroup == 0, DQ_ERR_SHAPE, "bad shape M=%d K=%d", M, K);
  DQ_REQUIRE(ldx >= K && ldx % 4 == 0, DQ_ERR_ALIGN, "ldx=%lld must be >= K and a multiple of 4", (long long)ldx);
  DQ_REQUIRE(aligned(x_bf16, 8) && (a == nullptr || aligned(a, 16)) && aligned(codes, 4), DQ_ERR_ALIGN,
             "x (8 B), a (16 B) and codes (4 B) must be aligned");
  const int64_t units = static_cast<int64_t>(M) * (K / kGroup);
  DQ_REQUIRE(units < (1ll << 31), DQ_ERR_SHAPE, "too many (token, group) units");
  const int per_cta = 8;
  DQ_CHECK_CUDA(launch_pdl(act_quant_grouped_kernel, dim3(static_cast<unsigned>((units + per_cta - 1) / per_cta)),
                           dim3(per_cta * 32), 0, static_cast<cudaStream_t>(stream),
                           static_cast<const __nv_bfloat16*>(x_bf16), ldx, a, M, K, codes, sx_groups,
                           scale_fp16, round_away));
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}

extern "C" int dq_quant_act_int4(const void* x_bf16, int64_t ldx, const float* a,
                                 const dq_hadamard_desc* had, int M, int K, int8_t* codes,
                                 float* sx, int scale_fp16, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(codes != nullptr && sx != nullptr, DQ_ERR_NULL, "codes / sx is null");
  return launch_act(static_cast<const __nv_bfloat16*>(x_bf16), ldx, a, had, M, K, codes, sx,
                    nullptr, MODE_CODES, scale_fp16, static_cast<cudaStream_t>(stream));
}

extern "C" int dq_quant_act_int4_f32(const float* x_f32, int64_t ldx, const float* a,
                                     const dq_hadamard_desc* had, int M, int K, int8_t* codes,
                                     float* sx, int scale_fp16, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(codes != nullptr && sx != nullptr, DQ_ERR_NULL, "codes / sx is null");
  return launch_act(x_f32, ldx, a, had, M, K, codes, sx, nullptr, MODE_CODES, scale_fp16,
                    static_cast<cudaStream_t>(stream));
}

extern "C" int dq_quant_act_int4_rmsnorm(const void* x_bf16, int64_t ldx, const void* norm_weight_bf16,
                                         float eps, const float* a, int M, int K, int8_t* codes,
                                         float* sx, int scale_fp16, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(codes != nullptr && sx != nullptr, DQ_ERR_NULL, "codes / sx is null");
  DQ_REQUIRE(eps >= 0.f, DQ_ERR_SHAPE, "eps must be >= 0 (got %g)", (double)eps);
  DQ_REQUIRE(norm_weight_bf16 == nullptr || aligned(norm_weight_bf16, 16), DQ_ERR_ALIGN,
             "norm weight must be 16-byte aligned");
  return launch_act(static_cast<const __nv_bfloat16*>(x_bf16), ldx, a, nullptr, M, K, codes, sx,
                    nullptr, MODE_CODES, scale_fp16, static_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(nullptr),
                    static_cast<const __nv_bfloat16*>(norm_weight_bf16), eps);
}

extern "C" int dq_fakequant_act_int4(const void* x, int x_is_f32, int64_t ldx, const float* a,
                                     const dq_hadamard_desc* had, int M, int K, float* out,
                                     int scale_fp16, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(out != nullptr, DQ_ERR_NULL, "out is null");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (x_is_f32)
    return launch_act(static_cast<const float*>(x), ldx, a, had, M, K, nullptr, nullptr, out,
                      MODE_FAKE, scale_fp16, s);
  return launch_act(static_cast<const __nv_bfloat16*>(x), ldx, a, had, M, K, nullptr, nullptr, out,
                    MODE_FAKE, scale_fp16, s);
}

extern "C" int dq_fakequant_act_int4_bf16(const void* x_bf16, int64_t ldx, int M, int K,
                                          void* out_bf16, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(out_bf16 != nullptr, DQ_ERR_NULL, "out is null");
  return launch_act(static_cast<const __nv_bfloat16*>(x_bf16), ldx, nullptr, nullptr, M, K, nullptr,
                    nullptr, static_cast<float*>(out_bf16), MODE_FAKE_BF16, 0,
                    static_cast<cudaStream_t>(stream));
}

extern "C" int dq_hadamard_f32(const float* x, float* out, int M, int K,
                               const dq_hadamard_desc* had, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  DQ_REQUIRE(out != nullptr, DQ_ERR_NULL, "out is null");
  DQ_REQUIRE(had != nullptr && had->kind != DQ_HAD_NONE, DQ_ERR_NULL, "no Hadamard described");
  return launch_act(x, static_cast<int64_t>(K), nullptr, had, M, K, nullptr, nullptr, out, MODE_RAW,
                    0, static_cast<cudaStream_t>(stream));
}

extern "C" int dq_quant_act_int4_gated(const void* gate_bf16, const void* up_bf16, int64_t ld,
                                       const float* a, const dq_hadamard_desc* had, int M, int K,
                                       int8_t* codes, float* sx, int scale_fp16, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  if (M == 0) return DQ_OK;
  DQ_REQUIRE(codes != nullptr && sx != nullptr && up_bf16 != nullptr, DQ_ERR_NULL, "codes / sx / up is null");
  DQ_REQUIRE(aligned(up_bf16, 16), DQ_ERR_ALIGN, "up must be 16-byte aligned");
  return launch_act(static_cast<const __nv_bfloat16*>(gate_bf16), ld, a, had, M, K, codes, sx, nullptr,
                    MODE_CODES, scale_fp16, static_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(up_bf16));
}
