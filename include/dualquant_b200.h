/*
 * dualquant_b200 -- C ABI of the Blackwell (sm_100a) W4A4 inference hot path.
 *
 * Every entry point is `extern "C"`, takes raw device pointers plus sizes, launches on the
 * caller's stream and returns an int status (0 = DQ_OK).  Nothing here allocates, frees,
 * synchronises or touches the legacy stream; scratch memory is caller-provided.  Pointers are
 * device pointers unless a comment says "host".  `stream` is a `cudaStream_t` passed as void*.
 *
 * The citations name the reference interface (path inside sayehs-dmatrix/dualquant : lines)
 * whose work the entry point takes over.
 */
#ifndef DUALQUANT_B200_H
#define DUALQUANT_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define DQ_API __attribute__((visibility("default")))
#else
#define DQ_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------------ */
enum {
  DQ_OK = 0,
  DQ_ERR_SHAPE = 1,       /* a size violates the kernel's divisibility / range rules          */
  DQ_ERR_ALIGN = 2,       /* a pointer or leading dimension is not aligned as required        */
  DQ_ERR_NULL = 3,        /* a required pointer is null                                       */
  DQ_ERR_ARCH = 4,        /* the current device is not compute capability 10.x                */
  DQ_ERR_CUDA = 5,        /* a CUDA runtime / driver call failed (see dq_last_error_string)   */
  DQ_ERR_WORKSPACE = 6,   /* caller-provided scratch is too small                             */
  DQ_ERR_UNSUPPORTED = 7, /* valid request that this build has no kernel for                  */
  DQ_ERR_NOT_INIT = 8,    /* dq_init was not called for the current device                    */
  DQ_ERR_TIMEOUT = 9      /* a bounded device-side wait expired (read via dq_device_status)   */
};

/* element types of the output matrix Y */
enum { DQ_DTYPE_F32 = 0, DQ_DTYPE_BF16 = 1 };

/* block-scaled FP4 flavours (formats/mx.py:23-31, formats/nvfp4.py:11-19) */
enum { DQ_FP4_MXFP4 = 0, DQ_FP4_NVFP4 = 1 };

/* online-Hadamard kinds (activations/perm_linear.py:76-106) */
enum {
  DQ_HAD_NONE = 0,
  DQ_HAD_FULL = 1,    /* x.view(-1, had_k, n/had_k): WHT over the last axis, * scale, had_K @   */
  DQ_HAD_PARTIAL = 2  /* x.view(-1, n/had_dim, had_dim): WHT across the head index, * scale     */
};

/*
 * Online Hadamard description.  Mirrors the attributes that
 * quarot/online_had_install.py:44-58 sets on a PermLinear (had_K, K, had_dim) and the
 * arithmetic of quarot/vendor/hadamard_utils.py:92-101 + quarot/__init__.py:39-64.
 */
typedef struct dq_hadamard_desc {
  int32_t kind;          /* DQ_HAD_*                                                         */
  int32_t had_k;         /* FULL: order of the +-1 matrix (1 = pure Walsh-Hadamard)          */
  int32_t had_dim;       /* PARTIAL: head_dim                                                */
  float scale;           /* fp32 factor applied after the Walsh-Hadamard butterflies         */
  const float* had_mat;  /* FULL with had_k > 1: device pointer to [had_k, had_k] fp32       */
} dq_hadamard_desc;

/* ---- library state ----------------------------------------------------------------------- */

/* One-time per-device set-up (kernel attributes, driver entry points, status word).  Call it
 * outside stream capture, with the device current.  Replaces the once-only
 * cudaFuncSetAttribute logic of the reference's launcher patch
 * (ablation/real_int4_kernel/nunchaku_patches/0001-dualquant-w4a4-modifications.patch:1136-1143). */
DQ_API int dq_init(int device);

/* Text of the last error raised on the calling thread (host pointer, never null). */
DQ_API const char* dq_last_error_string(void);

/* Reads (and clears) the device-side status word of `device`: 0, or DQ_ERR_TIMEOUT plus a
 * site code in the upper 16 bits when a bounded wait inside a kernel expired.  Synchronises
 * the device. */
DQ_API int dq_device_status(int device);

DQ_API int dq_abi_version(void);

/* Launch-shape overrides for measurement sweeps and tests (no counterpart in the reference, whose
 * Triton kernels autotune instead: vendor/dualscale_kernel_benchmark/fused_dual_scale_kernel.py:26-53).
 * name (host string): "linear_fused" (1 = dq_linear_w4a4_int4 runs decode batches, M <= 16, as one
 * launch that quantises inside the GEMM kernel; 0 = quantiser + GEMM, the default), "fused_stages", "fused_split", "fused_extra_cta"
 * (0 = the library's own choice), "ar_wait_log2" (the fused all-reduce waits 2^value SM cycles for a
 * peer before it gives up with DQ_ERR_TIMEOUT; 0 = 30, about half a second).  Process-wide, not thread-safe against concurrent launches. */
DQ_API int dq_set_tuning(const char* name, int value);

/* Tensor-core ceiling probe: launches, on every SM, a loop of `iters` x 4 tcgen05.mma instructions
 * (UMMA 128 x 256, 32 bytes of K each) on operands resident in shared / tensor memory; kind 0 =
 * kind::i8, 1 = kind::mxf4nvf4 with E8M0 block-32 scales, 2 = with E4M3 block-16 scales, 3 =
 * kind::f8f6f4 on E4M3 operands, 4 = the same with the operands re-fetched from L2 by bulk copies for
 * every four instructions (the K loop of the prefill GEMM without an epilogue).  *ops_out
 * (host, may be null) receives the arithmetic operations the launch performs (2 per multiply-add);
 * the caller times the launch with events.  Measurement helper in the spirit of the reference's
 * roofline estimate (ablation/real_int4_kernel/verification/ceiling_analysis.py:55-63), which
 * measures a cuBLAS bf16 GEMM and quotes datasheet figures for the integer rates. */
DQ_API int dq_mma_peak_probe(int kind, int iters, double* ops_out, void* stream);

/* ---- weights ----------------------------------------------------------------------------- */

/* Bytes of the packed weight matrix for (N, K): ceil(N/128) * (K/128) tiles of 8448 bytes
 * (8192 bytes of int4 codes + the tile's 128 fp16 group scales). */
DQ_API size_t dq_packed_w_bytes(int N, int K);

/*
 * Re-pack int4 weight codes into the streaming layout the GEMM consumes and transpose the
 * group scales.  Input is either signed codes (int8 [N,K], values in [-8,7]) or the
 * reference's packed form (uint8 [N,K/2], low nibble = even k, high nibble = odd k, biased
 * by +8: vendor/dualscale_kernel_benchmark/fused_dual_scale_kernel.py:156-189); give exactly
 * one of the two.  sw is fp16 [N, K/G]; sw_t receives ceil(N/128)*128*(K/G) fp16 values in the
 * same tile order as w_packed ([row tile][k group][row in tile]).
 */
DQ_API int dq_pack_w_int4(const int8_t* codes, const uint8_t* ref_packed, const void* sw,
                   int N, int K, int G, uint8_t* w_packed, void* sw_t, void* stream);

/* Inverse of dq_pack_w_int4: signed codes int8 [N,K] from the streaming layout. */
DQ_API int dq_unpack_w_int4(const uint8_t* w_packed, int N, int K, int8_t* codes, void* stream);

/*
 * Symmetric per-group int4 weight quantiser: W bf16 [N,K] -> codes int8 [N,K] and fp16
 * scales [N,K/G] (absmax/7, 1 for an all-zero group), the arithmetic of
 * formats/rtn_int.py:43-69 with the scale rounded to fp16 before the division.
 */
DQ_API int dq_quant_w_int4(const void* w_bf16, int N, int K, int G, int8_t* codes, void* sw,
                    void* stream);

/* ---- activations ------------------------------------------------------------------------- */

/*
 * Per-token int4 activation quantiser, the runtime half of PermLinear
 * (activations/perm_linear.py:108-134 with formats/rtn_int.py:43-69, block_size=-1):
 *   x32 = float(x) * a        (a may be null)
 *   x32 = hadamard(x32)       (had may be null / DQ_HAD_NONE)
 *   s   = absmax(x32)/7 (1 if 0), optionally rounded to fp16
 *   q   = clamp(round_half_even(x32/s), -8, 7)
 * x is bf16 [M,K] with leading dimension ldx (elements); codes int8 [M,K]; sx fp32 [M].
 * `a` is fp32 [K].  `had` is a host pointer.
 * scale_fp16 (here and in every entry point that takes it): 0 = fp32 token scale (the reference's
 * arithmetic when an activation scale or a Hadamard is configured), 1 = the scale rounded to fp16
 * (storage format of the benchmark configurations), 2 = the whole quantiser in bf16 arithmetic
 * (scale = bf16(absmax/7), q = round(bf16(x/s))): what the reference computes on a bf16 input with
 * neither activation scale nor Hadamard (activations/perm_linear.py:109-133).
 */
DQ_API int dq_quant_act_int4(const void* x_bf16, int64_t ldx, const float* a,
                      const dq_hadamard_desc* had, int M, int K, int8_t* codes, float* sx,
                      int scale_fp16, void* stream);

/* dq_quant_act_int4 for fp32 rows: the reference upcasts every input to fp32 before it scales
 * and quantises (activations/perm_linear.py:119-125), so fp32 (and fp16, widened by the caller)
 * activations are quantised from their fp32 values rather than through a bf16 rounding. */
DQ_API int dq_quant_act_int4_f32(const float* x_f32, int64_t ldx, const float* a,
                                 const dq_hadamard_desc* had, int M, int K, int8_t* codes,
                                 float* sx, int scale_fp16, void* stream);

/*
 * dq_quant_act_int4 with the MLP activation fused in front: the input row is
 * bf16(bf16(SiLU(gate)) * up), the bf16 arithmetic of the decoder MLP that feeds down_proj
 * (the reference leaves it to the HF model: hidden = act_fn(gate_proj(x)) * up_proj(x), then
 * PermLinear.forward of down_proj, activations/perm_linear.py:136-141).  gate and up are bf16
 * [M,K] with the same leading dimension ld (e.g. the two halves of a fused gate+up output).
 */
DQ_API int dq_quant_act_int4_gated(const void* gate_bf16, const void* up_bf16, int64_t ld,
                                   const float* a, const dq_hadamard_desc* had, int M, int K,
                                   int8_t* codes, float* sx, int scale_fp16, void* stream);

/* Same arithmetic, but writes the de-quantised value q*s as fp32 [M,K] (what
 * FormatSpec.cast returns, formats/base.py:33-39).  x is fp32 when x_is_f32 != 0. */
/*
 * RMSNorm fused in front of dq_quant_act_int4 (no Hadamard): per token
 * v = bf16(x * rsqrt(mean(x^2) + eps)), times the bf16 norm weight (rounded to bf16 again) when
 * norm_weight_bf16 is not null, then the column scale a and the per-token int4 quantiser.  This
 * is the reference's _RMSNbf16Safe (quarot/llama_quarot.py:135-141; HF LlamaRMSNorm when a
 * weight is given) followed by PermLinear._quantise_act (activations/perm_linear.py:108-134) in
 * one pass over the row; the bf16 normalised tensor is never written.
 */
DQ_API int dq_quant_act_int4_rmsnorm(const void* x_bf16, int64_t ldx, const void* norm_weight_bf16,
                                     float eps, const float* a, int M, int K, int8_t* codes,
                                     float* sx, int scale_fp16, void* stream);

DQ_API int dq_fakequant_act_int4(const void* x, int x_is_f32, int64_t ldx, const float* a,
                          const dq_hadamard_desc* had, int M, int K, float* out,
                          int scale_fp16, void* stream);

/* Per-token int4 fake-quantisation of bf16 rows with a bf16 result, in one pass: what PermLinear
 * does to its own output when quantize_bmm_input is set - act_fmt.cast(out.float()).to(bf16),
 * activations/perm_linear.py:139-140 - without the fp32 round trip through memory. */
DQ_API int dq_fakequant_act_int4_bf16(const void* x_bf16, int64_t ldx, int M, int K, void* out_bf16,
                                      void* stream);

/* The online Hadamard alone on fp32 rows: out = hadamard(x) (perm_linear.py:76-106). */
DQ_API int dq_hadamard_f32(const float* x, float* out, int M, int K, const dq_hadamard_desc* had,
                    void* stream);

/* ---- block-scaled FP4 (MXFP4 / NVFP4) quantisers ------------------------------------------ */

/*
 * Block-scaled FP4 quantiser along K - the work the reference hands to the external `blockfmt`
 * package (formats/mx.py:23-31 "MXFP4[E2M1]{32}", formats/nvfp4.py:11-19 "NVFP4[E2M1]{16}"),
 * element rounding as legacy_vendor/torch_quant.py:326-356, MX exponent rule as :359-375,
 * E4M3 scale rounding as scale_formats.py:39-45.
 *   x: bf16 or fp32 [M,K] (x_is_f32), optional column scale a fp32 [K]
 *   fmt: DQ_FP4_MXFP4 (block 32, sf = E8M0 byte) or DQ_FP4_NVFP4 (block 16, sf = E4M3 byte)
 *   codes: uint8 [M, K/2], element 2j in the low nibble, 2j+1 in the high nibble
 *   sf:    uint8 [M, K/block]
 *   NVFP4 second-level scale: tensor_scale (device pointer to one fp32) when given, else one
 *   scale per row = absmax_row/(6*448) which is written to row_scale[M] (may be null for MXFP4).
 */
DQ_API int dq_quant_fp4(const void* x, int x_is_f32, int64_t ldx, const float* a, int M, int K,
                        int fmt, const float* tensor_scale, uint8_t* codes, uint8_t* sf,
                        float* row_scale, void* stream);

/*
 * dq_quant_fp4 with the scale bytes written straight into the order dq_gemm_w4a4_fp4 streams
 * (what dq_fp4_sf_to_atoms would produce from the row-major bytes): sf_atoms has
 * dq_fp4_sf_atoms_bytes(M, K, fmt) bytes, rows past M of the last 128-row tile are written as
 * zero.  Needs K % 128 == 0 (MXFP4) / K % 64 == 0 (NVFP4).  Saves one pass per activation.
 */
DQ_API int dq_quant_fp4_atoms(const void* x, int x_is_f32, int64_t ldx, const float* a, int M, int K,
                              int fmt, const float* tensor_scale, uint8_t* codes, uint8_t* sf_atoms,
                              float* row_scale, void* stream);

/* Same arithmetic, de-quantised fp32 [M,K] out: what FormatSpec.cast returns for mxfp4 / nvfp4. */
DQ_API int dq_fakequant_fp4(const void* x, int x_is_f32, int64_t ldx, const float* a, int M, int K,
                            int fmt, const float* tensor_scale, float* out, void* stream);

/* Per-tensor NVFP4 second-level scale absmax(x)/(6*448) (1 for a zero tensor) into *scale. */
DQ_API int dq_nvfp4_tensor_scale(const void* x, int x_is_f32, int64_t numel, float* scale,
                                 void* stream);

/* Bytes of the scale factors of a [rows, K] operand in GEMM ("atom") order: rows padded to 128. */
DQ_API size_t dq_fp4_sf_atoms_bytes(int rows, int K, int fmt);

/* Re-orders row-major scale bytes [rows, K/block] into the order dq_gemm_w4a4_fp4 streams:
 * [row tile of 128][k][512-byte atom: (r % 32) * 16 + (r / 32) * 4 + (k % 4)], padding rows zero.
 * K must be a multiple of 256. */
DQ_API int dq_fp4_sf_to_atoms(const uint8_t* sf, int rows, int K, int fmt, uint8_t* out,
                              void* stream);

/*
 * Block-scaled FP4 W4A4 GEMM (tcgen05 kind::mxf4nvf4): the matmul PermLinear performs on
 * mxfp4 / nvfp4 fake-quantised operands (activations/perm_linear.py:136-141 with the casts of
 * formats/mx.py:23-31 / formats/nvfp4.py:11-19), computed on the packed operands:
 *   Y[m,n] = r[n] * w_scale * x_scale[m] * sum_k (qx[m,k]*sfx[m,k/B]) * (qw[n,k]*sfw[n,k/B])
 * x_codes uint8 [M,K/2], w_codes uint8 [N,K/2] (dq_quant_fp4 output), *_sf_atoms from
 * dq_fp4_sf_to_atoms, x_scale fp32 [M] / w_scale fp32 [1] (NVFP4 second-level scales; null = 1),
 * r fp32 [N] or null, y [M,N] fp32 or bf16.  K % 256 == 0.
 */
DQ_API int dq_gemm_w4a4_fp4(const uint8_t* x_codes, const uint8_t* x_sf_atoms, const float* x_scale,
                            const uint8_t* w_codes, const uint8_t* w_sf_atoms, const float* w_scale,
                            const float* r, int M, int N, int K, int fmt, void* y, int y_dtype,
                            void* stream);

/*
 * dq_gemm_w4a4_fp4 with the token tile chosen by the caller (same reference citation; the
 * reference has no tile notion).  token_tile = 32: 128 weight rows x 32 tokens per CTA (decode
 * batches, M <= 32 only: smaller stages, more weight bytes in flight).  128: 128 x 128, two CTAs per SM.  Both
 * split K over a cluster when the tiles alone leave SMs idle.  256: 128 x 256, one CTA per SM, the
 * weight tile of a stage fetched once for two token blocks (no split-K: fails with
 * DQ_ERR_UNSUPPORTED where the other tiles would split).  0 = the library's own choice, which is
 * what dq_gemm_w4a4_fp4 passes.  Results are identical for every choice that does not change
 * the split of K.
 */
DQ_API int dq_gemm_w4a4_fp4_tiled(const uint8_t* x_codes, const uint8_t* x_sf_atoms,
                                  const float* x_scale, const uint8_t* w_codes,
                                  const uint8_t* w_sf_atoms, const float* w_scale, const float* r,
                                  int M, int N, int K, int fmt, void* y, int y_dtype,
                                  int token_tile, void* stream);

/* ---- int4 dual-scale GEMM ------------------------------------------------------------------ */

/* Scratch bytes dq_gemm_w4a4_int4 needs for (M,N,K); may be 0. */
DQ_API size_t dq_gemm_w4a4_int4_workspace_bytes(int M, int N, int K);

/*
 * Y[m,n] = r[n] * sx[m] * sum_g sw[n,g] * (sum_{k in g} qx[m,k] * qw[n,k])
 * with exact int32 accumulation inside each weight group of G=128 and an fp32 epilogue: the
 * computation of ablation/real_int4_kernel/fused_w4a4_kernel.py:51-126 with one activation
 * scale per token, and of dequantise-and-matmul
 * (vendor/dualscale_kernel_benchmark/fused_dual_scale_kernel.py:192-206, 287-292).
 *   codes    int8 [M,K] (row stride K), values in [-8,7]
 *   sx       fp32 [M]
 *   w_packed, sw_t   from dq_pack_w_int4
 *   r        fp32 [N] or null (= 1)
 *   y        [M,N] row-major, fp32 or bf16 (y_dtype)
 */
DQ_API int dq_gemm_w4a4_int4(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                      const void* sw_t, const float* r, int M, int N, int K, int G, void* y,
                      int y_dtype, void* workspace, size_t workspace_bytes, void* stream);

/*
 * dq_gemm_w4a4_int4 with the decoder's residual connection fused into the epilogue:
 * Y = residual + linear.  residual is [M,N] of Y's element type and may be Y itself (in place).
 * For bf16 the linear's result is rounded to bf16 before the sum and the sum rounded again -
 * bit-identical to the separate `hidden = residual + o_proj(...)` of the HF decoder layer the
 * reference wraps (ablation/real_int4_kernel/full_model_nunchaku.py:81-114 leaves that add to HF).
 */
DQ_API int dq_gemm_w4a4_int4_residual(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                                      const void* sw_t, const float* r, const void* residual, int M,
                                      int N, int K, int G, void* y, int y_dtype, void* stream);

/*
 * The same GEMM for token counts where it is compute-bound (prefill), on the FP8 tensor-core path:
 * every int4 code is an exact E4M3 number and a group's 128 products sum to an integer below
 * 2^24, so tcgen05.mma kind::f8f6f4 with an fp32 accumulator yields the group sums exactly and
 * the result equals dq_gemm_w4a4_int4's bit for bit (same replacement target:
 * ablation/real_int4_kernel/fused_w4a4_kernel.py:60-130 / activations/perm_linear.py:104-131).
 * Operands are bytes: dq_expand_w_int4_e4m3 derives w8 [N,K] from the packed artefact (once, or
 * per call into scratch), dq_codes_to_e4m3 converts the quantiser's int8 codes [M,K] (row stride
 * ld) to x8 [M,K].  sw_t, r, sx, y, residual as in dq_gemm_w4a4_int4_residual (residual may be
 * NULL).  Any M >= 1 is accepted; the kernel works on tiles of 256 tokens.
 * The quantiser entries write their codes as E4M3 bytes directly when DQ_CODES_E4M3 is or-ed into
 * their scale_fp16 argument (codes then has to be read as uint8).
 */
#define DQ_CODES_E4M3 0x100
DQ_API int dq_expand_w_int4_e4m3(const uint8_t* w_packed, int N, int K, int G, uint8_t* w8, void* stream);
DQ_API int dq_codes_to_e4m3(const int8_t* codes, int64_t ld, int M, int K, uint8_t* x8, void* stream);
DQ_API int dq_gemm_w4a4_int4_e4m3(const uint8_t* x8, const float* sx, const uint8_t* w8, const void* sw_t,
                                  const float* r, int M, int N, int K, int G, void* y, int y_dtype,
                                  const void* residual, void* stream);

/*
 * The variant of the reference's fused W4A4 Triton kernel that scales activations per (token,
 * K tile) instead of per token (ablation/real_int4_kernel/fused_w4a4_kernel.py:93-100,119) and of
 * the per-group activation quantiser of its nunchaku path
 * (ablation/real_int4_kernel/full_model_nunchaku.py:81-114), with the activation group equal to
 * the weight group of this library's artefact (128; the Triton kernel uses 64 for both):
 *   s[m,g] = absmax_{k in g}(x[m,k]*a[k]) / 7 (1 if 0), q = clamp(round(x*a / s), -8, 7)
 *   Y[m,n] = r[n] * sum_g (sw[n,g] * s[m,g]) * (sum_{k in g} qx[m,k] * qw[n,k])
 * sx_groups is fp32 [K/128][M] (group-major).  round_away != 0 rounds halves away from zero like
 * the Triton kernel's libdevice.round (:98); 0 rounds them to even like formats/rtn_int.py:67.
 */
DQ_API int dq_quant_act_int4_grouped(const void* x_bf16, int64_t ldx, const float* a, int M, int K,
                                     int G, int8_t* codes, float* sx_groups, int scale_fp16,
                                     int round_away, void* stream);
DQ_API int dq_gemm_w4a4_int4_grouped(const int8_t* codes, const float* sx_groups,
                                     const uint8_t* w_packed, const void* sw_t, const float* r, int M,
                                     int N, int K, int G, void* y, int y_dtype, void* stream);

/* As above with an explicit kernel choice; used by tuning sweeps and tests.  token_tile: 0 = auto,
 * 16/32/64/128 = tcgen05 kernel with that token tile (weights through tensor memory for tiles up
 * to 64, int8 weight tiles in shared memory for 128; 1000 + tile / 2000 + tile force the
 * shared-memory / tensor-memory variant), -8/-16/-32 = decode-batch kernel with that token
 * capacity (needs M <= capacity).  split_k: 0 = auto, else 1/2/4/8. */
DQ_API int dq_gemm_w4a4_int4_ex(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                         const void* sw_t, const float* r, int M, int N, int K, int G, void* y,
                         int y_dtype, void* workspace, size_t workspace_bytes, void* stream,
                         int token_tile, int split_k);

/*
 * Peer-memory context of the all-reduce fused into dq_gemm_w4a4_int4_ar (host struct; every
 * pointer is a device pointer valid in THIS process: rank p's buffers mapped here, e.g. with
 * torch.distributed._symmetric_memory).  buf_ptrs[p]: 2 * buf_capacity_floats fp32;
 * flag_ptrs[p]: flag_units * 8 uint32, zero-initialised once; seq: this rank's own uint32 call
 * counter, zero-initialised.  All ranks must issue the same sequence of _ar calls.
 */
typedef struct dq_allreduce_ctx {
  int32_t world, rank;
  void* buf_ptrs[8];
  void* flag_ptrs[8];
  void* seq;
  uint64_t buf_capacity_floats;
  uint64_t flag_units;
} dq_allreduce_ctx;

/*
 * Row-parallel linear under tensor parallelism: each rank passes its K slice (codes, weights),
 * the partial products are summed across ranks inside the kernel's epilogue over NVLink peer
 * memory (bounded flag waits, sum in rank order, no NCCL, no multicast) and every rank receives
 * the full Y.  Replaces "F.linear then all-reduce" of a Megatron row-parallel layer; the
 * reference has no multi-GPU code.  Decode batches only (M <= 16); ctx null or world 1 = plain
 * GEMM.  Issues one extra one-thread kernel per call (call counter).
 */
DQ_API int dq_gemm_w4a4_int4_ar(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                                const void* sw_t, const float* r, int M, int N, int K, int G,
                                void* y, int y_dtype, void* stream, const dq_allreduce_ctx* ctx);
/* The same with the decoder's residual connection added to the cross-rank sum as it is stored:
 * Y = residual + sum over ranks (residual [M, N] in y's dtype, may alias y; NULL = none). */
DQ_API int dq_gemm_w4a4_int4_ar_residual(const int8_t* codes, const float* sx, const uint8_t* w_packed,
                                         const void* sw_t, const float* r, const void* residual, int M, int N,
                                         int K, int G, void* y, int y_dtype, void* stream,
                                         const dq_allreduce_ctx* ctx);

/*
 * Peer-memory context of the token-sharded prompt pass under tensor parallelism (host struct; every
 * pointer is a device pointer valid in THIS process: rank p's buffers mapped here).  Rank p owns
 * the tokens [p * tokens_per_rank, (p + 1) * tokens_per_rank) of the residual stream.
 *   part_ptrs[p]:  [world][tokens_per_rank][hidden] bf16 - slot s receives rank s's partial output
 *                  rows for rank p's tokens
 *   codes_ptrs[p]: [world * tokens_per_rank][hidden] bytes - the gathered activation codes
 *   sx_ptrs[p]:    [world * tokens_per_rank] fp32 - the gathered token scales
 *   flag_ptrs[p]:  8 uint32 barrier words, zero-initialised once
 *   barrier_count: this rank's own uint32 count of barriers, zero-initialised once (device memory;
 *                  may be NULL if every barrier call passes its epoch)
 * Replaces the all-reduce after a Megatron row-parallel linear plus the replicated norm in front of
 * the next column-parallel one; the reference has no multi-GPU code.
 */
typedef struct dq_exchange_ctx {
  int32_t world, rank;
  void* part_ptrs[8];
  void* codes_ptrs[8];
  void* sx_ptrs[8];
  void* flag_ptrs[8];
  int64_t tokens_per_rank;
  int32_t hidden;
  int32_t reserved;
  void* barrier_count;
} dq_exchange_ctx;

/*
 * Row-parallel int4 linear of the token-sharded prompt pass: dq_gemm_w4a4_int4_e4m3 whose bf16
 * output tiles [256 tokens x 128 rows] go, from the kernel's epilogue and while the other tiles
 * compute, into slot ctx->rank of the partial buffer of the rank that owns the tokens (plain
 * 16-byte stores to peer memory).  Needs N == ctx->hidden, N % 128 == 0,
 * M == world * tokens_per_rank and tokens_per_rank % 256 == 0.  Follow with dq_exchange_barrier,
 * then dq_exchange_sum.
 */
DQ_API int dq_gemm_w4a4_int4_e4m3_scatter(const uint8_t* x8, const float* sx, const uint8_t* w8, const void* sw_t,
                                          const float* r, int M, int N, int K, int G, const dq_exchange_ctx* ctx,
                                          void* stream);
/*
 * Barrier across the ranks of ctx on the device: publishes everything this rank's stream has
 * completed, then waits for every peer's word of the same epoch.  epoch: a counter the host
 * increments identically on all ranks (first call 1), or 0 - the kernel then counts in
 * ctx->barrier_count itself, which makes the call replayable inside a captured CUDA graph (do not
 * mix the two forms on one context).  The wait is bounded (2^34 SM cycles, about
 * nine seconds; dq_set_tuning("ar_wait_log2", n) changes it): on expiry the kernel records site 24 in
 * the device status word and returns, and while the word is set later barriers do not wait.
 */
DQ_API int dq_exchange_barrier(const dq_exchange_ctx* ctx, uint32_t epoch, void* stream);
/* x [tokens_per_rank, hidden] bf16 += bf16(sum over ranks, in rank order, of this rank's partial slots). */
DQ_API int dq_exchange_sum(const dq_exchange_ctx* ctx, void* x_bf16, void* stream);
/* This rank's codes [tokens_per_rank, hidden] bytes and token scales [tokens_per_rank] into its slice of
 * every rank's gathered buffers (its own included). */
DQ_API int dq_exchange_push(const dq_exchange_ctx* ctx, const void* codes, const float* sx, void* stream);

/* Test hook: the raw per-group int32 accumulators acc[M, N, K/G] (no scales applied). */
DQ_API int dq_gemm_w4a4_int4_acc(const int8_t* codes, const uint8_t* w_packed, int M, int N, int K,
                          int G, int32_t* acc, void* stream);

/*
 * One call for a whole PermLinear.forward (activations/perm_linear.py:136-141) on the real
 * int4 path: quantise x (as dq_quant_act_int4) into caller scratch, then the GEMM.
 * scratch must hold dq_linear_w4a4_int4_scratch_bytes(M,N,K) bytes.
 * Prefill batches (1024 tokens and more) run on the FP8-path GEMM (dq_gemm_w4a4_int4_e4m3, same
 * bits, about twice as fast) when the scratch also has room for the byte form of the weight:
 * dq_linear_w4a4_int4_prefill_scratch_bytes(M,N,K) (equal to the plain figure for smaller M).
 * The weight is expanded into the scratch on every call; callers that can keep N*K bytes per
 * weight call dq_expand_w_int4_e4m3 once and dq_gemm_w4a4_int4_e4m3 directly.
 */
DQ_API size_t dq_linear_w4a4_int4_scratch_bytes(int M, int N, int K);
DQ_API size_t dq_linear_w4a4_int4_prefill_scratch_bytes(int M, int N, int K);
DQ_API int dq_linear_w4a4_int4(const void* x_bf16, int64_t ldx, const float* a,
                        const dq_hadamard_desc* had, const uint8_t* w_packed, const void* sw_t,
                        const float* r, int M, int N, int K, int G, void* y, int y_dtype,
                        int scale_fp16, void* scratch, size_t scratch_bytes, void* stream);

/*
 * A16W4: 16-bit activations against the int4 weight artefact - the reference's fused-beta kernel
 * (vendor/dualscale_kernel_benchmark/fused_dual_scale_kernel.py:55-149, wrapper :220-262) and what
 * PermLinear computes when its activation cast is switched off (activations/perm_linear.py:108-141
 * with act_quant_enabled = False):
 *   Y[m,n] = r[n] * sum_k fp16(x[m,k] * a[k]) * fp16(qw[n,k] * sw[n,k/128])
 * on tcgen05 kind::f16 (fp16 operands, fp32 accumulation; with bf16 operands the reference's own
 * acceptance check, mean relative error < 1 % (:269-308), does not pass).  Activations beyond the fp16
 * range saturate at +-65504.  a may be null.  scratch holds fp16(x * a):
 * dq_linear_a16w4_scratch_bytes(M,N,K) bytes, 256-byte aligned.
 */
DQ_API size_t dq_linear_a16w4_scratch_bytes(int M, int N, int K);
DQ_API int dq_linear_a16w4(const void* x_bf16, int64_t ldx, const float* a, const uint8_t* w_packed,
                           const float* r, int M, int N, int K, int G, void* y, int y_dtype,
                           void* scratch, size_t scratch_bytes, void* stream);

/*
 * Attention glue of the end-to-end harness: rotary position embedding of the query and key heads
 * of S new tokens per sequence (S = 1 in decode, the prompt length in prefill) and the write of
 * their key / value heads into the cache, in one launch.
 * qkv is the bf16 output of the fused q/k/v linear, [B * S, (hq + 2 hkv) * head_dim] with row
 * stride ld_qkv, token (b, s) in row b * S + s; cos / sin tables are bf16 [max_len, head_dim];
 * token s goes to cache position pos0 + s, pos0 = *pos_dev (device int64) when pos_dev is given,
 * else pos_host; q_out [B, S, hq, head_dim]; caches [B, hkv, max_len, head_dim].  Arithmetic: the
 * bf16 tensor expression x * cos + rotate_half(x) * sin of the HF Llama layer the reference's
 * harness drives (ablation/real_int4_kernel/graph_bench_all.py:72-157 times that layer unchanged,
 * with a static cache): both products rounded to bf16, then their sum.  Tokens whose position
 * falls outside the cache are skipped.
 */
DQ_API int dq_rope_kv_append(const void* qkv_bf16, int64_t ld_qkv, const void* cos_tab_bf16,
                             const void* sin_tab_bf16, const int64_t* pos_dev, int64_t pos_host, int B,
                             int S, int hq, int hkv, int head_dim, int max_len, void* q_out_bf16,
                             void* k_cache_bf16, void* v_cache_bf16, void* stream);

/*
 * dq_linear_w4a4_int4 for callers that cannot hand the library any scratch memory.  (No
 * counterpart in the reference: its real-kernel path keeps torch-allocated buffers on the
 * module, ablation/real_int4_kernel/full_model_nunchaku.py:95-104.)
 *
 * Who needs it: code that runs where obtaining device memory is off the table - a serving loop
 * that has already handed every byte of HBM to its own pools, a plugin called from inside
 * another framework's execution callback where cudaMalloc would synchronise the device, or a
 * host that is only given input/output pointers.  Same arguments and results as
 * dq_linear_w4a4_int4 minus the scratch pair; the activation codes and token scales go to a
 * fixed array inside the library image instead.
 *
 * Limits and rules:
 *  - the array is dq_linear_w4a4_int4_static_max_bytes() = 2 MiB + 16 KiB and is resident on
 *    every GPU that loads the library for the life of the process; a call whose
 *    dq_linear_w4a4_int4_scratch_bytes(M,N,K) exceeds it fails with DQ_ERR_WORKSPACE
 *    (e.g. 128 tokens x K=16384 fits, 256 x 14336 does not);
 *  - the first call on each device resolves the array's device address (a host-side lookup);
 *    make that first call outside any stream capture, with the device current;
 *  - it never calls cudaMalloc / cudaFree or any allocating routine;
 *  - all calls share the one array and it keeps whatever the last call wrote.  Nothing in it
 *    has to start at zero: the quantiser overwrites every byte the GEMM later reads.  Two calls
 *    that overlap on the GPU (different streams, or graphs replayed concurrently) race on it -
 *    serialise them.
 */
DQ_API size_t dq_linear_w4a4_int4_static_max_bytes(void);
DQ_API int dq_linear_w4a4_int4_static(const void* x_bf16, int64_t ldx, const float* a,
                                      const dq_hadamard_desc* had, const uint8_t* w_packed,
                                      const void* sw_t, const float* r, int M, int N, int K,
                                      int G, void* y, int y_dtype, int scale_fp16, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DUALQUANT_B200_H */
