// Offline weight-side kernels: per-group int4 quantiser, re-packing of int4 codes into the
// streaming layout the GEMM consumes, and the inverse (test hook).
//
// Streaming layout ("w_packed", uint8, ceil(N/128)*(K/128)*8448 bytes): the matrix is cut into
// tiles of 128 rows x 128 k (one GEMM pipeline stage).  A tile is 8192 bytes of packed codes
// ([row in tile][64 bytes]) followed by the 128 fp16 group scales of its rows (256 bytes); tiles
// are stored in the order [row tile][k group], so a CTA that walks along K for its 128 rows reads
// one contiguous run of HBM and one bulk copy brings codes and scales of a stage.  Rows past N
// are zero.  Inside a tile row, 16-byte chunk ch covers
// k in [32ch, 32ch+32) of the group; byte b of the chunk holds code[32ch + b] in its low nibble
// and code[32ch + 16 + b] in its high nibble, both as two's-complement 4-bit values.  With this
// order `(w << 4) & 0xF0F0F0F0` and `w & 0xF0F0F0F0` on a 16-byte chunk yield two 16-byte runs of
// consecutive k (times 16) - the GEMM's unpack warps need no byte shuffles.
// The group scales are also kept on their own ("sw_t", fp16, ceil(N/128)*128*(K/G) values,
// [row tile][k group][row in tile], rows past N zero) for the kernel whose epilogue reads them
// from global memory.
#include "dq_common.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace dq {

__device__ __forceinline__ int code_at(const int8_t* codes, const uint8_t* ref_packed, int64_t row,
                                       int K, int k) {
  if (codes != nullptr) return codes[row * K + k];
  // reference packing: byte k/2, low nibble = even k, high nibble = odd k, value biased by +8
  const uint8_t byte = ref_packed[row * (K / 2) + (k >> 1)];
  const int nib = (k & 1) ? (byte >> 4) : (byte & 0xF);
  return nib - 8;
}

__global__ void pack_w_int4_kernel(const int8_t* __restrict__ codes,
                                   const uint8_t* __restrict__ ref_packed, int N, int K,
                                   uint8_t* __restrict__ w_packed) {
  // one thread per 16-byte output chunk; chunk index = ((tile * groups + g) * 128 + r) * 4 + ch
  const int64_t chunk = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int groups = K / kGroup;
  const int64_t tiles = (N + 127) / 128;
  if (chunk >= tiles * groups * 512) return;
  const int r = static_cast<int>((chunk >> 2) & 127);
  // chunk position inside the 64-byte row is swizzled: position p holds k chunk p ^ ((r >> 1) & 3)
  const int ch = static_cast<int>(chunk & 3) ^ ((r >> 1) & 3);
  const int64_t tg = chunk >> 9;
  const int g = static_cast<int>(tg % groups);
  const int64_t row = (tg / groups) * 128 + r;
  const int c = g * 4 + ch;  // 32-wide k chunk of the row
  uint32_t w[4] = {0, 0, 0, 0};
  if (row < N) {
#pragma unroll
    for (int b = 0; b < 16; ++b) {
      const uint32_t lo = static_cast<uint32_t>(code_at(codes, ref_packed, row, K, 32 * c + b)) & 0xFu;
      const uint32_t hi = static_cast<uint32_t>(code_at(codes, ref_packed, row, K, 32 * c + 16 + b)) & 0xFu;
      w[b >> 2] |= (lo | (hi << 4)) << (8 * (b & 3));
    }
  }
  *reinterpret_cast<uint4*>(w_packed + tg * kTileBytes + (chunk & 511) * 16) =
      make_uint4(w[0], w[1], w[2], w[3]);
}

__global__ void unpack_w_int4_kernel(const uint8_t* __restrict__ w_packed, int N, int K,
                                     int8_t* __restrict__ codes) {
  const int64_t chunk = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int groups = K / kGroup;
  const int64_t tiles = (N + 127) / 128;
  if (chunk >= tiles * groups * 512) return;
  const int r = static_cast<int>((chunk >> 2) & 127);
  const int ch = static_cast<int>(chunk & 3) ^ ((r >> 1) & 3);
  const int64_t tg = chunk >> 9;
  const int g = static_cast<int>(tg % groups);
  const int64_t row = (tg / groups) * 128 + r;
  if (row >= N) return;
  const int c = g * 4 + ch;
  const uint4 raw = *reinterpret_cast<const uint4*>(w_packed + tg * kTileBytes + (chunk & 511) * 16);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  int8_t* dst = codes + row * K + 32 * c;
#pragma unroll
  for (int b = 0; b < 16; ++b) {
    const uint32_t byte = (w[b >> 2] >> (8 * (b & 3))) & 0xFFu;
    dst[b] = static_cast<int8_t>(static_cast<int8_t>(byte << 4) >> 4);
    dst[16 + b] = static_cast<int8_t>(static_cast<int8_t>(byte & 0xF0u) >> 4);
  }
}

__global__ void transpose_sw_kernel(const __half* __restrict__ sw, int N, int groups,
                                    __half* __restrict__ sw_t, uint8_t* __restrict__ w_packed) {
  // output index = (tile * groups + g) * 128 + r
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t tiles = (N + 127) / 128;
  if (i >= tiles * groups * 128) return;
  const int r = static_cast<int>(i & 127);
  const int64_t tg = i >> 7;
  const int g = static_cast<int>(tg % groups);
  const int64_t n = (tg / groups) * 128 + r;
  const __half v = (n < N) ? sw[n * groups + g] : __float2half_rn(0.f);
  sw_t[i] = v;
  reinterpret_cast<__half*>(w_packed + tg * kTileBytes + kTileCodeBytes)[r] = v;
}

// One warp per (row, group of 128): s = absmax/7 rounded to fp16 (1 for a zero group),
// q = clamp(rint(w / s), -8, 7).
__global__ void quant_w_int4_kernel(const __nv_bfloat16* __restrict__ w, int N, int K,
                                    int8_t* __restrict__ codes, __half* __restrict__ sw) {
  const int64_t warp_id = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int groups = K / kGroup;
  if (warp_id >= static_cast<int64_t>(N) * groups) return;
  const int64_t row = warp_id / groups;
  const int g = static_cast<int>(warp_id % groups);
  const __nv_bfloat16* src = w + row * K + g * kGroup + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  float v[4];
  v[0] = __uint_as_float(raw.x << 16);
  v[1] = __uint_as_float(raw.x & 0xFFFF0000u);
  v[2] = __uint_as_float(raw.y << 16);
  v[3] = __uint_as_float(raw.y & 0xFFFF0000u);
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  float s = __fdiv_rn(amax, 7.0f);
  if (amax == 0.f) s = 1.0f;
  __half sh = __float2half_rn(fminf(s, 65504.0f));
  s = __half2float(sh);
  if (s == 0.f) { s = 1.0f; sh = __float2half_rn(1.0f); }
  uint32_t packed = 0;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float q = rintf(__fdiv_rn(v[e], s));
    q = fminf(fmaxf(q, -8.0f), 7.0f);
    packed |= (static_cast<uint32_t>(static_cast<int>(q)) & 0xFFu) << (8 * e);
  }
  *reinterpret_cast<uint32_t*>(codes + row * K + g * kGroup + lane * 4) = packed;
  if (lane == 0) sw[row * groups + g] = sh;
}

static int check_w_shape(int N, int K, int G) {
  DQ_REQUIRE(G == kGroup, DQ_ERR_UNSUPPORTED, "weight group size must be %d (got %d)", kGroup, G);
  DQ_REQUIRE(N >= 1 && K >= kGroup && K % kGroup == 0, DQ_ERR_SHAPE,
             "bad weight shape N=%d K=%d (K must be a multiple of %d)", N, K, kGroup);
  return DQ_OK;
}

}  // namespace dq

using namespace dq;

extern "C" size_t dq_packed_w_bytes(int N, int K) {
  if (N <= 0 || K <= 0) return 0;
  return (static_cast<size_t>(N) + 127) / 128 * (static_cast<size_t>(K) / kGroup) * kTileBytes;
}

extern "C" int dq_pack_w_int4(const int8_t* codes, const uint8_t* ref_packed, const void* sw, int N,
                              int K, int G, uint8_t* w_packed, void* sw_t, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  int rc = check_w_shape(N, K, G);
  if (rc != DQ_OK) return rc;
  DQ_REQUIRE((codes != nullptr) != (ref_packed != nullptr), DQ_ERR_NULL,
             "give exactly one of codes / ref_packed");
  DQ_REQUIRE(w_packed != nullptr && aligned(w_packed, 16), DQ_ERR_ALIGN,
             "w_packed must be non-null and 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t chunks = static_cast<int64_t>((N + 127) / 128) * (K / kGroup) * 512;
  pack_w_int4_kernel<<<static_cast<unsigned>((chunks + 255) / 256), 256, 0, s>>>(codes, ref_packed, N,
                                                                                 K, w_packed);
  DQ_CHECK_CUDA(cudaGetLastError());
  {
    DQ_REQUIRE(sw != nullptr && sw_t != nullptr, DQ_ERR_NULL, "sw and sw_t are required");
    const int groups = K / kGroup;
    const int64_t total = static_cast<int64_t>((N + 127) / 128) * 128 * groups;
    transpose_sw_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(
        static_cast<const __half*>(sw), N, groups, static_cast<__half*>(sw_t), w_packed);
    DQ_CHECK_CUDA(cudaGetLastError());
  }
  return DQ_OK;
}

extern "C" int dq_unpack_w_int4(const uint8_t* w_packed, int N, int K, int8_t* codes, void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  int rc = check_w_shape(N, K, kGroup);
  if (rc != DQ_OK) return rc;
  DQ_REQUIRE(w_packed != nullptr && codes != nullptr, DQ_ERR_NULL, "null pointer");
  DQ_REQUIRE(aligned(w_packed, 16), DQ_ERR_ALIGN, "w_packed must be 16-byte aligned");
  const int64_t chunks = static_cast<int64_t>((N + 127) / 128) * (K / kGroup) * 512;
  unpack_w_int4_kernel<<<static_cast<unsigned>((chunks + 255) / 256), 256, 0,
                         static_cast<cudaStream_t>(stream)>>>(w_packed, N, K, codes);
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}

extern "C" int dq_quant_w_int4(const void* w_bf16, int N, int K, int G, int8_t* codes, void* sw,
                               void* stream) {
  if (current_state() == nullptr) return DQ_ERR_NOT_INIT;
  int rc = check_w_shape(N, K, G);
  if (rc != DQ_OK) return rc;
  DQ_REQUIRE(w_bf16 != nullptr && codes != nullptr && sw != nullptr, DQ_ERR_NULL, "null pointer");
  DQ_REQUIRE(aligned(w_bf16, 8) && aligned(codes, 4), DQ_ERR_ALIGN, "w / codes misaligned");
  const int64_t warps = static_cast<int64_t>(N) * (K / kGroup);
  const int64_t threads = warps * 32;
  quant_w_int4_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0,
                        static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(w_bf16), N, K, codes, static_cast<__half*>(sw));
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}
