// Device helpers shared by the block-scaled FP4 GEMM kernels (tcgen05.mma kind::mxf4nvf4).
#pragma once
#include "dq_common.h"
#include "dq_ptx.cuh"

namespace dq {

constexpr int kFBN = 128;      // weight rows per CTA
constexpr int kFTN = 128;      // tokens per scale-factor block
constexpr int kFKStage = 256;  // k per stage (128 bytes of packed fp4 per row)
constexpr int kFTileBytes = 128 * 128;  // one operand tile of 128 rows

// Shared-memory descriptor of one scale-factor atom for tcgen05.cp: 32 rows x 16 bytes, no
// swizzle, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t sf_atom_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;  // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;         // descriptor version
  return d;
}

__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// Instruction descriptor, kind::mxf4nvf4: E2M1 operands (format code 1), both K-major.
//   [4,6) B scale id  [7,10) A format  [10,13) B format  [17,23) N >> 3  [23] scale format
//   (0 = E4M3, 1 = E8M0)  [24,29) M >> 4  [29,31) A scale id  [31] K size (0 = 64)
__device__ __forceinline__ uint32_t umma_idesc_fp4(int m, int n, int e8m0, uint32_t sf_id) {
  return (sf_id << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(e8m0) << 23) | (static_cast<uint32_t>(m >> 4) << 24) | (sf_id << 29);
}

template <int NVFP4>
__device__ __forceinline__ void umma_fp4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                         uint32_t accumulate) {
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

}  // namespace dq
