// Peer-memory exchange of the token-sharded prompt pass under tensor parallelism (one process per
// GPU, every rank's buffers mapped into every process):
//
//   * the row-parallel GEMM pushes its partial output tiles straight into the owner rank's
//     partial buffer while it computes (gemm_w4a4_int4_f8.cu, scatter output mode);
//   * exchange_barrier_kernel: every rank tells every peer "all I launched before this is done"
//     and waits - bounded - for the same word from each of them;
//   * exchange_sum_kernel: the owner adds the partial rows of all ranks, in rank order, onto its
//     slice of the residual stream;
//   * exchange_push_kernel: the owner copies its slice of quantised activations (codes, token
//     scales) into every rank's gathered buffer.
//
// Plain loads and stores over NVLink only: no multicast, no library collective.  Kernels of
// different ranks wait on one another, so they must run on different GPUs.
#include "dq_common.h"
#include "dq_ptx.cuh"

#include <cuda_bf16.h>

namespace dq {
namespace {

enum { XSITE_BARRIER = 24 };

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct BarrierArgs {
  uint32_t* flags[8];  // flags[p]: rank p's flag words, one per source rank
  int rank, world;
  uint32_t epoch;      // 0: take the epoch from *counter (device-side count of this rank's barriers)
  uint32_t* counter;   // this rank's own barrier count; advanced by the kernel when epoch == 0
  long long wait_cycles;
};

// One CTA, one thread per peer.  The kernels launched before this one on the stream have completed
// (stream order), so their stores - local and to peers - are performed; the fence and the release
// store publish them, the acquire load on the other side orders the peer's later reads after them.
// A wait that runs out records its site in the device status word and returns; once the word is
// set (by this or any earlier kernel) later barriers do not wait at all, so a lost rank costs one
// limit, not one per barrier.
// With epoch == 0 the epoch is this rank's own barrier count + 1, kept in device memory and advanced
// here: the ranks issue the same sequence of barriers, so their counts agree, and the launch carries
// no per-call value - a captured graph that holds barriers can be replayed.
__global__ void __launch_bounds__(32) exchange_barrier_kernel(BarrierArgs a, int* status) {
  const int p = threadIdx.x;
  const uint32_t epoch = (a.epoch != 0) ? a.epoch : *a.counter + 1u;
  __syncwarp();  // every lane has read the count before lane 0 advances it
  if (a.epoch == 0 && p == 0) *a.counter = epoch;
  if (p >= a.world || p == a.rank) return;
  __threadfence_system();
  st_release_sys_u32(a.flags[p] + a.rank, epoch);
  const uint32_t* mine = a.flags[a.rank] + p;
  const long long t_start = clock64();
  while (static_cast<int32_t>(ld_acquire_sys_u32(mine) - epoch) < 0) {
    if (*reinterpret_cast<volatile int*>(status) != 0) return;
    if (clock64() - t_start > a.wait_cycles) {
      atomicCAS(status, 0, XSITE_BARRIER);
      return;
    }
  }
}

__device__ __forceinline__ void bf16x8_to_f32(const uint4& raw, float* v) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint4 f32x8_to_bf16(const float* v) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 pr = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&pr);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// x[i] = bf16(x[i] + bf16(sum over ranks of part[rank][i])), the sum in fp32 and in rank order:
// what "reduce-scatter in bf16, then a bf16 residual add" computes.  part is this rank's own buffer
// [world][n] bf16; eight elements per thread and step.
__global__ void __launch_bounds__(256) exchange_sum_kernel(const uint4* __restrict__ part, int world, int64_t n8,
                                                           uint4* __restrict__ x) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float acc[8], v[8];
    bf16x8_to_f32(part[i], acc);
    for (int p = 1; p < world; ++p) {
      bf16x8_to_f32(part[static_cast<int64_t>(p) * n8 + i], v);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = __fadd_rn(acc[e], v[e]);
    }
    const uint4 s = f32x8_to_bf16(acc);
    bf16x8_to_f32(s, acc);
    bf16x8_to_f32(x[i], v);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = __fadd_rn(v[e], acc[e]);
    x[i] = f32x8_to_bf16(v);
  }
}

struct PushArgs {
  uint4* dst[8];  // every rank's gathered buffer, already offset to this rank's slice
  int world;
};

// src (n16 16-byte words, this rank's slice) -> the same slice of every rank's gathered buffer.
// blockIdx.y walks the destinations starting after this rank, so that at any moment the ranks
// write to different peers.
__global__ void __launch_bounds__(256) exchange_push_kernel(const uint4* __restrict__ src, int64_t n16, PushArgs a,
                                                            int rank) {
  const int p = (rank + 1 + static_cast<int>(blockIdx.y)) % a.world;
  uint4* dst = a.dst[p];
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}

bool ctx_ok(const dq_exchange_ctx* ctx) {
  if (ctx == nullptr || ctx->world < 1 || ctx->world > 8 || ctx->rank < 0 || ctx->rank >= ctx->world) return false;
  if (ctx->tokens_per_rank < 1 || ctx->hidden < 8 || ctx->hidden % 8 != 0) return false;
  for (int p = 0; p < ctx->world; ++p)
    if (ctx->part_ptrs[p] == nullptr || ctx->codes_ptrs[p] == nullptr || ctx->sx_ptrs[p] == nullptr ||
        ctx->flag_ptrs[p] == nullptr)
      return false;
  return true;
}

}  // namespace
}  // namespace dq

using namespace dq;

extern "C" int dq_exchange_barrier(const dq_exchange_ctx* ctx, uint32_t epoch, void* stream) {
  DeviceState* st = current_state();
  if (st == nullptr) return DQ_ERR_NOT_INIT;
  DQ_REQUIRE(ctx_ok(ctx), DQ_ERR_NULL, "bad exchange context");
  if (ctx->world == 1) return DQ_OK;
  BarrierArgs a;
  for (int p = 0; p < 8; ++p) a.flags[p] = p < ctx->world ? static_cast<uint32_t*>(ctx->flag_ptrs[p]) : nullptr;
  a.rank = ctx->rank;
  a.world = ctx->world;
  a.epoch = epoch;
  a.counter = static_cast<uint32_t*>(ctx->barrier_count);
  DQ_REQUIRE(epoch != 0 || a.counter != nullptr, DQ_ERR_NULL, "epoch 0 needs ctx->barrier_count");
  const int wl = tuning(DQ_TUNE_AR_WAIT_LOG2);
  // default: about nine seconds - the ranks' hosts enqueue a prompt pass with seconds of skew the
  // first time (lazy library set-up), and a peer that is merely late must not be taken for lost
  a.wait_cycles = 1ll << ((wl >= 10 && wl <= 40) ? wl : 34);
  exchange_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a, st->status_dev);
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}

extern "C" int dq_exchange_sum(const dq_exchange_ctx* ctx, void* x_bf16, void* stream) {
  DeviceState* st = current_state();
  if (st == nullptr) return DQ_ERR_NOT_INIT;
  DQ_REQUIRE(ctx_ok(ctx) && x_bf16 != nullptr, DQ_ERR_NULL, "bad exchange context / null x");
  DQ_REQUIRE(aligned(x_bf16, 16), DQ_ERR_ALIGN, "x must be 16-byte aligned");
  const int64_t n8 = ctx->tokens_per_rank * ctx->hidden / 8;
  int64_t blocks = (n8 + 255) / 256;
  if (blocks > st->sm_count * 8) blocks = st->sm_count * 8;
  exchange_sum_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(ctx->part_ptrs[ctx->rank]), ctx->world, n8, static_cast<uint4*>(x_bf16));
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}

extern "C" int dq_exchange_push(const dq_exchange_ctx* ctx, const void* codes, const float* sx, void* stream) {
  DeviceState* st = current_state();
  if (st == nullptr) return DQ_ERR_NOT_INIT;
  DQ_REQUIRE(ctx_ok(ctx) && codes != nullptr && sx != nullptr, DQ_ERR_NULL, "bad exchange context / null codes / sx");
  DQ_REQUIRE(aligned(codes, 16) && aligned(sx, 16) && ctx->tokens_per_rank % 4 == 0 && ctx->hidden % 16 == 0,
             DQ_ERR_ALIGN, "codes / sx must be 16-byte aligned, tokens_per_rank a multiple of 4, hidden of 16");
  const int64_t tq = ctx->tokens_per_rank;
  PushArgs pc, ps;
  pc.world = ps.world = ctx->world;
  for (int p = 0; p < 8; ++p) {
    pc.dst[p] = ps.dst[p] = nullptr;
    if (p < ctx->world) {
      pc.dst[p] = reinterpret_cast<uint4*>(static_cast<uint8_t*>(ctx->codes_ptrs[p]) + ctx->rank * tq * ctx->hidden);
      ps.dst[p] = reinterpret_cast<uint4*>(static_cast<float*>(ctx->sx_ptrs[p]) + ctx->rank * tq);
    }
  }
  const int64_t n16 = tq * ctx->hidden / 16;
  int64_t bx = (n16 + 255) / 256;
  const int64_t cap = (st->sm_count * 8 + ctx->world - 1) / ctx->world;
  if (bx > cap) bx = cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  exchange_push_kernel<<<dim3(static_cast<unsigned>(bx), ctx->world), 256, 0, s>>>(static_cast<const uint4*>(codes),
                                                                                     n16, pc, ctx->rank);
  DQ_CHECK_CUDA(cudaGetLastError());
  exchange_push_kernel<<<dim3(1, ctx->world), 256, 0, s>>>(reinterpret_cast<const uint4*>(sx), tq / 4, ps, ctx->rank);
  DQ_CHECK_CUDA(cudaGetLastError());
  return DQ_OK;
}
