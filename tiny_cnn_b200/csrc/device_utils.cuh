// Small device helpers: activation epilogues, warp/block reductions, cp.async.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "tinycnn_b200.h"

namespace b200 {

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == B200_ACT_RELU) return fmaxf(0.f, v);
  if (act == B200_ACT_TANH) return tanhf(v);
  return v;
}

// the default constructor parameters of leaky_relu_layer (epsilon) and elu_layer (alpha)
__host__ __device__ __forceinline__ float act_default_param(int act) {
  return act == B200_ACT_LEAKY_RELU ? 0.01f : act == B200_ACT_ELU ? 1.f : 0.f;
}

// relu / tanh as above; sigmoid_layer.h:26-30, leaky_relu_layer.h:74-78, elu_layer.h:38-42
__device__ __forceinline__ float apply_act_p(float v, int act, float param) {
  if (act == B200_ACT_RELU) return fmaxf(0.f, v);
  if (act == B200_ACT_TANH) return tanhf(v);
  if (act == B200_ACT_SIGMOID) return __fdiv_rn(1.f, __fadd_rn(1.f, expf(-v)));
  if (act == B200_ACT_LEAKY_RELU) return v > 0.f ? v : __fmul_rn(param, v);
  if (act == B200_ACT_ELU) return v < 0.f ? __fmul_rn(param, __fsub_rn(expf(v), 1.f)) : v;
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block (blockDim.x a multiple of 32, at most 1024).  Result valid
// in thread 0.  Fixed reduction tree, so repeated runs give identical bits.
__device__ __forceinline__ float block_sum(float v) {
  __shared__ float warp_part[32];
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();  // protects warp_part across back-to-back calls
  if (lane == 0) warp_part[wid] = v;
  __syncthreads();
  int nw = (blockDim.x + 31) >> 5;
  v = (threadIdx.x < nw) ? warp_part[threadIdx.x] : 0.f;
  if (wid == 0) v = warp_sum(v);
  return v;
}

__device__ __forceinline__ int warp_min_i(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ int warp_max_i(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// 4-byte asynchronous global->shared copy; writes 0 when !valid (src-size 0).
__device__ __forceinline__ void cp_async4(void *smem_dst, const void *gsrc, bool valid) {
  uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  int sz = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(d), "l"(gsrc), "r"(sz)
               : "memory");
}
// 16-byte form (both addresses 16-byte aligned).
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc, bool valid) {
  uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc), "r"(sz)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// ---- mbarrier + bulk asynchronous copy (one instruction moves a contiguous
// block global -> shared and signals an mbarrier with the byte count) ---------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(void *smem_dst, const void *gsrc, uint32_t bytes,
                                              uint64_t *bar) {
  asm volatile(
    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
      smem_u32(smem_dst)),
    "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
    : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
    "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
    : "=r"(ok)
    : "r"(smem_u32(bar)), "r"(parity)
    : "memory");
  return ok != 0;
}
// Bounded wait: polls until the phase completes or about two seconds of wall
// time (the device's nanosecond timer) have passed, and reports which.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity,
                                                  unsigned long long limit_ns = 2000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0, t1;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t0));
  do {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t1));
  } while (t1 - t0 < limit_ns);
  return false;
}

}  // namespace b200
