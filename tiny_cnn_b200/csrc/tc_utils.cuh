// tcgen05 (5th-generation tensor core), tensor-memory and TMA wrappers shared by the
// tensor-core GEMM and convolution kernels.  Everything here is inline PTX for sm_100a;
// every load is CTA-local.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "device_utils.cuh"

namespace b200 {

__device__ __forceinline__ void split_tf32(float x, float &hi, float &lo) {
  hi = __uint_as_float(__float_as_uint(x) & 0xffffe000u);  // keep the 10 TF32 mantissa bits
  lo = x - hi;                                              // exact in fp32
}

__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int c0, int c1,
                                            uint64_t *bar) {
  asm volatile(
    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(
      smem_u32(smem_dst)),
    "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
    : "memory");
}

// shared-memory matrix descriptor: K-major tile whose rows are 128 bytes, 128-byte
// swizzle, groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);  // start address
  d |= (uint64_t)1 << 16;                       // leading byte offset (unused for this layout)
  d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                       // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                       // 128-byte swizzle
  return d;
}

// instruction descriptor: TF32 x TF32 -> F32, both operands K-major, M x N tile
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int M, int N) {
  return (1u << 4)                    // D format F32
         | (2u << 7)                  // A format TF32
         | (2u << 10)                 // B format TF32
         | ((uint32_t)(N >> 3) << 17) // N / 8
         | ((uint32_t)(M >> 4) << 24); // M / 16
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
    "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
    " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
    "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
    : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(
                 smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float *v) {
  uint32_t r[32];
  asm volatile(
    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
      "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
      "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
      "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
    : "r"(taddr)
    : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// 3D tiled load (coordinates innermost first); the innermost coordinate must be a multiple of
// 4 floats.  Coordinates outside the tensor read the map's fill value (zero).
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const CUtensorMap *map, int c0, int c1,
                                            int c2, uint64_t *bar) {
  asm volatile(
    "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n" ::"r"(
      smem_u32(smem_dst)),
    "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
    : "memory");
}

__device__ __forceinline__ void tma_load_4d(void *smem_dst, const CUtensorMap *map, int c0, int c1,
                                            int c2, int c3, uint64_t *bar) {
  asm volatile(
    "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n" ::"r"(
      smem_u32(smem_dst)),
    "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
    : "memory");
}

// General shared-memory matrix descriptor.  `layout`: 2 = 128-byte swizzle of 16-byte chunks
// (K-major operands: rows of 32 floats, `sbo` bytes between groups of 8 rows), 1 = 128-byte
// swizzle of 32-byte chunks (the form 32-bit MN-major operands need: rows are 32 floats along
// M/N, one row per k; `lbo` bytes between successive 32-wide M/N blocks, `sbo` bytes between
// groups of 4 k-rows).  The swizzle is a function of the absolute shared address, so a start
// address offset by whole 128-byte rows addresses the rows that follow.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo,
                                              uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)layout << 61;
  return d;
}

// instruction descriptor with explicit operand majors (0 = K-major, 1 = MN-major)
__host__ __device__ constexpr uint32_t umma_idesc_tf32_major(int M, int N, int a_mn, int b_mn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0];\n}\n" ::"r"(smem_u32(bar))
               : "memory");
}

// round to the nearest TF32 (10 explicit mantissa bits, ties away from zero); lo = x - hi is exact
// in fp32.  Integer form of cvt.rna.tf32.f32 (same bits for every finite input): that instruction
// issues on the conversion pipe, a quarter-rate unit that a kernel converting an im2col tile in
// its inner loop saturates, while an add and a mask run at full rate.
__device__ __forceinline__ void split_tf32_rn(float x, float &hi, float &lo) {
  hi = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
  lo = x - hi;
}

__device__ __forceinline__ void tmem_alloc(uint32_t *slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                 smem_u32(slot)),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(base), "r"(cols)
               : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float *v) {
  uint32_t r[16];
  asm volatile(
    "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
      "=r"(r[15])
    : "r"(taddr)
    : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// the same load without the wait: issue several, then tmem_ld_wait() once before the values are used
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t *r) {
  asm volatile(
    "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
      "=r"(r[15])
    : "r"(taddr)
    : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

// A operand from tensor memory (lanes = rows of A, 8 columns per TF32 instruction)
__device__ __forceinline__ void umma_tf32_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
    "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
    " tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n}\n" ::"r"(tmem_d),
    "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
    : "memory");
}

// 16 consecutive TMEM columns of the warp's 32 lanes; complete with tcgen05.wait::st
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t *r) {
  asm volatile(
    "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
    "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n" ::"r"(taddr),
    "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
    "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
    : "memory");
}

// Cycle counter of the role-timing diagnostics.  They exist only in a build with
// -DB200_TC_TIMING (python -m tiny_cnn_b200.build --tc-timing); otherwise this is a constant and
// every counter update folds away.
__device__ __forceinline__ long long tc_clock() {
#ifdef B200_TC_TIMING
  return clock64();
#else
  return 0;
#endif
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}


// ---- host side: tensor-map encoder obtained from the driver at run time ----------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// fp32 matrix [rows][d0] (d0 a multiple of 4 floats), box b0 x box_rows, 128-byte swizzle, zero fill
static inline int make_map_2d(CUtensorMap *m, const float *base, uint64_t d0, uint64_t rows, uint32_t b0,
                              uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  B200_REQUIRE(fn != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {d0, rows};
  cuuint64_t strides[1] = {d0 * sizeof(float)};
  cuuint32_t box[2] = {b0, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed (%d) for a %llu x %llu matrix", (int)r,
               (unsigned long long)rows, (unsigned long long)d0);
  return 0;
}

// fp32 tensor [d2][d1][d0] (d0 innermost, a multiple of 4 floats), box b0 x b1 x b2, zero fill
static inline int make_map_3d(CUtensorMap *m, const float *base, uint64_t d0, uint64_t d1, uint64_t d2,
                              uint32_t b0, uint32_t b1, uint32_t b2, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_fn();
  B200_REQUIRE(fn != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {d0 * sizeof(float), d0 * d1 * sizeof(float)};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed (%d) for a %llu x %llu x %llu tensor",
               (int)r, (unsigned long long)d2, (unsigned long long)d1, (unsigned long long)d0);
  return 0;
}

// fp32 tensor [d3][d2][d1][d0] whose outermost dimension is `stride3` floats apart (the others are
// dense); box b0 x b1 x b2 x b3, zero fill
static inline int make_map_4d(CUtensorMap *m, const float *base, uint64_t d0, uint64_t d1, uint64_t d2,
                              uint64_t d3, uint64_t stride3, uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3,
                              CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_fn();
  B200_REQUIRE(fn != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {d0 * sizeof(float), d0 * d1 * sizeof(float), stride3 * sizeof(float)};
  cuuint32_t box[4] = {b0, b1, b2, b3};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed (%d) for a %llu x %llu x %llu x %llu tensor",
               (int)r, (unsigned long long)d3, (unsigned long long)d2, (unsigned long long)d1,
               (unsigned long long)d0);
  return 0;
}

}  // namespace b200
