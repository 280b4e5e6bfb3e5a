// FP32-accurate GEMM on the 5th-generation tensor cores (tcgen05) by the 3xTF32
// split: every fp32 operand x is written as hi + lo with hi = x truncated to
// TF32 and lo = x - hi (exact), and
//     A*B ~= A_lo*B_hi + A_hi*B_lo + A_hi*B_hi      (the lo*lo term, ~2^-22 relative, is dropped)
// is accumulated in fp32 in tensor memory.  Used for the large fully-connected
// GEMMs (the MLP configuration); the reference computes them with scalar
// loops (tiny_dnn/core/kernels/fully_connected_op_internal.h:15-71).
//
//   D[M][N] (+)= sum_k A[M][k] * Bt[N][k]         both operands K-major
//
// One block computes a 128 x BN tile of D:
//   warp 4 (one thread)  TMA producer: cp.async.bulk.tensor 2D loads of the
//                        A_hi/A_lo/B_hi/B_lo tiles of a 32-float k-block into a
//                        3-stage ring (128-byte swizzle), signalled on mbarriers
//   warp 5 (one thread)  tcgen05.mma issuer: 4 k-steps x 3 products per k-block
//                        into a 128 x BN fp32 accumulator in TMEM; tcgen05.commit
//                        frees the stage / publishes the accumulator
//   warps 0-3            epilogue: tcgen05.ld of their 32 TMEM lanes, bias /
//                        activation / accumulate, stores to D
// No multicast is used anywhere; every wait is bounded and a timeout sets the
// context's error word, releases TMEM and returns.
#include <cuda.h>

#include "common.cuh"
#include "device_utils.cuh"

namespace b200 {

constexpr int TC_BM = 128;
constexpr int TC_BK = 32;       // floats per k-block = 128 bytes = one swizzle row
constexpr int TC_STAGES = 3;
constexpr int TC_THREADS = 192;

// ---- operand preparation -----------------------------------------------------

__device__ __forceinline__ void split_tf32(float x, float &hi, float &lo) {
  hi = __uint_as_float(__float_as_uint(x) & 0xffffe000u);  // keep the 10 TF32 mantissa bits
  lo = x - hi;                                              // exact in fp32
}

// hi/lo[r][c] = split(src[r*ld + c]) for c < cols, 0 for cols <= c < pitch
__global__ void tc_split_kernel(const float *__restrict__ src, int rows, int cols, long long ld,
                                float *__restrict__ hi, float *__restrict__ lo, int pitch) {
  long long total = (long long)rows * pitch;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int c = (int)(i % pitch);
    long long r = i / pitch;
    float h = 0.f, l = 0.f;
    if (c < cols) split_tf32(src[r * ld + c], h, l);
    hi[i] = h;
    lo[i] = l;
  }
}

// hi/lo[c][r] = split(src[r*ld + c]): the transposed operand, rows of length
// `pitch` (r < rows, zero beyond); 32x32 tiles through shared memory
__global__ void tc_split_transpose_kernel(const float *__restrict__ src, int rows, int cols,
                                          long long ld, float *__restrict__ hi,
                                          float *__restrict__ lo, int pitch) {
  __shared__ float tile[32][33];
  const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    int r = r0 + j, c = c0 + threadIdx.x;
    tile[j][threadIdx.x] = (r < rows && c < cols) ? src[(long long)r * ld + c] : 0.f;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    int c = c0 + j, r = r0 + threadIdx.x;  // output row c, column r
    if (c < cols && r < pitch) {
      float h, l;
      split_tf32(tile[threadIdx.x][j], h, l);
      hi[(long long)c * pitch + r] = h;
      lo[(long long)c * pitch + r] = l;
    }
  }
}

// ---- tcgen05 / TMA wrappers ------------------------------------------------------

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

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}

struct TcArgs {
  float *D;
  const float *bias;
  int *err;
  int M, N, K;  // K = padded contraction length (multiple of 4)
  int accumulate, act;
};

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
  gemm3x_kernel(const __grid_constant__ CUtensorMap mapAhi, const __grid_constant__ CUtensorMap mapAlo,
                const __grid_constant__ CUtensorMap mapBhi, const __grid_constant__ CUtensorMap mapBlo,
                const TcArgs a) {
  constexpr uint32_t A_BYTES = TC_BM * TC_BK * 4;  // 16 KiB
  constexpr uint32_t B_BYTES = BN * TC_BK * 4;
  constexpr uint32_t STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // tiles need 1024-byte alignment (in the shared address space) for the 128-byte swizzle
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + TC_STAGES * STAGE_BYTES);
  uint64_t *empty = full + TC_STAGES;
  uint64_t *accum = empty + TC_STAGES;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(accum + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * BN;
  const int nkb = (a.K + TC_BK - 1) / TC_BK;

  if (tid == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum, 1);
    mbar_fence_init();
  }
  if (warp == 4) {  // one warp allocates the accumulator columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                   smem_u32(tmem_slot)),
                 "r"((uint32_t)BN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool failed = false;

  if (warp == 4 && lane == 0) {
    // ---- producer -------------------------------------------------------------
    for (int kb = 0; kb < nkb && !failed; ++kb) {
      const int s = kb % TC_STAGES;
      const uint32_t use = kb / TC_STAGES;
      if (use > 0 && !mbar_wait_bounded(&empty[s], (use - 1) & 1)) {
        failed = true;
        break;
      }
      uint8_t *st = smem + s * STAGE_BYTES;
      mbar_expect_tx(&full[s], STAGE_BYTES);
      tma_load_2d(st, &mapAhi, kb * TC_BK, m0, &full[s]);
      tma_load_2d(st + A_BYTES, &mapAlo, kb * TC_BK, m0, &full[s]);
      tma_load_2d(st + 2 * A_BYTES, &mapBhi, kb * TC_BK, n0, &full[s]);
      tma_load_2d(st + 2 * A_BYTES + B_BYTES, &mapBlo, kb * TC_BK, n0, &full[s]);
    }
  } else if (warp == 5 && lane == 0) {
    // ---- MMA issuer -------------------------------------------------------------
    constexpr uint32_t idesc = umma_idesc_tf32(TC_BM, BN);
    for (int kb = 0; kb < nkb && !failed; ++kb) {
      const int s = kb % TC_STAGES;
      if (!mbar_wait_bounded(&full[s], (kb / TC_STAGES) & 1)) {
        failed = true;
        break;
      }
      tc_fence_after();
      const uint32_t base = smem_u32(smem + s * STAGE_BYTES);
#pragma unroll
      for (int k4 = 0; k4 < TC_BK / 8; ++k4) {
        // one instruction consumes 8 floats (32 bytes) of k: advance inside the swizzle row
        const uint64_t ahi = umma_desc_k128(base + k4 * 32);
        const uint64_t alo = umma_desc_k128(base + A_BYTES + k4 * 32);
        const uint64_t bhi = umma_desc_k128(base + 2 * A_BYTES + k4 * 32);
        const uint64_t blo = umma_desc_k128(base + 2 * A_BYTES + B_BYTES + k4 * 32);
        umma_tf32(tmem_base, alo, bhi, idesc, (kb | k4) != 0);
        umma_tf32(tmem_base, ahi, blo, idesc, 1);
        umma_tf32(tmem_base, ahi, bhi, idesc, 1);
      }
      umma_commit(&empty[s]);  // the stage may be refilled once these MMAs have read it
    }
    if (!failed) umma_commit(accum);  // accumulator complete
  } else if (warp < 4) {
    // ---- epilogue ------------------------------------------------------------------
    if (!mbar_wait_bounded(accum, 0)) failed = true;
    tc_fence_after();
    if (!failed) {
      const int row = m0 + warp * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
        if (row < a.M) {
          float *drow = a.D + (size_t)row * a.N + n0 + c0;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            int col = n0 + c0 + j;
            if (col < a.N) {
              float x = v[j];
              if (a.bias) x += a.bias[col];
              if (a.accumulate) x += drow[j];
              drow[j] = apply_act(x, a.act);
            }
          }
        }
      }
    }
  }
  if (failed && a.err) atomicExch(a.err, 2);
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base),
                 "r"((uint32_t)BN)
                 : "memory");
  }
}

// ---- host side ---------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
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

// 2D fp32 tensor [rows][pitch]; box = 32 floats x box_rows, 128-byte swizzle, zero fill
static int make_map(CUtensorMap *m, const float *base, int rows, int cols, int pitch, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  B200_REQUIRE(fn != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch * sizeof(float)};
  cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed (%d) for a %d x %d tensor, pitch %d",
               (int)r, rows, cols, pitch);
  return 0;
}

static int tc_pitch(int k) { return (k + 3) / 4 * 4; }

// floats of scratch for the split operands of a GEMM with these extents
size_t gemm_tc_scratch_floats(int M, int N, int K) {
  return (size_t)2 * ((size_t)M + N) * tc_pitch(K) + 64;
}

template <int BN>
static int launch_tc(b200_ctx *ctx, const CUtensorMap maps[4], const TcArgs &a) {
  constexpr size_t smem = TC_STAGES * (2 * TC_BM * TC_BK * 4 + 2 * BN * TC_BK * 4) + 1024 + 128;
  B200_CUDA(cudaFuncSetAttribute(gemm3x_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem));
  dim3 grid(ceil_div(a.N, BN), ceil_div(a.M, TC_BM));
  gemm3x_kernel<BN><<<grid, TC_THREADS, smem, ctx->stream>>>(maps[0], maps[1], maps[2], maps[3], a);
  B200_LAUNCHED();
  return 0;
}

// D[M][N] (+)= A * Bt^T with A given as src_a (M x K when !a_transposed, else K x M
// to be transposed) and Bt as src_b (N x K when !b_transposed, else K x N).
int gemm_tc(b200_ctx *ctx, int M, int N, int K, const float *src_a, long long lda, bool a_transposed,
            const float *src_b, long long ldb, bool b_transposed, float *D, const float *bias,
            int accumulate, int act, float *scratch) {
  if (M == 0 || N == 0) return 0;
  const int Kp = tc_pitch(K);
  float *a_hi = scratch, *a_lo = a_hi + (size_t)M * Kp;
  float *b_hi = a_lo + (size_t)M * Kp, *b_lo = b_hi + (size_t)N * Kp;
  cudaStream_t st = ctx->stream;
  auto split = [&](const float *src, long long ld, bool transposed, int rows, float *hi, float *lo) {
    // result: rows x Kp (K-major)
    if (!transposed) {
      long long total = (long long)rows * Kp;
      int blocks = (int)((total + 255) / 256 < (long long)ctx->sm_count * 16 ? (total + 255) / 256
                                                                              : ctx->sm_count * 16);
      tc_split_kernel<<<blocks, 256, 0, st>>>(src, rows, K, ld, hi, lo, Kp);
    } else {
      // src is K x rows; zero the padding columns first when K is not a multiple of 4
      if (Kp != K) {
        cudaMemsetAsync(hi, 0, sizeof(float) * (size_t)rows * Kp, st);
        cudaMemsetAsync(lo, 0, sizeof(float) * (size_t)rows * Kp, st);
      }
      dim3 grid(ceil_div(rows, 32), ceil_div(K, 32));
      tc_split_transpose_kernel<<<grid, dim3(32, 8), 0, st>>>(src, K, rows, ld, hi, lo, Kp);
    }
  };
  split(src_a, lda, a_transposed, M, a_hi, a_lo);
  B200_LAUNCHED();
  split(src_b, ldb, b_transposed, N, b_hi, b_lo);
  B200_LAUNCHED();
  const int BN = N >= 128 ? 128 : 64;
  CUtensorMap maps[4];
  B200_TRY(make_map(&maps[0], a_hi, M, Kp, Kp, TC_BM));
  B200_TRY(make_map(&maps[1], a_lo, M, Kp, Kp, TC_BM));
  B200_TRY(make_map(&maps[2], b_hi, N, Kp, Kp, BN));
  B200_TRY(make_map(&maps[3], b_lo, N, Kp, Kp, BN));
  TcArgs a;
  a.D = D;
  a.bias = bias;
  a.err = ctx->dev_err;
  a.M = M;
  a.N = N;
  a.K = Kp;
  a.accumulate = accumulate;
  a.act = act;
  if (BN == 128) return launch_tc<128>(ctx, maps, a);
  return launch_tc<64>(ctx, maps, a);
}

}  // namespace b200
