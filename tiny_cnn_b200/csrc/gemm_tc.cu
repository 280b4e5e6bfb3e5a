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
// Every load is CTA-local; every wait is bounded and a timeout sets the
// context's error word, releases TMEM and returns.
#include "tc_utils.cuh"

namespace b200 {

constexpr int TC_BM = 128;
constexpr int TC_BK = 32;       // floats per k-block = 128 bytes = one swizzle row
constexpr int TC_STAGES = 3;
constexpr int TC_THREADS = 192;

// ---- operand preparation -----------------------------------------------------

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
          // all loads before the stores: interleaved, every load would wait for the store before it
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            int col = n0 + c0 + j;
            if (col < a.N) {
              if (a.bias) v[j] += __ldg(a.bias + col);
              if (a.accumulate) v[j] += drow[j];
            }
          }
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (n0 + c0 + j < a.N) drow[j] = apply_act(v[j], a.act);
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
