// Fully-connected forward / backward as FP32 tiled GEMMs on the reference's
// row-major [in][out] weight layout (no transposes on the hot path).
//
//   forward  out[B][N]  = in[B][K] * W[K][N] + b      (fully_connected_op_internal.h:15-36)
//   dX       din[B][K]  = dout[B][N] * W[K][N]^T      (:45-50)
//   dW       dW[K][N]  += in[B][K]^T * dout[B][N]     (:52-60)
//   db       db[N]     += column sums of dout         (:62-67)
//
// Large problems use 64x64 tiles.  Small ones (the CIFAR net's 1024->64 and
// 64->10 layers give 4..64 such tiles on 148 SMs) use 32x32 tiles and split
// the reduction dimension over gridDim.z; the slices are then summed in slice
// order by a second kernel, which also applies bias / activation / accumulate,
// so the result does not depend on scheduling.
#include "common.cuh"
#include "device_utils.cuh"

namespace b200 {

constexpr int GK = 16;  // tile depth

// C[m][n] (+)= sum_k A(m,k) * Bm(k,n) (+ bias[n]), then optional activation.
// A(m,k) = A[m*a_m + k*a_k], Bm(k,n) = Bm[k*b_k + n*b_n], C row-major ldc = N.
// A_KFAST / B_NFAST say which index is contiguous so tile loads coalesce.
// With gridDim.z > 1 block z reduces k in [z*k_per, (z+1)*k_per) and writes the
// raw partial sums to `partial + z*M*N`.
template <int BT, int TT, bool A_KFAST, bool B_NFAST>
__global__ void __launch_bounds__(256) sgemm_kernel(int M, int N, int K, const float *__restrict__ A,
                                                    long long a_m, long long a_k,
                                                    const float *__restrict__ Bm, long long b_k,
                                                    long long b_n, float *__restrict__ C,
                                                    const float *__restrict__ bias, int accumulate,
                                                    int act, int k_per, float *__restrict__ partial) {
  static_assert(BT / TT == 16, "256 threads as 16 x 16");
  __shared__ __align__(16) float As[GK][BT + 4];
  __shared__ __align__(16) float Bs[GK][BT + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BT, n0 = blockIdx.x * BT;
  const int tm = (tid / 16) * TT, tn = (tid % 16) * TT;
  const int kbeg = blockIdx.z * k_per;
  const int kend = min(K, kbeg + k_per);
  float acc[TT][TT];
#pragma unroll
  for (int i = 0; i < TT; ++i)
#pragma unroll
    for (int j = 0; j < TT; ++j) acc[i][j] = 0.f;

  constexpr int PER = BT * GK / 256;  // tile elements per thread
  for (int k0 = kbeg; k0 < kend; k0 += GK) {
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      int idx = tid + e * 256;
      int mm, kk;
      if (A_KFAST) {
        kk = idx % GK;
        mm = idx / GK;
      } else {
        mm = idx % BT;
        kk = idx / BT;
      }
      int m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < M && k < kend) ? A[m * a_m + k * a_k] : 0.f;
      int nn, kb;
      if (B_NFAST) {
        nn = idx % BT;
        kb = idx / BT;
      } else {
        kb = idx % GK;
        nn = idx / GK;
      }
      int n = n0 + nn;
      k = k0 + kb;
      Bs[kb][nn] = (n < N && k < kend) ? Bm[k * b_k + n * b_n] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      float av[TT], bv[TT];
#pragma unroll
      for (int i = 0; i < TT; ++i) {
        av[i] = As[kk][tm + i];
        bv[i] = Bs[kk][tn + i];
      }
#pragma unroll
      for (int i = 0; i < TT; ++i)
#pragma unroll
        for (int j = 0; j < TT; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  const bool split = gridDim.z > 1;
  float *dst = split ? partial + (size_t)blockIdx.z * M * N : C;
#pragma unroll
  for (int i = 0; i < TT; ++i) {
    int m = m0 + tm + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TT; ++j) {
      int n = n0 + tn + j;
      if (n >= N) continue;
      float v = acc[i][j];
      size_t ci = (size_t)m * N + n;
      if (!split) {
        if (bias) v += bias[n];
        if (accumulate) v += C[ci];
        v = apply_act(v, act);
      }
      dst[ci] = v;
    }
  }
}

// C[i] = act( (accumulate ? C[i] : 0) + bias[n] + sum_z partial[z][i] ), slices in order
__global__ void gemm_reduce_kernel(const float *__restrict__ partial, int slices, size_t MN, int N,
                                   float *__restrict__ C, const float *__restrict__ bias,
                                   int accumulate, int act) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < MN; i += step) {
    float v = partial[i];
    for (int z = 1; z < slices; ++z) v += partial[(size_t)z * MN + i];
    if (bias) v += bias[i % N];
    if (accumulate) v += C[i];
    C[i] = apply_act(v, act);
  }
}

// db[i] (+)= sum_n dout[n*N + i]: 32 columns x 8 row-lanes per block, lanes
// combined in a fixed order through shared memory
__global__ void col_sum_kernel(const float *__restrict__ d, float *__restrict__ db, int rows, int N,
                               int accumulate) {
  __shared__ float part[8][33];
  int col = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (col < N)
    for (int r = threadIdx.y; r < rows; r += 8) s += d[(size_t)r * N + col];
  part[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && col < N) {
    float t = part[0][threadIdx.x];
#pragma unroll
    for (int l = 1; l < 8; ++l) t += part[l][threadIdx.x];
    db[col] = accumulate ? db[col] + t : t;
  }
}

// Plan of one GEMM: tile size, k slices and the floats of scratch it needs.
struct GemmPlan {
  int tile;    // 64 or 32
  int slices;  // >= 1
  int k_per;
};

static GemmPlan plan_gemm(const b200_ctx *ctx, int M, int N, int K) {
  GemmPlan p;
  long long t64 = (long long)ceil_div(M, 64) * ceil_div(N, 64);
  if (t64 >= ctx->sm_count) {
    p.tile = 64;
    p.slices = 1;
    p.k_per = K > 0 ? K : 1;
    return p;
  }
  p.tile = 32;
  long long t32 = (long long)ceil_div(M, 32) * ceil_div(N, 32);
  int want = (int)((2LL * ctx->sm_count + t32 - 1) / t32);  // fill the machine twice
  int max_by_k = ceil_div(K > 0 ? K : 1, 64);               // at least 64 of k per slice
  int s = want < max_by_k ? want : max_by_k;
  if (s < 1) s = 1;
  int k_per = ceil_div(ceil_div(K > 0 ? K : 1, s), GK) * GK;
  p.k_per = k_per;
  p.slices = ceil_div(K > 0 ? K : 1, k_per);
  return p;
}

// A GEMM goes to the tensor cores when the context allows it and it is big enough
// to pay for splitting its operands.
static bool use_tc(const b200_ctx *ctx, int M, int N, int K) {
  if (ctx->fc_tensor_cores == 0) return false;
  if (M < 128 || N < 64 || K < 32) return false;  // at least one full tile in every direction
  if (ctx->fc_tensor_cores >= 2) return true;
  return (long long)M * N * K >= (1LL << 26);
}

// Upper bound, monotone in B, of the scratch any of the three GEMMs of a layer
// needs: slices * M * N <= (2*SMs/tiles32 + 1) * M * N <= 2*SMs*1024 + M*N; the
// tensor-core path needs the split operands instead.
size_t fc_scratch_floats(const b200_ctx *ctx, int in_size, int out_size, int B) {
  size_t need = 0;
  if (ctx->fc_tensor_cores != 0) {
    size_t t[3] = {gemm_tc_scratch_floats(B, out_size, in_size), gemm_tc_scratch_floats(B, in_size, out_size),
                   gemm_tc_scratch_floats(in_size, out_size, B)};
    for (size_t v : t)
      if (v > need) need = v;
  }
  size_t mn[3] = {(size_t)B * out_size, (size_t)B * in_size, (size_t)in_size * out_size};
  for (size_t v : mn) {
    size_t n = (size_t)2 * ctx->sm_count * 1024 + v;
    if (n > need) need = n;
  }
  return need;
}

template <bool A_KFAST, bool B_NFAST>
static int run_gemm(b200_ctx *ctx, int M, int N, int K, const float *A, long long a_m,
                    long long a_k, const float *Bm, long long b_k, long long b_n, float *C,
                    const float *bias, int accumulate, int act, float *scratch) {
  if (M == 0 || N == 0) return 0;
  GemmPlan p = plan_gemm(ctx, M, N, K);
  if (p.slices > 1 && !scratch) {  // no scratch supplied: single slice
    p.slices = 1;
    p.k_per = K;
  }
  dim3 grid(ceil_div(N, p.tile), ceil_div(M, p.tile), p.slices);
  if (p.tile == 64) {
    sgemm_kernel<64, 4, A_KFAST, B_NFAST><<<grid, 256, 0, ctx->stream>>>(
      M, N, K, A, a_m, a_k, Bm, b_k, b_n, C, bias, accumulate, act, p.k_per, scratch);
  } else {
    sgemm_kernel<32, 2, A_KFAST, B_NFAST><<<grid, 256, 0, ctx->stream>>>(
      M, N, K, A, a_m, a_k, Bm, b_k, b_n, C, bias, accumulate, act, p.k_per, scratch);
  }
  B200_LAUNCHED();
  if (p.slices > 1) {
    size_t MN = (size_t)M * N;
    size_t blocks = ceil_div_sz(MN, 256);
    if (blocks > (size_t)ctx->sm_count * 8) blocks = (size_t)ctx->sm_count * 8;
    gemm_reduce_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(scratch, p.slices, MN, N, C, bias,
                                                                 accumulate, act);
    B200_LAUNCHED();
  }
  return 0;
}

int fc_fwd(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W,
           const float *bias, float *out, int B, int act, float *scratch) {
  if (scratch && use_tc(ctx, B, out_size, in_size))
    // A = in [B][in]; Bt = W^T: W is [in][out], i.e. K x N, transposed while splitting
    return gemm_tc(ctx, B, out_size, in_size, in, in_size, false, W, out_size, true, out, bias, 0,
                   act, scratch);
  // M = B, N = out, K = in; A = in (k fast), Bm = W[k][n] (n fast)
  return run_gemm<true, true>(ctx, B, out_size, in_size, in, in_size, 1, W, out_size, 1, out, bias,
                              0, act, scratch);
}

int fc_bwd(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W,
           const float *dout, float *din, float *dW, float *db, int accumulate, int B,
           float *scratch) {
  if (din && scratch && use_tc(ctx, B, in_size, out_size)) {
    // din[B][in] = dout[B][out] * W^T: A = dout; Bt[n = c][k = o] = W[c*out + o] as stored
    B200_TRY(gemm_tc(ctx, B, in_size, out_size, dout, out_size, false, W, out_size, false, din,
                     nullptr, 0, 0, scratch));
  } else if (din) {
    // din[B][in] = dout[B][out] * W^T : M = B, N = in, K = out;
    // Bm(k = o, n = c) = W[c*out + o] -> b_k = 1, b_n = out (k fast)
    B200_TRY((run_gemm<true, false>(ctx, B, in_size, out_size, dout, out_size, 1, W, 1, out_size,
                                    din, nullptr, 0, 0, scratch)));
  }
  if (dW && scratch && use_tc(ctx, in_size, out_size, B)) {
    // dW[in][out] (+)= in^T * dout: A = in^T (in is B x in = K x M), Bt = dout^T (K x N)
    B200_TRY(gemm_tc(ctx, in_size, out_size, B, in, in_size, true, dout, out_size, true, dW, nullptr,
                     accumulate, 0, scratch));
  } else if (dW) {
    // dW[in][out] (+)= in^T * dout : M = in, N = out, K = B;
    // A(m = c, k = n) = in[n*in + c] -> a_m = 1, a_k = in (m fast)
    B200_TRY((run_gemm<false, true>(ctx, in_size, out_size, B, in, 1, in_size, dout, out_size, 1,
                                    dW, nullptr, accumulate, 0, scratch)));
  }
  if (db) {
    col_sum_kernel<<<ceil_div(out_size, 32), dim3(32, 8), 0, ctx->stream>>>(dout, db, B, out_size,
                                                                           accumulate);
    B200_LAUNCHED();
  }
  return 0;
}

}  // namespace b200
