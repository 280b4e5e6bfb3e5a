// Fully-connected forward / backward as FP32 tiled GEMMs on the reference's
// row-major [in][out] weight layout (no transposes on the hot path).
//
//   forward  out[B][N]  = in[B][K] * W[K][N] + b      (fully_connected_op_internal.h:15-36)
//   dX       din[B][K]  = dout[B][N] * W[K][N]^T      (:45-50)
//   dW       dW[K][N]  += in[B][K]^T * dout[B][N]     (:52-60)
//   db       db[N]     += column sums of dout         (:62-67)
#include "common.cuh"
#include "device_utils.cuh"

namespace b200 {

constexpr int GT = 64;   // tile edge in M and N
constexpr int GK = 16;   // tile depth

// C[m][n] (+)= sum_k A(m,k) * Bm(k,n) (+ bias[n]), then optional activation.
// A(m,k) = A[m*a_m + k*a_k], Bm(k,n) = Bm[k*b_k + n*b_n], C row-major ldc = N.
// A_KFAST / B_NFAST say which index is contiguous so tile loads coalesce.
template <bool A_KFAST, bool B_NFAST>
__global__ void __launch_bounds__(256) sgemm_kernel(int M, int N, int K, const float *__restrict__ A,
                                                    long long a_m, long long a_k,
                                                    const float *__restrict__ Bm, long long b_k,
                                                    long long b_n, float *__restrict__ C,
                                                    const float *__restrict__ bias, int accumulate,
                                                    int act) {
  __shared__ __align__(16) float As[GK][GT + 4];
  __shared__ __align__(16) float Bs[GK][GT + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int idx = tid + e * 256;
      int mm, kk;
      if (A_KFAST) {
        kk = idx % GK;
        mm = idx / GK;
      } else {
        mm = idx % GT;
        kk = idx / GT;
      }
      int m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < M && k < K) ? A[m * a_m + k * a_k] : 0.f;
      int nn, kb;
      if (B_NFAST) {
        nn = idx % GT;
        kb = idx / GT;
      } else {
        kb = idx % GK;
        nn = idx / GK;
      }
      int n = n0 + nn;
      k = k0 + kb;
      Bs[kb][nn] = (n < N && k < K) ? Bm[k * b_k + n * b_n] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      float4 a = *reinterpret_cast<const float4 *>(&As[kk][tm]);
      float4 b = *reinterpret_cast<const float4 *>(&Bs[kk][tn]);
      float av[4] = {a.x, a.y, a.z, a.w};
      float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int m = m0 + tm + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tn + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      size_t ci = (size_t)m * N + n;
      if (accumulate) v += C[ci];
      C[ci] = apply_act(v, act);
    }
  }
}

// db[i] (+)= sum_n dout[n*N + i]; one thread per column, rows in order
__global__ void col_sum_kernel(const float *__restrict__ d, float *__restrict__ db, int rows, int N,
                               int accumulate) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N) return;
  float s = 0.f;
  for (int r = 0; r < rows; ++r) s += d[(size_t)r * N + i];
  db[i] = accumulate ? db[i] + s : s;
}

template <bool A_KFAST, bool B_NFAST>
static int run_gemm(b200_ctx *ctx, int M, int N, int K, const float *A, long long a_m,
                    long long a_k, const float *Bm, long long b_k, long long b_n, float *C,
                    const float *bias, int accumulate, int act) {
  if (M == 0 || N == 0) return 0;
  dim3 grid(ceil_div(N, GT), ceil_div(M, GT));
  sgemm_kernel<A_KFAST, B_NFAST><<<grid, 256, 0, ctx->stream>>>(M, N, K, A, a_m, a_k, Bm, b_k, b_n,
                                                               C, bias, accumulate, act);
  B200_LAUNCHED();
  return 0;
}

int fc_fwd(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W,
           const float *bias, float *out, int B, int act) {
  // M = B, N = out, K = in; A = in (k fast), Bm = W[k][n] (n fast)
  return run_gemm<true, true>(ctx, B, out_size, in_size, in, in_size, 1, W, out_size, 1, out, bias,
                              0, act);
}

int fc_bwd(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W,
           const float *dout, float *din, float *dW, float *db, int accumulate, int B) {
  if (din) {
    // din[B][in] = dout[B][out] * W^T : M = B, N = in, K = out;
    // Bm(k = o, n = c) = W[c*out + o] -> b_k = 1, b_n = out (k fast)
    B200_TRY((run_gemm<true, false>(ctx, B, in_size, out_size, dout, out_size, 1, W, 1, out_size,
                                    din, nullptr, 0, 0)));
  }
  if (dW) {
    // dW[in][out] (+)= in^T * dout : M = in, N = out, K = B;
    // A(m = c, k = n) = in[n*in + c] -> a_m = 1, a_k = in (m fast)
    B200_TRY((run_gemm<false, true>(ctx, in_size, out_size, B, in, 1, in_size, dout, out_size, 1,
                                    dW, nullptr, accumulate, 0)));
  }
  if (db) {
    col_sum_kernel<<<ceil_div(out_size, 128), 128, 0, ctx->stream>>>(dout, db, B, out_size,
                                                                    accumulate);
    B200_LAUNCHED();
  }
  return 0;
}

}  // namespace b200
