// Activations (relu, tanh, softmax) forward/backward and the loss gradients
// that sit between the contraction kernels on the training step.
#include <float.h>

#include "common.cuh"
#include "device_utils.cuh"

namespace b200 {

// relu_layer.h:25-29, tanh_layer.h:24-28 -- elementwise, float4 where aligned
__global__ void act_fwd_kernel(int kind, float param, const float *__restrict__ x, float *__restrict__ y,
                               size_t n4, size_t n) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  size_t step = (size_t)gridDim.x * blockDim.x;
  const float4 *x4 = reinterpret_cast<const float4 *>(x);
  float4 *y4 = reinterpret_cast<float4 *>(y);
  for (size_t j = i; j < n4; j += step) {
    float4 v = x4[j];
    v.x = apply_act_p(v.x, kind, param);
    v.y = apply_act_p(v.y, kind, param);
    v.z = apply_act_p(v.z, kind, param);
    v.w = apply_act_p(v.w, kind, param);
    y4[j] = v;
  }
  for (size_t j = n4 * 4 + i; j < n; j += step) y[j] = apply_act_p(x[j], kind, param);
}

// relu_layer.h:31-39 dx = dy*(y>0); tanh_layer.h:30-38 dx = dy*(1-y*y)
// sigmoid_layer.h:32-39 dx = dy*y*(1-y); leaky_relu_layer.h:80-88 dx = dy*(y>0 ? 1 : epsilon);
// elu_layer.h:44-54 dx = dy*(y>0 ? 1 : alpha+y)
__device__ __forceinline__ float act_grad(int kind, float param, float y, float dy) {
  if (kind == B200_ACT_RELU) return dy * (y > 0.f ? 1.f : 0.f);
  if (kind == B200_ACT_TANH) return __fmul_rn(dy, __fsub_rn(1.f, __fmul_rn(y, y)));
  if (kind == B200_ACT_SIGMOID) return __fmul_rn(__fmul_rn(dy, y), __fsub_rn(1.f, y));
  if (kind == B200_ACT_LEAKY_RELU) return __fmul_rn(dy, y > 0.f ? 1.f : param);
  if (kind == B200_ACT_ELU) return __fmul_rn(dy, y > 0.f ? 1.f : __fadd_rn(param, y));
  return dy;
}

__global__ void act_bwd_kernel(int kind, float param, const float *__restrict__ y, const float *__restrict__ dy,
                               float *__restrict__ dx, size_t n4, size_t n) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  size_t step = (size_t)gridDim.x * blockDim.x;
  const float4 *y4 = reinterpret_cast<const float4 *>(y);
  const float4 *d4 = reinterpret_cast<const float4 *>(dy);
  float4 *o4 = reinterpret_cast<float4 *>(dx);
  for (size_t j = i; j < n4; j += step) {
    float4 a = y4[j], g = d4[j], o;
    o.x = act_grad(kind, param, a.x, g.x);
    o.y = act_grad(kind, param, a.y, g.y);
    o.z = act_grad(kind, param, a.z, g.z);
    o.w = act_grad(kind, param, a.w, g.w);
    o4[j] = o;
  }
  for (size_t j = n4 * 4 + i; j < n; j += step) dx[j] = act_grad(kind, param, y[j], dy[j]);
}

// softmax_layer.h:24-34: subtract the row max, exponentiate, divide by the sum
// accumulated in index order.  One thread per row (rows are 10 wide here); rows of at most
// SM_REG values are kept in registers between the passes.
constexpr int SM_REG = 16;

__global__ void softmax_fwd_kernel(const float *__restrict__ x, float *__restrict__ y, int dim,
                                   int B) {
  int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= B) return;
  const float *xr = x + (size_t)n * dim;
  float *yr = y + (size_t)n * dim;
  if (dim <= SM_REG) {
    float v[SM_REG];
#pragma unroll
    for (int j = 0; j < SM_REG; ++j) v[j] = j < dim ? xr[j] : 0.f;
    float alpha = v[0];
#pragma unroll
    for (int j = 1; j < SM_REG; ++j)
      if (j < dim) alpha = fmaxf(alpha, v[j]);
    float denom = 0.f;
#pragma unroll
    for (int j = 0; j < SM_REG; ++j)
      if (j < dim) {
        v[j] = expf(v[j] - alpha);
        denom += v[j];
      }
#pragma unroll
    for (int j = 0; j < SM_REG; ++j)
      if (j < dim) yr[j] = v[j] / denom;
    return;
  }
  float alpha = xr[0];
  for (int j = 1; j < dim; ++j) alpha = fmaxf(alpha, xr[j]);
  float denom = 0.f;
  for (int j = 0; j < dim; ++j) {
    float e = expf(xr[j] - alpha);
    yr[j] = e;
    denom += e;
  }
  for (int j = 0; j < dim; ++j) yr[j] = yr[j] / denom;
}

// Rows of at most 16 values, sixteen lanes per row: lane j exponentiates x_j, every lane adds the
// exponentials in index order (fetched from their lanes), so the result has the bits of the
// one-thread form above.
__global__ void __launch_bounds__(256) softmax_fwd16_kernel(const float *__restrict__ x, float *__restrict__ y, int dim,
                                                            int B) {
  const int n = (blockIdx.x * blockDim.x + threadIdx.x) >> 4, j = threadIdx.x & 15;
  const int base = threadIdx.x & 16;
  const bool live = n < B && j < dim;
  const float xj = live ? x[(size_t)n * dim + j] : 0.f;
  float alpha = __shfl_sync(0xffffffffu, xj, base);
  for (int k = 1; k < dim; ++k) alpha = fmaxf(alpha, __shfl_sync(0xffffffffu, xj, base + k));
  const float ej = expf(xj - alpha);
  float denom = 0.f;
  for (int k = 0; k < dim; ++k) denom += __shfl_sync(0xffffffffu, ej, base + k);
  if (live) y[(size_t)n * dim + j] = ej / denom;
}

__device__ __forceinline__ float loss_grad_one(int kind, float yi, float ti, float factor) {
  if (kind == B200_LOSS_MSE) return __fmul_rn(factor, __fsub_rn(yi, ti));
  if (kind == B200_LOSS_CROSS_ENTROPY)
    return __fdiv_rn(__fsub_rn(yi, ti), __fmul_rn(yi, __fsub_rn(1.f, yi)));
  return __fdiv_rn(-ti, yi);
}

// softmax_layer.h:36-55: dx_j = sum_k dy_k * (k == j ? y_j(1-y_j) : -y_k*y_j)
// With `t` != nullptr the incoming gradient is first computed as the loss gradient of (y, t)
// (loss_function.h) and stored to dy: the loss-gradient and softmax-gradient kernels in one.
// The same for rows of at most 16 values with sixteen lanes per row: lane j computes dx_j, fetching y_k
// and the incoming gradient g_k from lane k; the sum over k runs in index order as in the one-thread
// form below, so both give the same bits.
__global__ void __launch_bounds__(256) softmax_bwd16_kernel(const float *__restrict__ y, float *__restrict__ dy,
                                                            float *__restrict__ dx, int dim, int B,
                                                            const float *__restrict__ t, int loss_kind) {
  const int n = (blockIdx.x * blockDim.x + threadIdx.x) >> 4, j = threadIdx.x & 15;
  const int base = threadIdx.x & 16;  // first lane of this row's group inside the warp
  const bool live = n < B && j < dim;
  const float factor = 2.0f / (float)dim;
  float yj = 0.f, gj = 0.f;
  if (live) {
    yj = y[(size_t)n * dim + j];
    if (t != nullptr) {
      gj = loss_grad_one(loss_kind, yj, t[(size_t)n * dim + j], factor);
      dy[(size_t)n * dim + j] = gj;
    } else {
      gj = dy[(size_t)n * dim + j];
    }
  }
  float s = 0.f;
  for (int k = 0; k < dim; ++k) {
    const float yk = __shfl_sync(0xffffffffu, yj, base + k);
    const float gk = __shfl_sync(0xffffffffu, gj, base + k);
    const float df = (k == j) ? __fmul_rn(yj, __fsub_rn(1.f, yj)) : __fmul_rn(-yk, yj);
    s = __fadd_rn(s, __fmul_rn(gk, df));
  }
  if (live) dx[(size_t)n * dim + j] = s;
}

__global__ void softmax_bwd_kernel(const float *__restrict__ y, float *__restrict__ dy,
                                   float *__restrict__ dx, int dim, int B, const float *__restrict__ t,
                                   int loss_kind) {
  int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= B) return;
  const float *yr = y + (size_t)n * dim;
  float *gr = dy + (size_t)n * dim;
  float *dr = dx + (size_t)n * dim;
  const float factor = 2.0f / (float)dim;
  if (dim <= SM_REG) {
    float yv[SM_REG], gv[SM_REG];
#pragma unroll
    for (int j = 0; j < SM_REG; ++j) {
      yv[j] = j < dim ? yr[j] : 0.f;
      if (t != nullptr) {
        gv[j] = j < dim ? loss_grad_one(loss_kind, yv[j], t[(size_t)n * dim + j], factor) : 0.f;
        if (j < dim) gr[j] = gv[j];
      } else {
        gv[j] = j < dim ? gr[j] : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < SM_REG; ++j) {
      if (j < dim) {
        const float yj = yv[j];
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < SM_REG; ++k)
          if (k < dim) {
            float df = (k == j) ? __fmul_rn(yj, __fsub_rn(1.f, yj)) : __fmul_rn(-yv[k], yj);
            s = __fadd_rn(s, __fmul_rn(gv[k], df));
          }
        dr[j] = s;
      }
    }
    return;
  }
  if (t != nullptr)
    for (int j = 0; j < dim; ++j) gr[j] = loss_grad_one(loss_kind, yr[j], t[(size_t)n * dim + j], factor);
  for (int j = 0; j < dim; ++j) {
    float yj = yr[j];
    float s = 0.f;
    for (int k = 0; k < dim; ++k) {
      float df = (k == j) ? __fmul_rn(yj, __fsub_rn(1.f, yj)) : __fmul_rn(-yr[k], yj);
      s = __fadd_rn(s, __fmul_rn(gr[k], df));
    }
    dr[j] = s;
  }
}

// loss_function.h:28-36 (mse), :120-128 (cross_entropy), :143-150 (multiclass)
__global__ void loss_grad_kernel(int kind, const float *__restrict__ y, const float *__restrict__ t,
                                 float *__restrict__ dy, int dim, size_t n) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  size_t step = (size_t)gridDim.x * blockDim.x;
  const float factor = 2.0f / (float)dim;
  for (; i < n; i += step) {
    dy[i] = loss_grad_one(kind, y[i], t[i], factor);
  }
}

// sum over the batch of E::f (loss_function.h:17-26, :107-118, :132-141)
__global__ void loss_value_kernel(int kind, const float *__restrict__ y, const float *__restrict__ t,
                                  float *__restrict__ out, int dim, int B) {
  float acc = 0.f;
  for (int n = threadIdx.x; n < B; n += blockDim.x) {
    const float *yr = y + (size_t)n * dim;
    const float *tr = t + (size_t)n * dim;
    float d = 0.f;
    for (int j = 0; j < dim; ++j) {
      float yi = yr[j], ti = tr[j];
      if (kind == B200_LOSS_MSE)
        d += (yi - ti) * (yi - ti);
      else if (kind == B200_LOSS_CROSS_ENTROPY)
        d += -ti * logf(yi) - (1.f - ti) * logf(1.f - yi);
      else
        d += -ti * logf(yi);
    }
    if (kind == B200_LOSS_MSE) d /= (float)dim;
    acc += d;
  }
  acc = block_sum(acc);
  if (threadIdx.x == 0) *out = acc;
}

static int grid_for(size_t total, int block, int sm_count) {
  size_t blocks = (total + block - 1) / block;
  size_t cap = (size_t)sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int act_fwd(b200_ctx *ctx, int kind, const float *x, float *y, int dim, int B, float param) {
  B200_REQUIRE(kind >= B200_ACT_NONE && kind <= B200_ACT_ELU, "act_fwd: unknown activation %d", kind);
  size_t n = (size_t)dim * B;
  if (n == 0) return 0;
  if (kind == B200_ACT_SOFTMAX) {
    if (dim <= 16)
      softmax_fwd16_kernel<<<ceil_div(B * 16, 256), 256, 0, ctx->stream>>>(x, y, dim, B);
    else
      softmax_fwd_kernel<<<ceil_div(B, 32), 32, 0, ctx->stream>>>(x, y, dim, B);
  } else {
    size_t n4 = (aligned16(x) && aligned16(y)) ? n / 4 : 0;
    act_fwd_kernel<<<grid_for(n4 ? n4 : n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(kind, param, x,
                                                                                      y, n4, n);
  }
  B200_LAUNCHED();
  return 0;
}

int act_bwd(b200_ctx *ctx, int kind, const float *y, const float *dy, float *dx, int dim, int B, float param) {
  B200_REQUIRE(kind >= B200_ACT_NONE && kind <= B200_ACT_ELU, "act_bwd: unknown activation %d", kind);
  size_t n = (size_t)dim * B;
  if (n == 0) return 0;
  if (kind == B200_ACT_SOFTMAX) {
    if (dim <= 16)
      softmax_bwd16_kernel<<<ceil_div(B * 16, 256), 256, 0, ctx->stream>>>(y, const_cast<float *>(dy), dx, dim, B,
                                                                           nullptr, 0);
    else
      softmax_bwd_kernel<<<ceil_div(B, 32), 32, 0, ctx->stream>>>(y, const_cast<float *>(dy), dx, dim, B, nullptr, 0);
  } else {
    size_t n4 = (aligned16(y) && aligned16(dy) && aligned16(dx)) ? n / 4 : 0;
    act_bwd_kernel<<<grid_for(n4 ? n4 : n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
      kind, param, y, dy, dx, n4, n);
  }
  B200_LAUNCHED();
  return 0;
}

int loss_grad(b200_ctx *ctx, int kind, const float *y, const float *t, float *dy, int dim, int B) {
  B200_REQUIRE(kind >= B200_LOSS_MSE && kind <= B200_LOSS_CROSS_ENTROPY_MULTICLASS,
               "loss_grad: unknown loss %d", kind);
  size_t n = (size_t)dim * B;
  if (n == 0) return 0;
  loss_grad_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(kind, y, t, dy, dim,
                                                                             n);
  B200_LAUNCHED();
  return 0;
}

// loss gradient of (y, t) into dy, then the softmax gradient into dx: one launch
int softmax_loss_bwd(b200_ctx *ctx, int loss_kind, const float *y, const float *t, float *dy, float *dx, int dim,
                     int B) {
  B200_REQUIRE(loss_kind >= B200_LOSS_MSE && loss_kind <= B200_LOSS_CROSS_ENTROPY_MULTICLASS,
               "softmax_loss_bwd: unknown loss %d", loss_kind);
  if ((size_t)dim * B == 0) return 0;
  if (dim <= 16)
    softmax_bwd16_kernel<<<ceil_div(B * 16, 256), 256, 0, ctx->stream>>>(y, dy, dx, dim, B, t, loss_kind);
  else
    softmax_bwd_kernel<<<ceil_div(B, 32), 32, 0, ctx->stream>>>(y, dy, dx, dim, B, t, loss_kind);
  B200_LAUNCHED();
  return 0;
}

// ---- a narrow fully-connected layer followed by a softmax output layer ---------------------
// (the classifier's last two layers: 64 -> 10 in the CIFAR-10 net).  Sixteen lanes per sample as in
// the softmax kernels above; the weights (K x N floats, N <= 16) sit in shared memory.
constexpr int FCS_THREADS = 64;  // four samples per block: enough blocks to spread a small batch

// z = x W + b (fully_connected_op_internal.h:15-36: products added in input order, then the bias),
// y = softmax(z) (softmax_layer.h:24-34)
__global__ void __launch_bounds__(FCS_THREADS) fc_softmax_fwd16_kernel(const float *__restrict__ x,
                                                                       const float *__restrict__ W,
                                                                       const float *__restrict__ bias,
                                                                       float *__restrict__ z, float *__restrict__ y,
                                                                       int K, int N, int B) {
  extern __shared__ float fcs_w[];  // [K][N]
  for (int i = threadIdx.x; i < K * N; i += FCS_THREADS) fcs_w[i] = W[i];
  __syncthreads();
  const int n = (blockIdx.x * FCS_THREADS + threadIdx.x) >> 4, j = threadIdx.x & 15;
  const int base = threadIdx.x & 16;
  const bool row = n < B, live = row && j < N;
  const float *xr = x + (size_t)(row ? n : 0) * K;
  float acc = 0.f;
  for (int k0 = 0; k0 < K; k0 += 16) {
    const float xv = (row && k0 + j < K) ? xr[k0 + j] : 0.f;  // lane j holds x[k0 + j]
    const int kn = min(16, K - k0);
    for (int k = 0; k < kn; ++k) {
      const float xk = __shfl_sync(0xffffffffu, xv, base + k);
      if (j < N) acc = fmaf(xk, fcs_w[(k0 + k) * N + j], acc);
    }
  }
  const float zj = (bias != nullptr && j < N) ? acc + bias[j] : acc;
  if (live) z[(size_t)n * N + j] = zj;
  float alpha = __shfl_sync(0xffffffffu, zj, base);
  for (int k = 1; k < N; ++k) alpha = fmaxf(alpha, __shfl_sync(0xffffffffu, zj, base + k));
  const float ej = expf(zj - alpha);
  float denom = 0.f;
  for (int k = 0; k < N; ++k) denom += __shfl_sync(0xffffffffu, ej, base + k);
  if (live) y[(size_t)n * N + j] = ej / denom;
}

// dy = loss gradient of (y, t); dz = softmax gradient (as softmax_bwd16_kernel); dx = dz W^T
// (fully_connected_op_internal.h:45-50), multiplied by the gradient of a relu in front of the layer when
// `relu_x` (that relu's output = this layer's input) is given (relu_layer.h:31-39)
__global__ void __launch_bounds__(FCS_THREADS) fc_softmax_bwd16_kernel(const float *__restrict__ y,
                                                                       const float *__restrict__ t, int loss_kind,
                                                                       const float *__restrict__ W,
                                                                       const float *__restrict__ relu_x,
                                                                       float *__restrict__ dy, float *__restrict__ dz,
                                                                       float *__restrict__ dx, int K, int N, int B) {
  extern __shared__ float fcs_w[];  // [K][N]
  for (int i = threadIdx.x; i < K * N; i += FCS_THREADS) fcs_w[i] = W[i];
  __syncthreads();
  const int n = (blockIdx.x * FCS_THREADS + threadIdx.x) >> 4, j = threadIdx.x & 15;
  const int base = threadIdx.x & 16;
  const bool row = n < B, live = row && j < N;
  const float factor = 2.0f / (float)N;
  float yj = 0.f, gj = 0.f;
  if (live) {
    yj = y[(size_t)n * N + j];
    gj = loss_grad_one(loss_kind, yj, t[(size_t)n * N + j], factor);
    dy[(size_t)n * N + j] = gj;
  }
  float s = 0.f;
  for (int k = 0; k < N; ++k) {
    const float yk = __shfl_sync(0xffffffffu, yj, base + k);
    const float gk = __shfl_sync(0xffffffffu, gj, base + k);
    const float df = (k == j) ? __fmul_rn(yj, __fsub_rn(1.f, yj)) : __fmul_rn(-yk, yj);
    s = __fadd_rn(s, __fmul_rn(gk, df));
  }
  if (live) dz[(size_t)n * N + j] = s;
  if (dx == nullptr) return;
  // lane j owns inputs c = j, j + 16, ...: dx_c = sum_i dz_i W[c][i]
  for (int c0 = 0; c0 < K; c0 += 16) {
    const int c = c0 + j;
    float a = 0.f;
    for (int i = 0; i < N; ++i) {
      const float di = __shfl_sync(0xffffffffu, s, base + i);
      if (c < K) a = fmaf(di, fcs_w[c * N + i], a);
    }
    if (row && c < K) {
      if (relu_x != nullptr && !(relu_x[(size_t)n * K + c] > 0.f)) a = 0.f;
      dx[(size_t)n * K + c] = a;
    }
  }
}

bool fc_softmax_fusable(int K, int N) { return N >= 1 && N <= 16 && K >= 1 && (size_t)K * N * sizeof(float) <= 32 * 1024; }

int fc_softmax_fwd(b200_ctx *ctx, int K, int N, const float *x, const float *W, const float *bias, float *z, float *y,
                   int B) {
  B200_REQUIRE(fc_softmax_fusable(K, N), "fc_softmax_fwd: shape %d x %d not supported", K, N);
  if (B == 0) return 0;
  fc_softmax_fwd16_kernel<<<ceil_div(B * 16, FCS_THREADS), FCS_THREADS, (size_t)K * N * sizeof(float), ctx->stream>>>(
    x, W, bias, z, y, K, N, B);
  B200_LAUNCHED();
  return 0;
}

int fc_softmax_loss_bwd(b200_ctx *ctx, int loss_kind, int K, int N, const float *y, const float *t, const float *W,
                        const float *relu_x, float *dy, float *dz, float *dx, int B) {
  B200_REQUIRE(fc_softmax_fusable(K, N), "fc_softmax_loss_bwd: shape %d x %d not supported", K, N);
  B200_REQUIRE(loss_kind >= B200_LOSS_MSE && loss_kind <= B200_LOSS_CROSS_ENTROPY_MULTICLASS,
               "fc_softmax_loss_bwd: unknown loss %d", loss_kind);
  if (B == 0) return 0;
  fc_softmax_bwd16_kernel<<<ceil_div(B * 16, FCS_THREADS), FCS_THREADS, (size_t)K * N * sizeof(float), ctx->stream>>>(
    y, t, loss_kind, W, relu_x, dy, dz, dx, K, N, B);
  B200_LAUNCHED();
  return 0;
}

int loss_value(b200_ctx *ctx, int kind, const float *y, const float *t, float *loss_sum, int dim,
               int B) {
  B200_REQUIRE(kind >= B200_LOSS_MSE && kind <= B200_LOSS_CROSS_ENTROPY_MULTICLASS,
               "loss_value: unknown loss %d", kind);
  loss_value_kernel<<<1, 256, 0, ctx->stream>>>(kind, y, t, loss_sum, dim, B);
  B200_LAUNCHED();
  return 0;
}

}  // namespace b200
