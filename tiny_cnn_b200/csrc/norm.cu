// Layers that commonly sit between the hot operators of a tiny-dnn network: batch normalization
// (forward in both phases, backward), dropout with a mask supplied by the host, and the forward pass
// of local response normalization across channels (its backward pass does not exist in the
// reference).  All are HBM-bound: a per-channel reduction over batch x spatial positions, or one
// pass over the tensor.
#include "common.cuh"
#include "device_utils.cuh"

namespace b200 {

namespace {

constexpr int BN_THREADS = 256;

// Slices of the batch a channel's reduction is cut into: enough blocks to fill the GPU, few enough
// that every later block can add the slices up again by itself.
__host__ __device__ inline int bn_slices(int B, int channels, int sm_count) {
  int want = (4 * sm_count + channels - 1) / channels;
  if (want > 64) want = 64;
  if (want > B) want = B;
  return want < 1 ? 1 : want;
}

// sum of `vals` over the block, returned to every thread
__device__ __forceinline__ float block_sum_all(float v) {
  __shared__ float total;
  v = block_sum(v);
  if (threadIdx.x == 0) total = v;
  __syncthreads();
  v = total;
  __syncthreads();
  return v;
}

// the slices of channel c added in slice order (every block gets the same bits)
__device__ __forceinline__ float add_slices(const float *part, int c, int slices) {
  float s = 0.f;
  for (int z = 0; z < slices; ++z) s += part[(size_t)z * gridDim.x + c];
  return s;
}

// pass 1 of moments() (tiny_dnn/util/math_functions.h:25-37): per (channel, batch slice) the sum of x
// (two inputs: also the sum of x*y, for the backward pass)
__global__ void __launch_bounds__(BN_THREADS) bn_sum_kernel(const float *__restrict__ x, const float *__restrict__ y,
                                                            int S, int B, float *__restrict__ part_x,
                                                            float *__restrict__ part_xy, int vec4) {
  const int c = blockIdx.x, C = gridDim.x, z = blockIdx.y, Z = gridDim.y;
  const int n0 = (int)((long long)B * z / Z), n1 = (int)((long long)B * (z + 1) / Z);
  float sx = 0.f, sxy = 0.f;
  if (vec4) {  // 16-byte loads: S a multiple of 4 and the tensors 16-byte aligned (checked by the launcher)
    for (int n = n0; n < n1; ++n) {
      const size_t base = ((size_t)n * C + c) * S;
      const float4 *x4 = reinterpret_cast<const float4 *>(x + base);
      const float4 *y4 = y != nullptr ? reinterpret_cast<const float4 *>(y + base) : nullptr;
      for (int k = threadIdx.x; k < S / 4; k += BN_THREADS) {
        const float4 v = x4[k];
        sx += (v.x + v.y) + (v.z + v.w);
        if (y4 != nullptr) {
          const float4 w = y4[k];
          sxy += (v.x * w.x + v.y * w.y) + (v.z * w.z + v.w * w.w);
        }
      }
    }
  } else {
    for (int n = n0; n < n1; ++n) {
      const size_t base = ((size_t)n * C + c) * S;
      for (int k = threadIdx.x; k < S; k += BN_THREADS) {
        const float v = x[base + k];
        sx += v;
        if (y != nullptr) sxy += v * y[base + k];
      }
    }
  }
  sx = block_sum_all(sx);
  if (y != nullptr) sxy = block_sum_all(sxy);
  if (threadIdx.x == 0) {
    part_x[(size_t)z * C + c] = sx;
    if (y != nullptr) part_xy[(size_t)z * C + c] = sxy;
  }
}

// pass 2 (math_functions.h:39-61): per (channel, batch slice) the sum of (x - mean)^2
__global__ void __launch_bounds__(BN_THREADS) bn_var_kernel(const float *__restrict__ x, int S, int B, int slices,
                                                            const float *__restrict__ part_x,
                                                            float *__restrict__ part_v, int vec4) {
  const int c = blockIdx.x, C = gridDim.x, z = blockIdx.y, Z = gridDim.y;
  const float mean = __fdiv_rn(add_slices(part_x, c, slices), (float)B * (float)S);
  const int n0 = (int)((long long)B * z / Z), n1 = (int)((long long)B * (z + 1) / Z);
  float sv = 0.f;
  if (vec4) {
    for (int n = n0; n < n1; ++n) {
      const float4 *x4 = reinterpret_cast<const float4 *>(x + ((size_t)n * C + c) * S);
      for (int k = threadIdx.x; k < S / 4; k += BN_THREADS) {
        const float4 v = x4[k];
        const float a = v.x - mean, b = v.y - mean, e = v.z - mean, f = v.w - mean;
        sv += (a * a + b * b) + (e * e + f * f);
      }
    }
  } else {
    for (int n = n0; n < n1; ++n) {
      const size_t base = ((size_t)n * C + c) * S;
      for (int k = threadIdx.x; k < S; k += BN_THREADS) {
        const float d = __fsub_rn(x[base + k], mean);
        sv += __fmul_rn(d, d);
      }
    }
  }
  sv = block_sum_all(sv);
  if (threadIdx.x == 0) part_v[(size_t)z * C + c] = sv;
}

// y = (x - mean) / sqrt(variance + eps) (batch_normalization_layer.h:136-168).  Train phase
// (part_x != nullptr): mean and variance come from the slices (variance over max(1, B*S - 1)) and are
// stored by the channel's first block; test phase: they are read.
__global__ void __launch_bounds__(BN_THREADS) bn_apply_kernel(const float *__restrict__ x, float *__restrict__ y, int S,
                                                              int B, float eps, int slices,
                                                              const float *__restrict__ part_x,
                                                              const float *__restrict__ part_v, float *mean_io,
                                                              float *var_io, float *__restrict__ stddev, int vec4) {
  const int c = blockIdx.x, C = gridDim.x, z = blockIdx.y, Z = gridDim.y;
  float mean, var;
  if (part_x != nullptr) {
    mean = __fdiv_rn(add_slices(part_x, c, slices), (float)B * (float)S);
    var = __fdiv_rn(add_slices(part_v, c, slices), fmaxf(1.0f, __fsub_rn((float)((long long)B * S), 1.0f)));
  } else {
    mean = mean_io[c];
    var = var_io[c];
  }
  const float sd = __fsqrt_rn(__fadd_rn(var, eps));
  if (z == 0 && threadIdx.x == 0) {
    if (part_x != nullptr) {
      mean_io[c] = mean;
      var_io[c] = var;
    }
    stddev[c] = sd;
  }
  const int n0 = (int)((long long)B * z / Z), n1 = (int)((long long)B * (z + 1) / Z);
  if (vec4) {
    for (int n = n0; n < n1; ++n) {
      const size_t base = ((size_t)n * C + c) * S;
      const float4 *x4 = reinterpret_cast<const float4 *>(x + base);
      float4 *y4 = reinterpret_cast<float4 *>(y + base);
      for (int k = threadIdx.x; k < S / 4; k += BN_THREADS) {
        float4 v = x4[k];
        v.x = __fdiv_rn(__fsub_rn(v.x, mean), sd);
        v.y = __fdiv_rn(__fsub_rn(v.y, mean), sd);
        v.z = __fdiv_rn(__fsub_rn(v.z, mean), sd);
        v.w = __fdiv_rn(__fsub_rn(v.w, mean), sd);
        y4[k] = v;
      }
    }
    return;
  }
  for (int n = n0; n < n1; ++n) {
    const size_t base = ((size_t)n * C + c) * S;
    for (int k = threadIdx.x; k < S; k += BN_THREADS) y[base + k] = __fdiv_rn(__fsub_rn(x[base + k], mean), sd);
  }
}

// dx = (dy - mean(dy) - mean(dy*y) * y) / stddev (batch_normalization_layer.h:94-134)
__global__ void __launch_bounds__(BN_THREADS) bn_bwd_kernel(const float *__restrict__ y, const float *__restrict__ dy,
                                                            float *__restrict__ dx, int S, int B, int slices,
                                                            const float *__restrict__ part_d,
                                                            const float *__restrict__ part_dy,
                                                            const float *__restrict__ stddev, int vec4) {
  const int c = blockIdx.x, C = gridDim.x, z = blockIdx.y, Z = gridDim.y;
  const float count = (float)B * (float)S;
  const float mean_d = __fdiv_rn(add_slices(part_d, c, slices), count);
  const float mean_dy = __fdiv_rn(add_slices(part_dy, c, slices), count);
  const float sd = stddev[c];
  const int n0 = (int)((long long)B * z / Z), n1 = (int)((long long)B * (z + 1) / Z);
  if (vec4) {
    for (int n = n0; n < n1; ++n) {
      const size_t base = ((size_t)n * C + c) * S;
      const float4 *y4 = reinterpret_cast<const float4 *>(y + base), *g4 = reinterpret_cast<const float4 *>(dy + base);
      float4 *d4 = reinterpret_cast<float4 *>(dx + base);
      for (int k = threadIdx.x; k < S / 4; k += BN_THREADS) {
        const float4 a = y4[k], g = g4[k];
        float4 o;
        o.x = __fdiv_rn(__fsub_rn(__fsub_rn(g.x, mean_d), __fmul_rn(mean_dy, a.x)), sd);
        o.y = __fdiv_rn(__fsub_rn(__fsub_rn(g.y, mean_d), __fmul_rn(mean_dy, a.y)), sd);
        o.z = __fdiv_rn(__fsub_rn(__fsub_rn(g.z, mean_d), __fmul_rn(mean_dy, a.z)), sd);
        o.w = __fdiv_rn(__fsub_rn(__fsub_rn(g.w, mean_d), __fmul_rn(mean_dy, a.w)), sd);
        d4[k] = o;
      }
    }
    return;
  }
  for (int n = n0; n < n1; ++n) {
    const size_t base = ((size_t)n * C + c) * S;
    for (int k = threadIdx.x; k < S; k += BN_THREADS) {
      const float v = __fsub_rn(__fsub_rn(dy[base + k], mean_d), __fmul_rn(mean_dy, y[base + k]));
      dx[base + k] = __fdiv_rn(v, sd);
    }
  }
}

// running = momentum * running + (1 - momentum) * current (batch_normalization_layer.h:174-180)
__global__ void bn_post_update_kernel(int C, float momentum, float *__restrict__ mean, float *__restrict__ var,
                                      const float *__restrict__ mean_cur, const float *__restrict__ var_cur,
                                      const int *__restrict__ skip_if) {
  if (skip_if != nullptr && *skip_if != 0) return;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= C) return;
  const float one_m = __fsub_rn(1.0f, momentum);
  mean[i] = __fadd_rn(__fmul_rn(momentum, mean[i]), __fmul_rn(one_m, mean_cur[i]));
  var[i] = __fadd_rn(__fmul_rn(momentum, var[i]), __fmul_rn(one_m, var_cur[i]));
}

// dropout_layer.h:95-115 (train phase): out = mask * scale * in; :66-84: dx = mask * dy (no scale)
__global__ void dropout_kernel(const float *__restrict__ in, const uint8_t *__restrict__ mask, float scale,
                               float *__restrict__ out, size_t n) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) out[i] = __fmul_rn(__fmul_rn((float)mask[i], scale), in[i]);
}

// lrn_layer.h:110-143 (across channels): a window of `size` channels slides over the channel axis,
// the running sum of squares gains channel i + size/2 and loses channel i - size + size/2 in that
// order, out = in * (1 + alpha/size * sum)^-beta.  One thread per pixel walks the channels, so the
// running sum has the reference's additions and subtractions in the reference's order.
__global__ void lrn_across_fwd_kernel(const float *__restrict__ in, float *__restrict__ out, int C, int area, int size,
                                      float alpha_div_size, float beta, long long total) {
  long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += step) {
    const long long n = idx / area;
    const int j = (int)(idx - n * area);
    const float *ip = in + (size_t)n * C * area + j;
    float *op = out + (size_t)n * C * area + j;
    float sq = 0.f;
    for (int i = 0; i < size / 2 && i < C; ++i) {
      const float v = ip[(size_t)i * area];
      sq = __fadd_rn(sq, __fmul_rn(v, v));
    }
    int head = size / 2;
    long long tail = (long long)head - size;
    for (int i = 0; i < C; ++i, ++head, ++tail) {
      if (head < C) {
        const float v = ip[(size_t)head * area];
        sq = __fadd_rn(sq, __fmul_rn(v, v));
      }
      if (tail >= 0) {
        const float v = ip[(size_t)tail * area];
        sq = __fsub_rn(sq, __fmul_rn(v, v));
      }
      op[(size_t)i * area] = __fmul_rn(ip[(size_t)i * area], powf(__fadd_rn(1.0f, __fmul_rn(alpha_div_size, sq)), -beta));
    }
  }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int elementwise_grid(size_t n, int sm_count) {
  size_t blocks = (n + 255) / 256, cap = (size_t)sm_count * 16;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace

size_t batchnorm_scratch_floats(const b200_ctx *ctx, int channels, int B) {
  return (size_t)2 * bn_slices(B > 0 ? B : 1, channels, ctx->sm_count) * channels;
}

// `scratch`: batchnorm_scratch_floats floats.  train != 0: mean / variance are outputs (this batch's
// moments); train == 0: inputs.  stddev is always an output.
int batchnorm_fwd(b200_ctx *ctx, int channels, int spatial, float eps, const float *x, float *mean, float *variance,
                  float *stddev, float *y, int B, int train, float *scratch) {
  if (B == 0) return 0;
  const int Z = bn_slices(B, channels, ctx->sm_count);
  const dim3 grid(channels, Z);
  float *part_x = scratch, *part_v = scratch + (size_t)Z * channels;
  const int vec4 = spatial % 4 == 0 && aligned16(x) && aligned16(y);
  if (train) {
    bn_sum_kernel<<<grid, BN_THREADS, 0, ctx->stream>>>(x, nullptr, spatial, B, part_x, nullptr, vec4);
    B200_LAUNCHED();
    bn_var_kernel<<<grid, BN_THREADS, 0, ctx->stream>>>(x, spatial, B, Z, part_x, part_v, vec4);
    B200_LAUNCHED();
  }
  bn_apply_kernel<<<grid, BN_THREADS, 0, ctx->stream>>>(x, y, spatial, B, eps, Z, train ? part_x : nullptr,
                                                        train ? part_v : nullptr, mean, variance, stddev, vec4);
  B200_LAUNCHED();
  return 0;
}

int batchnorm_bwd(b200_ctx *ctx, int channels, int spatial, const float *y, const float *dy, const float *stddev,
                  float *dx, int B, float *scratch) {
  if (B == 0) return 0;
  const int Z = bn_slices(B, channels, ctx->sm_count);
  const dim3 grid(channels, Z);
  float *part_d = scratch, *part_dy = scratch + (size_t)Z * channels;
  const int vec4 = spatial % 4 == 0 && aligned16(y) && aligned16(dy) && aligned16(dx);
  bn_sum_kernel<<<grid, BN_THREADS, 0, ctx->stream>>>(dy, y, spatial, B, part_d, part_dy, vec4);
  B200_LAUNCHED();
  bn_bwd_kernel<<<grid, BN_THREADS, 0, ctx->stream>>>(y, dy, dx, spatial, B, Z, part_d, part_dy, stddev, vec4);
  B200_LAUNCHED();
  return 0;
}

int batchnorm_post_update(b200_ctx *ctx, int channels, float momentum, float *mean, float *variance,
                          const float *mean_cur, const float *var_cur, const int *skip_if) {
  bn_post_update_kernel<<<ceil_div(channels, 128), 128, 0, ctx->stream>>>(channels, momentum, mean, variance, mean_cur,
                                                                         var_cur, skip_if);
  B200_LAUNCHED();
  return 0;
}

int dropout_apply(b200_ctx *ctx, const float *in, const uint8_t *mask, float scale, float *out, size_t n) {
  if (n == 0) return 0;
  dropout_kernel<<<elementwise_grid(n, ctx->sm_count), 256, 0, ctx->stream>>>(in, mask, scale, out, n);
  B200_LAUNCHED();
  return 0;
}

int lrn_across_fwd(b200_ctx *ctx, const float *in, float *out, int channels, int area, int size, float alpha,
                   float beta, int B) {
  const long long total = (long long)B * area;
  if (total == 0) return 0;
  lrn_across_fwd_kernel<<<elementwise_grid((size_t)total, ctx->sm_count), 256, 0, ctx->stream>>>(
    in, out, channels, area, size, alpha / (float)size, beta, total);
  B200_LAUNCHED();
  return 0;
}

}  // namespace b200
