// Max and average pooling, forward and gradient.
//
// The reference drives both through index tables built once per layer
// (max: tiny_dnn/layers/max_pooling_layer.h:195-235; average:
// tiny_dnn/layers/average_pooling_layer.h:271-311).  Here the tables are
// closed-form index arithmetic evaluated per thread.
#include <float.h>

#include "common.cuh"
#include "device_utils.cuh"

namespace b200 {

// maxpool_op_internal (tiny_dnn/core/kernels/maxpool_op_internal.h:16-39):
// strict '>' against lowest(), window scanned dy-major, clipped at the border;
// the winning in-row index starts at 0 as the reference's `idx` does.
__global__ void maxpool_fwd_kernel(b200_pool_desc d, const float *__restrict__ in,
                                   float *__restrict__ out, int32_t *__restrict__ argmax,
                                   long long total) {
  long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long step = (long long)gridDim.x * blockDim.x;
  const int in_row = d.in_c * d.in_h * d.in_w;
  for (; idx < total; idx += step) {
    int ox = (int)(idx % d.out_w);
    long long r = idx / d.out_w;
    int oy = (int)(r % d.out_h);
    r /= d.out_h;
    int c = (int)(r % d.in_c);
    long long n = r / d.in_c;
    const float *ip = in + n * in_row;
    int y0 = oy * d.stride_h, x0 = ox * d.stride_w;
    int dymax = min(d.pool_h, d.in_h - y0);
    int dxmax = min(d.pool_w, d.in_w - x0);
    float best = -FLT_MAX;
    int besti = 0;
    for (int dy = 0; dy < dymax; ++dy)
      for (int dx = 0; dx < dxmax; ++dx) {
        int i = (d.in_h * c + y0 + dy) * d.in_w + x0 + dx;
        float v = ip[i];
        if (v > best) {
          best = v;
          besti = i;
        }
      }
    out[idx] = best;
    argmax[idx] = besti;
  }
}

// maxpool_grad_op_internal (maxpool_op_internal.h:41-57).  in2out[i] is the last
// window, in (y, x) order, that covers input i; 0 when no window does.
__global__ void maxpool_bwd_kernel(b200_pool_desc d, const float *__restrict__ dout,
                                   const int32_t *__restrict__ argmax, float *__restrict__ din,
                                   long long total) {
  long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long step = (long long)gridDim.x * blockDim.x;
  const int in_row = d.in_c * d.in_h * d.in_w;
  const int out_row = d.in_c * d.out_h * d.out_w;
  for (; idx < total; idx += step) {
    int i = (int)(idx % in_row);
    long long n = idx / in_row;
    int ix = i % d.in_w;
    int r = i / d.in_w;
    int iy = r % d.in_h;
    int c = r / d.in_h;
    int oy = min(iy / d.stride_h, d.out_h - 1);
    int ox = min(ix / d.stride_w, d.out_w - 1);
    bool covered = (iy < oy * d.stride_h + d.pool_h) && (ix < ox * d.stride_w + d.pool_w);
    int outi = covered ? (d.out_h * c + oy) * d.out_w + ox : 0;
    const long long ob = n * out_row;
    din[idx] = (argmax[ob + outi] == i) ? dout[ob + outi] : 0.f;
  }
}

// 2x2 windows with stride 2 on an even-width plane (every pooling layer of the
// benchmark networks): one thread owns two neighbouring outputs, reads the two
// input rows as float4 and writes float2 / int2.  Same scan order and strict
// '>' as the general kernel.
__global__ void maxpool2x2_fwd_kernel(int in_w, int in_h, int out_w, int out_h, long long planes,
                                      const float *__restrict__ in, float *__restrict__ out,
                                      int32_t *__restrict__ argmax, int in_c) {
  const int ow2 = out_w >> 1;  // output pairs per row
  long long total = planes * out_h * ow2;
  long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long step = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += step) {
    int xp = (int)(idx % ow2);
    long long r = idx / ow2;
    int oy = (int)(r % out_h);
    long long plane = r / out_h;  // n * in_c + c
    int c = (int)(plane % in_c);
    const float *ip = in + (plane * in_h + 2 * oy) * in_w + 4 * xp;
    float4 a = *reinterpret_cast<const float4 *>(ip);
    float4 b = *reinterpret_cast<const float4 *>(ip + in_w);
    // in-row index (c, y, x) of the window's first element
    int base = (in_h * c + 2 * (int)oy) * in_w + 4 * (int)xp;
    float best0 = -FLT_MAX, best1 = -FLT_MAX;
    int i0 = 0, i1 = 0;
    if (a.x > best0) { best0 = a.x; i0 = base; }
    if (a.y > best0) { best0 = a.y; i0 = base + 1; }
    if (b.x > best0) { best0 = b.x; i0 = base + in_w; }
    if (b.y > best0) { best0 = b.y; i0 = base + in_w + 1; }
    if (a.z > best1) { best1 = a.z; i1 = base + 2; }
    if (a.w > best1) { best1 = a.w; i1 = base + 3; }
    if (b.z > best1) { best1 = b.z; i1 = base + in_w + 2; }
    if (b.w > best1) { best1 = b.w; i1 = base + in_w + 3; }
    long long o = (plane * out_h + oy) * out_w + 2 * xp;
    *reinterpret_cast<float2 *>(out + o) = make_float2(best0, best1);
    *reinterpret_cast<int2 *>(argmax + o) = make_int2(i0, i1);
  }
}

// Gradient of the same layer; with `pooled_y` != nullptr (this layer's forward output) the
// gradient of a relu that precedes the pooling layer is applied on the way:
// din = (y > 0) ? pooled gradient : 0 at the window's winner, where the relu's output y equals the
// pooled value, and 0 at the other three positions either way -- so the mask needs one pooled
// value per window instead of the relu's whole output.
// I = unsigned when every index fits 32 bits (the usual case: the 64-bit divisions of the general
// form cost more than the memory traffic of this kernel), long long otherwise.
template <typename I>
__global__ void maxpool2x2_bwd_kernel(int in_w, int in_h, int out_w, int out_h, long long planes,
                                      const float *__restrict__ dout,
                                      const int32_t *__restrict__ argmax,
                                      const float *__restrict__ pooled_y, float *__restrict__ din,
                                      int in_c) {
  const I ow2 = (I)(out_w >> 1), oh = (I)out_h, ic = (I)in_c;
  const I total = (I)planes * oh * ow2;
  I idx = (I)blockIdx.x * (I)blockDim.x + (I)threadIdx.x;
  const I step = (I)gridDim.x * (I)blockDim.x;
  for (; idx < total; idx += step) {
    const I xp = idx % ow2;
    const I r = idx / ow2;
    const I oy = r % oh;
    const I plane = r / oh;
    const int c = (int)(plane % ic);
    const I o = (plane * oh + oy) * (I)out_w + 2 * xp;
    float2 g = *reinterpret_cast<const float2 *>(dout + o);
    int2 am = *reinterpret_cast<const int2 *>(argmax + o);
    if (pooled_y) {
      const float2 py = *reinterpret_cast<const float2 *>(pooled_y + o);
      g.x = py.x > 0.f ? g.x : 0.f;
      g.y = py.y > 0.f ? g.y : 0.f;
    }
    int base = (in_h * c + 2 * (int)oy) * in_w + 4 * (int)xp;
    float4 a, b;
    a.x = am.x == base ? g.x : 0.f;
    a.y = am.x == base + 1 ? g.x : 0.f;
    b.x = am.x == base + in_w ? g.x : 0.f;
    b.y = am.x == base + in_w + 1 ? g.x : 0.f;
    a.z = am.y == base + 2 ? g.y : 0.f;
    a.w = am.y == base + 3 ? g.y : 0.f;
    b.z = am.y == base + in_w + 2 ? g.y : 0.f;
    b.w = am.y == base + in_w + 3 ? g.y : 0.f;
    const I ioff = (plane * (I)in_h + 2 * oy) * (I)in_w + 4 * xp;
    *reinterpret_cast<float4 *>(din + ioff) = a;
    *reinterpret_cast<float4 *>(din + ioff + in_w) = b;
  }
}

// tiny_average_pooling_kernel (tiny_dnn/layers/average_pooling_layer.h:25-55):
// windows start at multiples of the stride while they fit entirely
// (init_connection :271-281); an output without a window is just the bias.
__global__ void avgpool_fwd_kernel(b200_pool_desc d, const float *__restrict__ in,
                                   const float *__restrict__ W, const float *__restrict__ bias,
                                   float *__restrict__ out, long long total) {
  long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long step = (long long)gridDim.x * blockDim.x;
  const int in_row = d.in_c * d.in_h * d.in_w;
  const float scale = 1.0f / (float)(d.pool_w * d.pool_h);
  for (; idx < total; idx += step) {
    int ox = (int)(idx % d.out_w);
    long long r = idx / d.out_w;
    int oy = (int)(r % d.out_h);
    r /= d.out_h;
    int c = (int)(r % d.in_c);
    long long n = r / d.in_c;
    const float *ip = in + n * in_row + (size_t)c * d.in_h * d.in_w;
    int y0 = oy * d.stride_h, x0 = ox * d.stride_w;
    float v = 0.f;
    if (y0 + d.pool_h <= d.in_h && x0 + d.pool_w <= d.in_w) {
      for (int dy = 0; dy < d.pool_h; ++dy)
        for (int dx = 0; dx < d.pool_w; ++dx) v += ip[(y0 + dy) * d.in_w + x0 + dx];
    }
    float w = __fmul_rn(W[c], scale);
    out[idx] = __fadd_rn(__fmul_rn(v, w), bias[c]);
  }
}

// prev_delta of tiny_average_pooling_back_kernel (average_pooling_layer.h:78-84):
// W[c]*scale*dout[first window covering the input].
__global__ void avgpool_bwd_dx_kernel(b200_pool_desc d, const float *__restrict__ W,
                                      const float *__restrict__ dout, float *__restrict__ din,
                                      long long total) {
  long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long step = (long long)gridDim.x * blockDim.x;
  const int in_row = d.in_c * d.in_h * d.in_w;
  const int out_row = d.in_c * d.out_h * d.out_w;
  const float scale = 1.0f / (float)(d.pool_w * d.pool_h);
  // number of windows that exist along each axis
  const int nwy = (d.in_h - d.pool_h) / d.stride_h + 1;
  const int nwx = (d.in_w - d.pool_w) / d.stride_w + 1;
  for (; idx < total; idx += step) {
    int i = (int)(idx % in_row);
    long long n = idx / in_row;
    int ix = i % d.in_w;
    int r = i / d.in_w;
    int iy = r % d.in_h;
    int c = r / d.in_h;
    // first window (smallest start) with start <= pos < start + pool
    int oy = iy < d.pool_h ? 0 : (iy - d.pool_h) / d.stride_h + 1;
    int ox = ix < d.pool_w ? 0 : (ix - d.pool_w) / d.stride_w + 1;
    bool covered = oy < nwy && ox < nwx && oy * d.stride_h <= iy && ox * d.stride_w <= ix &&
                   oy < d.out_h && ox < d.out_w;
    float v = 0.f;
    if (covered)
      v = __fmul_rn(__fmul_rn(W[c], scale), dout[n * out_row + (d.out_h * c + oy) * d.out_w + ox]);
    din[idx] = v;
  }
}

// dW[c] (+)= scale * sum_{n, window, tap} in*dout ; db[c] (+)= sum dout
// (average_pooling_layer.h:86-104).  One block per channel, fixed order.
__global__ void avgpool_bwd_dw_kernel(b200_pool_desc d, const float *__restrict__ in,
                                      const float *__restrict__ dout, float *__restrict__ dW,
                                      float *__restrict__ db, int B, int accumulate) {
  const int c = blockIdx.x;
  const int in_row = d.in_c * d.in_h * d.in_w;
  const int out_row = d.in_c * d.out_h * d.out_w;
  const int oplane = d.out_h * d.out_w;
  const float scale = 1.0f / (float)(d.pool_w * d.pool_h);
  float sw = 0.f, sb = 0.f;
  long long total = (long long)B * oplane;
  for (long long t = threadIdx.x; t < total; t += blockDim.x) {
    int n = (int)(t / oplane);
    int o = (int)(t % oplane);
    int oy = o / d.out_w, ox = o % d.out_w;
    float g = dout[(size_t)n * out_row + (size_t)c * oplane + o];
    sb += g;
    int y0 = oy * d.stride_h, x0 = ox * d.stride_w;
    if (y0 + d.pool_h <= d.in_h && x0 + d.pool_w <= d.in_w) {
      const float *ip = in + (size_t)n * in_row + (size_t)c * d.in_h * d.in_w;
      float s = 0.f;
      for (int dy = 0; dy < d.pool_h; ++dy)
        for (int dx = 0; dx < d.pool_w; ++dx) s += ip[(y0 + dy) * d.in_w + x0 + dx];
      sw = fmaf(s, g, sw);
    }
  }
  sw = block_sum(sw);
  sb = block_sum(sb);
  if (threadIdx.x == 0) {
    float vw = sw * scale;
    dW[c] = accumulate ? dW[c] + vw : vw;
    db[c] = accumulate ? db[c] + sb : sb;
  }
}

// entries in_c .. pool_w*pool_h*in_c of the weight gradient are never written
// by the reference; a fresh (non-accumulating) gradient holds 0 there.
__global__ void zero_tail_kernel(float *p, int from, int to) {
  int i = from + blockIdx.x * blockDim.x + threadIdx.x;
  if (i < to) p[i] = 0.f;
}

static int grid_for(long long total, int block, int sm_count) {
  long long blocks = (total + block - 1) / block;
  long long cap = (long long)sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

static int check_pool(const b200_pool_desc &d) {
  B200_REQUIRE(d.in_w > 0 && d.in_h > 0 && d.in_c > 0 && d.out_w > 0 && d.out_h > 0 &&
                 d.pool_w > 0 && d.pool_h > 0 && d.stride_w > 0 && d.stride_h > 0,
               "pool descriptor has a non-positive extent");
  B200_REQUIRE((d.out_h - 1) * d.stride_h < d.in_h && (d.out_w - 1) * d.stride_w < d.in_w,
               "pool descriptor: last window starts outside the input");
  return 0;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// 2x2/2 pooling of planes whose width is a multiple of 4 and whose height is even
static bool pool2x2_fast(const b200_pool_desc &d) {
  return d.pool_w == 2 && d.pool_h == 2 && d.stride_w == 2 && d.stride_h == 2 && (d.in_w % 4) == 0 &&
         (d.in_h % 2) == 0 && d.out_w * 2 == d.in_w && d.out_h * 2 == d.in_h;
}

int maxpool_fwd(b200_ctx *ctx, const b200_pool_desc &d, const float *in, float *out,
                int32_t *argmax, int B) {
  B200_TRY(check_pool(d));
  long long total = (long long)B * d.in_c * d.out_h * d.out_w;
  if (total == 0) return 0;
  if (pool2x2_fast(d) && aligned16(in) && aligned16(out) && aligned16(argmax)) {
    long long planes = (long long)B * d.in_c;
    maxpool2x2_fwd_kernel<<<grid_for(total / 2, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
      d.in_w, d.in_h, d.out_w, d.out_h, planes, in, out, argmax, d.in_c);
    B200_LAUNCHED();
    return 0;
  }
  maxpool_fwd_kernel<<<grid_for(total, 256, ctx->sm_count), 256, 0, ctx->stream>>>(d, in, out,
                                                                                   argmax, total);
  B200_LAUNCHED();
  return 0;
}

bool maxpool_can_fuse_relu(const b200_pool_desc &d) { return pool2x2_fast(d); }

int maxpool_bwd(b200_ctx *ctx, const b200_pool_desc &d, const float *dout, const int32_t *argmax,
                float *din, int B, const float *pooled_y) {
  B200_TRY(check_pool(d));
  long long total = (long long)B * d.in_c * d.in_h * d.in_w;
  if (total == 0) return 0;
  bool fast = pool2x2_fast(d) && aligned16(dout) && aligned16(din) && aligned16(argmax) &&
              (!pooled_y || aligned16(pooled_y));
  B200_REQUIRE(fast || !pooled_y, "maxpool_bwd: relu fusion needs the 2x2/2 aligned path");
  if (fast) {
    long long planes = (long long)B * d.in_c;
    long long work = planes * d.out_h * (d.out_w / 2);
    if (planes * d.in_h * d.in_w < (1LL << 31)) {
      maxpool2x2_bwd_kernel<unsigned><<<grid_for(work, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
        d.in_w, d.in_h, d.out_w, d.out_h, planes, dout, argmax, pooled_y, din, d.in_c);
    } else {
      maxpool2x2_bwd_kernel<long long><<<grid_for(work, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
        d.in_w, d.in_h, d.out_w, d.out_h, planes, dout, argmax, pooled_y, din, d.in_c);
    }
    B200_LAUNCHED();
    return 0;
  }
  maxpool_bwd_kernel<<<grid_for(total, 256, ctx->sm_count), 256, 0, ctx->stream>>>(d, dout, argmax,
                                                                                   din, total);
  B200_LAUNCHED();
  return 0;
}

static int check_avg(const b200_pool_desc &d) {
  B200_TRY(check_pool(d));
  // the reference dereferences in2wo[idx][0] for every input: each input must
  // lie in at least one window (average_pooling_layer.h:82)
  B200_REQUIRE(d.stride_w <= d.pool_w && d.stride_h <= d.pool_h &&
                 (d.in_w - d.pool_w) % d.stride_w == 0 && (d.in_h - d.pool_h) % d.stride_h == 0 &&
                 d.in_w >= d.pool_w && d.in_h >= d.pool_h,
               "average pooling: some input lies in no window (stride > pool or ragged edge)");
  return 0;
}

int avgpool_fwd(b200_ctx *ctx, const b200_pool_desc &d, const float *in, const float *W,
                const float *bias, float *out, int B) {
  B200_TRY(check_avg(d));
  long long total = (long long)B * d.in_c * d.out_h * d.out_w;
  if (total == 0) return 0;
  avgpool_fwd_kernel<<<grid_for(total, 256, ctx->sm_count), 256, 0, ctx->stream>>>(d, in, W, bias,
                                                                                   out, total);
  B200_LAUNCHED();
  return 0;
}

int avgpool_bwd(b200_ctx *ctx, const b200_pool_desc &d, const float *in, const float *W,
                const float *dout, float *din, float *dW, float *db, int accumulate, int B) {
  B200_TRY(check_avg(d));
  long long total = (long long)B * d.in_c * d.in_h * d.in_w;
  if (din && total > 0) {
    avgpool_bwd_dx_kernel<<<grid_for(total, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
      d, W, dout, din, total);
    B200_LAUNCHED();
  }
  if (dW && db) {
    avgpool_bwd_dw_kernel<<<d.in_c, 256, 0, ctx->stream>>>(d, in, dout, dW, db, B, accumulate);
    B200_LAUNCHED();
    int wlen = d.pool_w * d.pool_h * d.in_c;
    if (!accumulate && wlen > d.in_c) {
      zero_tail_kernel<<<ceil_div(wlen - d.in_c, 256), 256, 0, ctx->stream>>>(dW, d.in_c, wlen);
      B200_LAUNCHED();
    }
  }
  return 0;
}

}  // namespace b200
