// General convolution kernels: any stride, forward dilation, connection table
// and kernel size.  They are the path for shapes the tiled kernels do not take
// and the in-library cross-check of the tiled kernels.
//
// Semantics follow kernels::conv2d_op_internal
// (tiny_dnn/core/kernels/conv2d_op_internal.h:13-74 forward, :78-181 backward):
// forward honours dilation, dX and dW do not (:118-123, :139-160).
#include "common.cuh"
#include "device_utils.cuh"

namespace b200 {

// one thread per output element
__global__ void conv_general_fwd_kernel(ConvGeom g, const float *__restrict__ in,
                                        const float *__restrict__ W,
                                        const float *__restrict__ bias, float *__restrict__ out,
                                        long long total, int act) {
  long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long step = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += step) {
    int x = (int)(idx % g.OW);
    long long r = idx / g.OW;
    int y = (int)(r % g.OH);
    r /= g.OH;
    int o = (int)(r % g.OC);
    int n = (int)(r / g.OC);
    float acc = 0.f;
    const float *inb = in + (size_t)n * g.C * g.HI * g.WI;
    for (int inc = 0; inc < g.C; ++inc) {
      if (g.tbl && !g.tbl[inc * g.OC + o]) continue;
      const float *w = W + ((size_t)o * g.C + inc) * g.KH * g.KW;
      const float *ip = inb + (size_t)inc * g.HI * g.WI;
      float sum = 0.f;
      for (int wy = 0; wy < g.KH; ++wy) {
        int iy = y * g.SH + wy * g.DH - g.pad_t;
        if (iy < 0 || iy >= g.HI) continue;
        for (int wx = 0; wx < g.KW; ++wx) {
          int ix = x * g.SW + wx * g.DW - g.pad_l;
          if (ix < 0 || ix >= g.WI) continue;
          sum = fmaf(w[wy * g.KW + wx], ip[iy * g.WI + ix], sum);
        }
      }
      acc += sum;
    }
    if (g.has_bias) acc += bias[o];
    out[idx] = apply_act(acc, act);
  }
}

// one thread per input-gradient element (gather form of the reference scatter)
__global__ void conv_general_dx_kernel(ConvGeom g, const float *__restrict__ W,
                                       const float *__restrict__ dout, float *__restrict__ din,
                                       long long total) {
  long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long step = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += step) {
    int ix = (int)(idx % g.WI);
    long long r = idx / g.WI;
    int iy = (int)(r % g.HI);
    r /= g.HI;
    int inc = (int)(r % g.C);
    int n = (int)(r / g.C);
    int yp = iy + g.pad_t, xp = ix + g.pad_l;
    float acc = 0.f;
    const float *db = dout + (size_t)n * g.OC * g.OH * g.OW;
    for (int o = 0; o < g.OC; ++o) {
      if (g.tbl && !g.tbl[inc * g.OC + o]) continue;
      const float *w = W + ((size_t)o * g.C + inc) * g.KH * g.KW;
      const float *dp = db + (size_t)o * g.OH * g.OW;
      for (int wy = 0; wy < g.KH; ++wy) {
        int ty = yp - wy;
        if (ty < 0 || ty % g.SH) continue;
        int oy = ty / g.SH;
        if (oy >= g.OH) continue;
        for (int wx = 0; wx < g.KW; ++wx) {
          int tx = xp - wx;
          if (tx < 0 || tx % g.SW) continue;
          int ox = tx / g.SW;
          if (ox >= g.OW) continue;
          acc = fmaf(w[wy * g.KW + wx], dp[oy * g.OW + ox], acc);
        }
      }
    }
    din[idx] = acc;
  }
}

// one block per filter tap (o, inc, wy, wx): sum over samples and output plane
__global__ void conv_general_dw_kernel(ConvGeom g, const float *__restrict__ in,
                                       const float *__restrict__ dout, float *__restrict__ dW,
                                       int B, int accumulate) {
  int widx = blockIdx.x;
  int wx = widx % g.KW;
  int r = widx / g.KW;
  int wy = r % g.KH;
  r /= g.KH;
  int inc = r % g.C;
  int o = r / g.C;
  if (g.tbl && !g.tbl[inc * g.OC + o]) {
    if (!accumulate && threadIdx.x == 0) dW[widx] = 0.f;
    return;
  }
  int plane = g.OH * g.OW;
  long long total = (long long)B * plane;
  float acc = 0.f;
  for (long long i = threadIdx.x; i < total; i += blockDim.x) {
    int n = (int)(i / plane);
    int p = (int)(i % plane);
    int y = p / g.OW, x = p % g.OW;
    int iy = y * g.SH + wy - g.pad_t;
    int ix = x * g.SW + wx - g.pad_l;
    if (iy < 0 || iy >= g.HI || ix < 0 || ix >= g.WI) continue;
    acc = fmaf(in[((size_t)(n * g.C + inc) * g.HI + iy) * g.WI + ix],
               dout[((size_t)(n * g.OC + o)) * plane + p], acc);
  }
  acc = block_sum(acc);
  if (threadIdx.x == 0) dW[widx] = accumulate ? dW[widx] + acc : acc;
}

// one block per output channel: db[o] = sum over samples and plane of dout
__global__ void conv_db_kernel(const float *__restrict__ dout, float *__restrict__ db, int OC,
                               int plane, int B, int accumulate) {
  int o = blockIdx.x;
  long long total = (long long)B * plane;
  float acc = 0.f;
  for (long long i = threadIdx.x; i < total; i += blockDim.x) {
    int n = (int)(i / plane);
    int p = (int)(i % plane);
    acc += dout[((size_t)n * OC + o) * plane + p];
  }
  acc = block_sum(acc);
  if (threadIdx.x == 0) db[o] = accumulate ? db[o] + acc : acc;
}

static int grid_for(long long total, int block, int sm_count) {
  long long blocks = (total + block - 1) / block;
  long long cap = (long long)sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

int conv_general_fwd(b200_ctx *ctx, const ConvGeom &g, const float *in, const float *W,
                     const float *bias, float *out, int B, int act) {
  long long total = (long long)B * g.OC * g.OH * g.OW;
  if (total == 0) return 0;
  conv_general_fwd_kernel<<<grid_for(total, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
    g, in, W, bias, out, total, act);
  B200_LAUNCHED();
  return 0;
}

int conv_general_dx(b200_ctx *ctx, const ConvGeom &g, const float *W, const float *dout,
                    float *din, int B) {
  long long total = (long long)B * g.C * g.HI * g.WI;
  if (total == 0) return 0;
  conv_general_dx_kernel<<<grid_for(total, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
    g, W, dout, din, total);
  B200_LAUNCHED();
  return 0;
}

int conv_general_dw(b200_ctx *ctx, const ConvGeom &g, const float *in, const float *dout,
                    float *dW, float *db, int accumulate, int B) {
  int nw = (int)conv_weight_len(g);
  conv_general_dw_kernel<<<nw, 128, 0, ctx->stream>>>(g, in, dout, dW, B, accumulate);
  B200_LAUNCHED();
  if (g.has_bias && db) {
    conv_db_kernel<<<g.OC, 256, 0, ctx->stream>>>(dout, db, g.OC, g.OH * g.OW, B, accumulate);
    B200_LAUNCHED();
  }
  return 0;
}

}  // namespace b200
