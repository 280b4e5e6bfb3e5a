// extern "C" operator entry points: argument checks, algorithm choice, scratch
// management, and the HOST-buffer forms used by the reference-side OpKernel
// branches.
#include <string.h>

#include "common.cuh"
#include "device_utils.cuh"

using namespace b200;

namespace {

int check_ctx(b200_ctx *ctx) {
  B200_REQUIRE(ctx != nullptr, "context is NULL");
  B200_CUDA(cudaSetDevice(ctx->device));
  return 0;
}

bool use_tiled(const b200_conv_desc *d, const ConvGeom &g) {
  if (d->algo == 1) return false;
  return conv_tiled_ok(g);
}

int conv_fwd_impl(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W,
                  const float *bias, float *out, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(batch >= 0, "conv2d_fwd: negative batch");
  ConvGeom g;
  B200_TRY(conv_geom_from_desc(ctx, d, &g));
  if (batch == 0) return 0;  // empty batch: nothing to read or write
  B200_REQUIRE(in && W && out && (bias || !g.has_bias), "conv2d_fwd: NULL buffer");
  ConvTcUse tc = conv_tc_use(ctx, g, d->algo);
  B200_REQUIRE(d->algo != 3 || tc.fwd || tc.fwd_small,
               "conv2d_fwd: tensor-core kernels need stride 1, dilation 1, windows <= 8x8, <= 256 channels");
  if (tc.fwd_small) return conv_fwd_small(ctx, g, in, W, bias, out, batch, B200_ACT_NONE);
  if (tc.fwd) {
    size_t n_x = align_up(conv_tc_tall_floats(g, batch, 0), 64);
    void *scratch = nullptr;
    B200_TRY(ctx_scratch(ctx, (n_x + conv_tc_filter_floats(ctx, g, 0)) * sizeof(float), &scratch));
    float *xs = static_cast<float *>(scratch);
    B200_TRY(conv_tc_tall_x(ctx, g, in, batch, xs));
    return conv_tc_fwd(ctx, g, xs, W, bias, out, batch, B200_ACT_NONE, xs + n_x);
  }
  bool tiled = use_tiled(d, g);
  B200_REQUIRE(tiled || d->algo != 2, "conv2d_fwd: tiled kernels need stride 1, dilation 1, 3x3/5x5");
  if (tiled) {
    void *scratch = nullptr;
    B200_TRY(ctx_scratch(ctx, conv_tiled_fwd_scratch(g) * sizeof(float), &scratch));
    return conv_tiled_fwd(ctx, g, in, W, bias, out, batch, B200_ACT_NONE,
                          static_cast<float *>(scratch));
  }
  return conv_general_fwd(ctx, g, in, W, bias, out, batch, B200_ACT_NONE);
}

int conv_bwd_impl(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W,
                  const float *dout, float *din, float *dW, float *db, int accumulate,
                  int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(batch >= 0, "conv2d_bwd: negative batch");
  ConvGeom g;
  B200_TRY(conv_geom_from_desc(ctx, d, &g));
  B200_REQUIRE(dW && (db || !g.has_bias), "conv2d_bwd: NULL gradient buffer");
  B200_REQUIRE(batch == 0 || (in && W && dout), "conv2d_bwd: NULL buffer");
  size_t lenW = conv_weight_len(g);
  if (batch == 0) {
    if (!accumulate) {
      B200_CUDA(cudaMemsetAsync(dW, 0, lenW * sizeof(float), ctx->stream));
      if (g.has_bias) B200_CUDA(cudaMemsetAsync(db, 0, g.OC * sizeof(float), ctx->stream));
    }
    return 0;
  }
  ConvTcUse tc = conv_tc_use(ctx, g, d->algo);
  B200_REQUIRE(d->algo != 3 || tc.dw || tc.dw_small,
               "conv2d_bwd: tensor-core kernels need stride 1, dilation 1, windows <= 8x8, <= 256 channels");
  if (!din) tc.dx = false;
  bool tiled = use_tiled(d, g) && g.OW <= 64;
  B200_REQUIRE(tiled || d->algo != 2,
               "conv2d_bwd: tiled kernels need stride 1, dilation 1, 3x3/5x5, out width <= 64");
  // one carve-up of the context scratch for every pass of this call
  const bool need_dys = tc.dx || tc.dw;
  size_t n_dys = need_dys ? align_up(conv_tc_tall_floats(g, batch, 1), 64) : 0;
  int bs_rows = tc.dw && g.has_bias ? conv_tc_bsum_rows(g, batch) : 0;
  size_t n_bs = align_up((size_t)bs_rows * g.OC, 64);
  size_t n_xs = tc.dw ? align_up(conv_tc_tall_floats(g, batch, 0), 64) : 0;
  size_t n_wdx = tc.dx ? align_up(conv_tc_filter_floats(ctx, g, 1), 64) : 0;
  size_t n_part = tc.dw ? align_up(conv_tc_dw_floats(ctx, g, batch), 64) : 0;
  size_t n_tdx = (din && !tc.dx && tiled) ? align_up(conv_tiled_dx_scratch(g), 64) : 0;
  size_t n_small = tc.dw_small ? align_up(conv_dw_small_floats(ctx, g, batch), 64) : 0;
  size_t n_tdw = (!tc.dw && !tc.dw_small && tiled) ? conv_tiled_dw_scratch(ctx, g, batch) : 0;
  void *scratch = nullptr;
  B200_TRY(ctx_scratch(ctx, (n_dys + n_bs + n_xs + n_wdx + n_part + n_small + n_tdx + n_tdw + 64) * sizeof(float),
                       &scratch));
  float *dys = static_cast<float *>(scratch);
  float *bs = dys + n_dys, *xs = bs + n_bs, *wdx = xs + n_xs, *part = wdx + n_wdx;
  float *small = part + n_part;
  float *s_dx = small + n_small, *s_dw = s_dx + n_tdx;
  if (need_dys) B200_TRY(conv_tc_tall_dy(ctx, g, dout, batch, dys, bs_rows ? bs : nullptr));
  // dX
  if (din) {
    if (tc.dx)
      B200_TRY(conv_tc_dx(ctx, g, dys, W, din, batch, wdx));
    else if (tiled)
      B200_TRY(conv_tiled_dx(ctx, g, W, dout, din, batch, s_dx));
    else
      B200_TRY(conv_general_dx(ctx, g, W, dout, din, batch));
  }
  // dW, db
  if (tc.dw) {
    B200_TRY(conv_tc_tall_x(ctx, g, in, batch, xs));
    int splits = 0;
    B200_TRY(conv_tc_dw(ctx, g, xs, dys, batch, part, &splits));
    B200_TRY(conv_tc_dw_finish(ctx, g, part, splits, dW, accumulate, g.has_bias ? bs : nullptr, batch, db));
    return 0;
  }
  if (tc.dw_small) return conv_dw_small(ctx, g, in, dout, batch, small, dW, db, accumulate);
  if (!tiled) return conv_general_dw(ctx, g, in, dout, dW, db, accumulate, batch);
  int splits = 0;
  B200_TRY(conv_tiled_dw_partials(ctx, g, in, dout, batch, s_dw, &splits));
  size_t row = lenW + g.OC;
  B200_TRY(merge_rows(ctx, s_dw, splits, row, dW, lenW, accumulate, &g));
  if (g.has_bias) B200_TRY(merge_rows(ctx, s_dw + lenW, splits, row, db, g.OC, accumulate, nullptr));
  return 0;
}

// Device time of the main kernel of one pass (see b200_conv2d_time_pass).
int conv_time_pass_impl(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W,
                        const float *dout, int batch, int pass, int reps, float *ms, int *on_tc) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(batch >= 1 && reps >= 1 && pass >= 0 && pass <= 2 && ms, "conv2d_time_pass: bad argument");
  ConvGeom g;
  B200_TRY(conv_geom_from_desc(ctx, d, &g));
  B200_REQUIRE(in && W && (dout || pass == 0), "conv2d_time_pass: NULL buffer");
  ConvTcUse tc = conv_tc_use(ctx, g, d->algo);
  const bool tiled = use_tiled(d, g) && (pass == 0 || g.OW <= 64);
  const bool use_tc = pass == 0 ? (tc.fwd || tc.fwd_small) : pass == 1 ? tc.dx : (tc.dw || tc.dw_small);
  B200_REQUIRE(use_tc || tiled, "conv2d_time_pass: only the tensor-core and the tiled kernels are timed");
  const size_t in_len = (size_t)batch * g.C * g.HI * g.WI, out_len = (size_t)batch * g.OC * g.OH * g.OW;
  size_t n_res = align_up(in_len > out_len ? in_len : out_len, 64);
  size_t n_xs = align_up(conv_tc_tall_floats(g, batch, 0), 64), n_dys = align_up(conv_tc_tall_floats(g, batch, 1), 64);
  size_t n_wt = align_up(use_tc ? conv_tc_filter_floats(ctx, g, pass == 1) : 0, 64);
  size_t n_part = use_tc ? align_up(tc.dw_small ? conv_dw_small_floats(ctx, g, batch) + conv_weight_len(g) + g.OC
                                               : conv_tc_dw_floats(ctx, g, batch), 64) : 0;
  size_t n_tiled = 0;
  if (!use_tc)
    n_tiled = pass == 0 ? conv_tiled_fwd_scratch(g) : pass == 1 ? conv_tiled_dx_scratch(g)
                                                                 : conv_tiled_dw_scratch(ctx, g, batch);
  void *scratch = nullptr;
  B200_TRY(ctx_scratch(ctx, (n_res + n_xs + n_dys + n_wt + n_part + n_tiled + 64) * sizeof(float), &scratch));
  float *res = static_cast<float *>(scratch), *xs = res + n_res, *dys = xs + n_xs, *wt = dys + n_dys;
  float *part = wt + n_wt, *ts = part + n_part;
  cudaEvent_t e0, e1;
  B200_CUDA(cudaEventCreate(&e0));
  B200_CUDA(cudaEventCreate(&e1));
  int splits = 0, rc = 0;
  auto run = [&](int prep) -> int {
    if (use_tc) {
      if (pass == 0 && tc.fwd_small) return conv_fwd_small(ctx, g, in, W, nullptr, res, batch, B200_ACT_NONE);
      if (pass == 0) return conv_tc_fwd(ctx, g, xs, W, nullptr, res, batch, B200_ACT_NONE, wt, prep);
      if (pass == 1) return conv_tc_dx(ctx, g, dys, W, res, batch, wt, prep);
      if (tc.dw_small) {  // includes its finishing launch
        float *gw = part + conv_dw_small_floats(ctx, g, batch);
        return conv_dw_small(ctx, g, in, dout, batch, part, gw, gw + conv_weight_len(g), 0);
      }
      return conv_tc_dw(ctx, g, xs, dys, batch, part, &splits);
    }
    if (pass == 0) return conv_tiled_fwd(ctx, g, in, W, nullptr, res, batch, B200_ACT_NONE, ts);
    if (pass == 1) return conv_tiled_dx(ctx, g, W, dout, res, batch, ts);
    return conv_tiled_dw_partials(ctx, g, in, dout, batch, ts, &splits);
  };
  const bool slab = use_tc && !(pass == 2 && tc.dw_small) && !(pass == 0 && tc.fwd_small);
  if (slab && pass != 1) rc = conv_tc_tall_x(ctx, g, in, batch, xs);
  if (!rc && slab && pass != 0) rc = conv_tc_tall_dy(ctx, g, dout, batch, dys, nullptr);
  if (!rc) rc = run(1);  // warm-up, filter matrices, tile choice
  if (!rc) rc = cudaEventRecord(e0, ctx->stream) == cudaSuccess ? 0 : 1;
  for (int i = 0; i < reps && !rc; ++i) rc = run(0);
  if (!rc) rc = cudaEventRecord(e1, ctx->stream) == cudaSuccess ? 0 : 1;
  if (!rc) rc = cudaEventSynchronize(e1) == cudaSuccess ? 0 : 1;
  float t = 0.f;
  if (!rc) rc = cudaEventElapsedTime(&t, e0, e1) == cudaSuccess ? 0 : 1;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  B200_REQUIRE(rc == 0, "conv2d_time_pass: a launch or an event call failed (%s)", b200_last_error());
  *ms = t / reps;
  if (on_tc) *on_tc = use_tc ? 1 : 0;
  return 0;
}

// ---- host staging ------------------------------------------------------------

// Carves the context arena into device buffers for one *_host call.
struct Stage {
  b200_ctx *ctx;
  char *base = nullptr;
  size_t used = 0, cap = 0;
  std::vector<std::pair<size_t, size_t>> plan;  // bytes per buffer, planned first
};

struct HostBuf {
  const void *src;  // host source to upload (nullptr: none)
  void *dst;        // host destination to download (nullptr: none)
  size_t bytes;
  void *dev;
};

// Allocate all buffers of one call in the arena, upload inputs.
int stage_in(b200_ctx *ctx, HostBuf *bufs, int n) {
  size_t total = 0;
  for (int i = 0; i < n; ++i) total += align_up(bufs[i].bytes ? bufs[i].bytes : 4, 256);
  void *base = nullptr;
  B200_TRY(ctx_arena(ctx, total, &base));
  size_t off = 0;
  for (int i = 0; i < n; ++i) {
    bufs[i].dev = static_cast<char *>(base) + off;
    off += align_up(bufs[i].bytes ? bufs[i].bytes : 4, 256);
    if (bufs[i].src && bufs[i].bytes)
      B200_CUDA(cudaMemcpyAsync(bufs[i].dev, bufs[i].src, bufs[i].bytes, cudaMemcpyHostToDevice,
                                ctx->stream));
  }
  return 0;
}

int stage_out(b200_ctx *ctx, HostBuf *bufs, int n) {
  for (int i = 0; i < n; ++i)
    if (bufs[i].dst && bufs[i].bytes)
      B200_CUDA(cudaMemcpyAsync(bufs[i].dst, bufs[i].dev, bufs[i].bytes, cudaMemcpyDeviceToHost,
                                ctx->stream));
  B200_CUDA(cudaStreamSynchronize(ctx->stream));
  return 0;
}

size_t conv_in_len(const b200_conv_desc *d) {
  bool padded = d->input_is_padded || !d->pad_same;
  return padded ? (size_t)d->in_c * d->inp_h * d->inp_w : (size_t)d->in_c * d->in_h * d->in_w;
}
size_t conv_out_len(const b200_conv_desc *d) { return (size_t)d->out_c * d->out_h * d->out_w; }
size_t conv_w_len(const b200_conv_desc *d) {
  return (size_t)d->out_c * d->in_c * d->k_h * d->k_w;
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------- convolution
int b200_conv2d_fwd(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W,
                    const float *bias, float *out, int batch) {
  return conv_fwd_impl(ctx, d, in, W, bias, out, batch);
}

int b200_conv2d_bwd(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W,
                    const float *dout, float *din, float *dW, float *db, int accumulate,
                    int batch) {
  return conv_bwd_impl(ctx, d, in, W, dout, din, dW, db, accumulate, batch);
}

int b200_conv2d_time_pass(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W,
                          const float *dout, int batch, int pass, int reps, float *ms, int *on_tensor_cores) {
  return conv_time_pass_impl(ctx, d, in, W, dout, batch, pass, reps, ms, on_tensor_cores);
}

int b200_conv2d_fwd_host(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W,
                         const float *bias, float *out, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(d != nullptr && batch >= 0, "conv2d_fwd_host: bad argument");
  size_t f = sizeof(float);
  HostBuf b[4] = {{in, nullptr, conv_in_len(d) * batch * f, nullptr},
                  {W, nullptr, conv_w_len(d) * f, nullptr},
                  {d->has_bias ? bias : nullptr, nullptr, d->has_bias ? d->out_c * f : 0, nullptr},
                  {nullptr, out, conv_out_len(d) * batch * f, nullptr}};
  B200_TRY(stage_in(ctx, b, 4));
  B200_TRY(conv_fwd_impl(ctx, d, (const float *)b[0].dev, (const float *)b[1].dev,
                         (const float *)b[2].dev, (float *)b[3].dev, batch));
  return stage_out(ctx, b, 4);
}

int b200_conv2d_bwd_host(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W,
                         const float *dout, float *din, float *dW, float *db, int accumulate,
                         int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(d != nullptr && batch >= 0, "conv2d_bwd_host: bad argument");
  size_t f = sizeof(float);
  size_t nb = d->has_bias ? d->out_c * f : 0;
  HostBuf b[6] = {{in, nullptr, conv_in_len(d) * batch * f, nullptr},
                  {W, nullptr, conv_w_len(d) * f, nullptr},
                  {dout, nullptr, conv_out_len(d) * batch * f, nullptr},
                  {nullptr, din, din ? conv_in_len(d) * batch * f : 0, nullptr},
                  {accumulate ? dW : nullptr, dW, conv_w_len(d) * f, nullptr},
                  {accumulate && nb ? db : nullptr, nb ? db : nullptr, nb, nullptr}};
  B200_TRY(stage_in(ctx, b, 6));
  B200_TRY(conv_bwd_impl(ctx, d, (const float *)b[0].dev, (const float *)b[1].dev,
                         (const float *)b[2].dev, din ? (float *)b[3].dev : nullptr,
                         (float *)b[4].dev, nb ? (float *)b[5].dev : nullptr, accumulate, batch));
  return stage_out(ctx, b, 6);
}

// ---------------------------------------------------------------- fully connected
int b200_fc_fwd(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W,
                const float *bias, float *out, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(in_size > 0 && out_size > 0 && batch >= 0, "fc_fwd: bad size");
  B200_REQUIRE(in && W && out, "fc_fwd: NULL buffer");
  void *scratch = nullptr;
  B200_TRY(ctx_scratch(ctx, fc_scratch_floats(ctx, in_size, out_size, batch) * sizeof(float), &scratch));
  return fc_fwd(ctx, in_size, out_size, in, W, bias, out, batch, B200_ACT_NONE,
                static_cast<float *>(scratch));
}

int b200_fc_bwd(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W,
                const float *dout, float *din, float *dW, float *db, int accumulate, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(in_size > 0 && out_size > 0 && batch >= 0, "fc_bwd: bad size");
  B200_REQUIRE(in && W && dout && dW, "fc_bwd: NULL buffer");
  void *scratch = nullptr;
  B200_TRY(ctx_scratch(ctx, fc_scratch_floats(ctx, in_size, out_size, batch) * sizeof(float), &scratch));
  return fc_bwd(ctx, in_size, out_size, in, W, dout, din, dW, db, accumulate, batch,
                static_cast<float *>(scratch));
}

int b200_fc_fwd_host(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W,
                     const float *bias, float *out, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(in_size > 0 && out_size > 0 && batch >= 0, "fc_fwd_host: bad size");
  size_t f = sizeof(float);
  HostBuf b[4] = {{in, nullptr, (size_t)in_size * batch * f, nullptr},
                  {W, nullptr, (size_t)in_size * out_size * f, nullptr},
                  {bias, nullptr, bias ? out_size * f : 0, nullptr},
                  {nullptr, out, (size_t)out_size * batch * f, nullptr}};
  B200_TRY(stage_in(ctx, b, 4));
  void *scratch = nullptr;
  B200_TRY(ctx_scratch(ctx, fc_scratch_floats(ctx, in_size, out_size, batch) * sizeof(float), &scratch));
  B200_TRY(fc_fwd(ctx, in_size, out_size, (const float *)b[0].dev, (const float *)b[1].dev,
                  bias ? (const float *)b[2].dev : nullptr, (float *)b[3].dev, batch,
                  B200_ACT_NONE, static_cast<float *>(scratch)));
  return stage_out(ctx, b, 4);
}

int b200_fc_bwd_host(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W,
                     const float *dout, float *din, float *dW, float *db, int accumulate,
                     int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(in_size > 0 && out_size > 0 && batch >= 0, "fc_bwd_host: bad size");
  size_t f = sizeof(float);
  size_t nw = (size_t)in_size * out_size * f, nb = db ? out_size * f : 0;
  HostBuf b[6] = {{in, nullptr, (size_t)in_size * batch * f, nullptr},
                  {W, nullptr, nw, nullptr},
                  {dout, nullptr, (size_t)out_size * batch * f, nullptr},
                  {nullptr, din, din ? (size_t)in_size * batch * f : 0, nullptr},
                  {accumulate ? dW : nullptr, dW, nw, nullptr},
                  {accumulate && nb ? db : nullptr, db, nb, nullptr}};
  B200_TRY(stage_in(ctx, b, 6));
  void *scratch = nullptr;
  B200_TRY(ctx_scratch(ctx, fc_scratch_floats(ctx, in_size, out_size, batch) * sizeof(float), &scratch));
  B200_TRY(fc_bwd(ctx, in_size, out_size, (const float *)b[0].dev, (const float *)b[1].dev,
                  (const float *)b[2].dev, din ? (float *)b[3].dev : nullptr, (float *)b[4].dev,
                  db ? (float *)b[5].dev : nullptr, accumulate, batch, static_cast<float *>(scratch)));
  return stage_out(ctx, b, 6);
}

// ---------------------------------------------------------------- pooling
int b200_maxpool_fwd(b200_ctx *ctx, const b200_pool_desc *d, const float *in, float *out,
                     int32_t *argmax, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(d && in && out && argmax && batch >= 0, "maxpool_fwd: bad argument");
  return maxpool_fwd(ctx, *d, in, out, argmax, batch);
}
int b200_maxpool_bwd(b200_ctx *ctx, const b200_pool_desc *d, const float *dout,
                     const int32_t *argmax, float *din, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(d && dout && argmax && din && batch >= 0, "maxpool_bwd: bad argument");
  return maxpool_bwd(ctx, *d, dout, argmax, din, batch);
}
int b200_maxpool_fwd_host(b200_ctx *ctx, const b200_pool_desc *d, const float *in, float *out,
                          int32_t *argmax, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(d && batch >= 0, "maxpool_fwd_host: bad argument");
  size_t ni = (size_t)d->in_c * d->in_h * d->in_w * batch, no = (size_t)d->in_c * d->out_h * d->out_w * batch;
  HostBuf b[3] = {{in, nullptr, ni * 4, nullptr}, {nullptr, out, no * 4, nullptr},
                  {nullptr, argmax, no * 4, nullptr}};
  B200_TRY(stage_in(ctx, b, 3));
  B200_TRY(maxpool_fwd(ctx, *d, (const float *)b[0].dev, (float *)b[1].dev, (int32_t *)b[2].dev,
                       batch));
  return stage_out(ctx, b, 3);
}
int b200_maxpool_bwd_host(b200_ctx *ctx, const b200_pool_desc *d, const float *dout,
                          const int32_t *argmax, float *din, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(d && batch >= 0, "maxpool_bwd_host: bad argument");
  size_t ni = (size_t)d->in_c * d->in_h * d->in_w * batch, no = (size_t)d->in_c * d->out_h * d->out_w * batch;
  HostBuf b[3] = {{dout, nullptr, no * 4, nullptr}, {argmax, nullptr, no * 4, nullptr},
                  {nullptr, din, ni * 4, nullptr}};
  B200_TRY(stage_in(ctx, b, 3));
  B200_TRY(maxpool_bwd(ctx, *d, (const float *)b[0].dev, (const int32_t *)b[1].dev,
                       (float *)b[2].dev, batch));
  return stage_out(ctx, b, 3);
}

int b200_avgpool_fwd(b200_ctx *ctx, const b200_pool_desc *d, const float *in, const float *W,
                     const float *bias, float *out, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(d && in && W && bias && out && batch >= 0, "avgpool_fwd: bad argument");
  return avgpool_fwd(ctx, *d, in, W, bias, out, batch);
}
int b200_avgpool_bwd(b200_ctx *ctx, const b200_pool_desc *d, const float *in, const float *W,
                     const float *dout, float *din, float *dW, float *db, int accumulate,
                     int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(d && in && W && dout && dW && db && batch >= 0, "avgpool_bwd: bad argument");
  return avgpool_bwd(ctx, *d, in, W, dout, din, dW, db, accumulate, batch);
}
int b200_avgpool_fwd_host(b200_ctx *ctx, const b200_pool_desc *d, const float *in, const float *W,
                          const float *bias, float *out, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(d && batch >= 0, "avgpool_fwd_host: bad argument");
  size_t ni = (size_t)d->in_c * d->in_h * d->in_w * batch, no = (size_t)d->in_c * d->out_h * d->out_w * batch;
  size_t nw = (size_t)d->pool_w * d->pool_h * d->in_c;
  HostBuf b[4] = {{in, nullptr, ni * 4, nullptr}, {W, nullptr, nw * 4, nullptr},
                  {bias, nullptr, (size_t)d->in_c * 4, nullptr}, {nullptr, out, no * 4, nullptr}};
  B200_TRY(stage_in(ctx, b, 4));
  B200_TRY(avgpool_fwd(ctx, *d, (const float *)b[0].dev, (const float *)b[1].dev,
                       (const float *)b[2].dev, (float *)b[3].dev, batch));
  return stage_out(ctx, b, 4);
}
int b200_avgpool_bwd_host(b200_ctx *ctx, const b200_pool_desc *d, const float *in, const float *W,
                          const float *dout, float *din, float *dW, float *db, int accumulate,
                          int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(d && batch >= 0, "avgpool_bwd_host: bad argument");
  size_t ni = (size_t)d->in_c * d->in_h * d->in_w * batch, no = (size_t)d->in_c * d->out_h * d->out_w * batch;
  size_t nw = (size_t)d->pool_w * d->pool_h * d->in_c;
  HostBuf b[6] = {{in, nullptr, ni * 4, nullptr},
                  {W, nullptr, nw * 4, nullptr},
                  {dout, nullptr, no * 4, nullptr},
                  {nullptr, din, din ? ni * 4 : 0, nullptr},
                  {accumulate ? dW : nullptr, dW, nw * 4, nullptr},
                  {accumulate ? db : nullptr, db, (size_t)d->in_c * 4, nullptr}};
  B200_TRY(stage_in(ctx, b, 6));
  B200_TRY(avgpool_bwd(ctx, *d, (const float *)b[0].dev, (const float *)b[1].dev,
                       (const float *)b[2].dev, din ? (float *)b[3].dev : nullptr,
                       (float *)b[4].dev, (float *)b[5].dev, accumulate, batch));
  return stage_out(ctx, b, 6);
}

// ---------------------------------------------------------------- activations / loss
int b200_act_param_fwd(b200_ctx *ctx, int kind, float param, const float *x, float *y, int dim, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(x && y && dim > 0 && batch >= 0, "act_fwd: bad argument");
  return act_fwd(ctx, kind, x, y, dim, batch, param);
}
int b200_act_param_bwd(b200_ctx *ctx, int kind, float param, const float *y, const float *dy, float *dx, int dim,
                       int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(y && dy && dx && dim > 0 && batch >= 0, "act_bwd: bad argument");
  return act_bwd(ctx, kind, y, dy, dx, dim, batch, param);
}
int b200_act_param_fwd_host(b200_ctx *ctx, int kind, float param, const float *x, float *y, int dim, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(dim > 0 && batch >= 0, "act_fwd_host: bad argument");
  size_t n = (size_t)dim * batch * 4;
  HostBuf b[2] = {{x, nullptr, n, nullptr}, {nullptr, y, n, nullptr}};
  B200_TRY(stage_in(ctx, b, 2));
  B200_TRY(act_fwd(ctx, kind, (const float *)b[0].dev, (float *)b[1].dev, dim, batch, param));
  return stage_out(ctx, b, 2);
}
int b200_act_param_bwd_host(b200_ctx *ctx, int kind, float param, const float *y, const float *dy, float *dx,
                            int dim, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(dim > 0 && batch >= 0, "act_bwd_host: bad argument");
  size_t n = (size_t)dim * batch * 4;
  HostBuf b[3] = {{y, nullptr, n, nullptr}, {dy, nullptr, n, nullptr}, {nullptr, dx, n, nullptr}};
  B200_TRY(stage_in(ctx, b, 3));
  B200_TRY(act_bwd(ctx, kind, (const float *)b[0].dev, (const float *)b[1].dev, (float *)b[2].dev, dim, batch,
                   param));
  return stage_out(ctx, b, 3);
}
// the parameterless forms: the reference's default constructor arguments
int b200_act_fwd(b200_ctx *ctx, int kind, const float *x, float *y, int dim, int batch) {
  return b200_act_param_fwd(ctx, kind, act_default_param(kind), x, y, dim, batch);
}
int b200_act_bwd(b200_ctx *ctx, int kind, const float *y, const float *dy, float *dx, int dim, int batch) {
  return b200_act_param_bwd(ctx, kind, act_default_param(kind), y, dy, dx, dim, batch);
}
int b200_act_fwd_host(b200_ctx *ctx, int kind, const float *x, float *y, int dim, int batch) {
  return b200_act_param_fwd_host(ctx, kind, act_default_param(kind), x, y, dim, batch);
}
int b200_act_bwd_host(b200_ctx *ctx, int kind, const float *y, const float *dy, float *dx, int dim, int batch) {
  return b200_act_param_bwd_host(ctx, kind, act_default_param(kind), y, dy, dx, dim, batch);
}

// ---- batch normalization / dropout / LRN ------------------------------------------------------
static int bn_check(b200_ctx *ctx, int channels, int spatial, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(channels > 0 && spatial > 0 && batch >= 0, "batchnorm: bad shape %d x %d, batch %d", channels, spatial,
               batch);
  return 0;
}

int b200_batchnorm_fwd(b200_ctx *ctx, int channels, int spatial, float eps, const float *x, float *mean,
                       float *variance, float *stddev, float *y, int batch, int train) {
  B200_TRY(bn_check(ctx, channels, spatial, batch));
  B200_REQUIRE(x && mean && variance && stddev && y, "batchnorm_fwd: NULL argument");
  void *scratch = nullptr;
  B200_TRY(ctx_scratch(ctx, batchnorm_scratch_floats(ctx, channels, batch) * sizeof(float), &scratch));
  return batchnorm_fwd(ctx, channels, spatial, eps, x, mean, variance, stddev, y, batch, train,
                       static_cast<float *>(scratch));
}
int b200_batchnorm_bwd(b200_ctx *ctx, int channels, int spatial, const float *y, const float *dy,
                       const float *stddev, float *dx, int batch) {
  B200_TRY(bn_check(ctx, channels, spatial, batch));
  B200_REQUIRE(y && dy && stddev && dx, "batchnorm_bwd: NULL argument");
  void *scratch = nullptr;
  B200_TRY(ctx_scratch(ctx, batchnorm_scratch_floats(ctx, channels, batch) * sizeof(float), &scratch));
  return batchnorm_bwd(ctx, channels, spatial, y, dy, stddev, dx, batch, static_cast<float *>(scratch));
}
int b200_batchnorm_post_update(b200_ctx *ctx, int channels, float momentum, float *mean, float *variance,
                               const float *mean_cur, const float *var_cur) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(channels > 0 && mean && variance && mean_cur && var_cur, "batchnorm_post_update: bad argument");
  return batchnorm_post_update(ctx, channels, momentum, mean, variance, mean_cur, var_cur, nullptr);
}
int b200_batchnorm_fwd_host(b200_ctx *ctx, int channels, int spatial, float eps, const float *x, float *mean,
                            float *variance, float *stddev, float *y, int batch, int train) {
  B200_TRY(bn_check(ctx, channels, spatial, batch));
  const size_t n = (size_t)channels * spatial * batch * 4, c = (size_t)channels * 4;
  // the moments go in (test phase) or come out (train phase); stddev and y always come out
  HostBuf b[5] = {{x, nullptr, n, nullptr},
                  {train ? nullptr : mean, train ? mean : nullptr, c, nullptr},
                  {train ? nullptr : variance, train ? variance : nullptr, c, nullptr},
                  {nullptr, stddev, c, nullptr},
                  {nullptr, y, n, nullptr}};
  B200_TRY(stage_in(ctx, b, 5));
  void *scratch = nullptr;
  B200_TRY(ctx_scratch(ctx, batchnorm_scratch_floats(ctx, channels, batch) * sizeof(float), &scratch));
  B200_TRY(batchnorm_fwd(ctx, channels, spatial, eps, (const float *)b[0].dev, (float *)b[1].dev, (float *)b[2].dev,
                         (float *)b[3].dev, (float *)b[4].dev, batch, train, static_cast<float *>(scratch)));
  return stage_out(ctx, b, 5);
}
int b200_batchnorm_bwd_host(b200_ctx *ctx, int channels, int spatial, const float *y, const float *dy,
                            const float *stddev, float *dx, int batch) {
  B200_TRY(bn_check(ctx, channels, spatial, batch));
  const size_t n = (size_t)channels * spatial * batch * 4, c = (size_t)channels * 4;
  HostBuf b[4] = {{y, nullptr, n, nullptr}, {dy, nullptr, n, nullptr}, {stddev, nullptr, c, nullptr},
                  {nullptr, dx, n, nullptr}};
  B200_TRY(stage_in(ctx, b, 4));
  void *scratch = nullptr;
  B200_TRY(ctx_scratch(ctx, batchnorm_scratch_floats(ctx, channels, batch) * sizeof(float), &scratch));
  B200_TRY(batchnorm_bwd(ctx, channels, spatial, (const float *)b[0].dev, (const float *)b[1].dev,
                         (const float *)b[2].dev, (float *)b[3].dev, batch, static_cast<float *>(scratch)));
  return stage_out(ctx, b, 4);
}

int b200_dropout(b200_ctx *ctx, const float *in, const uint8_t *mask, float scale, float *out, long long n) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(in && mask && out && n >= 0, "dropout: bad argument");
  return dropout_apply(ctx, in, mask, scale, out, (size_t)n);
}
int b200_dropout_host(b200_ctx *ctx, const float *in, const uint8_t *mask, float scale, float *out, long long n) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(n >= 0, "dropout_host: bad argument");
  HostBuf b[3] = {{in, nullptr, (size_t)n * 4, nullptr}, {mask, nullptr, (size_t)n, nullptr},
                  {nullptr, out, (size_t)n * 4, nullptr}};
  B200_TRY(stage_in(ctx, b, 3));
  B200_TRY(dropout_apply(ctx, (const float *)b[0].dev, (const uint8_t *)b[1].dev, scale, (float *)b[2].dev, (size_t)n));
  return stage_out(ctx, b, 3);
}

int b200_lrn_fwd(b200_ctx *ctx, const float *in, float *out, int channels, int area, int size, float alpha, float beta,
                 int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(in && out && channels > 0 && area > 0 && size > 0 && batch >= 0, "lrn_fwd: bad argument");
  return lrn_across_fwd(ctx, in, out, channels, area, size, alpha, beta, batch);
}
int b200_lrn_fwd_host(b200_ctx *ctx, const float *in, float *out, int channels, int area, int size, float alpha,
                      float beta, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(channels > 0 && area > 0 && size > 0 && batch >= 0, "lrn_fwd_host: bad argument");
  const size_t n = (size_t)channels * area * batch * 4;
  HostBuf b[2] = {{in, nullptr, n, nullptr}, {nullptr, out, n, nullptr}};
  B200_TRY(stage_in(ctx, b, 2));
  B200_TRY(lrn_across_fwd(ctx, (const float *)b[0].dev, (float *)b[1].dev, channels, area, size, alpha, beta, batch));
  return stage_out(ctx, b, 2);
}

int b200_loss_grad(b200_ctx *ctx, int kind, const float *y, const float *t, float *dy, int dim,
                   int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(y && t && dy && dim > 0 && batch >= 0, "loss_grad: bad argument");
  return loss_grad(ctx, kind, y, t, dy, dim, batch);
}
int b200_loss_value(b200_ctx *ctx, int kind, const float *y, const float *t, float *loss_sum,
                    int dim, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(y && t && loss_sum && dim > 0 && batch >= 0, "loss_value: bad argument");
  return loss_value(ctx, kind, y, t, loss_sum, dim, batch);
}

// ---------------------------------------------------------------- merge + optimizer
int b200_merge_grads(b200_ctx *ctx, const float *grads, int rows, size_t len, float *dst) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(grads && dst && rows >= 1, "merge_grads: bad argument");
  return merge_rows(ctx, grads, rows, len, dst, len, 0, nullptr, /*in_order=*/1);
}
int b200_opt_update(b200_ctx *ctx, int kind, const b200_opt_hyper *h, const float *dW, float *W,
                    float *state0, float *state1, size_t len) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(h && dW && W, "opt_update: NULL argument");
  return opt_update(ctx, kind, *h, dW, 1, len, nullptr, W, state0, state1, len);
}
int b200_merge_update(b200_ctx *ctx, int kind, const b200_opt_hyper *h, const float *grads,
                      int rows, size_t stride, float *merged, float *W, float *state0,
                      float *state1, size_t len) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(h && grads && W, "merge_update: NULL argument");
  B200_REQUIRE(rows >= 1 && (rows == 1 || stride >= len), "merge_update: bad rows/stride");
  return opt_update(ctx, kind, *h, grads, rows, stride, merged, W, state0, state1, len);
}

// ---------------------------------------------------------------- quantized
int b200_qconv2d_fwd(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W,
                     const float *bias, float *out, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(d && in && W && out && batch >= 0 && (bias || !d->has_bias),
               "qconv2d_fwd: bad argument");
  return qconv_fwd(ctx, d, in, W, bias, out, batch);
}
int b200_qfc_fwd(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W,
                 const float *bias, float *out, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(in && W && out && batch >= 0, "qfc_fwd: bad argument");
  return qfc_fwd(ctx, in_size, out_size, in, W, bias, out, batch);
}
int b200_qconv2d_fwd_host(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W,
                          const float *bias, float *out, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(d && batch >= 0, "qconv2d_fwd_host: bad argument");
  size_t f = sizeof(float);
  size_t in_len = (size_t)d->in_c * d->inp_h * d->inp_w;
  HostBuf b[4] = {{in, nullptr, in_len * batch * f, nullptr},
                  {W, nullptr, conv_w_len(d) * f, nullptr},
                  {d->has_bias ? bias : nullptr, nullptr, d->has_bias ? d->out_c * f : 0, nullptr},
                  {nullptr, out, conv_out_len(d) * batch * f, nullptr}};
  B200_TRY(stage_in(ctx, b, 4));
  B200_TRY(qconv_fwd(ctx, d, (const float *)b[0].dev, (const float *)b[1].dev,
                     d->has_bias ? (const float *)b[2].dev : nullptr, (float *)b[3].dev, batch));
  return stage_out(ctx, b, 4);
}
int b200_qfc_fwd_host(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W,
                      const float *bias, float *out, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(in_size > 0 && out_size > 0 && batch >= 0, "qfc_fwd_host: bad argument");
  size_t f = sizeof(float);
  HostBuf b[4] = {{in, nullptr, (size_t)in_size * batch * f, nullptr},
                  {W, nullptr, (size_t)in_size * out_size * f, nullptr},
                  {bias, nullptr, bias ? out_size * f : 0, nullptr},
                  {nullptr, out, (size_t)out_size * batch * f, nullptr}};
  B200_TRY(stage_in(ctx, b, 4));
  B200_TRY(qfc_fwd(ctx, in_size, out_size, (const float *)b[0].dev, (const float *)b[1].dev,
                   bias ? (const float *)b[2].dev : nullptr, (float *)b[3].dev, batch));
  return stage_out(ctx, b, 4);
}

// ---- quantized layers chained without dequantizing ("eq") --------------------------------------
int b200_qconv2d_eq_fwd(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W, const float *bias,
                        const float *in_r, const float *W_r, const float *b_r, float *out, float *out_r, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(d && in && W && in_r && W_r && b_r && out && out_r && batch >= 0, "qconv2d_eq_fwd: bad argument");
  B200_REQUIRE(!d->has_bias || bias, "qconv2d_eq_fwd: the layer has a bias but none was given");
  return qconv_eq_fwd(ctx, d, in, W, bias, in_r, W_r, b_r, out, out_r, batch);
}
int b200_qfc_eq_fwd(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W, const float *bias,
                    const float *in_r, const float *W_r, const float *b_r, float *out, float *out_r, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(in_size > 0 && out_size > 0 && in && W && in_r && W_r && b_r && out && out_r && batch >= 0,
               "qfc_eq_fwd: bad argument");
  return qfc_eq_fwd(ctx, in_size, out_size, in, W, bias, in_r, W_r, b_r, out, out_r, batch);
}
int b200_qconv2d_eq_fwd_host(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W,
                             const float *bias, const float *in_r, const float *W_r, const float *b_r, float *out,
                             float *out_r, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(d && batch >= 0, "qconv2d_eq_fwd_host: bad argument");
  const size_t f = sizeof(float), in_len = (size_t)d->in_c * d->inp_h * d->inp_w;
  HostBuf b[8] = {{in, nullptr, in_len * batch * f, nullptr},
                  {W, nullptr, conv_w_len(d) * f, nullptr},
                  {d->has_bias ? bias : nullptr, nullptr, d->has_bias ? d->out_c * f : 0, nullptr},
                  {in_r, nullptr, (size_t)2 * batch * f, nullptr},
                  {W_r, nullptr, 2 * f, nullptr},
                  {b_r, nullptr, 2 * f, nullptr},
                  {nullptr, out, conv_out_len(d) * batch * f, nullptr},
                  {nullptr, out_r, (size_t)2 * batch * f, nullptr}};
  B200_TRY(stage_in(ctx, b, 8));
  B200_TRY(qconv_eq_fwd(ctx, d, (const float *)b[0].dev, (const float *)b[1].dev,
                        d->has_bias ? (const float *)b[2].dev : nullptr, (const float *)b[3].dev,
                        (const float *)b[4].dev, (const float *)b[5].dev, (float *)b[6].dev, (float *)b[7].dev, batch));
  return stage_out(ctx, b, 8);
}
int b200_qfc_eq_fwd_host(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W, const float *bias,
                         const float *in_r, const float *W_r, const float *b_r, float *out, float *out_r, int batch) {
  B200_TRY(check_ctx(ctx));
  B200_REQUIRE(in_size > 0 && out_size > 0 && batch >= 0, "qfc_eq_fwd_host: bad argument");
  const size_t f = sizeof(float);
  HostBuf b[8] = {{in, nullptr, (size_t)in_size * batch * f, nullptr},
                  {W, nullptr, (size_t)in_size * out_size * f, nullptr},
                  {bias, nullptr, bias ? out_size * f : 0, nullptr},
                  {in_r, nullptr, (size_t)2 * batch * f, nullptr},
                  {W_r, nullptr, 2 * f, nullptr},
                  {b_r, nullptr, 2 * f, nullptr},
                  {nullptr, out, (size_t)out_size * batch * f, nullptr},
                  {nullptr, out_r, (size_t)2 * batch * f, nullptr}};
  B200_TRY(stage_in(ctx, b, 8));
  B200_TRY(qfc_eq_fwd(ctx, in_size, out_size, (const float *)b[0].dev, (const float *)b[1].dev,
                      bias ? (const float *)b[2].dev : nullptr, (const float *)b[3].dev, (const float *)b[4].dev,
                      (const float *)b[5].dev, (float *)b[6].dev, (float *)b[7].dev, batch));
  return stage_out(ctx, b, 8);
}

}  // extern "C"
