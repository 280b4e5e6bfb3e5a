/*
 * oracle.c -- CPU restatement of tiny-dnn's training hot path, in plain C.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the parity tests, the
 * smoke test and the bench's CPU-baseline leg compare the CUDA path against.
 * Nothing in the product (the package, the C ABI library) may call it.
 *
 * Each function restates one reference routine with the same loop order and
 * the same float operations, so that, compiled without floating-point
 * contraction, it reproduces the reference bit for bit on the fp32 path.  It
 * is pinned against (a) the known-answer vectors of the reference's own tests
 * (tests/golden/reference_kats.json) and (b) outputs of the unmodified
 * reference compiled from its sources (oracle/_ref, see ref_shim.cpp).
 *
 * Layouts are the reference's: a batch is B rows of planar CHW
 * (tiny_dnn/util/util.h:168-173); conv weights [(in_c*o + inc)][ky][kx]
 * (core/kernels/conv2d_op_internal.h:41); fc weights [in][out]
 * (core/kernels/fully_connected_op_internal.h:28).
 */
#include <float.h>
#include <limits.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "tinycnn_b200.h"

#define ORC_API __attribute__((visibility("default")))

/* vectorize::dot with the scalar register type the default build selects
 * (tiny_dnn/util/product.h:321-364 over scalar_generic<float>, :28-62): four
 * interleaved accumulators, the tail added to the first, then (r0+r1)+(r2+r3). */
static float dot4(const float *f1, const float *f2, size_t size) {
  float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
  size_t n4 = size / 4, n1 = size % 4;
  for (size_t i = 0; i < n4; ++i) {
    r0 = f1[i * 4 + 0] * f2[i * 4 + 0] + r0;
    r1 = f1[i * 4 + 1] * f2[i * 4 + 1] + r1;
    r2 = f1[i * 4 + 2] * f2[i * 4 + 2] + r2;
    r3 = f1[i * 4 + 3] * f2[i * 4 + 3] + r3;
  }
  size_t idx = n4 * 4;
  for (size_t i = 0; i < n1; ++i) r0 = f1[idx + i] * f2[idx + i] + r0;
  r0 = r0 + r1;
  r2 = r2 + r3;
  r0 = r0 + r2;
  return r0;
}

/* ------------------------------------------------------------------------- */
/* convolution                                                                 */
/* ------------------------------------------------------------------------- */

static int tbl_connected(const b200_conv_desc *p, int o, int inc) {
  /* connection_table::is_connected(x = o, y = inc) -> connected_[y*cols + x]
   * (tiny_dnn/core/params/conv_params.h:52-54) */
  return p->tbl ? p->tbl[inc * p->out_c + o] != 0 : 1;
}

/* Conv2dPadding::copy_and_pad_input (core/params/conv_params.h:106-133) */
ORC_API void orc_conv_pad(const b200_conv_desc *p, const float *in, float *in_padded, int B) {
  size_t in_len = (size_t)p->in_c * p->in_h * p->in_w;
  size_t pad_len = (size_t)p->in_c * p->inp_h * p->inp_w;
  if (!p->pad_same) {
    memcpy(in_padded, in, sizeof(float) * in_len * B);
    return;
  }
  memset(in_padded, 0, sizeof(float) * pad_len * B);
  for (int n = 0; n < B; ++n)
    for (int c = 0; c < p->in_c; ++c)
      for (int y = 0; y < p->in_h; ++y)
        memcpy(in_padded + n * pad_len + ((size_t)p->inp_h * c + y + p->k_h / 2) * p->inp_w +
                 p->k_w / 2,
               in + n * in_len + ((size_t)p->in_h * c + y) * p->in_w, sizeof(float) * p->in_w);
}

/* Conv2dPadding::copy_and_unpad_delta (conv_params.h:140-166) */
ORC_API void orc_conv_unpad(const b200_conv_desc *p, const float *delta_padded, float *delta, int B) {
  size_t in_len = (size_t)p->in_c * p->in_h * p->in_w;
  size_t pad_len = (size_t)p->in_c * p->inp_h * p->inp_w;
  if (!p->pad_same) {
    memcpy(delta, delta_padded, sizeof(float) * in_len * B);
    return;
  }
  for (int n = 0; n < B; ++n)
    for (int c = 0; c < p->in_c; ++c)
      for (int y = 0; y < p->in_h; ++y)
        memcpy(delta + n * in_len + ((size_t)p->in_h * c + y) * p->in_w,
               delta_padded + n * pad_len + ((size_t)p->inp_h * c + y + p->k_h / 2) * p->inp_w +
                 p->k_w / 2,
               sizeof(float) * p->in_w);
}

/* kernels::conv2d_op_internal forward (core/kernels/conv2d_op_internal.h:13-74)
 * preceded by the fill_tensor(out, 0) of Conv2dOp::compute (conv2d_op.h:32-33).
 * `in` has in_padded geometry. */
ORC_API void orc_conv2d_fwd(const b200_conv_desc *p, const float *in, const float *W,
                            const float *bias, float *out, int B) {
  size_t iw = p->inp_w, ih = p->inp_h, id = p->in_c;
  size_t ow = p->out_w, oh = p->out_h, od = p->out_c;
  size_t kw = p->k_w, kh = p->k_h;
  size_t in_len = iw * ih * id, out_len = ow * oh * od, out_area = ow * oh;
  size_t elem_stride = p->stride_w, line_stride = iw * p->stride_h;
  memset(out, 0, sizeof(float) * out_len * B);
  for (int n = 0; n < B; ++n) {
    const float *inb = in + n * in_len;
    float *a = out + n * out_len;
    for (size_t o = 0; o < od; ++o) {
      float *pa = a + out_area * o;
      for (size_t inc = 0; inc < id; ++inc) {
        if (!tbl_connected(p, (int)o, (int)inc)) continue;
        const float *pw = W + kw * kh * (id * o + inc);
        const float *pin = inb + iw * ih * inc;
        float *pout = pa;
        for (size_t y = 0; y < oh; ++y) {
          const float *pin_line = pin;
          for (size_t x = 0; x < ow; ++x) {
            const float *pin_element = pin_line;
            const float *pw_element = pw;
            float sum = 0.f;
            for (size_t wy = 0; wy < kh; ++wy) {
              for (size_t wx = 0; wx < kw; ++wx)
                sum += pw_element[wx] * pin_element[wx * p->dil_w];
              pw_element += kw;
              pin_element += iw * p->dil_h;
            }
            pout[x] += sum;
            pin_line += elem_stride;
          }
          pout += ow;
          pin += line_stride;
        }
      }
      if (p->has_bias)
        for (size_t i = 0; i < out_area; ++i) pa[i] += bias[o]; /* vectorize::add */
    }
  }
}

/* kernels::conv2d_op_internal backward (conv2d_op_internal.h:78-181) preceded by
 * the fill_tensor(prev_delta, 0) of Conv2dGradOp::compute (conv2d_grad_op.h:33-34).
 * prev_delta has in_padded geometry and is overwritten.  dW / db are the
 * reference's per-sample rows (B x len), ADDED to, when per_sample != 0;
 * otherwise they are single rows that receive the sample rows summed in sample
 * order, the sum edge::merge_grads forms (node.h:89-103), again added to.
 */
ORC_API void orc_conv2d_bwd(const b200_conv_desc *p, const float *prev_out, const float *W,
                            const float *curr_delta, float *prev_delta, float *dW, float *db,
                            int per_sample, int B) {
  size_t iw = p->inp_w, ih = p->inp_h, id = p->in_c;
  size_t ow = p->out_w, oh = p->out_h, od = p->out_c;
  size_t kw = p->k_w, kh = p->k_h;
  size_t in_len = iw * ih * id, out_len = ow * oh * od, lenW = kw * kh * id * od;
  float *row_w = (float *)calloc(lenW ? lenW : 1, sizeof(float));
  float *row_b = (float *)calloc(od ? od : 1, sizeof(float));
  if (prev_delta) memset(prev_delta, 0, sizeof(float) * in_len * B);
  for (int n = 0; n < B; ++n) {
    const float *po = prev_out + n * in_len;
    const float *cd = curr_delta + n * out_len;
    /* propagate delta to previous layer */
    if (prev_delta) {
      float *pd = prev_delta + n * in_len;
      for (size_t inc = 0; inc < id; ++inc)
        for (size_t outc = 0; outc < od; ++outc) {
          if (!tbl_connected(p, (int)outc, (int)inc)) continue;
          const float *pw = W + kw * kh * (id * outc + inc);
          const float *pdelta_src = cd + ow * oh * outc;
          float *pdelta_dst = pd + iw * ih * inc;
          for (size_t y = 0; y < oh; ++y)
            for (size_t x = 0; x < ow; ++x) {
              const float *ppw = pw;
              const float ppdelta_src = pdelta_src[y * ow + x];
              float *ppdelta_dst = pdelta_dst + y * p->stride_h * iw + x * p->stride_w;
              for (size_t wy = 0; wy < kh; ++wy)
                for (size_t wx = 0; wx < kw; ++wx) ppdelta_dst[wy * iw + wx] += *ppw++ * ppdelta_src;
            }
        }
    }
    /* accumulate dw */
    float *dWn = per_sample ? dW + n * lenW : row_w;
    if (!per_sample) memset(row_w, 0, sizeof(float) * lenW);
    for (size_t inc = 0; inc < id; ++inc)
      for (size_t outc = 0; outc < od; ++outc) {
        if (!tbl_connected(p, (int)outc, (int)inc)) continue;
        for (size_t wy = 0; wy < kh; ++wy)
          for (size_t wx = 0; wx < kw; ++wx) {
            float dst = 0.f;
            const float *prevo = po + (ih * inc + wy) * iw + wx;
            const float *delta = cd + ow * oh * outc;
            if (p->stride_w > 1) {
              for (size_t y = 0; y < oh; ++y)
                for (size_t x = 0; x < ow; ++x)
                  dst += prevo[y * iw * p->stride_h + x * p->stride_w] * delta[y * ow + x];
            } else {
              for (size_t y = 0; y < oh; ++y)
                dst += dot4(prevo + y * iw * p->stride_h, delta + y * ow, ow);
            }
            dWn[(kh * (id * outc + inc) + wy) * kw + wx] += dst;
          }
      }
    /* accumulate db */
    float *dbn = per_sample ? (db ? db + n * od : NULL) : row_b;
    if (!per_sample) memset(row_b, 0, sizeof(float) * od);
    if (p->has_bias && dbn)
      for (size_t outc = 0; outc < od; ++outc) {
        const float *delta = cd + ow * oh * outc;
        float s = 0.f;
        for (size_t i = 0; i < ow * oh; ++i) s += delta[i];
        dbn[outc] += s;
      }
    if (!per_sample) {
      for (size_t i = 0; i < lenW; ++i) dW[i] += row_w[i];
      if (p->has_bias && db)
        for (size_t i = 0; i < od; ++i) db[i] += row_b[i];
    }
  }
  free(row_w);
  free(row_b);
}

/* ------------------------------------------------------------------------- */
/* fully connected                                                             */
/* ------------------------------------------------------------------------- */

/* kernels::fully_connected_op_internal forward
 * (core/kernels/fully_connected_op_internal.h:15-36) */
ORC_API void orc_fc_fwd(int in_size, int out_size, const float *in, const float *W,
                        const float *bias, float *out, int B) {
  for (int n = 0; n < B; ++n) {
    const float *x = in + (size_t)n * in_size;
    float *o = out + (size_t)n * out_size;
    for (int i = 0; i < out_size; ++i) {
      o[i] = 0.f;
      for (int c = 0; c < in_size; ++c) o[i] += W[(size_t)c * out_size + i] * x[c];
      if (bias) o[i] += bias[i];
    }
  }
}

/* kernels::fully_connected_op_internal backward (:38-71) after the
 * fill_tensor(prev_delta, 0) of FullyConnectedGradOp::compute
 * (fully_connected_grad_op.h:36-37).  dW/db as in orc_conv2d_bwd. */
ORC_API void orc_fc_bwd(int in_size, int out_size, const float *prev_out, const float *W,
                        const float *curr_delta, float *prev_delta, float *dW, float *db,
                        int per_sample, int B) {
  size_t lenW = (size_t)in_size * out_size;
  float *row_w = (float *)calloc(lenW ? lenW : 1, sizeof(float));
  float *row_b = (float *)calloc(out_size ? out_size : 1, sizeof(float));
  for (int n = 0; n < B; ++n) {
    const float *x = prev_out + (size_t)n * in_size;
    const float *d = curr_delta + (size_t)n * out_size;
    if (prev_delta) {
      float *pd = prev_delta + (size_t)n * in_size;
      for (int c = 0; c < in_size; ++c)
        pd[c] = 0.f + dot4(d, W + (size_t)c * out_size, out_size);
    }
    float *dWn = per_sample ? dW + (size_t)n * lenW : row_w;
    float *dbn = per_sample ? (db ? db + (size_t)n * out_size : NULL) : row_b;
    if (!per_sample) {
      memset(row_w, 0, sizeof(float) * lenW);
      memset(row_b, 0, sizeof(float) * out_size);
    }
    for (int c = 0; c < in_size; ++c) /* vectorize::muladd */
      for (int i = 0; i < out_size; ++i) dWn[(size_t)c * out_size + i] += d[i] * x[c];
    if (dbn)
      for (int i = 0; i < out_size; ++i) dbn[i] += d[i];
    if (!per_sample) {
      for (size_t i = 0; i < lenW; ++i) dW[i] += row_w[i];
      if (db)
        for (int i = 0; i < out_size; ++i) db[i] += row_b[i];
    }
  }
  free(row_w);
  free(row_b);
}

/* ------------------------------------------------------------------------- */
/* pooling                                                                     */
/* ------------------------------------------------------------------------- */

/* max_pooling_layer::init_connection / connect_kernel
 * (tiny_dnn/layers/max_pooling_layer.h:195-235): out2in lists and in2out. */
typedef struct {
  int *out2in;  /* [out_len][pool_w*pool_h], -1 padded */
  int *in2out;  /* [in_len], default 0 */
  int win;
} pool_tables;

static pool_tables build_max_tables(const b200_pool_desc *d) {
  pool_tables t;
  int in_len = d->in_c * d->in_h * d->in_w, out_len = d->in_c * d->out_h * d->out_w;
  t.win = d->pool_w * d->pool_h;
  t.out2in = (int *)malloc(sizeof(int) * (size_t)out_len * t.win);
  t.in2out = (int *)calloc(in_len, sizeof(int));
  for (size_t i = 0; i < (size_t)out_len * t.win; ++i) t.out2in[i] = -1;
  for (int c = 0; c < d->in_c; ++c)
    for (int y = 0; y < d->out_h; ++y)
      for (int x = 0; x < d->out_w; ++x) {
        int dxmax = d->pool_w < d->in_w - x * d->stride_w ? d->pool_w : d->in_w - x * d->stride_w;
        int dymax = d->pool_h < d->in_h - y * d->stride_h ? d->pool_h : d->in_h - y * d->stride_h;
        int out_index = (d->out_h * c + y) * d->out_w + x;
        int k = 0;
        for (int dy = 0; dy < dymax; ++dy)
          for (int dx = 0; dx < dxmax; ++dx) {
            int in_index = (d->in_h * c + y * d->stride_h + dy) * d->in_w + x * d->stride_w + dx;
            t.in2out[in_index] = out_index;
            t.out2in[(size_t)out_index * t.win + k++] = in_index;
          }
      }
  return t;
}

/* kernels::maxpool_op_internal (core/kernels/maxpool_op_internal.h:16-39) */
ORC_API void orc_maxpool_fwd(const b200_pool_desc *d, const float *in, float *out, int32_t *argmax,
                             int B) {
  pool_tables t = build_max_tables(d);
  int in_len = d->in_c * d->in_h * d->in_w, out_len = d->in_c * d->out_h * d->out_w;
  for (int n = 0; n < B; ++n) {
    const float *x = in + (size_t)n * in_len;
    for (int i = 0; i < out_len; ++i) {
      float max_value = -FLT_MAX;
      int idx = 0;
      for (int k = 0; k < t.win; ++k) {
        int j = t.out2in[(size_t)i * t.win + k];
        if (j < 0) break;
        if (x[j] > max_value) {
          max_value = x[j];
          idx = j;
        }
      }
      argmax[(size_t)n * out_len + i] = idx;
      out[(size_t)n * out_len + i] = max_value;
    }
  }
  free(t.out2in);
  free(t.in2out);
}

/* kernels::maxpool_grad_op_internal (maxpool_op_internal.h:41-57) */
ORC_API void orc_maxpool_bwd(const b200_pool_desc *d, const float *curr_delta,
                             const int32_t *argmax, float *prev_delta, int B) {
  pool_tables t = build_max_tables(d);
  int in_len = d->in_c * d->in_h * d->in_w, out_len = d->in_c * d->out_h * d->out_w;
  for (int n = 0; n < B; ++n)
    for (int i = 0; i < in_len; ++i) {
      int outi = t.in2out[i];
      prev_delta[(size_t)n * in_len + i] =
        (argmax[(size_t)n * out_len + outi] == i) ? curr_delta[(size_t)n * out_len + outi] : 0.f;
    }
  free(t.out2in);
  free(t.in2out);
}

/* tiny_average_pooling_kernel (tiny_dnn/layers/average_pooling_layer.h:25-55)
 * with the connections of init_connection / connect_kernel (:271-311). */
ORC_API void orc_avgpool_fwd(const b200_pool_desc *d, const float *in, const float *W,
                             const float *bias, float *out, int B) {
  int in_len = d->in_c * d->in_h * d->in_w, out_len = d->in_c * d->out_h * d->out_w;
  float scale = 1.0f / (float)(d->pool_w * d->pool_h);
  for (int n = 0; n < B; ++n)
    for (int c = 0; c < d->in_c; ++c) {
      float weight = W[c] * scale;
      for (int oy = 0; oy < d->out_h; ++oy)
        for (int ox = 0; ox < d->out_w; ++ox) {
          float value = 0.f;
          int y0 = oy * d->stride_h, x0 = ox * d->stride_w;
          if (y0 + d->pool_h <= d->in_h && x0 + d->pool_w <= d->in_w)
            for (int dy = 0; dy < d->pool_h; ++dy)
              for (int dx = 0; dx < d->pool_w; ++dx)
                value += in[(size_t)n * in_len + (d->in_h * c + y0 + dy) * d->in_w + x0 + dx];
          value *= weight;
          value += bias[c];
          out[(size_t)n * out_len + (d->out_h * c + oy) * d->out_w + ox] = value;
        }
    }
}

/* tiny_average_pooling_back_kernel (average_pooling_layer.h:58-106).
 * dW (pool_w*pool_h*in_c entries, only the first in_c touched) / db as in
 * orc_conv2d_bwd. */
ORC_API void orc_avgpool_bwd(const b200_pool_desc *d, const float *prev_out, const float *W,
                             const float *curr_delta, float *prev_delta, float *dW, float *db,
                             int per_sample, int B) {
  int in_len = d->in_c * d->in_h * d->in_w, out_len = d->in_c * d->out_h * d->out_w;
  int wlen = d->pool_w * d->pool_h * d->in_c;
  float scale = 1.0f / (float)(d->pool_w * d->pool_h);
  for (int n = 0; n < B; ++n) {
    const float *x = prev_out + (size_t)n * in_len;
    const float *g = curr_delta + (size_t)n * out_len;
    if (prev_delta)
      for (int c = 0; c < d->in_c; ++c) {
        float weight = W[c] * scale;
        for (int iy = 0; iy < d->in_h; ++iy)
          for (int ix = 0; ix < d->in_w; ++ix) {
            /* in2wo[idx][0]: first window, in (y, x) order, holding the input */
            int oy = iy < d->pool_h ? 0 : (iy - d->pool_h) / d->stride_h + 1;
            int ox = ix < d->pool_w ? 0 : (ix - d->pool_w) / d->stride_w + 1;
            prev_delta[(size_t)n * in_len + (d->in_h * c + iy) * d->in_w + ix] =
              weight * g[(d->out_h * c + oy) * d->out_w + ox];
          }
      }
    for (int c = 0; c < d->in_c; ++c) {
      float diff = 0.f, bdiff = 0.f;
      for (int y = 0; y + d->pool_h <= d->in_h; y += d->stride_h)
        for (int xx = 0; xx + d->pool_w <= d->in_w; xx += d->stride_w) {
          int outidx = (d->out_h * c + y / d->stride_h) * d->out_w + xx / d->stride_w;
          for (int dy = 0; dy < d->pool_h; ++dy)
            for (int dx = 0; dx < d->pool_w; ++dx)
              diff += x[(d->in_h * c + y + dy) * d->in_w + xx + dx] * g[outidx];
        }
      for (int i = 0; i < d->out_h * d->out_w; ++i) bdiff += g[d->out_h * d->out_w * c + i];
      if (per_sample) {
        dW[(size_t)n * wlen + c] += diff * scale;
        db[(size_t)n * d->in_c + c] += bdiff;
      } else {
        dW[c] += 0.f + diff * scale;
        db[c] += 0.f + bdiff;
      }
    }
  }
}

/* ------------------------------------------------------------------------- */
/* activations and losses                                                      */
/* ------------------------------------------------------------------------- */

static float act_default_param(int kind) {
  return kind == B200_ACT_LEAKY_RELU ? 0.01f : kind == B200_ACT_ELU ? 1.f : 0.f;
}

/* relu_layer.h:25-29, tanh_layer.h:24-28, softmax_layer.h:24-34, sigmoid_layer.h:26-30,
   leaky_relu_layer.h:74-78 (param = epsilon_), elu_layer.h:38-42 (param = alpha_) */
ORC_API void orc_act_param_fwd(int kind, float param, const float *x, float *y, int dim, int B) {
  for (int n = 0; n < B; ++n) {
    const float *xr = x + (size_t)n * dim;
    float *yr = y + (size_t)n * dim;
    if (kind == B200_ACT_RELU) {
      for (int j = 0; j < dim; ++j) yr[j] = xr[j] > 0.f ? xr[j] : 0.f;
    } else if (kind == B200_ACT_TANH) {
      for (int j = 0; j < dim; ++j) yr[j] = tanhf(xr[j]);
    } else if (kind == B200_ACT_SIGMOID) {
      for (int j = 0; j < dim; ++j) yr[j] = 1.f / (1.f + expf(-xr[j]));
    } else if (kind == B200_ACT_LEAKY_RELU) {
      for (int j = 0; j < dim; ++j) yr[j] = xr[j] > 0.f ? xr[j] : param * xr[j];
    } else if (kind == B200_ACT_ELU) {
      for (int j = 0; j < dim; ++j) yr[j] = xr[j] < 0.f ? param * (expf(xr[j]) - 1.f) : xr[j];
    } else if (kind == B200_ACT_SOFTMAX) {
      float alpha = xr[0];
      for (int j = 1; j < dim; ++j) alpha = xr[j] > alpha ? xr[j] : alpha;
      float denominator = 0.f;
      for (int j = 0; j < dim; ++j) {
        yr[j] = expf(xr[j] - alpha);
        denominator += yr[j];
      }
      for (int j = 0; j < dim; ++j) yr[j] /= denominator;
    } else {
      memcpy(yr, xr, sizeof(float) * dim);
    }
  }
}

/* relu_layer.h:31-39, tanh_layer.h:30-38, softmax_layer.h:36-55, sigmoid_layer.h:32-39,
   leaky_relu_layer.h:80-88, elu_layer.h:44-54 */
ORC_API void orc_act_param_bwd(int kind, float param, const float *y, const float *dy, float *dx, int dim,
                               int B) {
  for (int n = 0; n < B; ++n) {
    const float *yr = y + (size_t)n * dim, *gr = dy + (size_t)n * dim;
    float *dr = dx + (size_t)n * dim;
    if (kind == B200_ACT_RELU) {
      for (int j = 0; j < dim; ++j) dr[j] = gr[j] * (yr[j] > 0.f ? 1.f : 0.f);
    } else if (kind == B200_ACT_TANH) {
      for (int j = 0; j < dim; ++j) dr[j] = gr[j] * (1.f - yr[j] * yr[j]);
    } else if (kind == B200_ACT_SIGMOID) {
      for (int j = 0; j < dim; ++j) dr[j] = gr[j] * yr[j] * (1.f - yr[j]);
    } else if (kind == B200_ACT_LEAKY_RELU) {
      for (int j = 0; j < dim; ++j) dr[j] = gr[j] * (yr[j] > 0.f ? 1.f : param);
    } else if (kind == B200_ACT_ELU) {
      for (int j = 0; j < dim; ++j) dr[j] = gr[j] * (yr[j] > 0.f ? 1.f : (param + yr[j]));
    } else if (kind == B200_ACT_SOFTMAX) {
      float *df = (float *)malloc(sizeof(float) * dim);
      for (int j = 0; j < dim; ++j) {
        for (int k = 0; k < dim; ++k)
          df[k] = (k == j) ? yr[j] * (1.f - yr[j]) : -yr[k] * yr[j];
        dr[j] = dot4(gr, df, dim);
      }
      free(df);
    } else {
      memcpy(dr, gr, sizeof(float) * dim);
    }
  }
}

/* the reference's default constructor arguments */
ORC_API void orc_act_fwd(int kind, const float *x, float *y, int dim, int B) {
  orc_act_param_fwd(kind, act_default_param(kind), x, y, dim, B);
}
ORC_API void orc_act_bwd(int kind, const float *y, const float *dy, float *dx, int dim, int B) {
  orc_act_param_bwd(kind, act_default_param(kind), y, dy, dx, dim, B);
}

/* ------------------------------------------------------------------------- */
/* batch normalization, dropout, local response normalization                  */
/* ------------------------------------------------------------------------- */

/* moments() (tiny_dnn/util/math_functions.h:25-96): per channel, samples in order, std::accumulate
   over the spatial positions of each; then the division */
static void moments_mean(const float *x, int C, int S, int B, float *mean) {
  for (int j = 0; j < C; ++j) mean[j] = 0.f;
  for (int i = 0; i < B; ++i)
    for (int j = 0; j < C; ++j) {
      float r = mean[j];
      const float *it = x + ((size_t)i * C + j) * S;
      for (int k = 0; k < S; ++k) r = r + it[k];
      mean[j] = r;
    }
  const float div = (float)B * S;
  for (int j = 0; j < C; ++j) mean[j] = mean[j] / div;
}

static void moments_variance(const float *x, int C, int S, int B, const float *mean, float *var) {
  for (int j = 0; j < C; ++j) var[j] = 0.f;
  for (int i = 0; i < B; ++i)
    for (int j = 0; j < C; ++j) {
      float r = var[j];
      const float ex = mean[j];
      const float *it = x + ((size_t)i * C + j) * S;
      /* `current + pow(x - ex, float_t{2.0})`: x - ex is formed in float, the square and the addition
         in double (the C library's pow(double, double) is the overload that unqualified call finds),
         and std::accumulate stores the sum back into its float accumulator */
      for (int k = 0; k < S; ++k) r = (float)((double)r + pow((double)(it[k] - ex), 2.0));
      var[j] = r;
    }
  float div = (float)((size_t)B * S) - 1.0f;
  if (div < 1.0f) div = 1.0f;
  for (int j = 0; j < C; ++j) var[j] = var[j] / div;
}

/* batch_normalization_layer::forward_propagation (batch_normalization_layer.h:136-168) */
ORC_API void orc_batchnorm_fwd(int C, int S, float eps, const float *x, float *mean, float *variance, float *stddev,
                               float *y, int B, int train) {
  if (train) {
    moments_mean(x, C, S, B, mean);
    moments_variance(x, C, S, B, mean, variance);
  }
  for (int j = 0; j < C; ++j) stddev[j] = sqrtf(variance[j] + eps);
  for (int i = 0; i < B; ++i)
    for (int j = 0; j < C; ++j) {
      const float m = mean[j];
      const float *ip = x + ((size_t)i * C + j) * S;
      float *op = y + ((size_t)i * C + j) * S;
      for (int k = 0; k < S; ++k) op[k] = (ip[k] - m) / stddev[j];
    }
}

/* batch_normalization_layer::back_propagation (:94-134) */
ORC_API void orc_batchnorm_bwd(int C, int S, const float *y, const float *dy, const float *stddev, float *dx, int B) {
  const size_t n = (size_t)B * C * S;
  float *ddy = (float *)malloc(sizeof(float) * (n ? n : 1));
  float *mean_ddy = (float *)malloc(sizeof(float) * C), *mean_d = (float *)malloc(sizeof(float) * C);
  for (size_t i = 0; i < n; ++i) ddy[i] = y[i] * dy[i];
  moments_mean(ddy, C, S, B, mean_ddy);
  moments_mean(dy, C, S, B, mean_d);
  for (int i = 0; i < B; ++i)
    for (int j = 0; j < C; ++j)
      for (int k = 0; k < S; ++k) {
        const size_t idx = ((size_t)i * C + j) * S + k;
        float v = dy[idx] - mean_d[j] - mean_ddy[j] * y[idx];
        dx[idx] = v / stddev[j];
      }
  free(ddy);
  free(mean_ddy);
  free(mean_d);
}

/* batch_normalization_layer::post_update (:174-180) */
ORC_API void orc_batchnorm_post_update(int C, float momentum, float *mean, float *variance, const float *mean_cur,
                                       const float *var_cur) {
  for (int i = 0; i < C; ++i) {
    mean[i] = momentum * mean[i] + (1 - momentum) * mean_cur[i];
    variance[i] = momentum * variance[i] + (1 - momentum) * var_cur[i];
  }
}

/* dropout_layer in the train phase with a given mask (dropout_layer.h:95-115); with scale 1 on a
   gradient it is the backward pass (:66-84) */
ORC_API void orc_dropout(const float *in, const uint8_t *mask, float scale, float *out, long long n) {
  for (long long i = 0; i < n; ++i) out[i] = mask[i] * scale * in[i];
}

/* lrn_layer::forward_across (lrn_layer.h:110-143) */
ORC_API void orc_lrn_fwd(const float *in, float *out, int C, int area, int size, float alpha, float beta, int B) {
  float *sq = (float *)malloc(sizeof(float) * area);
  const float alpha_div_size = alpha / size;
  for (int n = 0; n < B; ++n) {
    const float *ip = in + (size_t)n * C * area;
    float *op = out + (size_t)n * C * area;
    for (int j = 0; j < area; ++j) sq[j] = 0.f;
    for (int i = 0; i < size / 2 && i < C; ++i)
      for (int j = 0; j < area; ++j) sq[j] += ip[(size_t)i * area + j] * ip[(size_t)i * area + j];
    int head = size / 2;
    long tail = (long)head - (long)size;
    for (int i = 0; i < C; ++i, ++head, ++tail) {
      if (head < C)
        for (int j = 0; j < area; ++j) sq[j] += ip[(size_t)head * area + j] * ip[(size_t)head * area + j];
      if (tail >= 0)
        for (int j = 0; j < area; ++j) sq[j] -= ip[(size_t)tail * area + j] * ip[(size_t)tail * area + j];
      for (int j = 0; j < area; ++j)
        op[(size_t)i * area + j] = ip[(size_t)i * area + j] * powf(1.f + alpha_div_size * sq[j], -beta);
    }
  }
  free(sq);
}

/* mse::df, cross_entropy::df, cross_entropy_multiclass::df
 * (tiny_dnn/lossfunctions/loss_function.h:28-36,120-128,143-150) */
ORC_API void orc_loss_grad(int kind, const float *y, const float *t, float *dy, int dim, int B) {
  float factor = 2.0f / (float)dim;
  for (size_t i = 0; i < (size_t)dim * B; ++i) {
    if (kind == B200_LOSS_MSE)
      dy[i] = factor * (y[i] - t[i]);
    else if (kind == B200_LOSS_CROSS_ENTROPY)
      dy[i] = (y[i] - t[i]) / (y[i] * (1.f - y[i]));
    else
      dy[i] = -t[i] / y[i];
  }
}

/* sum over samples of E::f (loss_function.h:17-26,107-118,132-141) */
ORC_API float orc_loss_value(int kind, const float *y, const float *t, int dim, int B) {
  float total = 0.f;
  for (int n = 0; n < B; ++n) {
    float d = 0.f;
    for (int j = 0; j < dim; ++j) {
      float yi = y[(size_t)n * dim + j], ti = t[(size_t)n * dim + j];
      if (kind == B200_LOSS_MSE)
        d += (yi - ti) * (yi - ti);
      else if (kind == B200_LOSS_CROSS_ENTROPY)
        d += -ti * logf(yi) - (1.f - ti) * logf(1.f - yi);
      else
        d += -ti * logf(yi);
    }
    if (kind == B200_LOSS_MSE) d /= (float)dim;
    total += d;
  }
  return total;
}

/* ------------------------------------------------------------------------- */
/* merge + optimizers                                                          */
/* ------------------------------------------------------------------------- */

/* edge::merge_grads (tiny_dnn/node.h:89-103) */
ORC_API void orc_merge_grads(const float *grads, int rows, size_t len, float *dst) {
  memcpy(dst, grads, sizeof(float) * len);
  for (int r = 1; r < rows; ++r)
    for (size_t i = 0; i < len; ++i) dst[i] += grads[(size_t)r * len + i];
}

/* adagrad::update (optimizers/optimizer.h:60-66), adam::update (:112-127,
 * WITHOUT the trailing b1_t/b2_t advance, which the caller does),
 * momentum::update (:205-213) */
ORC_API void orc_opt_update(int kind, const b200_opt_hyper *h, const float *dW, float *W,
                            float *s0, float *s1, size_t len) {
  for (size_t i = 0; i < len; ++i) {
    if (kind == B200_OPT_ADAGRAD) {
      s0[i] += dW[i] * dW[i];
      W[i] -= h->alpha * dW[i] / (sqrtf(s0[i]) + h->eps);
    } else if (kind == B200_OPT_ADAM) {
      s0[i] = h->b1 * s0[i] + (1.f - h->b1) * dW[i];
      s1[i] = h->b2 * s1[i] + (1.f - h->b2) * dW[i] * dW[i];
      W[i] -= h->alpha * (s0[i] / (1.f - h->b1_t)) / sqrtf((s1[i] / (1.f - h->b2_t)) + h->eps);
    } else if (kind == B200_OPT_MOMENTUM) {
      float V = h->mu * s0[i] - h->alpha * (dW[i] + W[i] * h->lambda);
      W[i] += V;
      s0[i] = V;
    } else if (kind == B200_OPT_RMSPROP) { /* optimizer.h:82-89 */
      s0[i] = h->mu * s0[i] + (1 - h->mu) * dW[i] * dW[i];
      W[i] -= h->alpha * dW[i] / sqrtf(s0[i] + h->eps);
    } else if (kind == B200_OPT_ADAMAX) { /* optimizer.h:153-166; the literal 1.0 makes the step size a double */
      s0[i] = h->b1 * s0[i] + (1.f - h->b1) * dW[i];
      s1[i] = fmaxf(h->b2 * s1[i], fabsf(dW[i]));
      W[i] -= (h->alpha / (1.0 - h->b1_t)) * (s0[i] / (s1[i] + h->eps));
    } else if (kind == B200_OPT_GRADIENT_DESCENT) { /* optimizer.h:185-188 */
      W[i] = W[i] - h->alpha * (dW[i] + h->lambda * W[i]);
    } else { /* nesterov_momentum, optimizer.h:233-240 */
      float V = h->mu * s0[i] - h->alpha * (dW[i] + W[i] * h->lambda);
      W[i] += (-h->mu) * s0[i] + (1 + h->mu) * V;
      s0[i] = V;
    }
  }
}

/* ------------------------------------------------------------------------- */
/* quantization helpers (core/kernels/tiny_quantization_kernel.h)              */
/* ------------------------------------------------------------------------- */

/* float_to_quantized_unclamped<T> (:32-49); bits = 8 (uint8) or 32 (int32) */
ORC_API int64_t orc_f2q_unclamped(int bits, float input, float range_min, float range_max) {
  if (range_min == range_max) return 0;
  const int64_t number_of_steps = (int64_t)1 << bits;
  const double range_adjust = (number_of_steps / (number_of_steps - 1.0));
  const double range = ((range_max - range_min) * range_adjust);
  const double range_scale = (number_of_steps / range);
  int64_t quantized = (int64_t)(round(input * range_scale) - round(range_min * range_scale));
  const int64_t lowest_quantized = bits == 8 ? 0 : (int64_t)INT32_MIN;
  quantized += lowest_quantized;
  return quantized;
}

/* float_to_quantized<T> (:59-68) */
ORC_API int64_t orc_f2q(int bits, float input, float range_min, float range_max) {
  int64_t q = orc_f2q_unclamped(bits, input, range_min, range_max);
  const int64_t lo = bits == 8 ? 0 : (int64_t)INT32_MIN;
  const int64_t hi = bits == 8 ? 255 : (int64_t)INT32_MAX;
  if (q < lo) q = lo;
  if (q > hi) q = hi;
  return q;
}

/* quantized_to_float<T> (:70-84) */
ORC_API float orc_q2f(int bits, int64_t input, float range_min, float range_max) {
  if (range_min == range_max) return range_min;
  const int64_t number_of_steps = (int64_t)1 << bits;
  const double range_adjust = (number_of_steps / (number_of_steps - 1.0));
  const double range = ((range_max - range_min) * range_adjust);
  const double range_scale = (range / number_of_steps);
  const int64_t lowest_quantized = bits == 8 ? 0 : (int64_t)INT32_MIN;
  const double offset_input = (double)input - lowest_quantized;
  const double result = range_min + (offset_input * range_scale);
  return (float)result;
}

/* float_for_one_quantized_level<uint8_t> (:86-93) */
static float one_level_u8(float range_min, float range_max) {
  const int64_t highest_ = 255, lowest_ = 0;
  return (range_max - range_min) / (highest_ - lowest_);
}

/* quantization_range_for_multiplication<uint8,uint8,int32> (:95-114) */
ORC_API void orc_range_for_multiplication(float min_a, float max_a, float min_b, float max_b,
                                          float *min_c, float *max_c) {
  const float a = one_level_u8(min_a, max_a);
  const float b = one_level_u8(min_b, max_b);
  const int64_t c_highest = (int64_t)INT32_MAX, c_lowest = (int64_t)INT32_MIN;
  const float c = a * b;
  *min_c = c * c_lowest;
  *max_c = c * c_highest;
}

/* requantize_in_new_range<T1,T2> (:116-126): bits_in -> bits_out */
ORC_API int64_t orc_requantize_in_new_range(int bits_in, int bits_out, int64_t input, float min_in,
                                            float max_in, float min_new, float max_new) {
  const float f = orc_q2f(bits_in, input, min_in, max_in);
  return orc_f2q(bits_out, f, min_new, max_new);
}

/* requantize_many_in_new_range<int32_t, uint8_t> (:145-186) */
ORC_API void orc_requantize_many_i32_u8(const int32_t *input, size_t count, float min_input,
                                        float max_input, float min_output, float max_output,
                                        uint8_t *output) {
  const int fp_shift = 16;
  const float input_range = max_input - min_input;
  const float output_range = max_output - min_output;
  const float recip_output_range = (255.0f / output_range);
  const int64_t recip_output_range_fp = (int64_t)(recip_output_range * (1 << fp_shift));
  const int64_t range_scale_fp =
    (int64_t)(255.0f * (1 << fp_shift) * input_range / output_range);
  const int64_t input_offset_fp =
    (int64_t)((min_input * recip_output_range_fp) + (range_scale_fp >> 1));
  const int64_t output_offset_fp = (int64_t)(round((min_output * 255.0f) / output_range));
  const int64_t rounding_delta = 1 << (fp_shift - 1);
  for (size_t index = 0; index < count; ++index) {
    const int64_t input_value = (int64_t)input[index];
    const int64_t fp_value = ((input_value * range_scale_fp) >> 32) + input_offset_fp;
    const int64_t round_intermediate =
      ((fp_value >= 0) ? (fp_value + rounding_delta) : (fp_value - rounding_delta)) >> fp_shift;
    int64_t q = (round_intermediate - output_offset_fp);
    if (q < 0) q = 0;
    if (q > 255) q = 255;
    output[index] = (uint8_t)(int32_t)q;
  }
}

/* quantize_down_and_shrink_range<int32_t, uint8_t> (:230-254) */
ORC_API void orc_quantize_down_and_shrink_range(const int32_t *input, size_t count, float min_input,
                                                float max_input, float *min_new, float *max_new,
                                                uint8_t *output) {
  int32_t actual_min = INT32_MAX, actual_max = INT32_MIN;
  for (size_t i = 0; i < count; ++i) {
    if (input[i] < actual_min) actual_min = input[i];
    if (input[i] > actual_max) actual_max = input[i];
  }
  float mn = orc_q2f(32, actual_min, min_input, max_input);
  *min_new = 0.0f < mn ? 0.0f : mn; /* std::min(0.0f, mn) */
  if (!(mn < 0.0f)) *min_new = 0.0f;
  *max_new = orc_q2f(32, actual_max, min_input, max_input);
  orc_requantize_many_i32_u8(input, count, min_input, max_input, *min_new, *max_new, output);
}

/* tiny_quantized_conv2d_kernel for every sample
 * (core/kernels/tiny_quantized_conv2d_kernel.h:20-148, loop backend_tiny.h:107-110).
 * `in` has in_padded geometry.  Optional debug outputs (may be NULL): the uint8
 * input, the int32 accumulators. */
ORC_API int orc_qconv2d_fwd(const b200_conv_desc *p, const float *in, const float *W,
                            const float *bias, float *out, int B, uint8_t *dbg_in_q,
                            int32_t *dbg_acc) {
  size_t iw = p->inp_w, ih = p->inp_h, id = p->in_c;
  size_t ow = p->out_w, oh = p->out_h, od = p->out_c;
  size_t kw = p->k_w, kh = p->k_h;
  size_t in_len = iw * ih * id, out_len = ow * oh * od, lenW = kw * kh * id * od;
  /* the reference's range scans must stay inside the buffers */
  if ((id - 1) * iw * ih + ih * ih > in_len) return 1;
  if ((id - 1) * iw * ih + kh * kh > lenW) return 2;
  uint8_t *in_q = (uint8_t *)malloc(in_len);
  uint8_t *W_q = (uint8_t *)malloc(lenW);
  uint8_t *b_q = (uint8_t *)malloc(od ? od : 1);
  int32_t *a_q = (int32_t *)malloc(sizeof(int32_t) * out_len);
  uint8_t *a_rq = (uint8_t *)malloc(out_len);
  for (int n = 0; n < B; ++n) {
    const float *x = in + n * in_len;
    /* image quantization (:27-38) */
    float min_input = x[0], max_input = x[0];
    for (size_t inc = 0; inc < id; ++inc)
      for (size_t ins = 0; ins < ih * ih; ++ins) {
        float v = x[iw * ih * inc + ins];
        min_input = v < min_input ? v : min_input;
        max_input = max_input < v ? v : max_input;
      }
    for (size_t i = 0; i < in_len; ++i) in_q[i] = (uint8_t)orc_f2q(8, x[i], min_input, max_input);
    /* filter quantization (:40-55) */
    float min_filter = W[0], max_filter = W[0];
    for (size_t inc = 0; inc < id; ++inc)
      for (size_t ins = 0; ins < kh * kh; ++ins) {
        float v = W[iw * ih * inc + ins];
        min_filter = v < min_filter ? v : min_filter;
        max_filter = max_filter < v ? v : max_filter;
      }
    if (min_filter == max_filter) {
      max_filter = W[0] + 1e-3f;
      min_filter = W[0] - 1e-3f;
    }
    for (size_t i = 0; i < lenW; ++i) W_q[i] = (uint8_t)orc_f2q(8, W[i], min_filter, max_filter);
    /* bias quantization (:57-71) */
    float min_bias = 0.f, max_bias = 0.f;
    if (p->has_bias) {
      for (size_t o = 0; o < od; ++o) {
        min_bias = bias[o] < min_bias ? bias[o] : min_bias;
        max_bias = max_bias < bias[o] ? bias[o] : max_bias;
      }
      if (min_bias == max_bias) {
        max_bias = bias[0] + 1e-3f;
        min_bias = bias[0] - 1e-3f;
      }
      for (size_t o = 0; o < od; ++o) b_q[o] = (uint8_t)orc_f2q(8, bias[o], min_bias, max_bias);
    }
    /* output range and offsets (:73-87) */
    float min_output_value, max_output_value;
    orc_range_for_multiplication(min_input, max_input, min_filter, max_filter, &min_output_value,
                                 &max_output_value);
    const int32_t offset_input = (int32_t)orc_f2q_unclamped(8, 0.0f, min_input, max_input);
    const int32_t offset_filter = (int32_t)orc_f2q_unclamped(8, 0.0f, min_filter, max_filter);
    const int32_t zero_in_total_space =
      (int32_t)orc_f2q(32, 0.0f, min_output_value, max_output_value);
    memset(a_q, 0, sizeof(int32_t) * out_len);
    for (size_t o = 0; o < od; ++o) {
      for (size_t inc = 0; inc < id; ++inc) {
        if (!tbl_connected(p, (int)o, (int)inc)) continue;
        const uint8_t *pw = W_q + kw * kh * (id * o + inc);
        const uint8_t *pi = in_q + iw * ih * inc;
        int32_t *pa = a_q + ow * oh * o;
        for (size_t y = 0; y < oh; ++y)
          for (size_t xx = 0; xx < ow; ++xx) {
            const uint8_t *ppw = pw;
            const uint8_t *ppi = pi + iw * (y * p->stride_h) + xx * p->stride_w;
            int32_t sum = 0;
            for (size_t wy = 0; wy < kh; ++wy)
              for (size_t wx = 0; wx < kw; ++wx)
                sum += ((int32_t)(*ppw++) - offset_filter) *
                       ((int32_t)ppi[wy * iw + wx] - offset_input);
            pa[y * ow + xx] += sum;
          }
      }
      if (p->has_bias) {
        int32_t *pa = a_q + ow * oh * o;
        for (size_t i = 0; i < ow * oh; ++i) pa[i] += (b_q[o] - zero_in_total_space);
      }
    }
    if (dbg_in_q) memcpy(dbg_in_q + n * in_len, in_q, in_len);
    if (dbg_acc) memcpy(dbg_acc + n * out_len, a_q, sizeof(int32_t) * out_len);
    /* requantize and dequantize (:135-147) */
    float min_rq, max_rq;
    orc_quantize_down_and_shrink_range(a_q, out_len, min_output_value, max_output_value, &min_rq,
                                       &max_rq, a_rq);
    for (size_t i = 0; i < out_len; ++i) out[n * out_len + i] = orc_q2f(8, a_rq[i], min_rq, max_rq);
  }
  free(in_q);
  free(W_q);
  free(b_q);
  free(a_q);
  free(a_rq);
  return 0;
}

/* tiny_quantized_fully_connected_kernel for every sample
 * (core/kernels/tiny_quantized_fully_connected_kernel.h:22-128, loop
 * backend_tiny.h:306-311).  bias may be NULL (has_bias_ false). */
ORC_API int orc_qfc_fwd(int in_size, int out_size, const float *in, const float *W,
                        const float *bias, float *out, int B) {
  size_t lenW = (size_t)in_size * out_size;
  uint8_t *in_q = (uint8_t *)malloc(in_size);
  uint8_t *W_q = (uint8_t *)malloc(lenW);
  uint8_t *b_q = (uint8_t *)malloc(out_size);
  int32_t *o_q = (int32_t *)malloc(sizeof(int32_t) * out_size);
  uint8_t *o_rq = (uint8_t *)malloc(out_size);
  for (int n = 0; n < B; ++n) {
    const float *x = in + (size_t)n * in_size;
    float min_input = x[0], max_input = x[0];
    for (int c = 0; c < in_size; ++c) {
      min_input = x[c] < min_input ? x[c] : min_input;
      max_input = max_input < x[c] ? x[c] : max_input;
    }
    for (int c = 0; c < in_size; ++c) in_q[c] = (uint8_t)orc_f2q(8, x[c], min_input, max_input);
    float min_filter = W[0], max_filter = W[0];
    for (size_t c = 0; c < lenW; ++c) {
      min_filter = W[c] < min_filter ? W[c] : min_filter;
      max_filter = max_filter < W[c] ? W[c] : max_filter;
    }
    if (min_filter == max_filter) {
      max_filter = W[0] + 1e-3f;
      min_filter = W[0] - 1e-3f;
    }
    for (size_t c = 0; c < lenW; ++c) W_q[c] = (uint8_t)orc_f2q(8, W[c], min_filter, max_filter);
    float min_output_value, max_output_value;
    orc_range_for_multiplication(min_input, max_input, min_filter, max_filter, &min_output_value,
                                 &max_output_value);
    float min_bias = 0.f, max_bias = 0.f;
    if (bias) {
      for (int i = 0; i < out_size; ++i) {
        min_bias = bias[i] < min_bias ? bias[i] : min_bias;
        max_bias = max_bias < bias[i] ? bias[i] : max_bias;
      }
      if (min_bias == max_bias) {
        max_bias = bias[0] + 1e-3f;
        min_bias = bias[0] - 1e-3f;
      }
      for (int i = 0; i < out_size; ++i) b_q[i] = (uint8_t)orc_f2q(8, bias[i], min_bias, max_bias);
    }
    min_output_value += min_bias;
    max_output_value += max_bias;
    const int32_t offset_input = (int32_t)orc_f2q_unclamped(8, 0.0f, min_input, max_input);
    const int32_t offset_filter = (int32_t)orc_f2q_unclamped(8, 0.0f, min_filter, max_filter);
    const int32_t zero_in_total_space =
      (int32_t)orc_f2q(32, 0.0f, min_output_value, max_output_value);
    for (int i = 0; i < out_size; ++i) {
      o_q[i] = 0;
      for (int c = 0; c < in_size; ++c)
        o_q[i] += (int32_t)(W_q[(size_t)c * out_size + i] - offset_filter) *
                  (int32_t)(in_q[c] - offset_input);
      if (bias) o_q[i] += (b_q[i] - zero_in_total_space);
    }
    float min_rq, max_rq;
    orc_quantize_down_and_shrink_range(o_q, out_size, min_output_value, max_output_value, &min_rq,
                                       &max_rq, o_rq);
    for (int i = 0; i < out_size; ++i)
      out[(size_t)n * out_size + i] = orc_q2f(8, o_rq[i], min_rq, max_rq);
  }
  free(in_q);
  free(W_q);
  free(b_q);
  free(o_q);
  free(o_rq);
  return 0;
}

/* The "efficient" forms for chained quantized layers: operands arrive as uint8 values held in
   floats with their ranges, results leave the same way (no quantize at the input, no dequantize at
   the output).  tiny_quantized_conv2d_kernel, nine-argument overload
   (tiny_quantized_conv2d_kernel.h:353-466), per sample as tiny_backend::conv2d_eq calls it
   (backend_tiny.h:115-135): in [B][in_len] (padded), in_r [B][2], W_r / b_r [2], out [B][out_len],
   out_r [B][2]. */
ORC_API int orc_qconv2d_eq_fwd(const b200_conv_desc *p, const float *in, const float *W, const float *bias,
                               const float *in_r, const float *W_r, const float *b_r, float *out, float *out_r,
                               int B) {
  (void)b_r; /* the kernel takes the bias range and never reads it */
  size_t iw = p->inp_w, ih = p->inp_h, id = p->in_c;
  size_t ow = p->out_w, oh = p->out_h, od = p->out_c;
  size_t kw = p->k_w, kh = p->k_h;
  size_t in_len = iw * ih * id, out_len = ow * oh * od, lenW = kw * kh * id * od;
  uint8_t *in_q = (uint8_t *)malloc(in_len);
  uint8_t *W_q = (uint8_t *)malloc(lenW);
  int32_t *a_q = (int32_t *)malloc(sizeof(int32_t) * out_len);
  uint8_t *a_rq = (uint8_t *)malloc(out_len);
  for (size_t i = 0; i < lenW; ++i) W_q[i] = (uint8_t)W[i];
  for (int n = 0; n < B; ++n) {
    const float *x = in + n * in_len;
    float min_filter = W_r[0], max_filter = W_r[1];
    if (W_r[0] == W_r[1]) {
      max_filter = W_r[1] + 1e-3f;
      min_filter = W_r[0] - 1e-3f;
    }
    const float min_input = in_r[2 * n], max_input = in_r[2 * n + 1];
    float min_output_value, max_output_value;
    orc_range_for_multiplication(min_input, max_input, min_filter, max_filter, &min_output_value,
                                 &max_output_value);
    for (size_t i = 0; i < in_len; ++i) in_q[i] = (uint8_t)x[i];
    const int32_t offset_input = (int32_t)orc_f2q_unclamped(8, 0.0f, min_input, max_input);
    const int32_t offset_filter = (int32_t)orc_f2q_unclamped(8, 0.0f, min_filter, max_filter);
    const int32_t zero_in_total_space = (int32_t)orc_f2q(32, 0.0f, min_output_value, max_output_value);
    memset(a_q, 0, sizeof(int32_t) * out_len);
    for (size_t o = 0; o < od; ++o) {
      for (size_t inc = 0; inc < id; ++inc) {
        if (!tbl_connected(p, (int)o, (int)inc)) continue;
        const uint8_t *pw = W_q + kw * kh * (id * o + inc);
        const uint8_t *pi = in_q + iw * ih * inc;
        int32_t *pa = a_q + ow * oh * o;
        for (size_t y = 0; y < oh; ++y)
          for (size_t xx = 0; xx < ow; ++xx) {
            const uint8_t *ppw = pw;
            const uint8_t *ppi = pi + iw * (y * p->stride_h) + xx * p->stride_w;
            int32_t sum = 0;
            for (size_t wy = 0; wy < kh; ++wy)
              for (size_t wx = 0; wx < kw; ++wx)
                sum += ((int32_t)(*ppw++) - offset_filter) * ((int32_t)ppi[wy * iw + wx] - offset_input);
            pa[y * ow + xx] += sum;
          }
      }
      if (p->has_bias) {
        /* `bias[o] - zero_in_total_space`: the FLOAT bias entry minus the int, formed in float, then
           cast to int32 (:436-441) -- not the integer form of the plain kernel */
        int32_t *pa = a_q + ow * oh * o;
        const int32_t add = (int32_t)(bias[o] - (float)zero_in_total_space);
        for (size_t i = 0; i < ow * oh; ++i) pa[i] += add;
      }
    }
    float min_rq, max_rq;
    orc_quantize_down_and_shrink_range(a_q, out_len, min_output_value, max_output_value, &min_rq, &max_rq, a_rq);
    for (size_t i = 0; i < out_len; ++i) out[n * out_len + i] = (float)a_rq[i];
    out_r[2 * n] = min_rq;
    out_r[2 * n + 1] = max_rq;
  }
  free(in_q);
  free(W_q);
  free(a_q);
  free(a_rq);
  return 0;
}

/* tiny_quantized_fully_connected_kernel, eleven-argument overload
   (tiny_quantized_fully_connected_kernel.h:269-370), per sample as tiny_backend::fully_eq would
   (backend_tiny.h:321-345) */
ORC_API int orc_qfc_eq_fwd(int in_size, int out_size, const float *in, const float *W, const float *bias,
                           const float *in_r, const float *W_r, const float *b_r, float *out, float *out_r, int B) {
  const int has_bias = bias != NULL;
  uint8_t *in_q = (uint8_t *)malloc(in_size ? in_size : 1);
  uint8_t *W_q = (uint8_t *)malloc((size_t)in_size * out_size + 1);
  uint8_t *b_q = (uint8_t *)malloc(out_size ? out_size : 1);
  int32_t *o_q = (int32_t *)malloc(sizeof(int32_t) * (out_size ? out_size : 1));
  uint8_t *o_rq = (uint8_t *)malloc(out_size ? out_size : 1);
  for (size_t i = 0; i < (size_t)in_size * out_size; ++i) W_q[i] = (uint8_t)W[i];
  if (has_bias)
    for (int i = 0; i < out_size; ++i) b_q[i] = (uint8_t)bias[i];
  for (int n = 0; n < B; ++n) {
    const float *x = in + (size_t)n * in_size;
    float min_filter = W_r[0], max_filter = W_r[1];
    if (min_filter == max_filter) {
      max_filter = W_r[1] + 1e-3f;
      min_filter = W_r[0] - 1e-3f;
    }
    float min_bias = b_r[0], max_bias = b_r[1];
    if (has_bias && min_bias == max_bias) {
      max_bias = b_r[1] + 1e-3f;
      min_bias = b_r[0] - 1e-3f;
    }
    const float min_input = in_r[2 * n], max_input = in_r[2 * n + 1];
    float min_output_value, max_output_value;
    orc_range_for_multiplication(min_input, max_input, min_filter, max_filter, &min_output_value,
                                 &max_output_value);
    for (int i = 0; i < in_size; ++i) in_q[i] = (uint8_t)x[i];
    min_output_value += min_bias;
    max_output_value += max_bias;
    const int32_t offset_input = (int32_t)orc_f2q_unclamped(8, 0.0f, min_input, max_input);
    const int32_t offset_filter = (int32_t)orc_f2q_unclamped(8, 0.0f, min_filter, max_filter);
    const int32_t zero_in_total_space = (int32_t)orc_f2q(32, 0.0f, min_output_value, max_output_value);
    for (int i = 0; i < out_size; ++i) {
      int32_t acc = 0;
      for (int c = 0; c < in_size; ++c)
        acc += ((int32_t)W_q[(size_t)c * out_size + i] - offset_filter) * ((int32_t)in_q[c] - offset_input);
      if (has_bias) acc += (b_q[i] - zero_in_total_space);
      o_q[i] = acc;
    }
    float min_rq, max_rq;
    orc_quantize_down_and_shrink_range(o_q, out_size, min_output_value, max_output_value, &min_rq, &max_rq, o_rq);
    for (int i = 0; i < out_size; ++i) out[(size_t)n * out_size + i] = (float)o_rq[i];
    out_r[2 * n] = min_rq;
    out_r[2 * n + 1] = max_rq;
  }
  free(in_q);
  free(W_q);
  free(b_q);
  free(o_q);
  free(o_rq);
  return 0;
}

/* ------------------------------------------------------------------------- */
/* one training step of a sequential network                                   */
/* ------------------------------------------------------------------------- */

typedef struct {
  b200_layer_spec s;
  size_t in_dim, out_dim, w_off, w_len, b_off, b_len;
  float *out, *grad;   /* [B][out_dim] */
  float *padded, *padded_grad; /* conv: padded input / padded prev_delta */
  int32_t *argmax;
  /* batch normalization: this batch's moments, stddev_, the moving averages (5 x channels floats) */
  float *bn_mean_cur, *bn_var_cur, *bn_stddev, *bn_mean, *bn_var;
} orc_layer;

typedef struct orc_net {
  int n_layers, max_batch;
  orc_layer *L;
  size_t n_params;
  int n_tensors;
  size_t *t_off, *t_len;
  float *params, *grads, *s0, *s1, *in_grad;
  float b1_t, b2_t; /* adam powers, advanced once per update call */
  int powers_init;
  int test_phase;   /* net_phase::test: batch normalization reads its moving averages */
} orc_net;

static size_t layer_dims(const b200_layer_spec *s, size_t prev, size_t *in_dim, size_t *w_len,
                         size_t *b_len) {
  *w_len = *b_len = 0;
  switch (s->kind) {
    case B200_LAYER_CONV:
      *in_dim = (size_t)s->conv.in_c * s->conv.in_h * s->conv.in_w;
      *w_len = (size_t)s->conv.out_c * s->conv.in_c * s->conv.k_h * s->conv.k_w;
      *b_len = s->conv.has_bias ? s->conv.out_c : 0;
      return (size_t)s->conv.out_c * s->conv.out_h * s->conv.out_w;
    case B200_LAYER_FC:
      *in_dim = s->fc_in;
      *w_len = (size_t)s->fc_in * s->fc_out;
      *b_len = s->fc_has_bias ? s->fc_out : 0;
      return s->fc_out;
    case B200_LAYER_MAXPOOL:
    case B200_LAYER_AVGPOOL:
      *in_dim = (size_t)s->pool.in_c * s->pool.in_h * s->pool.in_w;
      if (s->kind == B200_LAYER_AVGPOOL) {
        *w_len = (size_t)s->pool.pool_w * s->pool.pool_h * s->pool.in_c;
        *b_len = s->pool.in_c;
      }
      return (size_t)s->pool.in_c * s->pool.out_h * s->pool.out_w;
    case B200_LAYER_BATCHNORM:
      *in_dim = (size_t)s->bn_channels * s->bn_spatial;
      return *in_dim;
    default: *in_dim = prev; return prev;
  }
}

ORC_API orc_net *orc_net_create(const b200_layer_spec *specs, int n_layers, int max_batch) {
  orc_net *net = (orc_net *)calloc(1, sizeof(orc_net));
  net->n_layers = n_layers;
  net->max_batch = max_batch;
  net->L = (orc_layer *)calloc(n_layers, sizeof(orc_layer));
  net->t_off = (size_t *)calloc(2 * n_layers, sizeof(size_t));
  net->t_len = (size_t *)calloc(2 * n_layers, sizeof(size_t));
  size_t off = 0, prev = 0;
  for (int i = 0; i < n_layers; ++i) {
    orc_layer *L = &net->L[i];
    L->s = specs[i];
    L->out_dim = layer_dims(&specs[i], prev, &L->in_dim, &L->w_len, &L->b_len);
    if (i > 0 && L->in_dim != prev) return NULL;
    prev = L->out_dim;
    if (L->w_len) {
      L->w_off = off;
      net->t_off[net->n_tensors] = off;
      net->t_len[net->n_tensors++] = L->w_len;
      off += L->w_len;
    }
    if (L->b_len) {
      L->b_off = off;
      net->t_off[net->n_tensors] = off;
      net->t_len[net->n_tensors++] = L->b_len;
      off += L->b_len;
    }
    L->out = (float *)calloc(L->out_dim * max_batch, sizeof(float));
    L->grad = (float *)calloc(L->out_dim * max_batch, sizeof(float));
    if (specs[i].kind == B200_LAYER_CONV) {
      size_t pl = (size_t)specs[i].conv.in_c * specs[i].conv.inp_h * specs[i].conv.inp_w;
      L->padded = (float *)calloc(pl * max_batch, sizeof(float));
      L->padded_grad = (float *)calloc(pl * max_batch, sizeof(float));
    }
    if (specs[i].kind == B200_LAYER_MAXPOOL)
      L->argmax = (int32_t *)calloc(L->out_dim * max_batch, sizeof(int32_t));
    if (specs[i].kind == B200_LAYER_BATCHNORM) {
      const size_t c = specs[i].bn_channels;
      L->bn_mean_cur = (float *)calloc(5 * c, sizeof(float));  /* init(): zeros */
      L->bn_var_cur = L->bn_mean_cur + c;
      L->bn_stddev = L->bn_mean_cur + 2 * c;
      L->bn_mean = L->bn_mean_cur + 3 * c;
      L->bn_var = L->bn_mean_cur + 4 * c;
    }
  }
  net->n_params = off;
  net->params = (float *)calloc(off ? off : 1, sizeof(float));
  net->grads = (float *)calloc(off ? off : 1, sizeof(float));
  net->s0 = (float *)calloc(off ? off : 1, sizeof(float));
  net->s1 = (float *)calloc(off ? off : 1, sizeof(float));
  net->in_grad = (float *)calloc(net->L[0].in_dim * max_batch, sizeof(float));
  return net;
}

ORC_API void orc_net_destroy(orc_net *net) {
  if (!net) return;
  for (int i = 0; i < net->n_layers; ++i) {
    free(net->L[i].out);
    free(net->L[i].grad);
    free(net->L[i].padded);
    free(net->L[i].padded_grad);
    free(net->L[i].argmax);
    free(net->L[i].bn_mean_cur);
  }
  free(net->L);
  free(net->t_off);
  free(net->t_len);
  free(net->params);
  free(net->grads);
  free(net->s0);
  free(net->s1);
  free(net->in_grad);
  free(net);
}

ORC_API size_t orc_net_param_count(const orc_net *net) { return net->n_params; }
ORC_API float *orc_net_params(orc_net *net) { return net->params; }
ORC_API float *orc_net_grads(orc_net *net) { return net->grads; }
ORC_API float *orc_net_output(orc_net *net) { return net->L[net->n_layers - 1].out; }
ORC_API float *orc_net_layer_out(orc_net *net, int i) { return net->L[i].out; }
ORC_API float *orc_net_layer_grad(orc_net *net, int i) { return i < 0 ? net->in_grad : net->L[i].grad; }
/* network::set_netphase (network.h:438-442) */
ORC_API void orc_net_set_phase(orc_net *net, int train) { net->test_phase = !train; }
/* moving averages of batch normalization layer i: mean_ then variance_ */
ORC_API float *orc_net_bn_mean(orc_net *net, int i) { return net->L[i].bn_mean; }
ORC_API float *orc_net_bn_var(orc_net *net, int i) { return net->L[i].bn_var; }

static int act_kind(int layer_kind) {
  return layer_kind == B200_LAYER_RELU         ? B200_ACT_RELU
         : layer_kind == B200_LAYER_TANH       ? B200_ACT_TANH
         : layer_kind == B200_LAYER_SIGMOID    ? B200_ACT_SIGMOID
         : layer_kind == B200_LAYER_LEAKY_RELU ? B200_ACT_LEAKY_RELU
         : layer_kind == B200_LAYER_ELU        ? B200_ACT_ELU
                                               : B200_ACT_SOFTMAX;
}

/* sequential::forward (tiny_dnn/nodes.h:288-303) */
ORC_API void orc_net_forward(orc_net *net, const float *x, int B) {
  const float *in = x;
  for (int i = 0; i < net->n_layers; ++i) {
    orc_layer *L = &net->L[i];
    const float *W = net->params + L->w_off;
    const float *b = L->b_len ? net->params + L->b_off : NULL;
    switch (L->s.kind) {
      case B200_LAYER_CONV:
        orc_conv_pad(&L->s.conv, in, L->padded, B);
        orc_conv2d_fwd(&L->s.conv, L->padded, W, b, L->out, B);
        break;
      case B200_LAYER_FC: orc_fc_fwd(L->s.fc_in, L->s.fc_out, in, W, b, L->out, B); break;
      case B200_LAYER_MAXPOOL: orc_maxpool_fwd(&L->s.pool, in, L->out, L->argmax, B); break;
      case B200_LAYER_AVGPOOL: orc_avgpool_fwd(&L->s.pool, in, W, b, L->out, B); break;
      case B200_LAYER_BATCHNORM:
        orc_batchnorm_fwd(L->s.bn_channels, L->s.bn_spatial, L->s.bn_eps, in,
                          net->test_phase ? L->bn_mean : L->bn_mean_cur, net->test_phase ? L->bn_var : L->bn_var_cur,
                          L->bn_stddev, L->out, B, !net->test_phase);
        break;
      default: orc_act_param_fwd(act_kind(L->s.kind), L->s.act_param, in, L->out, (int)L->out_dim, B); break;
    }
    in = L->out;
  }
}

/* gradient<E> + sequential::backward (loss_function.h:190-218, nodes.h:276-286)
 * + the merge_grads of layer::update_weight; leaves the batch-summed gradient
 * of every parameter in the flat gradient buffer. */
ORC_API void orc_net_backward(orc_net *net, const float *x, const float *t, int loss_kind, int B) {
  int n = net->n_layers;
  orc_layer *last = &net->L[n - 1];
  orc_loss_grad(loss_kind, last->out, t, last->grad, (int)last->out_dim, B);
  memset(net->grads, 0, sizeof(float) * net->n_params);
  for (int i = n - 1; i >= 0; --i) {
    orc_layer *L = &net->L[i];
    const float *in = i == 0 ? x : net->L[i - 1].out;
    float *din = i == 0 ? net->in_grad : net->L[i - 1].grad;
    const float *W = net->params + L->w_off;
    float *dW = net->grads + L->w_off;
    float *db = L->b_len ? net->grads + L->b_off : NULL;
    switch (L->s.kind) {
      case B200_LAYER_CONV:
        orc_conv2d_bwd(&L->s.conv, L->padded, W, L->grad, L->padded_grad, dW, db, 0, B);
        orc_conv_unpad(&L->s.conv, L->padded_grad, din, B);
        break;
      case B200_LAYER_FC:
        orc_fc_bwd(L->s.fc_in, L->s.fc_out, in, W, L->grad, din, dW, db, 0, B);
        break;
      case B200_LAYER_MAXPOOL: orc_maxpool_bwd(&L->s.pool, L->grad, L->argmax, din, B); break;
      case B200_LAYER_AVGPOOL:
        orc_avgpool_bwd(&L->s.pool, in, W, L->grad, din, dW, db, 0, B);
        break;
      case B200_LAYER_BATCHNORM:
        orc_batchnorm_bwd(L->s.bn_channels, L->s.bn_spatial, L->out, L->grad, L->bn_stddev, din, B);
        break;
      default: orc_act_param_bwd(act_kind(L->s.kind), L->s.act_param, L->out, L->grad, din, (int)L->out_dim, B); break;
    }
  }
}

/* nodes::update_weights -> layer::update_weight (nodes.h:103-107,
 * layer.h:663-682): one optimizer::update per trainable tensor in network
 * order; adam's powers advance after every call (optimizer.h:125-126). */
ORC_API void orc_net_update(orc_net *net, int opt_kind, const b200_opt_hyper *h) {
  b200_opt_hyper hh = *h;
  if ((opt_kind == B200_OPT_ADAM || opt_kind == B200_OPT_ADAMAX) && !net->powers_init) {
    net->b1_t = h->b1;
    net->b2_t = h->b2;
    net->powers_init = 1;
  }
  for (int k = 0; k < net->n_tensors; ++k) {
    hh.b1_t = net->b1_t;
    hh.b2_t = net->b2_t;
    orc_opt_update(opt_kind, &hh, net->grads + net->t_off[k], net->params + net->t_off[k],
                   net->s0 + net->t_off[k], net->s1 + net->t_off[k], net->t_len[k]);
    if (opt_kind == B200_OPT_ADAM || opt_kind == B200_OPT_ADAMAX) {
      net->b1_t *= h->b1;
      net->b2_t *= h->b2; /* adamax has no b2_t; the value is unused there */
    }
  }
  /* layer::update_weight ends with post_update() (layer.h:681) */
  for (int i = 0; i < net->n_layers; ++i) {
    orc_layer *L = &net->L[i];
    if (L->s.kind == B200_LAYER_BATCHNORM)
      orc_batchnorm_post_update(L->s.bn_channels, L->s.bn_momentum, L->bn_mean, L->bn_var, L->bn_mean_cur,
                                L->bn_var_cur);
  }
}

/* network::fit (tiny_dnn/network.h:840-926) for `epochs` passes over n samples: the loop over
 * mini-batches with the reference's batch buffers.  in_batch_ / t_batch_ are sized to the
 * mini-batch once (:858-859); train_onebatch copies the step's `size` samples over their first
 * rows and runs fprop / bprop on the whole buffers (:918-924), so a last mini-batch of
 * 1 < size < batch samples is a full step whose remaining rows are the previous step's; a single
 * left-over sample takes train_once's one-sample branch (:893-895). */
ORC_API void orc_net_train_step(orc_net *net, const float *x, const float *t, int B, int loss_kind,
                                int opt_kind, const b200_opt_hyper *h);

ORC_API int orc_net_fit(orc_net *net, const float *x, const float *t, long long n, int batch, int epochs,
                        int loss_kind, int opt_kind, const b200_opt_hyper *h) {
  const size_t in_dim = net->L[0].in_dim, out_dim = net->L[net->n_layers - 1].out_dim;
  if (batch < 1 || batch > net->max_batch) return 1;
  float *xb = (float *)calloc((size_t)batch * in_dim, sizeof(float));
  float *tb = (float *)calloc((size_t)batch * out_dim, sizeof(float));
  for (int e = 0; e < epochs; ++e)
    for (long long i = 0; i < n; i += batch) {
      const int size = (int)((n - i) < batch ? (n - i) : batch);
      if (size == 1) {
        orc_net_train_step(net, x + (size_t)i * in_dim, t + (size_t)i * out_dim, 1, loss_kind, opt_kind, h);
      } else {
        memcpy(xb, x + (size_t)i * in_dim, (size_t)size * in_dim * sizeof(float));
        memcpy(tb, t + (size_t)i * out_dim, (size_t)size * out_dim * sizeof(float));
        orc_net_train_step(net, xb, tb, batch, loss_kind, opt_kind, h);
      }
    }
  free(xb);
  free(tb);
  return 0;
}

/* ---- the callers' data formats ------------------------------------------------------------- */
/* parse_cifar10 (tiny_dnn/io/cifar10_parser.h:47-85, mode 0) and detail::parse_mnist_image
 * (tiny_dnn/io/mnist_parser.h:43-68, mode 1): n planar uint8 images [c][h][w] -> float rows
 * [c][h + 2*y_pad][w + 2*x_pad], border filled with scale_min. */
ORC_API void orc_images_u8_to_float(const b200_image_desc *d, const uint8_t *src, long long n, float *dst) {
  const int W = d->width, H = d->height, Wo = W + 2 * d->x_padding, Ho = H + 2 * d->y_padding;
  const float smin = d->scale_min, smax = d->scale_max;
  for (long long p = 0; p < n * d->channels; ++p) {
    float *o = dst + (size_t)p * Wo * Ho;
    for (int i = 0; i < Wo * Ho; ++i) o[i] = smin;
    for (int y = 0; y < H; ++y)
      for (int x = 0; x < W; ++x) {
        const uint8_t c = src[(size_t)p * W * H + (size_t)y * W + x];
        float v;
        if (d->mode == B200_IMAGE_CIFAR10)
          v = smin + (smax - smin) * c / 255;
        else
          v = (c / 255.0f) * (smax - smin) + smin;
        o[(size_t)(y + d->y_padding) * Wo + x + d->x_padding] = v;
      }
  }
}

/* nodes::label2vec (tiny_dnn/nodes.h:180-189) */
ORC_API void orc_labels_to_targets(const uint8_t *labels, long long n, int out_dim, float tmin, float tmax,
                                   float *dst) {
  for (long long s = 0; s < n; ++s) {
    for (int j = 0; j < out_dim; ++j) dst[s * out_dim + j] = tmin;
    dst[s * out_dim + labels[s]] = tmax;
  }
}

/* network::fit calls optimizer.reset() (network.h:856): stateful_optimizer::reset clears the
 * per-weight state (optimizer.h:36-38) but adam's powers b1_t / b2_t carry on.  `keep_powers` = 0
 * also restarts the powers (a new optimizer object). */
ORC_API void orc_net_opt_reset(orc_net *net, int keep_powers) {
  memset(net->s0, 0, net->n_params * sizeof(float));
  memset(net->s1, 0, net->n_params * sizeof(float));
  if (!keep_powers) net->powers_init = 0;
}

ORC_API void orc_net_adam_powers(const orc_net *net, float *b1_t, float *b2_t) {
  *b1_t = net->b1_t;
  *b2_t = net->b2_t;
}

/* network::train_onebatch (tiny_dnn/network.h:911-926) */
ORC_API void orc_net_train_step(orc_net *net, const float *x, const float *t, int B, int loss_kind,
                                int opt_kind, const b200_opt_hyper *h) {
  orc_net_forward(net, x, B);
  orc_net_backward(net, x, t, loss_kind, B);
  orc_net_update(net, opt_kind, h);
}
