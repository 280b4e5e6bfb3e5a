// uint8 quantized convolution and fully-connected forward, bit-exact with the
// reference's per-sample pipeline
//   tiny_quantized_conv2d_kernel          (core/kernels/tiny_quantized_conv2d_kernel.h:20-148)
//   tiny_quantized_fully_connected_kernel (core/kernels/tiny_quantized_fully_connected_kernel.h:22-128)
// built on the scalar helpers of core/kernels/tiny_quantization_kernel.h.
//
// Every float / double expression below is written with explicit
// round-to-nearest intrinsics in the operand order of the reference so that no
// multiply-add contraction or reassociation can change a bit; this file is also
// compiled with -fmad=false.
//
// Pipeline (all samples of the batch at once):
//   1. per-sample min/max of the input            (conv :27-36, fc :30-35)
//   2. min/max of the filter subset the reference scans, and of the bias
//      (conv :40-71, fc :38-67) -- sample independent, done once
//   3. quantize input, filter, bias to uint8      (float_to_quantized, :59-68)
//   4. per-sample output range, offsets, zero point (conv :73-87, fc :49-81)
//   5. int32 accumulate of (w - off_w)*(x - off_x) + (bias_q - zero)
//   6. per-sample min/max of the accumulators, shrink range, fixed-point
//      requantize to uint8, dequantize to float   (:140-147; kernel.h:145-186,230-254)
#include <limits.h>

#include "common.cuh"
#include "device_utils.cuh"

namespace b200 {

// ---- scalar helpers (tiny_quantization_kernel.h) ---------------------------

// float_to_quantized_unclamped<T> (:32-49); BITS = 8 (uint8, lowest 0) or 32
// (int32, lowest -2^31)
template <int BITS>
__device__ __forceinline__ long long f2q_unclamped(float input, float rmin, float rmax) {
  if (rmin == rmax) return 0;
  const long long steps = 1LL << BITS;
  const double range_adjust = __ddiv_rn((double)steps, __dsub_rn((double)steps, 1.0));
  const double range = __dmul_rn((double)__fsub_rn(rmax, rmin), range_adjust);
  const double range_scale = __ddiv_rn((double)steps, range);
  long long q = (long long)__dsub_rn(round(__dmul_rn((double)input, range_scale)),
                                     round(__dmul_rn((double)rmin, range_scale)));
  const long long lowest = BITS == 8 ? 0LL : -(1LL << 31);
  return q + lowest;
}

// float_to_quantized<T> (:59-68)
template <int BITS>
__device__ __forceinline__ long long f2q(float input, float rmin, float rmax) {
  long long q = f2q_unclamped<BITS>(input, rmin, rmax);
  const long long lowest = BITS == 8 ? 0LL : -(1LL << 31);
  const long long highest = BITS == 8 ? 255LL : (1LL << 31) - 1;
  q = q > lowest ? q : lowest;
  q = q < highest ? q : highest;
  return q;
}

// quantized_to_float<T> (:70-84)
template <int BITS>
__device__ __forceinline__ float q2f(long long input, float rmin, float rmax) {
  if (rmin == rmax) return rmin;
  const long long steps = 1LL << BITS;
  const double range_adjust = __ddiv_rn((double)steps, __dsub_rn((double)steps, 1.0));
  const double range = __dmul_rn((double)__fsub_rn(rmax, rmin), range_adjust);
  const double range_scale = __ddiv_rn(range, (double)steps);
  const long long lowest = BITS == 8 ? 0LL : -(1LL << 31);
  const double offset_input = __dsub_rn((double)input, (double)lowest);
  const double result = __dadd_rn((double)rmin, __dmul_rn(offset_input, range_scale));
  return (float)result;
}

// float_for_one_quantized_level<uint8_t> (:86-93)
__device__ __forceinline__ float one_level_u8(float rmin, float rmax) {
  return __fdiv_rn(__fsub_rn(rmax, rmin), 255.0f);
}

struct QSample {
  float min_in, max_in;    // input range
  float min_out, max_out;  // int32 accumulator range
  int off_in;              // quantized 0.0 of the input
  int zero_total;          // quantized 0.0 of the accumulator space
  int acc_min, acc_max;    // observed accumulator extremes
  // requantize_many_in_new_range<int32,uint8> constants (:159-171)
  long long range_scale_fp, input_offset_fp, output_offset_fp;
  float min_new, max_new;  // shrunk output range
};

struct QGlobal {
  float min_f, max_f;
  float min_b, max_b;
  int off_f;
};

// ---- 1. per-sample input range ----------------------------------------------

// One block per sample.  The scanned region is `nseg` segments of `seg_len`
// elements starting every `seg_stride` elements: the conv kernel scans
// in_padded.height^2 elements per channel plane (:29-35), the fc kernel scans
// the whole row.  Both seed the range with element 0.
__global__ void q_input_range_kernel(const float *__restrict__ in, size_t row_len, int nseg,
                                     size_t seg_stride, size_t seg_len, QSample *qs) {
  const float *r = in + (size_t)blockIdx.x * row_len;
  float mn = r[0], mx = r[0];
  size_t total = (size_t)nseg * seg_len;
  for (size_t t = threadIdx.x; t < total; t += blockDim.x) {
    size_t s = t / seg_len, e = t - s * seg_len;
    float v = r[s * seg_stride + e];
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
  __shared__ float smn[32], smx[32];
  mn = warp_min(mn);
  mx = warp_max(mx);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) {
    smn[wid] = mn;
    smx[wid] = mx;
  }
  __syncthreads();
  if (wid == 0) {
    int nw = blockDim.x >> 5;
    mn = lane < nw ? smn[lane] : smn[0];
    mx = lane < nw ? smx[lane] : smx[0];
    mn = warp_min(mn);
    mx = warp_max(mx);
    if (lane == 0) {
      qs[blockIdx.x].min_in = mn;
      qs[blockIdx.x].max_in = mx;
    }
  }
}

// ---- 2. filter / bias ranges ---------------------------------------------------

// Single block.  Filter: `nseg` segments of `seg_len` elements every
// `seg_stride`, seeded with W[0]; equal min/max widen to W[0] -+ 1e-3.
// Bias: all `nbias` elements, seeded with 0; equal min/max widen to b[0] -+ 1e-3.
__global__ void q_filter_range_kernel(const float *__restrict__ W, int nseg, size_t seg_stride,
                                      size_t seg_len, const float *__restrict__ bias, int nbias,
                                      QGlobal *qg) {
  float mn = W[0], mx = W[0];
  size_t total = (size_t)nseg * seg_len;
  for (size_t t = threadIdx.x; t < total; t += blockDim.x) {
    size_t s = t / seg_len, e = t - s * seg_len;
    float v = W[s * seg_stride + e];
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
  float bmn = 0.f, bmx = 0.f;
  for (int t = threadIdx.x; t < nbias; t += blockDim.x) {
    bmn = fminf(bmn, bias[t]);
    bmx = fmaxf(bmx, bias[t]);
  }
  __shared__ float s4[4][32];
  mn = warp_min(mn);
  mx = warp_max(mx);
  bmn = warp_min(bmn);
  bmx = warp_max(bmx);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) {
    s4[0][wid] = mn;
    s4[1][wid] = mx;
    s4[2][wid] = bmn;
    s4[3][wid] = bmx;
  }
  __syncthreads();
  if (wid == 0) {
    int nw = blockDim.x >> 5;
    mn = warp_min(lane < nw ? s4[0][lane] : s4[0][0]);
    mx = warp_max(lane < nw ? s4[1][lane] : s4[1][0]);
    bmn = warp_min(lane < nw ? s4[2][lane] : s4[2][0]);
    bmx = warp_max(lane < nw ? s4[3][lane] : s4[3][0]);
    if (lane == 0) {
      if (mn == mx) {
        mx = __fadd_rn(W[0], 1e-3f);
        mn = __fsub_rn(W[0], 1e-3f);
      }
      if (nbias > 0 && bmn == bmx) {
        bmx = __fadd_rn(bias[0], 1e-3f);
        bmn = __fsub_rn(bias[0], 1e-3f);
      }
      qg->min_f = mn;
      qg->max_f = mx;
      qg->min_b = bmn;
      qg->max_b = bmx;
      qg->off_f = (int)f2q_unclamped<8>(0.0f, mn, mx);
    }
  }
}

// ---- 3. quantize --------------------------------------------------------------

__global__ void q_quantize_filter_kernel(const float *__restrict__ W, size_t lenW,
                                         const float *__restrict__ bias, int nbias,
                                         const QGlobal *__restrict__ qg, uint8_t *__restrict__ Wq,
                                         uint8_t *__restrict__ bq) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  size_t step = (size_t)gridDim.x * blockDim.x;
  const float mn = qg->min_f, mx = qg->max_f;
  for (size_t j = i; j < lenW; j += step) Wq[j] = (uint8_t)f2q<8>(W[j], mn, mx);
  const float bmn = qg->min_b, bmx = qg->max_b;
  for (size_t j = i; j < (size_t)nbias; j += step) bq[j] = (uint8_t)f2q<8>(bias[j], bmn, bmx);
}

__global__ void q_quantize_input_kernel(const float *__restrict__ in, size_t row_len,
                                        const QSample *__restrict__ qs, uint8_t *__restrict__ inq) {
  const int n = blockIdx.y;
  const float mn = qs[n].min_in, mx = qs[n].max_in;
  const float *r = in + (size_t)n * row_len;
  uint8_t *q = inq + (size_t)n * row_len;
  size_t step = (size_t)gridDim.x * blockDim.x;
  for (size_t j = blockIdx.x * (size_t)blockDim.x + threadIdx.x; j < row_len; j += step)
    q[j] = (uint8_t)f2q<8>(r[j], mn, mx);
}

// ---- 4. per-sample output range and offsets -------------------------------------

// quantization_range_for_multiplication<u8,u8,i32> (:95-114); the fc kernel
// then adds the bias range to it (fc :67-68).
__global__ void q_sample_params_kernel(QSample *qs, const QGlobal *__restrict__ qg, int B,
                                       int add_bias_range) {
  int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= B) return;
  QSample s = qs[n];
  float a_level = one_level_u8(s.min_in, s.max_in);
  float b_level = one_level_u8(qg->min_f, qg->max_f);
  float c_level = __fmul_rn(a_level, b_level);
  float mn = __fmul_rn(c_level, (float)(-(1LL << 31)));
  float mx = __fmul_rn(c_level, (float)((1LL << 31) - 1));
  if (add_bias_range) {
    mn = __fadd_rn(mn, qg->min_b);
    mx = __fadd_rn(mx, qg->max_b);
  }
  s.min_out = mn;
  s.max_out = mx;
  s.off_in = (int)f2q_unclamped<8>(0.0f, s.min_in, s.max_in);
  s.zero_total = (int)f2q<32>(0.0f, mn, mx);
  s.acc_min = INT_MAX;
  s.acc_max = INT_MIN;
  qs[n] = s;
}

// ---- 5. int32 accumulate ----------------------------------------------------------

__device__ __forceinline__ void block_minmax_atomic(int mn, int mx, int *gmin, int *gmax) {
  __shared__ int smn[32], smx[32];
  mn = warp_min_i(mn);
  mx = warp_max_i(mx);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) {
    smn[wid] = mn;
    smx[wid] = mx;
  }
  __syncthreads();
  if (wid == 0) {
    int nw = (blockDim.x + 31) >> 5;
    mn = warp_min_i(lane < nw ? smn[lane] : INT_MAX);
    mx = warp_max_i(lane < nw ? smx[lane] : INT_MIN);
    if (lane == 0) {
      atomicMin(gmin, mn);
      atomicMax(gmax, mx);
    }
  }
}

// conv :89-133.  grid = (blocks per sample, B); one thread per output element.
__global__ void q_conv_acc_kernel(ConvGeom g, const uint8_t *__restrict__ inq,
                                  const uint8_t *__restrict__ Wq, const uint8_t *__restrict__ bq,
                                  const QGlobal *__restrict__ qg, QSample *qs,
                                  int *__restrict__ acc) {
  const int n = blockIdx.y;
  const int out_len = g.OC * g.OH * g.OW;
  const int in_len = g.C * g.HI * g.WI;
  const int off_f = qg->off_f;
  const int off_in = qs[n].off_in;
  const int zero_total = qs[n].zero_total;
  const uint8_t *ib = inq + (size_t)n * in_len;
  int mn = INT_MAX, mx = INT_MIN;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < out_len;
       idx += gridDim.x * blockDim.x) {
    int x = idx % g.OW;
    int r = idx / g.OW;
    int y = r % g.OH;
    int o = r / g.OH;
    int sum = 0;
    for (int inc = 0; inc < g.C; ++inc) {
      if (g.tbl && !g.tbl[inc * g.OC + o]) continue;
      const uint8_t *w = Wq + ((size_t)o * g.C + inc) * g.KH * g.KW;
      const uint8_t *ip = ib + ((size_t)inc * g.HI + y * g.SH) * g.WI + x * g.SW;
      for (int wy = 0; wy < g.KH; ++wy)
        for (int wx = 0; wx < g.KW; ++wx)
          sum += ((int)w[wy * g.KW + wx] - off_f) * ((int)ip[wy * g.WI + wx] - off_in);
    }
    if (g.has_bias) sum += (int)bq[o] - zero_total;
    acc[(size_t)n * out_len + idx] = sum;
    mn = min(mn, sum);
    mx = max(mx, sum);
  }
  block_minmax_atomic(mn, mx, &qs[n].acc_min, &qs[n].acc_max);
}

// fc :100-112.  grid = (blocks per sample, B); one thread per output.
__global__ void q_fc_acc_kernel(int in_size, int out_size, int has_bias,
                                const uint8_t *__restrict__ inq, const uint8_t *__restrict__ Wq,
                                const uint8_t *__restrict__ bq, const QGlobal *__restrict__ qg,
                                QSample *qs, int *__restrict__ acc) {
  const int n = blockIdx.y;
  const int off_f = qg->off_f;
  const int off_in = qs[n].off_in;
  const int zero_total = qs[n].zero_total;
  const uint8_t *ib = inq + (size_t)n * in_size;
  int mn = INT_MAX, mx = INT_MIN;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < out_size;
       i += gridDim.x * blockDim.x) {
    int sum = 0;
    for (int c = 0; c < in_size; ++c)
      sum += ((int)Wq[(size_t)c * out_size + i] - off_f) * ((int)ib[c] - off_in);
    if (has_bias) sum += (int)bq[i] - zero_total;
    acc[(size_t)n * out_size + i] = sum;
    mn = min(mn, sum);
    mx = max(mx, sum);
  }
  block_minmax_atomic(mn, mx, &qs[n].acc_min, &qs[n].acc_max);
}

// ---- 6. shrink range, requantize, dequantize ---------------------------------------

// quantize_down_and_shrink_range (:230-254) and the constants of
// requantize_many_in_new_range<int32,uint8> (:159-171), once per sample.
__global__ void q_requant_params_kernel(QSample *qs, int B) {
  int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= B) return;
  QSample s = qs[n];
  float min_new = fminf(0.0f, q2f<32>((long long)s.acc_min, s.min_out, s.max_out));
  float max_new = q2f<32>((long long)s.acc_max, s.min_out, s.max_out);
  const float input_range = __fsub_rn(s.max_out, s.min_out);
  const float output_range = __fsub_rn(max_new, min_new);
  const float recip_output_range = __fdiv_rn(255.0f, output_range);
  const long long recip_output_range_fp =
    (long long)__fmul_rn(recip_output_range, (float)(1 << 16));
  s.range_scale_fp = (long long)__fdiv_rn(
    __fmul_rn(__fmul_rn(255.0f, (float)(1 << 16)), input_range), output_range);
  s.input_offset_fp =
    (long long)__fadd_rn(__fmul_rn(s.min_out, __ll2float_rn(recip_output_range_fp)),
                         __ll2float_rn(s.range_scale_fp >> 1));
  s.output_offset_fp = (long long)roundf(__fdiv_rn(__fmul_rn(min_new, 255.0f), output_range));
  s.min_new = min_new;
  s.max_new = max_new;
  qs[n] = s;
}

// inner loop of requantize_many_in_new_range<int32,uint8> (:172-185) followed
// by quantized_to_float<uint8_t> (:70-84)
__global__ void q_requant_dequant_kernel(const int *__restrict__ acc, size_t out_len,
                                         const QSample *__restrict__ qs, float *__restrict__ out) {
  const int n = blockIdx.y;
  const QSample s = qs[n];
  const int *a = acc + (size_t)n * out_len;
  float *o = out + (size_t)n * out_len;
  const long long rounding_delta = 1LL << 15;
  size_t step = (size_t)gridDim.x * blockDim.x;
  for (size_t j = blockIdx.x * (size_t)blockDim.x + threadIdx.x; j < out_len; j += step) {
    long long v = (long long)a[j];
    long long fp_value = ((v * s.range_scale_fp) >> 32) + s.input_offset_fp;
    long long ri = ((fp_value >= 0) ? (fp_value + rounding_delta) : (fp_value - rounding_delta)) >> 16;
    long long q = ri - s.output_offset_fp;
    q = q > 0 ? q : 0;
    q = q < 255 ? q : 255;
    o[j] = q2f<8>(q, s.min_new, s.max_new);
  }
}

// ---- host side -------------------------------------------------------------------------

static int blocks_for(size_t n, int block) {
  size_t b = (n + block - 1) / block;
  if (b > 1024) b = 1024;
  if (b < 1) b = 1;
  return (int)b;
}

struct QScratch {
  QSample *qs;
  QGlobal *qg;
  uint8_t *inq, *Wq, *bq;
  int *acc;
};

static int q_carve(b200_ctx *ctx, int B, size_t in_len, size_t lenW, size_t nbias, size_t out_len,
                   QScratch *s) {
  size_t o_qs = 0;
  size_t o_qg = align_up(o_qs + sizeof(QSample) * (size_t)B, 256);
  size_t o_in = align_up(o_qg + sizeof(QGlobal), 256);
  size_t o_w = align_up(o_in + in_len * B, 256);
  size_t o_b = align_up(o_w + lenW, 256);
  size_t o_acc = align_up(o_b + nbias + 1, 256);
  size_t total = o_acc + sizeof(int) * out_len * B;
  void *base = nullptr;
  B200_TRY(ctx_scratch(ctx, total, &base));
  char *p = static_cast<char *>(base);
  s->qs = reinterpret_cast<QSample *>(p + o_qs);
  s->qg = reinterpret_cast<QGlobal *>(p + o_qg);
  s->inq = reinterpret_cast<uint8_t *>(p + o_in);
  s->Wq = reinterpret_cast<uint8_t *>(p + o_w);
  s->bq = reinterpret_cast<uint8_t *>(p + o_b);
  s->acc = reinterpret_cast<int *>(p + o_acc);
  return 0;
}

int qconv_fwd(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W,
              const float *bias, float *out, int B) {
  b200_conv_desc dd = *d;
  dd.input_is_padded = 1;  // the quantized layer pads before its backend call
                           // (quantized_convolutional_layer.h:402-437)
  ConvGeom g;
  B200_TRY(conv_geom_from_desc(ctx, &dd, &g));
  B200_REQUIRE(g.DH == 1 && g.DW == 1, "quantized convolution has no dilation");
  if (B == 0) return 0;
  const size_t plane = (size_t)g.HI * g.WI;
  const size_t in_len = plane * g.C, out_len = (size_t)g.OC * g.OH * g.OW;
  const size_t lenW = conv_weight_len(g);
  // The reference scans height*height elements per input plane and
  // k_h*k_h filter elements at input-plane offsets; refuse shapes where those
  // scans would leave the buffers (the reference reads out of bounds there).
  B200_REQUIRE((size_t)(g.C - 1) * plane + (size_t)g.HI * g.HI <= in_len,
               "quantized convolution: in_padded height %d > width %d makes the reference scan "
               "past the input row", g.HI, g.WI);
  B200_REQUIRE((size_t)(g.C - 1) * plane + (size_t)g.KH * g.KH <= lenW,
               "quantized convolution: the reference's filter range scan leaves the filter "
               "tensor for this shape");
  QScratch s;
  B200_TRY(q_carve(ctx, B, in_len, lenW, g.OC, out_len, &s));
  cudaStream_t st = ctx->stream;
  q_input_range_kernel<<<B, 256, 0, st>>>(in, in_len, g.C, plane, (size_t)g.HI * g.HI, s.qs);
  B200_LAUNCHED();
  q_filter_range_kernel<<<1, 256, 0, st>>>(W, g.C, plane, (size_t)g.KH * g.KH, bias,
                                          g.has_bias ? g.OC : 0, s.qg);
  B200_LAUNCHED();
  q_quantize_filter_kernel<<<blocks_for(lenW, 256), 256, 0, st>>>(W, lenW, bias,
                                                                  g.has_bias ? g.OC : 0, s.qg,
                                                                  s.Wq, s.bq);
  B200_LAUNCHED();
  q_sample_params_kernel<<<ceil_div(B, 128), 128, 0, st>>>(s.qs, s.qg, B, 0);
  B200_LAUNCHED();
  q_quantize_input_kernel<<<dim3(blocks_for(in_len, 256), B), 256, 0, st>>>(in, in_len, s.qs,
                                                                           s.inq);
  B200_LAUNCHED();
  q_conv_acc_kernel<<<dim3(blocks_for(out_len, 256), B), 256, 0, st>>>(g, s.inq, s.Wq, s.bq, s.qg,
                                                                      s.qs, s.acc);
  B200_LAUNCHED();
  q_requant_params_kernel<<<ceil_div(B, 128), 128, 0, st>>>(s.qs, B);
  B200_LAUNCHED();
  q_requant_dequant_kernel<<<dim3(blocks_for(out_len, 256), B), 256, 0, st>>>(s.acc, out_len, s.qs,
                                                                             out);
  B200_LAUNCHED();
  return 0;
}

int qfc_fwd(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W,
            const float *bias, float *out, int B) {
  B200_REQUIRE(in_size > 0 && out_size > 0, "quantized fc: non-positive size");
  if (B == 0) return 0;
  const size_t lenW = (size_t)in_size * out_size;
  const int nbias = bias ? out_size : 0;
  QScratch s;
  B200_TRY(q_carve(ctx, B, in_size, lenW, out_size, out_size, &s));
  cudaStream_t st = ctx->stream;
  q_input_range_kernel<<<B, 256, 0, st>>>(in, in_size, 1, 0, in_size, s.qs);
  B200_LAUNCHED();
  q_filter_range_kernel<<<1, 1024, 0, st>>>(W, 1, 0, lenW, bias, nbias, s.qg);
  B200_LAUNCHED();
  q_quantize_filter_kernel<<<blocks_for(lenW, 256), 256, 0, st>>>(W, lenW, bias, nbias, s.qg, s.Wq,
                                                                  s.bq);
  B200_LAUNCHED();
  q_sample_params_kernel<<<ceil_div(B, 128), 128, 0, st>>>(s.qs, s.qg, B, 1);
  B200_LAUNCHED();
  q_quantize_input_kernel<<<dim3(blocks_for(in_size, 256), B), 256, 0, st>>>(in, in_size, s.qs,
                                                                            s.inq);
  B200_LAUNCHED();
  q_fc_acc_kernel<<<dim3(blocks_for(out_size, 128), B), 128, 0, st>>>(in_size, out_size, nbias > 0,
                                                                     s.inq, s.Wq, s.bq, s.qg, s.qs,
                                                                     s.acc);
  B200_LAUNCHED();
  q_requant_params_kernel<<<ceil_div(B, 128), 128, 0, st>>>(s.qs, B);
  B200_LAUNCHED();
  q_requant_dequant_kernel<<<dim3(blocks_for(out_size, 256), B), 256, 0, st>>>(s.acc, out_size,
                                                                              s.qs, out);
  B200_LAUNCHED();
  return 0;
}

}  // namespace b200
