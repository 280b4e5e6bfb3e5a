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
  int sum_in;              // sum of the quantized input bytes (dp4a path)
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
  for (int s = 0; s < nseg; ++s) {
    const float *seg = r + s * seg_stride;
    for (size_t e = threadIdx.x; e < seg_len; e += blockDim.x) {
      float v = seg[e];
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
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
  s.sum_in = 0;
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
// `bias_f` != nullptr: the nine-argument kernel's bias term, `bias[o] - zero_in_total_space` formed
// in FLOAT from the float-held bias entry and cast to int32 (tiny_quantized_conv2d_kernel.h:436-441)
__global__ void q_conv_acc_kernel(ConvGeom g, const uint8_t *__restrict__ inq,
                                  const uint8_t *__restrict__ Wq, const uint8_t *__restrict__ bq,
                                  const QGlobal *__restrict__ qg, QSample *qs,
                                  int *__restrict__ acc, const float *__restrict__ bias_f) {
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
    if (g.has_bias)
      sum += bias_f != nullptr ? (int)__fsub_rn(bias_f[o], (float)zero_total) : (int)bq[o] - zero_total;
    acc[(size_t)n * out_len + idx] = sum;
    mn = min(mn, sum);
    mx = max(mx, sum);
  }
  block_minmax_atomic(mn, mx, &qs[n].acc_min, &qs[n].acc_max);
}

// ---- 5b. the same accumulators through dp4a --------------------------------------------
//
// sum (w - off_w)(x - off_x) = sum w*x - off_x * sum w - off_w * sum x + n * off_w * off_x is exact
// in integers, so the products can be taken four bytes at a time (dp4a on unsigned bytes) from
// operands laid out with the contracted index fastest.  All arithmetic is modulo 2^32 and the
// true value fits an int32, so intermediate wrap-around is harmless.

// min / max of a long vector, many blocks: per-block results, reduced by q_filter_range_kernel
__global__ void q_minmax_partial_kernel(const float *__restrict__ v, size_t n, float *__restrict__ part) {
  float mn = v[0], mx = v[0];
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    mn = fminf(mn, v[i]);
    mx = fmaxf(mx, v[i]);
  }
  __shared__ float s2[2][32];
  mn = warp_min(mn);
  mx = warp_max(mx);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) {
    s2[0][wid] = mn;
    s2[1][wid] = mx;
  }
  __syncthreads();
  if (wid == 0) {
    int nw = blockDim.x >> 5;
    mn = warp_min(lane < nw ? s2[0][lane] : s2[0][0]);
    mx = warp_max(lane < nw ? s2[1][lane] : s2[1][0]);
    if (lane == 0) {
      part[2 * blockIdx.x] = mn;
      part[2 * blockIdx.x + 1] = mx;
    }
  }
}

// fully-connected filter, quantized and transposed: Wt[i][c] (row pitch `pitch` bytes, zero padded)
// from W[c*out + i]; 32 x 32 tiles through shared memory
__global__ void q_quantize_filter_t_kernel(const float *__restrict__ W, int in_size, int out_size, int pitch,
                                           const float *__restrict__ bias, int nbias,
                                           const QGlobal *__restrict__ qg, uint8_t *__restrict__ Wt,
                                           uint8_t *__restrict__ bq) {
  __shared__ uint8_t tile[32][33];
  const float mn = qg->min_f, mx = qg->max_f;
  if (blockIdx.x == 0 && blockIdx.y == 0) {
    const float bmn = qg->min_b, bmx = qg->max_b;
    for (int j = threadIdx.y * 32 + threadIdx.x; j < nbias; j += 256) bq[j] = (uint8_t)f2q<8>(bias[j], bmn, bmx);
  }
  const int c0 = blockIdx.y * 32, i0 = blockIdx.x * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    int c = c0 + j, i = i0 + threadIdx.x;
    tile[j][threadIdx.x] = (c < in_size && i < out_size) ? (uint8_t)f2q<8>(W[(size_t)c * out_size + i], mn, mx) : 0;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    int i = i0 + j, c = c0 + threadIdx.x;
    if (i < out_size && c < pitch) Wt[(size_t)i * pitch + c] = tile[threadIdx.x][j];
  }
}

// input rows quantized with a row pitch (zero padded) and their byte sums (sum_in starts at 0:
// q_sample_params_kernel); grid = (slices of 1024 bytes, B)
__global__ void __launch_bounds__(256) q_quantize_input_pitch_kernel(const float *__restrict__ in, int row_len,
                                                                    int pitch, QSample *qs,
                                                                    uint8_t *__restrict__ inq) {
  const int n = blockIdx.y;
  const float mn = qs[n].min_in, mx = qs[n].max_in;
  const float *r = in + (size_t)n * row_len;
  const int j0 = blockIdx.x * 1024 + threadIdx.x * 4;
  int sum = 0;
  if (j0 < pitch) {  // pitch is a multiple of 4
    unsigned w = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      unsigned v = j0 + k < row_len ? (unsigned)f2q<8>(r[j0 + k], mn, mx) : 0u;
      w |= v << (8 * k);
      sum += (int)v;
    }
    *reinterpret_cast<unsigned *>(inq + (size_t)n * pitch + j0) = w;
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if ((threadIdx.x & 31) == 0 && sum) atomicAdd(&qs[n].sum_in, sum);
}

// fc :100-112.  One warp per pair of outputs and group of 8 samples; lanes split the contraction
// in 16-byte pieces (pitch is a multiple of 16).
constexpr int QFC_SAMPLES = 8, QFC_OUTS = 2;
__device__ __forceinline__ unsigned dp4a4(const uint4 &a, const uint4 &b, unsigned c) {
  c = __dp4a(a.x, b.x, c);
  c = __dp4a(a.y, b.y, c);
  c = __dp4a(a.z, b.z, c);
  return __dp4a(a.w, b.w, c);
}
__global__ void __launch_bounds__(128) q_fc_acc_dp4a_kernel(int in_size, int out_size, int pitch, int has_bias,
                                                           int B, const uint8_t *__restrict__ inq,
                                                           const uint8_t *__restrict__ Wt,
                                                           const uint8_t *__restrict__ bq,
                                                           const QGlobal *__restrict__ qg, QSample *qs,
                                                           int *__restrict__ acc) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i0 = (blockIdx.x * 4 + warp) * QFC_OUTS, n0 = blockIdx.y * QFC_SAMPLES;
  if (i0 >= out_size) return;
  const int vecs = pitch >> 4;
  const uint4 ones = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
  const uint4 *wrow[QFC_OUTS];
#pragma unroll
  for (int k = 0; k < QFC_OUTS; ++k)
    wrow[k] = reinterpret_cast<const uint4 *>(Wt + (size_t)min(i0 + k, out_size - 1) * pitch);
  const uint4 *xrow[QFC_SAMPLES];
#pragma unroll
  for (int s = 0; s < QFC_SAMPLES; ++s)
    xrow[s] = reinterpret_cast<const uint4 *>(inq + (size_t)min(n0 + s, B - 1) * pitch);
  unsigned a[QFC_OUTS][QFC_SAMPLES], sw[QFC_OUTS];
#pragma unroll
  for (int k = 0; k < QFC_OUTS; ++k) {
    sw[k] = 0;
#pragma unroll
    for (int s = 0; s < QFC_SAMPLES; ++s) a[k][s] = 0;
  }
  for (int q = lane; q < vecs; q += 32) {
    uint4 w[QFC_OUTS];
#pragma unroll
    for (int k = 0; k < QFC_OUTS; ++k) {
      w[k] = __ldg(wrow[k] + q);
      sw[k] = dp4a4(w[k], ones, sw[k]);
    }
#pragma unroll
    for (int s = 0; s < QFC_SAMPLES; ++s) {
      const uint4 x = __ldg(xrow[s] + q);
#pragma unroll
      for (int k = 0; k < QFC_OUTS; ++k) a[k][s] = dp4a4(w[k], x, a[k][s]);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
#pragma unroll
    for (int k = 0; k < QFC_OUTS; ++k) {
      sw[k] += __shfl_xor_sync(0xffffffffu, sw[k], o);
#pragma unroll
      for (int s = 0; s < QFC_SAMPLES; ++s) a[k][s] += __shfl_xor_sync(0xffffffffu, a[k][s], o);
    }
  // lanes 0..15 each finish one (output, sample) pair
  const int k = lane >> 3, sl = lane & 7;
  unsigned mine = 0, msw = 0;
#pragma unroll
  for (int kk = 0; kk < QFC_OUTS; ++kk)
#pragma unroll
    for (int s = 0; s < QFC_SAMPLES; ++s)
      if (kk == k && s == sl) {
        mine = a[kk][s];
        msw = sw[kk];
      }
  if (k < QFC_OUTS && i0 + k < out_size && n0 + sl < B) {
    const int n = n0 + sl, i = i0 + k;
    const unsigned off_f = (unsigned)qg->off_f, off_in = (unsigned)qs[n].off_in;
    unsigned v = mine - off_in * msw - off_f * (unsigned)qs[n].sum_in + (unsigned)in_size * off_f * off_in;
    int sum = (int)v;
    if (has_bias) sum += (int)bq[i] - qs[n].zero_total;
    acc[(size_t)n * out_size + i] = sum;
    atomicMin(&qs[n].acc_min, sum);
    atomicMax(&qs[n].acc_max, sum);
  }
}

// convolution operands with the channel index fastest: input [n][y][x][c], filter [o][tap][c]
__global__ void q_quantize_input_nhwc_kernel(const float *__restrict__ in, int C, int HW, const QSample *__restrict__ qs,
                                             uint8_t *__restrict__ inq) {
  const int n = blockIdx.y;
  const float mn = qs[n].min_in, mx = qs[n].max_in;
  const float *r = in + (size_t)n * C * HW;
  unsigned *q = reinterpret_cast<unsigned *>(inq + (size_t)n * C * HW);
  const int Cw = C >> 2, total = HW * Cw;
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < total; j += gridDim.x * blockDim.x) {
    const int p = j % HW, cw = j / HW;  // pixel fastest: the four plane reads are coalesced
    unsigned w = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) w |= (unsigned)f2q<8>(r[(size_t)(cw * 4 + k) * HW + p], mn, mx) << (8 * k);
    q[(size_t)p * Cw + cw] = w;
  }
}

__global__ void q_quantize_filter_otc_kernel(const float *__restrict__ W, int C, int OC, int KK,
                                             const float *__restrict__ bias, int nbias,
                                             const QGlobal *__restrict__ qg, uint8_t *__restrict__ Wq,
                                             uint8_t *__restrict__ bq) {
  const float mn = qg->min_f, mx = qg->max_f;
  const int total = OC * KK * C;
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < total; j += gridDim.x * blockDim.x) {
    const int c = j % C, r = j / C, tap = r % KK, o = r / KK;
    Wq[j] = (uint8_t)f2q<8>(W[((size_t)o * C + c) * KK + tap], mn, mx);
  }
  const float bmn = qg->min_b, bmx = qg->max_b;
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < nbias; j += gridDim.x * blockDim.x)
    bq[j] = (uint8_t)f2q<8>(bias[j], bmn, bmx);
}

// conv :89-133.  Block = one sample, 128 output pixels, all output channels; thread = 4 pixels x 8
// output channels (a warp shares the channels, so its filter loads are broadcasts); the whole
// quantized filter sits in shared memory.
constexpr int QCV_PPT = 4, QCV_OPT = 8, QCV_PIX = 32 * QCV_PPT, QCV_WARPS = 8;
template <bool VEC>
__global__ void __launch_bounds__(256) q_conv_acc_dp4a_kernel(ConvGeom g, const uint8_t *__restrict__ inq,
                                                             const uint8_t *__restrict__ Wq,
                                                             const uint8_t *__restrict__ bq,
                                                             const QGlobal *__restrict__ qg, QSample *qs,
                                                             int *__restrict__ acc) {
  extern __shared__ __align__(16) uint8_t qsm[];
  const int KK = g.KH * g.KW, Cw = g.C >> 2;
  const int wlen = g.OC * KK * g.C;                         // bytes of the filter
  unsigned *wsm = reinterpret_cast<unsigned *>(qsm);         // [o][tap][Cw] words
  unsigned *wsum = wsm + ((wlen >> 2) + 3) / 4 * 4;         // [OC]
  const int n = blockIdx.y, tid = threadIdx.x;
  for (int j = tid; j < (wlen >> 2); j += 256) wsm[j] = reinterpret_cast<const unsigned *>(Wq)[j];
  __syncthreads();
  for (int o = tid; o < g.OC; o += 256) {
    unsigned t = 0;
    for (int j = 0; j < KK * Cw; ++j) t = __dp4a(wsm[o * KK * Cw + j], 0x01010101u, t);
    wsum[o] = t;
  }
  __syncthreads();
  const int npix = g.OH * g.OW;
  const int p0 = blockIdx.x * QCV_PIX + (tid & 31) * QCV_PPT, og = tid >> 5;
  const unsigned off_f = (unsigned)qg->off_f, off_in = (unsigned)qs[n].off_in;
  const int zero_total = qs[n].zero_total;
  const unsigned *ib = reinterpret_cast<const unsigned *>(inq + (size_t)n * g.C * g.HI * g.WI);
  int pbase[QCV_PPT];  // word offset of the window origin of each pixel (pixels past the end repeat the last)
#pragma unroll
  for (int k = 0; k < QCV_PPT; ++k) {
    const int p = min(p0 + k, npix - 1);
    const int y = p / g.OW, x = p - y * g.OW;
    pbase[k] = (y * g.SH * g.WI + x * g.SW) * Cw;
  }
  int mn = INT_MAX, mx = INT_MIN;
  for (int o0 = og * QCV_OPT; o0 < g.OC; o0 += QCV_WARPS * QCV_OPT) {
    unsigned a[QCV_PPT][QCV_OPT], sx[QCV_PPT];
#pragma unroll
    for (int k = 0; k < QCV_PPT; ++k) {
      sx[k] = 0;
#pragma unroll
      for (int j = 0; j < QCV_OPT; ++j) a[k][j] = 0;
    }
    for (int wy = 0; wy < g.KH; ++wy)
      for (int wx = 0; wx < g.KW; ++wx) {
        const int ioff = (wy * g.WI + wx) * Cw;
        const unsigned *wp = wsm + (size_t)(o0 * KK + wy * g.KW + wx) * Cw;
        if (VEC) {  // 16 channels per load
          for (int cw = 0; cw < Cw; cw += 4) {
            uint4 xv[QCV_PPT];
#pragma unroll
            for (int k = 0; k < QCV_PPT; ++k) {
              xv[k] = *reinterpret_cast<const uint4 *>(ib + pbase[k] + ioff + cw);
              sx[k] = dp4a4(xv[k], make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u), sx[k]);
            }
#pragma unroll
            for (int j = 0; j < QCV_OPT; ++j) {
              const int o = min(o0 + j, g.OC - 1);
              const uint4 wv = *reinterpret_cast<const uint4 *>(wp + (o - o0) * KK * Cw + cw);
#pragma unroll
              for (int k = 0; k < QCV_PPT; ++k) a[k][j] = dp4a4(wv, xv[k], a[k][j]);
            }
          }
        } else {
          for (int cw = 0; cw < Cw; ++cw) {
            unsigned xv[QCV_PPT];
#pragma unroll
            for (int k = 0; k < QCV_PPT; ++k) {
              xv[k] = ib[pbase[k] + ioff + cw];
              sx[k] = __dp4a(xv[k], 0x01010101u, sx[k]);
            }
#pragma unroll
            for (int j = 0; j < QCV_OPT; ++j) {
              const int o = min(o0 + j, g.OC - 1);
              const unsigned wv = wp[(o - o0) * KK * Cw + cw];
#pragma unroll
              for (int k = 0; k < QCV_PPT; ++k) a[k][j] = __dp4a(wv, xv[k], a[k][j]);
            }
          }
        }
      }
#pragma unroll
    for (int j = 0; j < QCV_OPT; ++j) {
      const int o = o0 + j;
      if (o < g.OC) {
        int sums[QCV_PPT];
#pragma unroll
        for (int k = 0; k < QCV_PPT; ++k) {
          unsigned v = a[k][j] - off_in * wsum[o] - off_f * sx[k] + (unsigned)(KK * g.C) * off_f * off_in;
          int sum = (int)v;
          if (g.has_bias) sum += (int)bq[o] - zero_total;
          sums[k] = sum;
          if (p0 + k < npix) {
            mn = min(mn, sum);
            mx = max(mx, sum);
          }
        }
        int *dst = acc + (size_t)n * g.OC * npix + (size_t)o * npix + p0;
        if (p0 + QCV_PPT <= npix && (npix & 3) == 0) {
          *reinterpret_cast<int4 *>(dst) = make_int4(sums[0], sums[1], sums[2], sums[3]);
        } else {
#pragma unroll
          for (int k = 0; k < QCV_PPT; ++k)
            if (p0 + k < npix) dst[k] = sums[k];
        }
      }
    }
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

// ---- 7. the forms for chained quantized layers ("eq") -----------------------------------------
// Operands are uint8 values held in floats, with their ranges; the result leaves the same way
// (tiny_quantized_conv2d_kernel.h:353-466, tiny_quantized_fully_connected_kernel.h:269-370).

// ranges, offsets and the accumulator range of every sample from the supplied ranges
__global__ void q_eq_params_kernel(QSample *qs, QGlobal *qg, const float *__restrict__ in_r,
                                   const float *__restrict__ W_r, const float *__restrict__ b_r, int B, int fc,
                                   int has_bias) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= B) return;
  float min_f = W_r[0], max_f = W_r[1];
  if (min_f == max_f) {
    max_f = __fadd_rn(W_r[1], 1e-3f);
    min_f = __fsub_rn(W_r[0], 1e-3f);
  }
  float min_b = 0.f, max_b = 0.f;
  if (fc) {  // only the fully-connected kernel reads the bias range (:286-293, :313-314)
    min_b = b_r[0];
    max_b = b_r[1];
    if (has_bias && min_b == max_b) {
      max_b = __fadd_rn(b_r[1], 1e-3f);
      min_b = __fsub_rn(b_r[0], 1e-3f);
    }
  }
  QSample s = qs[n];
  s.min_in = in_r[2 * n];
  s.max_in = in_r[2 * n + 1];
  const float c_level = __fmul_rn(one_level_u8(s.min_in, s.max_in), one_level_u8(min_f, max_f));
  float mn = __fmul_rn(c_level, (float)(-(1LL << 31)));
  float mx = __fmul_rn(c_level, (float)((1LL << 31) - 1));
  if (fc) {
    mn = __fadd_rn(mn, min_b);
    mx = __fadd_rn(mx, max_b);
  }
  s.min_out = mn;
  s.max_out = mx;
  s.off_in = (int)f2q_unclamped<8>(0.0f, s.min_in, s.max_in);
  s.zero_total = (int)f2q<32>(0.0f, mn, mx);
  s.acc_min = INT_MAX;
  s.acc_max = INT_MIN;
  s.sum_in = 0;
  qs[n] = s;
  if (n == 0) {
    qg->min_f = min_f;
    qg->max_f = max_f;
    qg->min_b = min_b;
    qg->max_b = max_b;
    qg->off_f = (int)f2q_unclamped<8>(0.0f, min_f, max_f);
  }
}

// static_cast<uint8_t>(float) of values that are uint8 already
__global__ void q_cast_u8_kernel(const float *__restrict__ src, uint8_t *__restrict__ dst, size_t n) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) dst[i] = (uint8_t)__float2int_rz(src[i]);
}

// fully-connected accumulate on the reference's [in][out] byte filter: one thread per (sample, output)
__global__ void q_fc_acc_kernel(int in_size, int out_size, int has_bias, const uint8_t *__restrict__ inq,
                                const uint8_t *__restrict__ Wq, const uint8_t *__restrict__ bq,
                                const QGlobal *__restrict__ qg, QSample *qs, int *__restrict__ acc) {
  const int n = blockIdx.y;
  const int off_f = qg->off_f, off_in = qs[n].off_in, zero_total = qs[n].zero_total;
  const uint8_t *x = inq + (size_t)n * in_size;
  int mn = INT_MAX, mx = INT_MIN;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < out_size; i += gridDim.x * blockDim.x) {
    int sum = 0;
    for (int c = 0; c < in_size; ++c) sum += ((int)Wq[(size_t)c * out_size + i] - off_f) * ((int)x[c] - off_in);
    if (has_bias) sum += (int)bq[i] - zero_total;
    acc[(size_t)n * out_size + i] = sum;
    mn = min(mn, sum);
    mx = max(mx, sum);
  }
  block_minmax_atomic(mn, mx, &qs[n].acc_min, &qs[n].acc_max);
}

// requantize to uint8 held in floats, and hand the shrunk range out (:455-465 / :358-369)
__global__ void q_requant_u8_kernel(const int *__restrict__ acc, size_t out_len, const QSample *__restrict__ qs,
                                    float *__restrict__ out, float *__restrict__ out_r) {
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
    o[j] = (float)q;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    out_r[2 * n] = s.min_new;
    out_r[2 * n + 1] = s.max_new;
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
  float *part;
  int *acc;
};

constexpr int Q_PART_BLOCKS = 592;

static int q_carve(b200_ctx *ctx, int B, size_t in_len, size_t lenW, size_t nbias, size_t out_len,
                   QScratch *s) {
  size_t o_qs = 0;
  size_t o_qg = align_up(o_qs + sizeof(QSample) * (size_t)B, 256);
  size_t o_part = align_up(o_qg + sizeof(QGlobal), 256);
  size_t o_in = align_up(o_part + sizeof(float) * 2 * Q_PART_BLOCKS, 256);
  size_t o_w = align_up(o_in + in_len * B, 256);
  size_t o_b = align_up(o_w + lenW, 256);
  size_t o_acc = align_up(o_b + nbias + 1, 256);
  size_t total = o_acc + sizeof(int) * out_len * B;
  void *base = nullptr;
  B200_TRY(ctx_scratch(ctx, total, &base));
  char *p = static_cast<char *>(base);
  s->qs = reinterpret_cast<QSample *>(p + o_qs);
  s->qg = reinterpret_cast<QGlobal *>(p + o_qg);
  s->part = reinterpret_cast<float *>(p + o_part);
  s->inq = reinterpret_cast<uint8_t *>(p + o_in);
  s->Wq = reinterpret_cast<uint8_t *>(p + o_w);
  s->bq = reinterpret_cast<uint8_t *>(p + o_b);
  s->acc = reinterpret_cast<int *>(p + o_acc);
  return 0;
}

// shared memory of q_conv_acc_dp4a_kernel: the quantized filter and one byte sum per output channel
static size_t qconv_dp4a_smem(const ConvGeom &g) {
  size_t words = (size_t)g.OC * g.KH * g.KW * g.C / 4;
  return ((words + 3) / 4 * 4 + g.OC) * 4;
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
  // channel-fastest operands and dp4a when every window position is connected
  const size_t smem = qconv_dp4a_smem(g);
  const bool fast = !g.tbl && g.C % 4 == 0 && smem <= 200 * 1024;
  q_input_range_kernel<<<B, 1024, 0, st>>>(in, in_len, g.C, plane, (size_t)g.HI * g.HI, s.qs);
  B200_LAUNCHED();
  q_filter_range_kernel<<<1, 256, 0, st>>>(W, g.C, plane, (size_t)g.KH * g.KH, bias,
                                          g.has_bias ? g.OC : 0, s.qg);
  B200_LAUNCHED();
  if (fast)
    q_quantize_filter_otc_kernel<<<blocks_for(lenW, 256), 256, 0, st>>>(
      W, g.C, g.OC, g.KH * g.KW, bias, g.has_bias ? g.OC : 0, s.qg, s.Wq, s.bq);
  else
    q_quantize_filter_kernel<<<blocks_for(lenW, 256), 256, 0, st>>>(W, lenW, bias,
                                                                    g.has_bias ? g.OC : 0, s.qg,
                                                                    s.Wq, s.bq);
  B200_LAUNCHED();
  q_sample_params_kernel<<<ceil_div(B, 128), 128, 0, st>>>(s.qs, s.qg, B, 0);
  B200_LAUNCHED();
  if (fast) {
    q_quantize_input_nhwc_kernel<<<dim3(blocks_for(in_len / 4, 256), B), 256, 0, st>>>(
      in, g.C, (int)plane, s.qs, s.inq);
    B200_LAUNCHED();
    static bool attr_set = false;
    if (!attr_set) {
      B200_CUDA(cudaFuncSetAttribute(q_conv_acc_dp4a_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     200 * 1024));
      B200_CUDA(cudaFuncSetAttribute(q_conv_acc_dp4a_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     200 * 1024));
      attr_set = true;
    }
    dim3 grid(ceil_div(g.OH * g.OW, QCV_PIX), B);
    if (g.C % 16 == 0)
      q_conv_acc_dp4a_kernel<true><<<grid, 256, smem, st>>>(g, s.inq, s.Wq, s.bq, s.qg, s.qs, s.acc);
    else
      q_conv_acc_dp4a_kernel<false><<<grid, 256, smem, st>>>(g, s.inq, s.Wq, s.bq, s.qg, s.qs, s.acc);
  } else {
    q_quantize_input_kernel<<<dim3(blocks_for(in_len, 256), B), 256, 0, st>>>(in, in_len, s.qs,
                                                                             s.inq);
    B200_LAUNCHED();
    q_conv_acc_kernel<<<dim3(blocks_for(out_len, 256), B), 256, 0, st>>>(g, s.inq, s.Wq, s.bq,
                                                                        s.qg, s.qs, s.acc, nullptr);
  }
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
  const int pitch = (in_size + 15) / 16 * 16;  // bytes per quantized row, zero padded
  QScratch s;
  B200_TRY(q_carve(ctx, B, pitch, (size_t)pitch * out_size, out_size, out_size, &s));
  cudaStream_t st = ctx->stream;
  q_input_range_kernel<<<B, 1024, 0, st>>>(in, in_size, 1, 0, in_size, s.qs);
  B200_LAUNCHED();
  int pblocks = blocks_for(lenW, 1024);
  if (pblocks > Q_PART_BLOCKS) pblocks = Q_PART_BLOCKS;
  q_minmax_partial_kernel<<<pblocks, 1024, 0, st>>>(W, lenW, s.part);
  B200_LAUNCHED();
  // the partial results stand in for the filter: same extremes, and when all are equal so is W[0]
  q_filter_range_kernel<<<1, 1024, 0, st>>>(s.part, 1, 0, (size_t)2 * pblocks, bias, nbias, s.qg);
  B200_LAUNCHED();
  q_quantize_filter_t_kernel<<<dim3(ceil_div(out_size, 32), ceil_div(pitch, 32)), dim3(32, 8), 0, st>>>(
    W, in_size, out_size, pitch, bias, nbias, s.qg, s.Wq, s.bq);
  B200_LAUNCHED();
  q_sample_params_kernel<<<ceil_div(B, 128), 128, 0, st>>>(s.qs, s.qg, B, 1);
  B200_LAUNCHED();
  q_quantize_input_pitch_kernel<<<dim3(ceil_div(pitch, 1024), B), 256, 0, st>>>(in, in_size, pitch, s.qs, s.inq);
  B200_LAUNCHED();
  q_fc_acc_dp4a_kernel<<<dim3(ceil_div(out_size, 4 * QFC_OUTS), ceil_div(B, QFC_SAMPLES)), 128, 0, st>>>(
    in_size, out_size, pitch, nbias > 0, B, s.inq, s.Wq, s.bq, s.qg, s.qs, s.acc);
  B200_LAUNCHED();
  q_requant_params_kernel<<<ceil_div(B, 128), 128, 0, st>>>(s.qs, B);
  B200_LAUNCHED();
  q_requant_dequant_kernel<<<dim3(blocks_for(out_size, 256), B), 256, 0, st>>>(s.acc, out_size,
                                                                              s.qs, out);
  B200_LAUNCHED();
  return 0;
}

// tiny_backend::conv2d_eq (backend_tiny.h:115-135): padded rows of uint8 values held in floats
int qconv_eq_fwd(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W, const float *bias,
                 const float *in_r, const float *W_r, const float *b_r, float *out, float *out_r, int B) {
  b200_conv_desc dd = *d;
  dd.input_is_padded = 1;
  ConvGeom g;
  B200_TRY(conv_geom_from_desc(ctx, &dd, &g));
  B200_REQUIRE(g.DH == 1 && g.DW == 1, "quantized convolution has no dilation");
  if (B == 0) return 0;
  const size_t in_len = (size_t)g.HI * g.WI * g.C, out_len = (size_t)g.OC * g.OH * g.OW;
  const size_t lenW = conv_weight_len(g);
  QScratch s;
  B200_TRY(q_carve(ctx, B, in_len, lenW, g.OC, out_len, &s));
  cudaStream_t st = ctx->stream;
  q_eq_params_kernel<<<ceil_div(B, 128), 128, 0, st>>>(s.qs, s.qg, in_r, W_r, b_r, B, 0, g.has_bias);
  B200_LAUNCHED();
  q_cast_u8_kernel<<<blocks_for(in_len * B, 256), 256, 0, st>>>(in, s.inq, in_len * B);
  B200_LAUNCHED();
  q_cast_u8_kernel<<<blocks_for(lenW, 256), 256, 0, st>>>(W, s.Wq, lenW);
  B200_LAUNCHED();
  q_conv_acc_kernel<<<dim3(blocks_for(out_len, 256), B), 256, 0, st>>>(g, s.inq, s.Wq, s.bq, s.qg, s.qs, s.acc,
                                                                      g.has_bias ? bias : nullptr);
  B200_LAUNCHED();
  q_requant_params_kernel<<<ceil_div(B, 128), 128, 0, st>>>(s.qs, B);
  B200_LAUNCHED();
  q_requant_u8_kernel<<<dim3(blocks_for(out_len, 256), B), 256, 0, st>>>(s.acc, out_len, s.qs, out, out_r);
  B200_LAUNCHED();
  return 0;
}

// tiny_backend::fully_eq (backend_tiny.h:321-345)
int qfc_eq_fwd(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W, const float *bias,
               const float *in_r, const float *W_r, const float *b_r, float *out, float *out_r, int B) {
  if (B == 0) return 0;
  const size_t lenW = (size_t)in_size * out_size;
  QScratch s;
  B200_TRY(q_carve(ctx, B, in_size, lenW, out_size, out_size, &s));
  cudaStream_t st = ctx->stream;
  const int has_bias = bias != nullptr;
  q_eq_params_kernel<<<ceil_div(B, 128), 128, 0, st>>>(s.qs, s.qg, in_r, W_r, b_r, B, 1, has_bias);
  B200_LAUNCHED();
  q_cast_u8_kernel<<<blocks_for((size_t)in_size * B, 256), 256, 0, st>>>(in, s.inq, (size_t)in_size * B);
  B200_LAUNCHED();
  q_cast_u8_kernel<<<blocks_for(lenW, 256), 256, 0, st>>>(W, s.Wq, lenW);
  B200_LAUNCHED();
  if (has_bias) {
    q_cast_u8_kernel<<<blocks_for(out_size, 256), 256, 0, st>>>(bias, s.bq, out_size);
    B200_LAUNCHED();
  }
  q_fc_acc_kernel<<<dim3(blocks_for(out_size, 128), B), 128, 0, st>>>(in_size, out_size, has_bias, s.inq, s.Wq, s.bq,
                                                                     s.qg, s.qs, s.acc);
  B200_LAUNCHED();
  q_requant_params_kernel<<<ceil_div(B, 128), 128, 0, st>>>(s.qs, B);
  B200_LAUNCHED();
  q_requant_u8_kernel<<<dim3(blocks_for(out_size, 256), B), 256, 0, st>>>(s.acc, out_size, s.qs, out, out_r);
  B200_LAUNCHED();
  return 0;
}

}  // namespace b200
