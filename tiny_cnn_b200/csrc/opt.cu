// Per-sample gradient merge fused with the optimizer update.
//
// The reference sums the B per-sample gradient rows of a parameter tensor
// (edge::merge_grads, tiny_dnn/node.h:89-103), multiplies by 1.0
// (tiny_dnn/layers/layer.h:669-673) and hands the sum to optimizer::update
// (adagrad tiny_dnn/optimizers/optimizer.h:60-66, adam :112-127, momentum
// :205-213).  Here the row sum is formed in registers and consumed by the
// update formula in the same thread; the arithmetic of each formula is written
// with explicit round-to-nearest operations so no multiply-add contraction
// changes the rounding sequence of the reference.
#include "common.cuh"
#include "device_utils.cuh"

namespace b200 {

struct OptParams {
  float alpha, b1, b2, b1_t, b2_t, mu, lambda, eps;
};

__device__ __forceinline__ void opt_apply(int kind, const OptParams &h, float g, float &w,
                                          float &s0, float &s1) {
  if (kind == B200_OPT_ADAGRAD) {
    // g[i] += dW*dW ; W -= alpha*dW/(sqrt(g)+eps)
    s0 = __fadd_rn(s0, __fmul_rn(g, g));
    w = __fsub_rn(w, __fdiv_rn(__fmul_rn(h.alpha, g), __fadd_rn(__fsqrt_rn(s0), h.eps)));
  } else if (kind == B200_OPT_ADAM) {
    // mt = b1*mt + (1-b1)*dW ; vt = b2*vt + (1-b2)*dW*dW
    // W -= alpha*(mt/(1-b1_t)) / sqrt(vt/(1-b2_t) + eps)
    s0 = __fadd_rn(__fmul_rn(h.b1, s0), __fmul_rn(__fsub_rn(1.f, h.b1), g));
    s1 = __fadd_rn(__fmul_rn(h.b2, s1), __fmul_rn(__fmul_rn(__fsub_rn(1.f, h.b2), g), g));
    float mhat = __fdiv_rn(s0, __fsub_rn(1.f, h.b1_t));
    float vhat = __fdiv_rn(s1, __fsub_rn(1.f, h.b2_t));
    w = __fsub_rn(w, __fdiv_rn(__fmul_rn(h.alpha, mhat), __fsqrt_rn(__fadd_rn(vhat, h.eps))));
  } else if (kind == B200_OPT_MOMENTUM) {
    // V = mu*dWprev - alpha*(dW + W*lambda) ; W += V ; dWprev = V
    float v = __fsub_rn(__fmul_rn(h.mu, s0),
                        __fmul_rn(h.alpha, __fadd_rn(g, __fmul_rn(w, h.lambda))));
    w = __fadd_rn(w, v);
    s0 = v;
  } else if (kind == B200_OPT_RMSPROP) {
    // g = mu*g + (1-mu)*dW*dW ; W -= alpha*dW/sqrt(g+eps)   (optimizer.h:82-89)
    s0 = __fadd_rn(__fmul_rn(h.mu, s0), __fmul_rn(__fmul_rn(__fsub_rn(1.f, h.mu), g), g));
    w = __fsub_rn(w, __fdiv_rn(__fmul_rn(h.alpha, g), __fsqrt_rn(__fadd_rn(s0, h.eps))));
  } else if (kind == B200_OPT_ADAMAX) {
    // mt = b1*mt + (1-b1)*dW ; ut = max(b2*ut, |dW|) ; W -= (alpha/(1.0-b1_t)) * (mt/(ut+eps))
    // (optimizer.h:153-166).  The literal 1.0 is a double: the step size, its product with the
    // float quotient and the subtraction from W are double operations rounded to float once.
    s0 = __fadd_rn(__fmul_rn(h.b1, s0), __fmul_rn(__fsub_rn(1.f, h.b1), g));
    s1 = fmaxf(__fmul_rn(h.b2, s1), fabsf(g));
    const double step = __ddiv_rn((double)h.alpha, __dsub_rn(1.0, (double)h.b1_t));
    const float q = __fdiv_rn(s0, __fadd_rn(s1, h.eps));
    w = (float)__dsub_rn((double)w, __dmul_rn(step, (double)q));
  } else if (kind == B200_OPT_GRADIENT_DESCENT) {
    // W = W - alpha*(dW + lambda*W)   (optimizer.h:185-188)
    w = __fsub_rn(w, __fmul_rn(h.alpha, __fadd_rn(g, __fmul_rn(h.lambda, w))));
  } else {
    // nesterov: V = mu*dWprev - alpha*(dW + W*lambda) ; W += (-mu)*dWprev + (1+mu)*V ; dWprev = V
    // (optimizer.h:233-240)
    float v = __fsub_rn(__fmul_rn(h.mu, s0),
                        __fmul_rn(h.alpha, __fadd_rn(g, __fmul_rn(w, h.lambda))));
    w = __fadd_rn(w, __fadd_rn(__fmul_rn(-h.mu, s0), __fmul_rn(__fadd_rn(1.f, h.mu), v)));
    s0 = v;
  }
}

// optimizers that keep a second state vector / per-tensor powers
__host__ __device__ __forceinline__ bool opt_two_states(int kind) { return kind == B200_OPT_ADAM || kind == B200_OPT_ADAMAX; }

__global__ void opt_update_kernel(int kind, OptParams h, const float *__restrict__ grads, int rows,
                                  size_t stride, float *__restrict__ merged, float *__restrict__ W,
                                  float *__restrict__ s0, float *__restrict__ s1, size_t len) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < len; i += step) {
    float g = grads[i];
    for (int r = 1; r < rows; ++r) g = __fadd_rn(g, grads[(size_t)r * stride + i]);
    if (merged) merged[i] = g;
    float w = W[i], a = s0 ? s0[i] : 0.f, b = opt_two_states(kind) ? s1[i] : 0.f;
    opt_apply(kind, h, g, w, a, b);
    W[i] = w;
    if (s0) s0[i] = a;
    if (opt_two_states(kind)) s1[i] = b;
  }
}

// Whole flat parameter buffer in one launch; the segment an element belongs to
// selects Adam's (b1_t, b2_t), which differ per tensor because adam::update
// advances them once per call (optimizer.h:125-126).
__global__ void opt_update_segments_kernel(int kind, OptParams h, const float *__restrict__ grads,
                                           float *__restrict__ W, float *__restrict__ s0,
                                           float *__restrict__ s1,
                                           const OptSegment *__restrict__ segs, int n_segs,
                                           size_t total, const float *__restrict__ pow_tab,
                                           const int *__restrict__ skip_if) {
  if (skip_if && *skip_if != 0) return;
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    OptParams hp = h;
    if (opt_two_states(kind)) {
      // binary search of the segment containing i
      int lo = 0, hi = n_segs - 1;
      while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (segs[mid].offset <= i)
          lo = mid;
        else
          hi = mid - 1;
      }
      hp.b1_t = pow_tab[2 * lo];
      hp.b2_t = pow_tab[2 * lo + 1];
    }
    float g = grads[i];
    float w = W[i], a = s0[i], b = opt_two_states(kind) ? s1[i] : 0.f;
    opt_apply(kind, hp, g, w, a, b);
    W[i] = w;
    s0[i] = a;
    if (opt_two_states(kind)) s1[i] = b;
  }
}

// One step of the network performs n_tensors update calls; tensor t sees the
// power after t further multiplies, and every entry then moves on by n_tensors
// sequential float multiplies -- the same products, in the same order, that
// `b1_t *= b1` produces on the host.
__global__ void opt_advance_powers_kernel(float *pow_tab, int n_tensors, float b1, float b2,
                                          const int *__restrict__ skip_if) {
  if (skip_if && *skip_if != 0) return;
  int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tensors) return;
  float p1 = pow_tab[2 * t], p2 = pow_tab[2 * t + 1];
  for (int k = 0; k < n_tensors; ++k) {
    p1 = __fmul_rn(p1, b1);
    p2 = __fmul_rn(p2, b2);
  }
  pow_tab[2 * t] = p1;
  pow_tab[2 * t + 1] = p2;
}

static OptParams to_params(const b200_opt_hyper &h) {
  OptParams p;
  p.alpha = h.alpha;
  p.b1 = h.b1;
  p.b2 = h.b2;
  p.b1_t = h.b1_t;
  p.b2_t = h.b2_t;
  p.mu = h.mu;
  p.lambda = h.lambda;
  p.eps = h.eps;
  return p;
}

static int grid_for(size_t total, int block, int sm_count) {
  size_t blocks = (total + block - 1) / block;
  size_t cap = (size_t)sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

int opt_update(b200_ctx *ctx, int kind, const b200_opt_hyper &h, const float *grads, int rows,
               size_t stride, float *merged, float *W, float *s0, float *s1, size_t len) {
  B200_REQUIRE(kind >= B200_OPT_ADAGRAD && kind <= B200_OPT_NESTEROV_MOMENTUM, "unknown optimizer %d", kind);
  B200_REQUIRE(rows >= 1, "opt_update: rows must be >= 1");
  B200_REQUIRE((s0 != nullptr || kind == B200_OPT_GRADIENT_DESCENT) && (!opt_two_states(kind) || s1 != nullptr),
               "opt_update: optimizer state buffer is NULL");
  if (len == 0) return 0;
  opt_update_kernel<<<grid_for(len, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
    kind, to_params(h), grads, rows, stride, merged, W, s0, s1, len);
  B200_LAUNCHED();
  return 0;
}

int opt_update_segments(b200_ctx *ctx, int kind, const b200_opt_hyper &h, const float *grads,
                        float *W, float *s0, float *s1, const OptSegment *segs_dev, int n_segs,
                        size_t total, float *pow_tab, const int *skip_if) {
  B200_REQUIRE(kind >= B200_OPT_ADAGRAD && kind <= B200_OPT_NESTEROV_MOMENTUM, "unknown optimizer %d", kind);
  if (total == 0) return 0;
  opt_update_segments_kernel<<<grid_for(total, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
    kind, to_params(h), grads, W, s0, s1, segs_dev, n_segs, total, pow_tab, skip_if);
  B200_LAUNCHED();
  return 0;
}

int opt_advance_powers(b200_ctx *ctx, float *pow_tab, int n_tensors, float b1, float b2,
                       const int *skip_if) {
  if (n_tensors == 0) return 0;
  opt_advance_powers_kernel<<<ceil_div(n_tensors, 64), 64, 0, ctx->stream>>>(pow_tab, n_tensors, b1,
                                                                            b2, skip_if);
  B200_LAUNCHED();
  return 0;
}

}  // namespace b200
