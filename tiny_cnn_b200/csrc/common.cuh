// Shared plumbing of the B200 hot-path library: context, error reporting,
// launch accounting and the internal launcher prototypes the C ABI and the
// device-resident training step both use.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>
#include <map>
#include <string>
#include <vector>

#include "tinycnn_b200.h"

namespace b200 {

// ----------------------------------------------------------------------------
// errors
// ----------------------------------------------------------------------------
void set_error(const char *fmt, ...);
void clear_error();

#define B200_CUDA(expr)                                                              \
  do {                                                                               \
    cudaError_t e__ = (expr);                                                        \
    if (e__ != cudaSuccess) {                                                        \
      ::b200::set_error("%s:%d: %s -> %s", __FILE__, __LINE__, #expr,               \
                        cudaGetErrorString(e__));                                    \
      return 1;                                                                      \
    }                                                                                \
  } while (0)

#define B200_REQUIRE(cond, ...)                                                      \
  do {                                                                               \
    if (!(cond)) {                                                                   \
      ::b200::set_error(__VA_ARGS__);                                                \
      return 2;                                                                      \
    }                                                                                \
  } while (0)

#define B200_TRY(expr)                                                               \
  do {                                                                               \
    int r__ = (expr);                                                                \
    if (r__ != 0) return r__;                                                        \
  } while (0)

extern std::atomic<unsigned long long> g_launches;

// Check the launch just issued and count it.
#define B200_LAUNCHED()                                                              \
  do {                                                                               \
    ::b200::g_launches.fetch_add(1, std::memory_order_relaxed);                     \
    B200_CUDA(cudaGetLastError());                                                   \
  } while (0)

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline size_t ceil_div_sz(size_t a, size_t b) { return (a + b - 1) / b; }
static inline size_t align_up(size_t a, size_t b) { return (a + b - 1) / b * b; }

}  // namespace b200

// Tile shape of the direct-convolution kernel chosen for one problem.
struct TileChoice {
  int OCT, OCB, TH, TWG, NSB, ICB;
};

// ----------------------------------------------------------------------------
// context
// ----------------------------------------------------------------------------
struct b200_ctx {
  int device = 0;
  int sm_count = 148;
  size_t smem_optin = 0;  // max dynamic shared memory per block (opt-in)
  cudaStream_t stream = nullptr;
  bool own_stream = false;

  // grow-only device scratch used by kernels that need global scratch
  // (split partial sums, re-laid-out filters).  One op at a time per context.
  void *scratch = nullptr;
  size_t scratch_bytes = 0;

  // grow-only device arena + pinned host buffer for the *_host entry points
  void *arena = nullptr;
  size_t arena_bytes = 0;
  void *pinned = nullptr;
  size_t pinned_bytes = 0;

  // device word a kernel sets when a bounded wait ran out; read by b200_ctx_sync
  int *dev_err = nullptr;

  // fully-connected GEMMs on the tensor cores (3xTF32): 0 never, 1 when large, 2 whenever legal
  int fc_tensor_cores = 1;
  // convolutions on the tensor cores: 0 never, 1 for layers with at least 16 channels on
  // both sides, 2 whenever the geometry allows
  int conv_tensor_cores = 1;

  // tile shapes already chosen, keyed by the problem's dimensions
  std::map<std::string, TileChoice> tile_cache;

  // device copies of connection tables, keyed by their bytes
  std::map<std::string, uint8_t *> tbl_cache;
};

namespace b200 {

int ctx_scratch(b200_ctx *ctx, size_t bytes, void **out);
int ctx_arena(b200_ctx *ctx, size_t bytes, void **out);
int ctx_pinned(b200_ctx *ctx, size_t bytes, void **out);
int ctx_device_table(b200_ctx *ctx, const uint8_t *host_tbl, size_t n, const uint8_t **out);
// Remember a measured tile choice (and append it to the file named by the
// environment variable B200_TUNE_CACHE, which ctx creation reads back, so a
// later process starts with the choices already made).
void ctx_remember_tile(b200_ctx *ctx, const std::string &key, const TileChoice &c);

// ----------------------------------------------------------------------------
// convolution geometry shared by the general and the tiled kernels
// ----------------------------------------------------------------------------
struct ConvGeom {
  int C, HI, WI;   // geometry of the `in` / `din` buffers
  int OC, OH, OW;  // geometry of `out` / `dout`
  int KH, KW, SH, SW, DH, DW;
  int pad_t, pad_l;  // in(y) = oy*SH + wy*DH - pad_t
  int has_bias;
  const uint8_t *tbl;  // DEVICE connected[inc*OC + o] or nullptr
};

int conv_geom_from_desc(b200_ctx *ctx, const b200_conv_desc *d, ConvGeom *g);
size_t conv_weight_len(const ConvGeom &g);

// true when the tiled (stride 1, dilation 1, 3x3 or 5x5) kernels apply
bool conv_tiled_ok(const ConvGeom &g);

// scratch sizes (in floats) of the tiled path
size_t conv_tiled_fwd_scratch(const ConvGeom &g);
size_t conv_tiled_dx_scratch(const ConvGeom &g);
size_t conv_tiled_dw_scratch(const b200_ctx *ctx, const ConvGeom &g, int B);

// general kernels (any stride / dilation / table)
int conv_general_fwd(b200_ctx *ctx, const ConvGeom &g, const float *in, const float *W,
                     const float *bias, float *out, int B, int act);
int conv_general_dx(b200_ctx *ctx, const ConvGeom &g, const float *W, const float *dout,
                    float *din, int B);
int conv_general_dw(b200_ctx *ctx, const ConvGeom &g, const float *in, const float *dout,
                    float *dW, float *db, int accumulate, int B);

// tiled kernels; `scratch` must hold the matching conv_tiled_*_scratch floats
int conv_tiled_fwd(b200_ctx *ctx, const ConvGeom &g, const float *in, const float *W,
                   const float *bias, float *out, int B, int act, float *scratch);
int conv_tiled_dx_prep(b200_ctx *ctx, const ConvGeom &g, const float *W, float *scratch);
int conv_tiled_dx(b200_ctx *ctx, const ConvGeom &g, const float *W, const float *dout,
                  float *din, int B, float *scratch, int prep = 1);
// Writes `*splits` partial sums of [dW | db] (row length conv_weight_len + OC)
// into scratch; the caller merges them in row order.
int conv_tiled_dw_partials(b200_ctx *ctx, const ConvGeom &g, const float *in,
                           const float *dout, int B, float *scratch, int *splits);

// tensor-core path (conv_tc.cu): stride 1, dilation 1, windows up to 8x8, at most 256 channels
// either side.  The passes read "tall" split copies of the input (xs) and of dY (dys) that
// conv_tc_tall_x / conv_tc_tall_dy write; sizes in floats from the *_floats functions.
bool conv_tc_ok(const b200_ctx *ctx, const ConvGeom &g);
// which passes of a layer run on the tensor cores: `algo` 3 = all (when conv_tc_ok), 1 / 2 =
// none, 0 = by the context's conv_tensor_cores option
struct ConvTcUse {
  bool fwd, dx, dw;
  bool dw_small;   // dW through the im2col form for layers with few input channels (conv_dw_small)
  bool fwd_small;  // forward through the im2col form for the same layers (conv_fwd_small)
};
// forward of layers with few input channels (in_c*KH*KW <= 96, <= 64 out channels) from the CHW input
bool conv_fwd_small_ok(const b200_ctx *ctx, const ConvGeom &g);
int conv_fwd_small(b200_ctx *ctx, const ConvGeom &g, const float *in, const float *W, const float *bias, float *out,
                   int B, int act);
ConvTcUse conv_tc_use(const b200_ctx *ctx, const ConvGeom &g, int algo);
size_t conv_tc_tall_floats(const ConvGeom &g, int B, int which);  // 0: input, 1: dY
size_t conv_tc_filter_floats(const b200_ctx *ctx, const ConvGeom &g, int for_dx);
int conv_tc_bsum_rows(const ConvGeom &g, int B);
size_t conv_tc_dw_floats(const b200_ctx *ctx, const ConvGeom &g, int B);
int conv_tc_tall_x(b200_ctx *ctx, const ConvGeom &g, const float *in, int B, float *xs);
int conv_tc_tall_dy(b200_ctx *ctx, const ConvGeom &g, const float *dout, int B, float *dys, float *bsum);
// the same conversions fused with the 2x2/2 max-pooling layer before the convolution (forward) and
// with the gradient of the pooling layer (and relu) after it (backward)
int conv_tc_tall_x_pool(b200_ctx *ctx, const ConvGeom &g, const float *in, float *pooled, int32_t *argmax, int B,
                        float *xs);
int conv_tc_tall_dy_unpool(b200_ctx *ctx, const ConvGeom &g, const float *gpool, const int32_t *argmax,
                           const float *pooled_y, float *dout_chw, int B, float *dys, float *bsum);
// filter matrices of the forward and / or dX pass (either may be nullptr) in one launch
int conv_tc_prep(b200_ctx *ctx, const ConvGeom &g, const float *W, float *wt_fwd, float *wt_dx);
// `prep` = 0 reuses the filter matrices an earlier call left in `wt` (same weights)
int conv_tc_fwd(b200_ctx *ctx, const ConvGeom &g, const float *xs, const float *W, const float *bias,
                float *out, int B, int act, float *wt, int prep = 1);
int conv_tc_dx(b200_ctx *ctx, const ConvGeom &g, const float *dys, const float *W, float *din, int B,
               float *wt, int prep = 1);
int conv_tc_dw(b200_ctx *ctx, const ConvGeom &g, const float *xs, const float *dys, int B, float *part,
               int *splits);
// Arguments of one finishing pass of a tensor-core dW kernel: sums the partial rows in fixed order
// and stores the totals in the reference layout.  Elements [0, row_w) are weight-gradient entries in
// the producing kernel's own order; `layout` says which: 0 = [unit][j][ky][inc][o] of
// conv_dw_tc_kernel (kx = KW-1-j), 1 = [k][o] of conv_dw_small_tc_kernel.  Elements
// [row_w, row_w + OC) are bias-gradient sums taken from `bsrc` (bs_rows rows of bs_stride floats,
// entry bs_off + o of each).  Unconnected pairs get no gradient.
struct DwFinishArgs {
  const float *part;
  long long part_stride;
  int splits;
  const float *bsrc;
  long long bs_stride, bs_off;
  int bs_rows;
  float *dW, *db;
  int layout, row_w;
  int C, OC, OCp, KH, KW, ic_slabs;
  const uint8_t *tbl;
  int accumulate;
};
constexpr int DW_FINISH_MAX = 4;  // layers per launch of dw_finish_many
// finish: fixed-order sum of the partial rows into the reference layout, and (with bsum / db) the bias
// gradient.  With `defer` the pass is not launched but described there, for dw_finish_many.
int conv_tc_dw_finish(b200_ctx *ctx, const ConvGeom &g, float *part, int splits, float *dW, int accumulate,
                      const float *bsum, int B, float *db, DwFinishArgs *defer = nullptr);
// the finishing passes of several layers in one launch (same sums, element by element)
int dw_finish_many(b200_ctx *ctx, const DwFinishArgs *list, int n);

// dW of stride-1 layers with in_c*KH*KW <= 128 on the tensor cores, straight from the CHW tensors
bool conv_dw_small_ok(const b200_ctx *ctx, const ConvGeom &g);
size_t conv_dw_small_floats(const b200_ctx *ctx, const ConvGeom &g, int B);
int conv_dw_small(b200_ctx *ctx, const ConvGeom &g, const float *in, const float *dout, int B, float *part,
                  float *dW, float *db, int accumulate, DwFinishArgs *defer = nullptr);

// dst (+)= sum_r src[r*stride + i], rows summed in order; optional connection
// mask for convolution weights (entries of unconnected pairs are left alone
// when accumulating and zeroed otherwise).
// `mask` (may be nullptr) names a convolution whose connection table zeroes the
// gradient of unconnected (o, inc) pairs within the first conv_weight_len entries.
// `in_order` != 0 adds the rows strictly one after the other (the order of
// edge::merge_grads); otherwise four interleaved running sums are combined at the end.
int merge_rows(b200_ctx *ctx, const float *src, int rows, size_t stride, float *dst, size_t len,
               int accumulate, const ConvGeom *mask, int in_order = 0);

// ----------------------------------------------------------------------------
// other ops
// ----------------------------------------------------------------------------
// tensor-core GEMM (gemm_tc.cu): D[M][N] (+)= A * Bt^T, operands split into TF32 hi/lo
// pairs in `scratch` (gemm_tc_scratch_floats floats)
size_t gemm_tc_scratch_floats(int M, int N, int K);
int gemm_tc(b200_ctx *ctx, int M, int N, int K, const float *src_a, long long lda, bool a_transposed,
            const float *src_b, long long ldb, bool b_transposed, float *D, const float *bias,
            int accumulate, int act, float *scratch);

// `scratch` (fc_scratch_floats floats, may be nullptr) holds the k-slice partial
// sums small GEMMs are split into, or the split operands of the tensor-core path.
size_t fc_scratch_floats(const b200_ctx *ctx, int in_size, int out_size, int B);
int fc_fwd(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W,
           const float *bias, float *out, int B, int act, float *scratch);
// sum of a bucket over the ranks of a data-parallel job through peer memory (peer_reduce.cu)
struct PeerReduce {
  int rank = 0, world = 0;
  long long n = 0;
  long long split = 0;           // [split, n) is pushed early, [0, split) by the summing kernel
  long long ll_n = 0;            // words per rank and half when the late region travels as flagged 8-byte words
  unsigned long long timeout_ns = 0;
  float **bases_dev = nullptr;   // [world] every rank's buffer as mapped in this process
  unsigned *step_dev = nullptr;  // [0] reductions done so far, [1] blocks of the running sum that ended
};
size_t peer_reduce_bytes(long long n, long long split, int world);
// `timeout_ms` bounds every wait of the summing kernel (0 = 10 s)
int peer_reduce_init(b200_ctx *ctx, PeerReduce *pr, long long n, long long split, int rank, int world,
                     const unsigned long long *bases, int timeout_ms);
void peer_reduce_free(PeerReduce *pr);
int peer_reduce_push_early(b200_ctx *ctx, const PeerReduce *pr, float *grads);
int peer_reduce_push_all(b200_ctx *ctx, const PeerReduce *pr, float *grads);
int peer_reduce_sum_early(b200_ctx *ctx, const PeerReduce *pr, float *grads);
int peer_reduce_finish(b200_ctx *ctx, const PeerReduce *pr, float *grads, int late_pushed, int early_summed);
int peer_reduce_run(b200_ctx *ctx, const PeerReduce *pr, float *grads);

int fc_bwd(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W,
           const float *dout, float *din, float *dW, float *db, int accumulate, int B,
           float *scratch);

int maxpool_fwd(b200_ctx *ctx, const b200_pool_desc &d, const float *in, float *out,
                int32_t *argmax, int B);
// `pooled_y` (optional): this layer's forward output, given when a relu layer feeds the pooling
// layer; the relu's gradient mask (its output at a window's winner is the pooled value) is applied
// to din on the way (2x2/2 aligned layers only, see maxpool_can_fuse_relu).
int maxpool_bwd(b200_ctx *ctx, const b200_pool_desc &d, const float *dout, const int32_t *argmax,
                float *din, int B, const float *pooled_y = nullptr);
bool maxpool_can_fuse_relu(const b200_pool_desc &d);
int avgpool_fwd(b200_ctx *ctx, const b200_pool_desc &d, const float *in, const float *W,
                const float *bias, float *out, int B);
int avgpool_bwd(b200_ctx *ctx, const b200_pool_desc &d, const float *in, const float *W,
                const float *dout, float *din, float *dW, float *db, int accumulate, int B);

// `param`: epsilon of leaky relu / alpha of elu (ignored by the other kinds)
int act_fwd(b200_ctx *ctx, int kind, const float *x, float *y, int dim, int B, float param = 0.f);
int act_bwd(b200_ctx *ctx, int kind, const float *y, const float *dy, float *dx, int dim, int B,
            float param = 0.f);
// batch normalization, dropout with a host-made mask, local response normalization (norm.cu)
size_t batchnorm_scratch_floats(const b200_ctx *ctx, int channels, int B);
int batchnorm_fwd(b200_ctx *ctx, int channels, int spatial, float eps, const float *x, float *mean, float *variance,
                  float *stddev, float *y, int B, int train, float *scratch);
int batchnorm_bwd(b200_ctx *ctx, int channels, int spatial, const float *y, const float *dy, const float *stddev,
                  float *dx, int B, float *scratch);
int batchnorm_post_update(b200_ctx *ctx, int channels, float momentum, float *mean, float *variance,
                          const float *mean_cur, const float *var_cur, const int *skip_if);
int dropout_apply(b200_ctx *ctx, const float *in, const uint8_t *mask, float scale, float *out, size_t n);
int lrn_across_fwd(b200_ctx *ctx, const float *in, float *out, int channels, int area, int size, float alpha,
                   float beta, int B);

int loss_grad(b200_ctx *ctx, int kind, const float *y, const float *t, float *dy, int dim, int B);
// loss gradient (into dy) and the gradient of a softmax layer whose output is y (into dx) in one launch
int softmax_loss_bwd(b200_ctx *ctx, int loss_kind, const float *y, const float *t, float *dy, float *dx, int dim,
                     int B);
// a fully-connected layer of at most 16 outputs followed by a softmax output layer, as one kernel
// per direction: forward z = x W + b, y = softmax(z); backward dy = loss gradient, dz = softmax
// gradient, dx = dz W^T (times the gradient of the relu whose output `relu_x` is the layer's input,
// when given; dx may be nullptr)
bool fc_softmax_fusable(int K, int N);
int fc_softmax_fwd(b200_ctx *ctx, int K, int N, const float *x, const float *W, const float *bias, float *z, float *y,
                   int B);
int fc_softmax_loss_bwd(b200_ctx *ctx, int loss_kind, int K, int N, const float *y, const float *t, const float *W,
                        const float *relu_x, float *dy, float *dz, float *dx, int B);
int loss_value(b200_ctx *ctx, int kind, const float *y, const float *t, float *loss_sum, int dim,
               int B);

// Per-tensor segment of the flat parameter buffer for the fused update.
struct OptSegment {
  unsigned long long offset;
  unsigned long long len;
};
int opt_update(b200_ctx *ctx, int kind, const b200_opt_hyper &h, const float *grads, int rows,
               size_t stride, float *merged, float *W, float *s0, float *s1, size_t len);
// All tensors in one launch; Adam powers are read per tensor from the device
// table pow_tab[2*t] = b1_t, pow_tab[2*t+1] = b2_t and advanced afterwards by
// opt_advance_powers (one sequential float multiply per update call, which is
// how adam::update evolves them).
// `skip_if` (may be nullptr): device word; when it is non-zero as the kernel starts, nothing is
// changed (a reduction over the replicas that gave up leaves the parameters of the step before).
int opt_update_segments(b200_ctx *ctx, int kind, const b200_opt_hyper &h, const float *grads,
                        float *W, float *s0, float *s1, const OptSegment *segs_dev,
                        int n_segs, size_t total, float *pow_tab, const int *skip_if = nullptr);
int opt_advance_powers(b200_ctx *ctx, float *pow_tab, int n_tensors, float b1, float b2,
                       const int *skip_if = nullptr);

// raw dataset bytes -> the first layer's float rows and the target rows (data.cu)
int check_image_desc(const b200_image_desc *d);
size_t image_in_len(const b200_image_desc *d);
size_t image_out_len(const b200_image_desc *d);
int images_u8_to_float(b200_ctx *ctx, const b200_image_desc *d, const uint8_t *src, long long n, float *dst);
int labels_to_targets(b200_ctx *ctx, const uint8_t *labels, long long n, int out_dim, float tmin, float tmax,
                      float *dst);

int qconv_fwd(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W,
              const float *bias, float *out, int B);
int qfc_fwd(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W,
            const float *bias, float *out, int B);
// the forms for chained quantized layers: uint8 values held in floats with their ranges in and out
int qconv_eq_fwd(b200_ctx *ctx, const b200_conv_desc *d, const float *in, const float *W, const float *bias,
                 const float *in_r, const float *W_r, const float *b_r, float *out, float *out_r, int B);
int qfc_eq_fwd(b200_ctx *ctx, int in_size, int out_size, const float *in, const float *W, const float *bias,
               const float *in_r, const float *W_r, const float *b_r, float *out, float *out_r, int B);

}  // namespace b200
