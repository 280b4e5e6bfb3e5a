// Device-resident twin of a network<sequential>: the whole training step
// (network::train_onebatch, tiny_dnn/network.h:911-926) runs on the GPU with
// activations, gradients, parameters and optimizer state resident in HBM.
//
//   forward   sequential::forward   (tiny_dnn/nodes.h:288-303)
//   backward  gradient<E> + sequential::backward (loss_function.h:190-218, nodes.h:276-286)
//   update    nodes::update_weights -> layer::update_weight (nodes.h:103-107, layer.h:663-682)
//
// Memory layout: one flat parameter buffer in network order (per layer W then
// b), a gradient bucket and optimizer state buffers of the same shape, so the
// data-parallel exchange is a single sum all-reduce of the bucket and the
// update is one launch over the whole buffer.
#include <string.h>

#include "common.cuh"

using namespace b200;

namespace {

struct Layer {
  int kind = 0;
  b200_conv_desc cd{};
  ConvGeom g{};
  b200_pool_desc pd{};
  int fc_in = 0, fc_out = 0, fc_bias = 0;
  size_t in_dim = 0, out_dim = 0;
  size_t w_off = 0, w_len = 0, b_off = 0, b_len = 0;
  float *out = nullptr;   // [max_batch][out_dim]
  float *grad = nullptr;  // dE/d out
  int32_t *argmax = nullptr;
  bool tiled = false;
  float *wt_fwd = nullptr, *wt_dx = nullptr, *dw_part = nullptr;
  // tensor-core passes: tall split copies of the input and of dY, per-block bias partials,
  // filter matrices, partial weight gradients
  ConvTcUse tc = {false, false, false, false};
  float *tc_xs = nullptr, *tc_dys = nullptr, *tc_bsum = nullptr;
  float *tc_wt_fwd = nullptr, *tc_wt_dx = nullptr, *tc_part = nullptr, *tc_small_part = nullptr;
  float *fc_scratch = nullptr;  // k-slice partial sums of the small GEMMs
  float *fc_scratch_side = nullptr;  // the same for the dW GEMM when it runs on the side stream
  float act_param = 0.f;  // leaky relu: epsilon; elu: alpha
  // batch normalization: shape, constants, this batch's moments, stddev, moving averages, slice sums
  int bn_c = 0, bn_s = 0;
  float bn_eps = 0.f, bn_momentum = 0.f;
  float *bn_mean_cur = nullptr, *bn_var_cur = nullptr, *bn_stddev = nullptr, *bn_mean = nullptr, *bn_var = nullptr,
        *bn_scratch = nullptr;
  int fused_act = 0;      // activation of the NEXT layer folded into this epilogue
  bool skipped = false;   // activation layer folded into the previous layer
  bool relu_bwd_fused = false;   // max-pool: also applies the gradient of the relu before it
  bool bwd_done_by_next = false; // relu: its gradient is produced by the pooling layer after it
  // 2x2 max-pool next to a tensor-core convolution: the pooling kernels also write the tall split
  // copies that convolution reads (its input in the forward pass, its dY in the backward pass)
  cudaEvent_t ev_prep = nullptr;  // convolution: its filter matrices / copies are ready (side stream)
  bool dx_prep_side = false;      // the FFMA dX filter copy of this step was made beside the forward pass
  int feeds_conv = -1;     // max-pool: convolution layer whose input copy it writes
  int grad_to_conv = -1;   // max-pool: convolution layer whose dY copy it writes
  bool xs_from_pool = false, dys_from_pool = false;  // convolution: copies come from the pooling layers
};

}  // namespace

struct b200_net {
  b200_ctx *ctx = nullptr;
  int max_batch = 0;
  std::vector<Layer> layers;
  // a narrow fully-connected layer + softmax output layer run as one kernel per direction:
  // index of that fully-connected layer (-1: none) and of a relu directly before it (-1: none)
  int head_fc = -1, head_relu = -1;
  bool train_phase = true;  // net_phase::train (b200_net_set_phase)
  bool batch_finishes = false;  // B200_NET_BATCH_FINISH=1
  std::vector<OptSegment> segs;  // trainable tensors in update order
  size_t n_params = 0;
  float *params = nullptr, *grads = nullptr, *state0 = nullptr, *state1 = nullptr;
  OptSegment *segs_dev = nullptr;
  float *pow_tab = nullptr;  // device [2*T] Adam powers per tensor
  std::vector<float> pow_host;
  bool pow_init = false;
  float pow_b1 = 0.f, pow_b2 = 0.f;
  float *in_grad = nullptr;  // dE/d input of the first layer
  float *x_dev = nullptr, *t_dev = nullptr;  // staging for the HOST step
  // side stream for independent work of one layer's backward pass (a tensor-core dW beside an
  // FFMA dX use different units of the SM and share it)
  cudaStream_t side = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  // b200_net_fit_host: uploads of the next mini-batch overlap the step of the current one
  cudaStream_t copy_stream = nullptr;
  float *x_stage[2] = {nullptr, nullptr}, *t_stage[2] = {nullptr, nullptr};
  // b200_net_fit_u8_host: raw image bytes and labels of a mini-batch
  uint8_t *u8_stage[2] = {nullptr, nullptr}, *label_stage[2] = {nullptr, nullptr};
  size_t u8_stage_bytes = 0;
  cudaEvent_t up_done[2] = {nullptr, nullptr}, stage_free[2] = {nullptr, nullptr};
  // a full mini-batch of b200_net_fit_host is read where the upload left it, and its forward output
  // leaves through a copy the step itself makes, fetched by a third stream: between two steps the
  // compute stream has nothing but the next graph
  cudaStream_t d2h_stream = nullptr;
  float *out_stage[2] = {nullptr, nullptr};
  cudaEvent_t step_done[2] = {nullptr, nullptr}, d2h_done[2] = {nullptr, nullptr};
  bool stage_used[2] = {false, false}, out_stage_used[2] = {false, false};
  unsigned fit_toggle = 0;        // staging buffer of the next step (persists across fit calls)
  int fit_last = -1;              // staging buffer holding the latest full mini-batch; -1: x_dev / t_dev do
  float *fit_out_copy = nullptr;  // where the step being issued leaves a copy of its forward output
  int cur_batch = 0;
  const float *cur_x = nullptr;
  int fit_rows = 0;  // rows of x_dev / t_dev the last step of a fit call ran on
  bool fuse = true;
  bool input_grad = true;
  bool keep_layer_grads = false;  // B200_NET_KEEP_GRADS=1: every layer's dE/d out also in CHW form
  PeerReduce peer;  // data-parallel replicas: the gradient bucket is summed over the ranks inside the step
  // the layers after `peer_early_layer` (inclusive) own bucket entries [peer.split, n): once their weight
  // gradients exist they are pushed to the peers from `comm`, beside the rest of the backward pass
  int peer_early_layer = -1;
  cudaStream_t comm = nullptr;
  cudaEvent_t ev_comm_main = nullptr, ev_comm_side = nullptr, ev_comm_done = nullptr;
  bool peer_early_sum = true;   // sum the early region on the communication stream (B200_PEER_EARLY_SUM=0: in the last kernel)
  bool early_summed = false;    // the backward pass just issued did so
  // captured launch sequences: slot 0 = whole step, slot 1 = forward + backward.  A slot keeps
  // the graphs of the last few configurations (buffers, batch size, hyper-parameters), so the
  // ragged last mini-batch of an epoch does not evict the graph of the full ones.
  struct GraphEntry {
    cudaGraphExec_t exec = nullptr;
    int seen = 0;
    unsigned long long kernels = 0;  // kernels recorded in the graph
    unsigned long long last_use = 0;
  };
  struct GraphSlot {
    std::map<std::string, GraphEntry> entries;
    unsigned long long clock = 0;
    void clear() {
      for (auto &kv : entries)
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
      entries.clear();
    }
  } slots[2];
  static constexpr size_t kGraphsPerSlot = 8;
  bool use_graph = true;
};

namespace {

int net_alloc(void **p, size_t bytes) {
  B200_CUDA(cudaMalloc(p, bytes ? bytes : 4));
  B200_CUDA(cudaMemset(*p, 0, bytes ? bytes : 4));
  return 0;
}

bool is_foldable_act(int kind) { return kind == B200_LAYER_RELU || kind == B200_LAYER_TANH; }
int act_of_layer(int kind) {
  if (kind == B200_LAYER_RELU) return B200_ACT_RELU;
  if (kind == B200_LAYER_TANH) return B200_ACT_TANH;
  if (kind == B200_LAYER_SOFTMAX) return B200_ACT_SOFTMAX;
  if (kind == B200_LAYER_SIGMOID) return B200_ACT_SIGMOID;
  if (kind == B200_LAYER_LEAKY_RELU) return B200_ACT_LEAKY_RELU;
  if (kind == B200_LAYER_ELU) return B200_ACT_ELU;
  return B200_ACT_NONE;
}

int net_forward_impl(b200_net *net, const float *x, int B) {
  b200_ctx *ctx = net->ctx;
  const float *in = x;
  size_t n = net->layers.size();
  // The filter matrices of the tensor-core layers depend on the weights only: they are made on the
  // side stream while the first layers compute; each layer waits for its own.
  bool prep_on_side = false;
  if (net->side) {
    cudaStream_t main_stream = ctx->stream;
    // first what the forward pass waits for (the tensor-core layers' filter matrices), then the
    // flipped filter copies of FFMA dX passes, which only the backward pass reads
    for (int pass = 0; pass < 2; ++pass) {
      for (size_t i = 0; i < n; ++i) {
        Layer &L = net->layers[i];
        if (L.kind != B200_LAYER_CONV || !L.ev_prep) continue;
        const bool dx_copy = L.tiled && !L.tc.dx && L.g.OW <= 64 && L.wt_dx && (i > 0 || net->input_grad);
        if (pass == 0) L.dx_prep_side = false;
        if (pass == 0 ? !L.tc.fwd : !dx_copy) continue;
        if (!prep_on_side) {
          B200_CUDA(cudaEventRecord(net->ev_fork, main_stream));
          B200_CUDA(cudaStreamWaitEvent(net->side, net->ev_fork, 0));
          prep_on_side = true;
        }
        ctx->stream = net->side;
        int rc;
        if (pass == 0) {
          rc = conv_tc_prep(ctx, L.g, net->params + L.w_off, L.tc_wt_fwd, L.tc.dx ? L.tc_wt_dx : nullptr);
        } else {
          rc = conv_tiled_dx_prep(ctx, L.g, net->params + L.w_off, L.wt_dx);
          L.dx_prep_side = rc == 0;
        }
        ctx->stream = main_stream;
        B200_TRY(rc);
        B200_CUDA(cudaEventRecord(L.ev_prep, net->side));
      }
    }
  }
  for (size_t i = 0; i < n; ++i) {
    Layer &L = net->layers[i];
    if (L.skipped || (net->head_fc >= 0 && i == n - 1)) {
      in = L.out;  // already written by the previous layer's kernel
      continue;
    }
    float *dst = L.fused_act ? net->layers[i + 1].out : L.out;
    const float *W = net->params + L.w_off;
    const float *b = L.b_len ? net->params + L.b_off : nullptr;
    switch (L.kind) {
      case B200_LAYER_CONV:
        if (L.tc.fwd) {
          if (!L.xs_from_pool) B200_TRY(conv_tc_tall_x(ctx, L.g, in, B, L.tc_xs));
          // the dX pass of this step reads the same weights: both filter matrices in one launch
          if (prep_on_side && L.ev_prep && L.tc.fwd)
            B200_CUDA(cudaStreamWaitEvent(ctx->stream, L.ev_prep, 0));
          else
            B200_TRY(conv_tc_prep(ctx, L.g, W, L.tc_wt_fwd, L.tc.dx ? L.tc_wt_dx : nullptr));
          B200_TRY(conv_tc_fwd(ctx, L.g, L.tc_xs, W, b, dst, B, L.fused_act, L.tc_wt_fwd, 0));
        } else if (L.tc.fwd_small)
          B200_TRY(conv_fwd_small(ctx, L.g, in, W, b, dst, B, L.fused_act));
        else if (L.tiled)
          B200_TRY(conv_tiled_fwd(ctx, L.g, in, W, b, dst, B, L.fused_act, L.wt_fwd));
        else
          B200_TRY(conv_general_fwd(ctx, L.g, in, W, b, dst, B, L.fused_act));
        break;
      case B200_LAYER_FC:
        if ((int)i == net->head_fc)
          B200_TRY(fc_softmax_fwd(ctx, L.fc_in, L.fc_out, in, W, b, dst, net->layers[n - 1].out, B));
        else
          B200_TRY(fc_fwd(ctx, L.fc_in, L.fc_out, in, W, b, dst, B, L.fused_act, L.fc_scratch));
        break;
      case B200_LAYER_MAXPOOL:
        if (L.feeds_conv >= 0) {
          Layer &Cv = net->layers[L.feeds_conv];
          B200_TRY(conv_tc_tall_x_pool(ctx, Cv.g, in, dst, L.argmax, B, Cv.tc_xs));
        } else {
          B200_TRY(maxpool_fwd(ctx, L.pd, in, dst, L.argmax, B));
        }
        break;
      case B200_LAYER_AVGPOOL:
        B200_TRY(avgpool_fwd(ctx, L.pd, in, W, b, dst, B));
        break;
      case B200_LAYER_BATCHNORM:
        B200_TRY(batchnorm_fwd(ctx, L.bn_c, L.bn_s, L.bn_eps, in, net->train_phase ? L.bn_mean_cur : L.bn_mean,
                               net->train_phase ? L.bn_var_cur : L.bn_var, L.bn_stddev, dst, B, net->train_phase ? 1 : 0,
                               L.bn_scratch));
        break;
      case B200_LAYER_RELU:
      case B200_LAYER_TANH:
      case B200_LAYER_SOFTMAX:
      case B200_LAYER_SIGMOID:
      case B200_LAYER_LEAKY_RELU:
      case B200_LAYER_ELU:
        B200_TRY(act_fwd(ctx, act_of_layer(L.kind), in, dst, (int)L.out_dim, B, L.act_param));
        break;
      default: B200_REQUIRE(false, "net_forward: unknown layer kind %d", L.kind);
    }
    in = dst;
  }
  if (prep_on_side) {
    // everything the side stream was given in this pass ends here (a filter copy made for the
    // backward pass has no reader in the forward pass), so a forward pass alone leaves no open branch
    B200_CUDA(cudaEventRecord(net->ev_join, net->side));
    B200_CUDA(cudaStreamWaitEvent(ctx->stream, net->ev_join, 0));
  }
  net->cur_batch = B;
  net->cur_x = x;
  return 0;
}

int net_backward_impl(b200_net *net, const float *t, int loss_kind, bool peer_in_step = false) {
  b200_ctx *ctx = net->ctx;
  int B = net->cur_batch;
  int n = (int)net->layers.size();
  Layer &last = net->layers[n - 1];
  // a softmax output layer: loss gradient and softmax gradient in one launch
  const bool tail_fused = net->fuse && last.kind == B200_LAYER_SOFTMAX && n >= 2;
  if (net->head_fc >= 0) {
    // loss gradient, softmax gradient, the narrow layer's dX and the gradient of a relu in front of
    // it in one launch; the layer's dW / db follow in the loop below
    Layer &F = net->layers[net->head_fc];
    const int first = net->head_relu >= 0 ? net->head_relu : net->head_fc;  // first layer the kernel covers
    float *target = first == 0 ? (net->input_grad ? net->in_grad : nullptr) : net->layers[first - 1].grad;
    B200_TRY(fc_softmax_loss_bwd(ctx, loss_kind, F.fc_in, F.fc_out, last.out, t, net->params + F.w_off,
                                 net->head_relu >= 0 ? net->layers[net->head_relu].out : nullptr, last.grad, F.grad,
                                 target, B));
  } else if (tail_fused)
    B200_TRY(softmax_loss_bwd(ctx, loss_kind, last.out, t, last.grad, net->layers[n - 2].grad, (int)last.out_dim, B));
  else
    B200_TRY(loss_grad(ctx, loss_kind, last.out, t, last.grad, (int)last.out_dim, B));
  // The gradients with respect to the weights are leaves of the backward pass: nothing in it
  // reads them.  They go to the side stream, so the chain of dX kernels -- the critical path --
  // does not wait for them, and kernels that leave SMs idle overlap.  One join at the end.
  cudaStream_t main_stream = ctx->stream;
  bool side_used = false, comm_used = false;
  int rc_side = 0;
  net->early_summed = false;
  // One side branch, not one per layer: the large kernels of both branches each fill the SMs, so
  // more branches only interleave them and delay the dX chain (measured: two branches 0.387 ms
  // against 0.374 ms with one).
  auto fork = [&]() -> int {
    B200_CUDA(cudaEventRecord(net->ev_fork, main_stream));
    B200_CUDA(cudaStreamWaitEvent(net->side, net->ev_fork, 0));
    ctx->stream = net->side;
    side_used = true;
    return 0;
  };
  // The finishing passes of the tensor-core dW kernels (partial rows -> gradient in the reference
  // layout) can be collected and launched together (before the gradients leave for the other
  // replicas, and at the end of the pass) instead of after each dW kernel: B200_NET_BATCH_FINISH=1.
  // Measured slower on the benchmark step (0.335 against 0.323 ms: the one launch then shares the SMs
  // with the first layer's dX), so each pass follows its kernel by default.
  std::vector<DwFinishArgs> finishes;
  auto flush_finishes = [&]() -> int {
    if (finishes.empty()) return 0;
    ctx->stream = net->side;  // they were produced there (fork() ran)
    int rc = dw_finish_many(ctx, finishes.data(), (int)finishes.size());
    ctx->stream = main_stream;
    finishes.clear();
    return rc;
  };
  for (int i = tail_fused ? n - 2 : n - 1; i >= 0 && rc_side == 0; --i) {
    Layer &L = net->layers[i];
    const float *in = i == 0 ? net->cur_x : net->layers[i - 1].out;
    float *din = i == 0 ? (net->input_grad ? net->in_grad : nullptr) : net->layers[i - 1].grad;
    const float *W = net->params + L.w_off;
    float *dW = net->grads + L.w_off;
    float *db = L.b_len ? net->grads + L.b_off : nullptr;
    if (net->head_fc >= 0 && i == net->head_relu) continue;  // its gradient came with the head kernel
    const bool head = i == net->head_fc && net->head_fc >= 0;
    if (head) din = nullptr;                                  // so did this layer's dX
    const bool can_fork = net->side != nullptr && (din != nullptr || head);
    switch (L.kind) {
      case B200_LAYER_CONV: {
        bool tiled_bwd = L.tiled && L.g.OW <= 64;
        const bool tc_dx = L.tc.dx && din != nullptr;
        if ((tc_dx || L.tc.dw) && !L.dys_from_pool)
          B200_TRY(conv_tc_tall_dy(ctx, L.g, L.grad, B, L.tc_dys, L.tc.dw && db ? L.tc_bsum : nullptr));
        // dW first: its launch precedes the dX launch, so a one-block-per-SM dW kernel is resident
        // when the small blocks of an FFMA dX arrive and both share the SMs
        const bool forked = can_fork && (L.tc.dw || L.tc.dw_small);
        const bool batch_fin = forked && net->batch_finishes;
        if (forked) B200_TRY(fork());
        if (L.tc.dw) {
          if (!L.tc.fwd && !L.xs_from_pool) rc_side = conv_tc_tall_x(ctx, L.g, in, B, L.tc_xs);
          int splits = 0;
          if (!rc_side) rc_side = conv_tc_dw(ctx, L.g, L.tc_xs, L.tc_dys, B, L.tc_part, &splits);
          DwFinishArgs later;
          if (!rc_side)
            rc_side = conv_tc_dw_finish(ctx, L.g, L.tc_part, splits, dW, 0, db ? L.tc_bsum : nullptr, B, db,
                                        batch_fin ? &later : nullptr);
          if (!rc_side && batch_fin) finishes.push_back(later);
        } else if (L.tc.dw_small) {
          DwFinishArgs later;
          rc_side = conv_dw_small(ctx, L.g, in, L.grad, B, L.tc_small_part, dW, db, 0, batch_fin ? &later : nullptr);
          if (!rc_side && batch_fin) finishes.push_back(later);
        } else if (tiled_bwd) {
          int splits = 0;
          rc_side = conv_tiled_dw_partials(ctx, L.g, in, L.grad, B, L.dw_part, &splits);
          size_t row = L.w_len + L.g.OC;
          if (!rc_side && db && L.b_off == L.w_off + L.w_len) {
            // [W | b] are neighbours in the bucket as in a partial row: one merge
            rc_side = merge_rows(ctx, L.dw_part, splits, row, dW, row, 0, &L.g);
          } else if (!rc_side) {
            rc_side = merge_rows(ctx, L.dw_part, splits, row, dW, L.w_len, 0, &L.g);
            if (!rc_side && db)
              rc_side = merge_rows(ctx, L.dw_part + L.w_len, splits, row, db, L.b_len, 0, nullptr);
          }
        } else {
          rc_side = conv_general_dw(ctx, L.g, in, L.grad, dW, db, 0, B);
        }
        ctx->stream = main_stream;
        if (rc_side) break;
        if (din) {
          if (tc_dx)
            B200_TRY(conv_tc_dx(ctx, L.g, L.tc_dys, W, din, B, L.tc_wt_dx, L.tc.fwd ? 0 : 1));
          else if (tiled_bwd) {
            // the filter copy was made beside the forward pass (same weights: nothing updates
            // them between the two passes of a step)
            if (L.dx_prep_side) B200_CUDA(cudaStreamWaitEvent(ctx->stream, L.ev_prep, 0));
            B200_TRY(conv_tiled_dx(ctx, L.g, W, L.grad, din, B, L.wt_dx, L.dx_prep_side ? 0 : 1));
          }
          else
            B200_TRY(conv_general_dx(ctx, L.g, W, L.grad, din, B));
        }
        break;
      }
      case B200_LAYER_FC:
        if (can_fork && L.fc_scratch_side) {
          B200_TRY(fork());
          rc_side = fc_bwd(ctx, L.fc_in, L.fc_out, in, W, L.grad, nullptr, dW, db, 0, B, L.fc_scratch_side);
          ctx->stream = main_stream;
          if (rc_side) break;
          B200_TRY(fc_bwd(ctx, L.fc_in, L.fc_out, in, W, L.grad, din, nullptr, nullptr, 0, B, L.fc_scratch));
        } else {
          B200_TRY(fc_bwd(ctx, L.fc_in, L.fc_out, in, W, L.grad, din, dW, db, 0, B, L.fc_scratch));
        }
        break;
      case B200_LAYER_MAXPOOL:
        if (L.grad_to_conv >= 0) {
          // gradient of this layer (and of the relu before it) written straight into the forms the
          // tensor-core convolution reads: tall split copy, CHW gradient, bias partials
          Layer &Cv = net->layers[L.grad_to_conv];
          // the CHW form of the convolution's dY is written only when one of its backward kernels
          // reads it (the tensor-core dW and dX passes read the tall copy)
          const bool cv_din = L.grad_to_conv > 0 || net->input_grad;
          const bool chw_read = !Cv.tc.dw || (cv_din && !Cv.tc.dx) || net->keep_layer_grads;
          B200_TRY(conv_tc_tall_dy_unpool(ctx, Cv.g, L.grad, L.argmax,
                                          L.relu_bwd_fused ? L.out : nullptr,
                                          chw_read ? Cv.grad : nullptr, B, Cv.tc_dys,
                                          Cv.tc.dw && Cv.b_len ? Cv.tc_bsum : nullptr));
        } else if (L.relu_bwd_fused) {
          // the relu before this layer was folded into the producer's epilogue: apply
          // its gradient mask here and write straight into the producer's gradient
          B200_TRY(maxpool_bwd(ctx, L.pd, L.grad, L.argmax, net->layers[i - 2].grad, B, L.out));
        } else if (din) {
          B200_TRY(maxpool_bwd(ctx, L.pd, L.grad, L.argmax, din, B));
        }
        break;
      case B200_LAYER_AVGPOOL:
        B200_TRY(avgpool_bwd(ctx, L.pd, in, W, L.grad, din, dW, db, 0, B));
        break;
      case B200_LAYER_BATCHNORM:
        if (din) B200_TRY(batchnorm_bwd(ctx, L.bn_c, L.bn_s, L.out, L.grad, L.bn_stddev, din, B, L.bn_scratch));
        break;
      case B200_LAYER_RELU:
      case B200_LAYER_TANH:
      case B200_LAYER_SOFTMAX:
      case B200_LAYER_SIGMOID:
      case B200_LAYER_LEAKY_RELU:
      case B200_LAYER_ELU:
        if (L.bwd_done_by_next) break;  // the pooling layer after it already wrote din
        if (din)
          B200_TRY(act_bwd(ctx, act_of_layer(L.kind), L.out, L.grad, din, (int)L.out_dim, B, L.act_param));
        break;
      default: B200_REQUIRE(false, "net_backward: unknown layer kind %d", L.kind);
    }
    if (peer_in_step && i == net->peer_early_layer && rc_side == 0 && net->comm) {
      B200_TRY(flush_finishes());
      // every weight gradient of layers i.. has been issued (main or side stream): send them to
      // the peers now, from a third stream, while the remaining layers still compute
      B200_CUDA(cudaEventRecord(net->ev_comm_main, main_stream));
      B200_CUDA(cudaStreamWaitEvent(net->comm, net->ev_comm_main, 0));
      if (side_used) {
        B200_CUDA(cudaEventRecord(net->ev_comm_side, net->side));
        B200_CUDA(cudaStreamWaitEvent(net->comm, net->ev_comm_side, 0));
      }
      ctx->stream = net->comm;
      int rc = peer_reduce_push_early(ctx, &net->peer, net->grads);
      // ... and add the other ranks' copies as they arrive, still beside the remaining layers
      if (rc == 0 && net->peer_early_sum) {
        rc = peer_reduce_sum_early(ctx, &net->peer, net->grads);
        net->early_summed = rc == 0;
      }
      ctx->stream = main_stream;
      B200_TRY(rc);
      B200_CUDA(cudaEventRecord(net->ev_comm_done, net->comm));
      comm_used = true;
    }
  }
  ctx->stream = main_stream;
  if (rc_side == 0) B200_TRY(flush_finishes());
  if (side_used) {  // the optimizer (or the caller's all-reduce) follows on the main stream
    B200_CUDA(cudaEventRecord(net->ev_join, net->side));
    B200_CUDA(cudaStreamWaitEvent(main_stream, net->ev_join, 0));
  }
  if (comm_used) B200_CUDA(cudaStreamWaitEvent(main_stream, net->ev_comm_done, 0));

  return rc_side;
}

// Adam powers: an optimizer object whose powers currently are (b1_t, b2_t) -- a fresh one has
// (b1, b2) -- gives tensor j of the next step b1_t * b1^j, reached by j sequential float
// multiplies (optimizer.h:104-110,125-126).
int net_init_powers(b200_net *net, float b1, float b2, float b1_t, float b2_t) {
  size_t T = net->segs.size();
  net->pow_host.assign(2 * T + 2, 0.f);
  float p1 = b1_t, p2 = b2_t;
  for (size_t j = 0; j < T; ++j) {
    net->pow_host[2 * j] = p1;
    net->pow_host[2 * j + 1] = p2;
    p1 *= b1;
    p2 *= b2;
  }
  B200_CUDA(cudaMemcpyAsync(net->pow_tab, net->pow_host.data(), sizeof(float) * 2 * T,
                            cudaMemcpyHostToDevice, net->ctx->stream));
  B200_CUDA(cudaStreamSynchronize(net->ctx->stream));
  net->pow_init = true;
  net->pow_b1 = b1;
  net->pow_b2 = b2;
  return 0;
}

int net_update_impl(b200_net *net, int opt_kind, const b200_opt_hyper *h) {
  b200_ctx *ctx = net->ctx;
  int T = (int)net->segs.size();
  // after a reduction over the replicas whose wait ran out the update changes nothing
  const int *skip_if = net->peer.world > 1 ? ctx->dev_err : nullptr;
  B200_TRY(opt_update_segments(ctx, opt_kind, *h, net->grads, net->params, net->state0,
                               net->state1, net->segs_dev, T, net->n_params, net->pow_tab, skip_if));
  // adam and adamax advance their powers once per update call (optimizer.h:125-126, :165)
  if (opt_kind == B200_OPT_ADAM || opt_kind == B200_OPT_ADAMAX)
    B200_TRY(opt_advance_powers(ctx, net->pow_tab, T, h->b1, h->b2, skip_if));
  // layer::update_weight ends with post_update() (layer.h:681): batch normalization moves its averages
  for (Layer &L : net->layers)
    if (L.kind == B200_LAYER_BATCHNORM)
      B200_TRY(batchnorm_post_update(ctx, L.bn_c, L.bn_momentum, L.bn_mean, L.bn_var, L.bn_mean_cur, L.bn_var_cur,
                                     skip_if));
  return 0;
}

int ensure_powers(b200_net *net, int opt_kind, const b200_opt_hyper *h) {
  if ((opt_kind == B200_OPT_ADAM || opt_kind == B200_OPT_ADAMAX) && !net->pow_init)
    B200_TRY(net_init_powers(net, h->b1, h->b2, h->b1, h->b2));
  return 0;
}

int check_net(b200_net *net) {
  B200_REQUIRE(net != nullptr, "net is NULL");
  B200_CUDA(cudaSetDevice(net->ctx->device));
  return 0;
}

int step_eager(b200_net *net, const float *x, const float *t, int B, int loss_kind, int opt_kind,
               const b200_opt_hyper *h) {
  B200_TRY(net_forward_impl(net, x, B));
  const bool peer = net->peer.world > 1;
  const bool early = peer && net->comm && net->peer_early_layer >= 0 && net->peer.split < net->peer.n;
  B200_TRY(net_backward_impl(net, t, loss_kind, early));
  if (peer) {
    if (!early) B200_TRY(peer_reduce_push_early(net->ctx, &net->peer, net->grads));
    B200_TRY(peer_reduce_finish(net->ctx, &net->peer, net->grads, 0, early && net->early_summed));
  }
  B200_TRY(net_update_impl(net, opt_kind, h));
  if (net->fit_out_copy) {  // fit from host buffers: the forward output of this step, for the stream that fetches it
    const Layer &last = net->layers.back();
    B200_CUDA(cudaMemcpyAsync(net->fit_out_copy, last.out, (size_t)B * last.out_dim * sizeof(float),
                              cudaMemcpyDeviceToDevice, net->ctx->stream));
  }
  return 0;
}

}  // namespace

extern "C" {

int b200_net_create(b200_ctx *ctx, const b200_layer_spec *specs, int n_layers, int max_batch,
                    b200_net **out) {
  B200_REQUIRE(ctx && specs && out && n_layers > 0 && max_batch > 0, "net_create: bad argument");
  B200_CUDA(cudaSetDevice(ctx->device));
  b200_net *net = new b200_net();
  net->ctx = ctx;
  net->max_batch = max_batch;
  net->layers.resize(n_layers);
  if (const char *e = getenv("B200_NET_NO_FUSE")) net->fuse = !(e[0] == '1');
  if (const char *e = getenv("B200_NET_BATCH_FINISH")) net->batch_finishes = e[0] == '1';
  if (const char *e = getenv("B200_NET_NO_GRAPH")) net->use_graph = !(e[0] == '1');
  if (const char *e = getenv("B200_NET_KEEP_GRADS")) net->keep_layer_grads = e[0] == '1';
  if (!getenv("B200_NET_NO_SIDE")) {
    cudaStreamCreateWithFlags(&net->side, cudaStreamNonBlocking);
    cudaEventCreateWithFlags(&net->ev_fork, cudaEventDisableTiming);
    cudaEventCreateWithFlags(&net->ev_join, cudaEventDisableTiming);
  }
  size_t off = 0;
  size_t prev_out = 0;
  for (int i = 0; i < n_layers; ++i) {
    Layer &L = net->layers[i];
    const b200_layer_spec &S = specs[i];
    L.kind = S.kind;
    switch (S.kind) {
      case B200_LAYER_CONV: {
        L.cd = S.conv;
        L.cd.input_is_padded = 0;
        if (int r = conv_geom_from_desc(ctx, &L.cd, &L.g)) {
          delete net;
          return r;
        }
        L.in_dim = (size_t)L.g.C * L.g.HI * L.g.WI;
        L.out_dim = (size_t)L.g.OC * L.g.OH * L.g.OW;
        L.w_len = conv_weight_len(L.g);
        L.b_len = L.g.has_bias ? L.g.OC : 0;
        L.tiled = conv_tiled_ok(L.g) && L.cd.algo != 1;
        L.tc = conv_tc_use(ctx, L.g, L.cd.algo);
        break;
      }
      case B200_LAYER_FC:
        L.fc_in = S.fc_in;
        L.fc_out = S.fc_out;
        L.fc_bias = S.fc_has_bias;
        L.in_dim = S.fc_in;
        L.out_dim = S.fc_out;
        L.w_len = (size_t)S.fc_in * S.fc_out;
        L.b_len = S.fc_has_bias ? S.fc_out : 0;
        break;
      case B200_LAYER_MAXPOOL:
      case B200_LAYER_AVGPOOL:
        L.pd = S.pool;
        L.in_dim = (size_t)S.pool.in_c * S.pool.in_h * S.pool.in_w;
        L.out_dim = (size_t)S.pool.in_c * S.pool.out_h * S.pool.out_w;
        if (S.kind == B200_LAYER_AVGPOOL) {
          // weight vector has pool_w*pool_h*C entries (average_pooling_layer.h:231-233)
          L.w_len = (size_t)S.pool.pool_w * S.pool.pool_h * S.pool.in_c;
          L.b_len = S.pool.in_c;
        }
        break;
      case B200_LAYER_RELU:
      case B200_LAYER_TANH:
      case B200_LAYER_SOFTMAX:
      case B200_LAYER_SIGMOID:
      case B200_LAYER_LEAKY_RELU:
      case B200_LAYER_ELU:
        L.in_dim = L.out_dim = prev_out;
        L.act_param = S.act_param;
        break;
      case B200_LAYER_BATCHNORM:
        L.bn_c = S.bn_channels;
        L.bn_s = S.bn_spatial;
        L.bn_eps = S.bn_eps;
        L.bn_momentum = S.bn_momentum;
        if (L.bn_c <= 0 || L.bn_s <= 0) {
          set_error("net_create: batch normalization layer %d has shape %d x %d", i, L.bn_c, L.bn_s);
          delete net;
          return 2;
        }
        L.in_dim = L.out_dim = (size_t)L.bn_c * L.bn_s;
        break;
      default:
        set_error("net_create: unknown layer kind %d at %d", S.kind, i);
        delete net;
        return 2;
    }
    if (i > 0 && L.in_dim != prev_out) {
      set_error("net_create: layer %d expects %zu inputs, previous layer gives %zu", i, L.in_dim,
                prev_out);
      delete net;
      return 2;
    }
    if (L.in_dim == 0 || L.out_dim == 0) {
      set_error("net_create: layer %d has an empty shape", i);
      delete net;
      return 2;
    }
    prev_out = L.out_dim;
    if (L.w_len) {
      L.w_off = off;
      net->segs.push_back({off, L.w_len});
      off += L.w_len;
    }
    if (L.b_len) {
      L.b_off = off;
      net->segs.push_back({off, L.b_len});
      off += L.b_len;
    }
  }
  net->n_params = off;
  // fold relu/tanh into the producing convolution / fully-connected epilogue
  if (net->fuse) {
    for (int i = 0; i + 1 < n_layers; ++i) {
      Layer &L = net->layers[i];
      Layer &N = net->layers[i + 1];
      if ((L.kind == B200_LAYER_CONV || L.kind == B200_LAYER_FC) && is_foldable_act(N.kind)) {
        L.fused_act = act_of_layer(N.kind);
        N.skipped = true;
      }
    }
  }
  // relu -> 2x2 max-pool: the pooling gradient kernel applies the relu mask itself
  if (net->fuse) {
    for (int i = 2; i < n_layers; ++i) {
      Layer &P = net->layers[i];
      Layer &R = net->layers[i - 1];
      if (P.kind == B200_LAYER_MAXPOOL && R.kind == B200_LAYER_RELU && R.skipped &&
          maxpool_can_fuse_relu(P.pd)) {
        P.relu_bwd_fused = true;
        R.bwd_done_by_next = true;
      }
    }
  }
  // narrow fully-connected layer -> softmax output layer: one kernel per direction
  if (net->fuse && n_layers >= 2) {
    Layer &S = net->layers[n_layers - 1];
    Layer &F = net->layers[n_layers - 2];
    if (S.kind == B200_LAYER_SOFTMAX && F.kind == B200_LAYER_FC && fc_softmax_fusable(F.fc_in, F.fc_out)) {
      net->head_fc = n_layers - 2;
      if (n_layers >= 3 && net->layers[n_layers - 3].kind == B200_LAYER_RELU) net->head_relu = n_layers - 3;
    }
  }
  // 2x2 max-pool beside a tensor-core convolution: fuse the tall conversions into the pooling kernels
  if (net->fuse) {
    for (int i = 0; i < n_layers; ++i) {
      Layer &P = net->layers[i];
      if (P.kind != B200_LAYER_MAXPOOL || !maxpool_can_fuse_relu(P.pd)) continue;
      if (i + 1 < n_layers) {
        Layer &N = net->layers[i + 1];
        if (N.kind == B200_LAYER_CONV && (N.tc.fwd || N.tc.dw) && N.g.C == P.pd.in_c &&
            N.g.HI == P.pd.out_h && N.g.WI == P.pd.out_w) {
          P.feeds_conv = i + 1;
          N.xs_from_pool = true;
        }
      }
      int j = P.relu_bwd_fused ? i - 2 : i - 1;
      if (j >= 0 && (P.relu_bwd_fused || !net->layers[i - 1].skipped)) {
        Layer &Cv = net->layers[j];
        if (Cv.kind == B200_LAYER_CONV && (Cv.tc.dx || Cv.tc.dw) && Cv.g.OC == P.pd.in_c &&
            Cv.g.OH == P.pd.in_h && Cv.g.OW == P.pd.in_w && (P.relu_bwd_fused || j == i - 1) &&
            (P.relu_bwd_fused || Cv.fused_act == 0)) {
          P.grad_to_conv = j;
          Cv.dys_from_pool = true;
        }
      }
    }
  }
  // device memory
  size_t f = sizeof(float);
  B200_TRY(net_alloc((void **)&net->params, off * f));
  B200_TRY(net_alloc((void **)&net->grads, off * f));
  B200_TRY(net_alloc((void **)&net->state0, off * f));
  B200_TRY(net_alloc((void **)&net->state1, off * f));
  B200_TRY(net_alloc((void **)&net->segs_dev, sizeof(OptSegment) * (net->segs.size() + 1)));
  B200_CUDA(cudaMemcpy(net->segs_dev, net->segs.data(), sizeof(OptSegment) * net->segs.size(),
                       cudaMemcpyHostToDevice));
  B200_TRY(net_alloc((void **)&net->pow_tab, f * 2 * (net->segs.size() + 1)));
  size_t in0 = net->layers[0].in_dim;
  B200_TRY(net_alloc((void **)&net->in_grad, in0 * max_batch * f));
  B200_TRY(net_alloc((void **)&net->x_dev, in0 * max_batch * f));
  B200_TRY(net_alloc((void **)&net->t_dev, net->layers[n_layers - 1].out_dim * max_batch * f));
  for (int i = 0; i < n_layers; ++i) {
    Layer &L = net->layers[i];
    B200_TRY(net_alloc((void **)&L.out, L.out_dim * max_batch * f));
    if (L.kind == B200_LAYER_BATCHNORM) {
      float **bufs[5] = {&L.bn_mean_cur, &L.bn_var_cur, &L.bn_stddev, &L.bn_mean, &L.bn_var};
      for (float **b : bufs) {  // the reference's init(): all zeros
        B200_TRY(net_alloc((void **)b, (size_t)L.bn_c * f));
        B200_CUDA(cudaMemset(*b, 0, (size_t)L.bn_c * f));
      }
      B200_TRY(net_alloc((void **)&L.bn_scratch, batchnorm_scratch_floats(ctx, L.bn_c, max_batch) * f));
    }
    B200_TRY(net_alloc((void **)&L.grad, L.out_dim * max_batch * f));
    if (L.kind == B200_LAYER_MAXPOOL)
      B200_TRY(net_alloc((void **)&L.argmax, L.out_dim * max_batch * sizeof(int32_t)));
    if (L.kind == B200_LAYER_FC) {
      B200_TRY(net_alloc((void **)&L.fc_scratch,
                         fc_scratch_floats(ctx, L.fc_in, L.fc_out, max_batch) * f));
      if (net->side)
        B200_TRY(net_alloc((void **)&L.fc_scratch_side,
                           fc_scratch_floats(ctx, L.fc_in, L.fc_out, max_batch) * f));
    }
    if (L.kind == B200_LAYER_CONV && L.tiled) {
      B200_TRY(net_alloc((void **)&L.wt_fwd, conv_tiled_fwd_scratch(L.g) * f));
      B200_TRY(net_alloc((void **)&L.wt_dx, conv_tiled_dx_scratch(L.g) * f));
      size_t need = conv_tiled_dw_scratch(ctx, L.g, max_batch);
      B200_TRY(net_alloc((void **)&L.dw_part, need * f));
    }
    if (L.kind == B200_LAYER_CONV && L.tc.dw_small)
      B200_TRY(net_alloc((void **)&L.tc_small_part, conv_dw_small_floats(ctx, L.g, max_batch) * f));
    if (L.kind == B200_LAYER_CONV && (L.tc.fwd || L.tiled) && net->side)
      B200_CUDA(cudaEventCreateWithFlags(&L.ev_prep, cudaEventDisableTiming));
    if (L.kind == B200_LAYER_CONV && (L.tc.fwd || L.tc.dx || L.tc.dw)) {
      if (L.tc.fwd || L.tc.dw)
        B200_TRY(net_alloc((void **)&L.tc_xs, conv_tc_tall_floats(L.g, max_batch, 0) * f));
      if (L.tc.dx || L.tc.dw)
        B200_TRY(net_alloc((void **)&L.tc_dys, conv_tc_tall_floats(L.g, max_batch, 1) * f));
      if (L.tc.fwd) B200_TRY(net_alloc((void **)&L.tc_wt_fwd, conv_tc_filter_floats(ctx, L.g, 0) * f));
      if (L.tc.dx) B200_TRY(net_alloc((void **)&L.tc_wt_dx, conv_tc_filter_floats(ctx, L.g, 1) * f));
      if (L.tc.dw) {
        B200_TRY(net_alloc((void **)&L.tc_part, conv_tc_dw_floats(ctx, L.g, max_batch) * f));
        B200_TRY(net_alloc((void **)&L.tc_bsum, (size_t)conv_tc_bsum_rows(L.g, max_batch) * L.g.OC * f + 64));
      }
    }
  }
  *out = net;
  return 0;
}

int b200_net_destroy(b200_net *net) {
  if (!net) return 0;
  cudaSetDevice(net->ctx->device);
  cudaStreamSynchronize(net->ctx->stream);
  for (auto &slot : net->slots) slot.clear();
  for (auto &L : net->layers) {
    cudaFree(L.out);
    cudaFree(L.grad);
    cudaFree(L.argmax);
    cudaFree(L.bn_mean_cur);
    cudaFree(L.bn_var_cur);
    cudaFree(L.bn_stddev);
    cudaFree(L.bn_mean);
    cudaFree(L.bn_var);
    cudaFree(L.bn_scratch);
    cudaFree(L.wt_fwd);
    cudaFree(L.wt_dx);
    if (L.ev_prep) cudaEventDestroy(L.ev_prep);
    cudaFree(L.dw_part);
    cudaFree(L.fc_scratch_side);
    cudaFree(L.tc_xs);
    cudaFree(L.tc_dys);
    cudaFree(L.tc_bsum);
    cudaFree(L.tc_wt_fwd);
    cudaFree(L.tc_wt_dx);
    cudaFree(L.tc_part);
    cudaFree(L.tc_small_part);
    cudaFree(L.fc_scratch);
  }
  cudaFree(net->params);
  cudaFree(net->grads);
  cudaFree(net->state0);
  cudaFree(net->state1);
  cudaFree(net->segs_dev);
  cudaFree(net->pow_tab);
  cudaFree(net->in_grad);
  for (int i = 0; i < 2; ++i) {
    cudaFree(net->x_stage[i]);
    cudaFree(net->t_stage[i]);
    cudaFree(net->u8_stage[i]);
    cudaFree(net->label_stage[i]);
    if (net->up_done[i]) cudaEventDestroy(net->up_done[i]);
    if (net->stage_free[i]) cudaEventDestroy(net->stage_free[i]);
    cudaFree(net->out_stage[i]);
    if (net->step_done[i]) cudaEventDestroy(net->step_done[i]);
    if (net->d2h_done[i]) cudaEventDestroy(net->d2h_done[i]);
  }
  if (net->copy_stream) cudaStreamDestroy(net->copy_stream);
  if (net->d2h_stream) cudaStreamDestroy(net->d2h_stream);
  peer_reduce_free(&net->peer);
  if (net->comm) cudaStreamDestroy(net->comm);
  if (net->ev_comm_main) cudaEventDestroy(net->ev_comm_main);
  if (net->ev_comm_side) cudaEventDestroy(net->ev_comm_side);
  if (net->ev_comm_done) cudaEventDestroy(net->ev_comm_done);
  if (net->side) cudaStreamDestroy(net->side);
  if (net->ev_fork) cudaEventDestroy(net->ev_fork);
  if (net->ev_join) cudaEventDestroy(net->ev_join);
  cudaFree(net->x_dev);
  cudaFree(net->t_dev);
  delete net;
  return 0;
}

size_t b200_net_param_count(const b200_net *net) { return net ? net->n_params : 0; }
int b200_net_tensor_count(const b200_net *net) { return net ? (int)net->segs.size() : 0; }
int b200_net_tensor_info(const b200_net *net, int i, size_t *offset, size_t *len) {
  B200_REQUIRE(net && i >= 0 && i < (int)net->segs.size(), "net_tensor_info: index out of range");
  if (offset) *offset = net->segs[i].offset;
  if (len) *len = net->segs[i].len;
  return 0;
}
int b200_net_in_dim(const b200_net *net) { return net ? (int)net->layers.front().in_dim : 0; }
int b200_net_out_dim(const b200_net *net) { return net ? (int)net->layers.back().out_dim : 0; }

int b200_net_set_params(b200_net *net, const float *host_params) {
  B200_TRY(check_net(net));
  B200_CUDA(cudaMemcpyAsync(net->params, host_params, net->n_params * sizeof(float),
                            cudaMemcpyHostToDevice, net->ctx->stream));
  B200_CUDA(cudaStreamSynchronize(net->ctx->stream));
  return 0;
}
int b200_net_get_params(b200_net *net, float *host_params) {
  B200_TRY(check_net(net));
  B200_CUDA(cudaMemcpyAsync(host_params, net->params, net->n_params * sizeof(float),
                            cudaMemcpyDeviceToHost, net->ctx->stream));
  B200_CUDA(cudaStreamSynchronize(net->ctx->stream));
  return 0;
}
int b200_net_get_grads(b200_net *net, float *host_grads) {
  B200_TRY(check_net(net));
  B200_CUDA(cudaMemcpyAsync(host_grads, net->grads, net->n_params * sizeof(float),
                            cudaMemcpyDeviceToHost, net->ctx->stream));
  B200_CUDA(cudaStreamSynchronize(net->ctx->stream));
  return 0;
}

float *b200_net_params_ptr(b200_net *net) { return net ? net->params : nullptr; }
float *b200_net_grads_ptr(b200_net *net) { return net ? net->grads : nullptr; }
float *b200_net_output_ptr(b200_net *net) { return net ? net->layers.back().out : nullptr; }
float *b200_net_layer_out_ptr(b200_net *net, int i) {
  if (!net || i < 0 || i >= (int)net->layers.size()) return nullptr;
  // a layer whose activation was folded away never materialises its own output
  if (net->layers[i].fused_act) return nullptr;
  return net->layers[i].out;
}
float *b200_net_layer_grad_ptr(b200_net *net, int i) {
  if (!net || i < -1 || i >= (int)net->layers.size()) return nullptr;
  if (i == -1) return net->in_grad;
  return net->layers[i].grad;
}

int b200_net_forward(b200_net *net, const float *x, int batch) {
  B200_TRY(check_net(net));
  B200_REQUIRE(x != nullptr, "net_forward: x is NULL");
  B200_REQUIRE(batch >= 1 && batch <= net->max_batch, "net_forward: batch %d outside 1..%d", batch,
               net->max_batch);
  return net_forward_impl(net, x, batch);
}

int b200_net_backward(b200_net *net, const float *t, int loss_kind) {
  B200_TRY(check_net(net));
  B200_REQUIRE(t != nullptr, "net_backward: t is NULL");
  B200_REQUIRE(net->cur_batch > 0, "net_backward: no forward pass to differentiate");
  return net_backward_impl(net, t, loss_kind);
}

int b200_net_set_phase(b200_net *net, int train) {
  B200_TRY(check_net(net));
  net->train_phase = train != 0;
  return 0;
}

int b200_net_set_input_grad(b200_net *net, int on) {
  B200_TRY(check_net(net));
  if (net->input_grad != (on != 0)) {
    net->input_grad = on != 0;
    for (auto &slot : net->slots) slot.clear();  // the step's launch sequence changes
  }
  return 0;
}

int b200_net_bn_stats(b200_net *net, int layer, float *mean, float *variance, int set) {
  B200_TRY(check_net(net));
  B200_REQUIRE(layer >= 0 && layer < (int)net->layers.size() && net->layers[layer].kind == B200_LAYER_BATCHNORM,
               "net_bn_stats: layer %d is not a batch normalization layer", layer);
  B200_REQUIRE(mean && variance, "net_bn_stats: NULL argument");
  Layer &L = net->layers[layer];
  const size_t bytes = (size_t)L.bn_c * sizeof(float);
  cudaStream_t st = net->ctx->stream;
  if (set) {
    B200_CUDA(cudaMemcpyAsync(L.bn_mean, mean, bytes, cudaMemcpyHostToDevice, st));
    B200_CUDA(cudaMemcpyAsync(L.bn_var, variance, bytes, cudaMemcpyHostToDevice, st));
  } else {
    B200_CUDA(cudaMemcpyAsync(mean, L.bn_mean, bytes, cudaMemcpyDeviceToHost, st));
    B200_CUDA(cudaMemcpyAsync(variance, L.bn_var, bytes, cudaMemcpyDeviceToHost, st));
  }
  B200_CUDA(cudaStreamSynchronize(st));
  return 0;
}

int b200_net_opt_reset(b200_net *net, int reset_powers) {
  B200_TRY(check_net(net));
  size_t bytes = net->n_params * sizeof(float);
  B200_CUDA(cudaMemsetAsync(net->state0, 0, bytes, net->ctx->stream));
  B200_CUDA(cudaMemsetAsync(net->state1, 0, bytes, net->ctx->stream));
  if (reset_powers) net->pow_init = false;
  return 0;
}

// The first layer with parameters finishes its gradients last; everything after it in the
// bucket can leave early.  The boundary is rounded up to 16 bytes (entries below it that are
// ready early simply travel with the late part).
static long long peer_split_of(const b200_net *net, int *early_layer) {
  int first = -1, second = -1;
  for (int i = 0; i < (int)net->layers.size(); ++i) {
    if (net->layers[i].w_len == 0 && net->layers[i].b_len == 0) continue;
    if (first < 0) first = i;
    else if (second < 0) second = i;
  }
  long long n = (long long)net->n_params, split = n;
  if (second >= 0) {
    const Layer &L = net->layers[second];
    split = (long long)((L.w_len ? L.w_off : L.b_off) + 3) / 4 * 4;
    if (split > n) split = n;
  }
  if (early_layer) *early_layer = split < n ? second : -1;
  return split;
}

size_t b200_net_peer_reduce_bytes(b200_net *net, int world) {
  if (!net || world < 2) return 0;
  return peer_reduce_bytes((long long)net->n_params, peer_split_of(net, nullptr), world);
}

int b200_net_peer_reduce_init(b200_net *net, int rank, int world, const unsigned long long *buffers,
                              int timeout_ms) {
  B200_TRY(check_net(net));
  const long long n = (long long)net->n_params;
  const long long split = peer_split_of(net, &net->peer_early_layer);
  B200_TRY(peer_reduce_init(net->ctx, &net->peer, n, split, rank, world, buffers, timeout_ms));
  if (const char *e = getenv("B200_PEER_EARLY_SUM")) net->peer_early_sum = atoi(e) != 0;
  if (!net->comm) {
    B200_CUDA(cudaStreamCreateWithFlags(&net->comm, cudaStreamNonBlocking));
    B200_CUDA(cudaEventCreateWithFlags(&net->ev_comm_main, cudaEventDisableTiming));
    B200_CUDA(cudaEventCreateWithFlags(&net->ev_comm_side, cudaEventDisableTiming));
    B200_CUDA(cudaEventCreateWithFlags(&net->ev_comm_done, cudaEventDisableTiming));
  }
  // the step's launch sequence changes: captured graphs are rebuilt
  for (auto &slot : net->slots) slot.clear();
  return 0;
}

int b200_net_peer_reduce(b200_net *net) {
  B200_TRY(check_net(net));
  B200_REQUIRE(net->peer.world > 1, "net_peer_reduce: b200_net_peer_reduce_init was not called");
  return peer_reduce_run(net->ctx, &net->peer, net->grads);
}

int b200_net_peer_push(b200_net *net) {
  B200_TRY(check_net(net));
  B200_REQUIRE(net->peer.world > 1, "net_peer_push: b200_net_peer_reduce_init was not called");
  return peer_reduce_push_all(net->ctx, &net->peer, net->grads);
}

int b200_net_peer_sum(b200_net *net) {
  B200_TRY(check_net(net));
  B200_REQUIRE(net->peer.world > 1, "net_peer_sum: b200_net_peer_reduce_init was not called");
  return peer_reduce_finish(net->ctx, &net->peer, net->grads, 1, 0);
}

int b200_net_update(b200_net *net, int opt_kind, const b200_opt_hyper *h) {
  B200_TRY(check_net(net));
  B200_REQUIRE(h != nullptr, "net_update: hyper-parameters are NULL");
  B200_TRY(ensure_powers(net, opt_kind, h));
  return net_update_impl(net, opt_kind, h);
}

int b200_net_set_adam_powers(b200_net *net, float b1, float b2, float b1_t, float b2_t) {
  B200_TRY(check_net(net));
  return net_init_powers(net, b1, b2, b1_t, b2_t);
}

static int opt_state_ptr(b200_net *net, int which, float **p) {
  B200_REQUIRE(which == 0 || which == 1, "optimizer state %d: there are two state buffers, 0 and 1", which);
  *p = which == 0 ? net->state0 : net->state1;
  return 0;
}

int b200_net_get_opt_state(b200_net *net, int which, float *host_state) {
  B200_TRY(check_net(net));
  B200_REQUIRE(host_state != nullptr, "net_get_opt_state: NULL buffer");
  float *src = nullptr;
  B200_TRY(opt_state_ptr(net, which, &src));
  B200_CUDA(cudaMemcpyAsync(host_state, src, net->n_params * sizeof(float), cudaMemcpyDeviceToHost,
                            net->ctx->stream));
  B200_CUDA(cudaStreamSynchronize(net->ctx->stream));
  return 0;
}

int b200_net_set_opt_state(b200_net *net, int which, const float *host_state) {
  B200_TRY(check_net(net));
  B200_REQUIRE(host_state != nullptr, "net_set_opt_state: NULL buffer");
  float *dst = nullptr;
  B200_TRY(opt_state_ptr(net, which, &dst));
  B200_CUDA(cudaMemcpyAsync(dst, host_state, net->n_params * sizeof(float), cudaMemcpyHostToDevice,
                            net->ctx->stream));
  B200_CUDA(cudaStreamSynchronize(net->ctx->stream));
  return 0;
}

int b200_net_adam_powers(const b200_net *net, float *b1_t, float *b2_t) {
  B200_REQUIRE(net != nullptr, "net is NULL");
  size_t T = net->segs.size();
  std::vector<float> tab(2 * T + 2, 0.f);
  if (net->pow_init) {
    B200_CUDA(cudaStreamSynchronize(net->ctx->stream));
    B200_CUDA(cudaMemcpy(tab.data(), net->pow_tab, sizeof(float) * 2 * T, cudaMemcpyDeviceToHost));
  }
  // entry 0 is what the NEXT update call of the first tensor will use
  if (b1_t) *b1_t = tab[0];
  if (b2_t) *b2_t = tab[1];
  return 0;
}

}  // extern "C"

// Runs `body` (a sequence of launches on the context stream) directly the first
// time a configuration `key` is seen, captures it into a CUDA graph the second
// time, and replays the graph afterwards.
template <typename F>
static int run_captured(b200_net *net, int slot_idx, const std::string &key, F body) {
  if (!net->use_graph) return body();
  b200_net::GraphSlot &table = net->slots[slot_idx];
  auto it = table.entries.find(key);
  if (it == table.entries.end()) {
    if (table.entries.size() >= b200_net::kGraphsPerSlot) {  // drop the configuration used longest ago
      auto victim = table.entries.begin();
      for (auto e = table.entries.begin(); e != table.entries.end(); ++e)
        if (e->second.last_use < victim->second.last_use) victim = e;
      if (victim->second.exec) B200_CUDA(cudaGraphExecDestroy(victim->second.exec));
      table.entries.erase(victim);
    }
    it = table.entries.emplace(key, b200_net::GraphEntry()).first;
  }
  b200_net::GraphEntry &slot = it->second;
  slot.last_use = ++table.clock;
  cudaStream_t st = net->ctx->stream;
  if (slot.exec) {
    B200_CUDA(cudaGraphLaunch(slot.exec, st));
    g_launches.fetch_add(slot.kernels, std::memory_order_relaxed);
    return 0;
  }
  if (slot.seen++ == 0) return body();  // sets kernel attributes; nothing allocates afterwards
  cudaGraph_t graph = nullptr;
  unsigned long long before = g_launches.load();
  B200_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed));
  int r = body();
  cudaError_t ce = cudaStreamEndCapture(st, &graph);
  unsigned long long recorded = g_launches.load() - before;
  if (r != 0) {
    if (graph) cudaGraphDestroy(graph);
    return r;
  }
  if (ce != cudaSuccess) {
    set_error("stream capture failed: %s", cudaGetErrorString(ce));
    return 1;
  }
  B200_CUDA(cudaGraphInstantiate(&slot.exec, graph, 0));
  B200_CUDA(cudaGraphDestroy(graph));
  slot.kernels = recorded;
  B200_CUDA(cudaGraphLaunch(slot.exec, st));
  return 0;
}

static std::string step_key(const float *x, const float *t, int batch, int loss_kind, int opt_kind,
                            const b200_opt_hyper *h) {
  std::string key;
  key.append(reinterpret_cast<const char *>(&x), sizeof(x));
  key.append(reinterpret_cast<const char *>(&t), sizeof(t));
  key.append(reinterpret_cast<const char *>(&batch), sizeof(batch));
  key.append(reinterpret_cast<const char *>(&loss_kind), sizeof(loss_kind));
  key.append(reinterpret_cast<const char *>(&opt_kind), sizeof(opt_kind));
  if (h) key.append(reinterpret_cast<const char *>(h), sizeof(*h));
  return key;
}
// the phase decides which kernels a batch normalization layer launches
static std::string step_key(const b200_net *net, const float *x, const float *t, int batch, int loss_kind,
                            int opt_kind, const b200_opt_hyper *h) {
  std::string key = step_key(x, t, batch, loss_kind, opt_kind, h);
  key.push_back(net->train_phase ? 't' : 'e');
  key.append(reinterpret_cast<const char *>(&net->fit_out_copy), sizeof(net->fit_out_copy));
  return key;
}

// Rows a step of network::fit runs on when `nb` new samples are left (network.h:883-926).  The
// reference copies the new samples over the first rows of its batch buffers in_batch_ / t_batch_
// (members sized to the mini-batch once per fit) and then runs forward / backward on the WHOLE
// buffers, so a last mini-batch of 1 < nb < batch samples is a full step whose rows nb.. are
// still the previous step's rows nb..; a single left-over sample takes train_once's one-sample
// branch instead.  The device keeps the same rows in x_dev / t_dev between steps (and between fit
// calls, like the members), so copying only the new rows reproduces it.
static int fit_step_rows(b200_net *net, int nb, int batch, int *rows) {
  if (nb == batch || nb == 1) {
    *rows = nb;
    return 0;
  }
  B200_REQUIRE(net->fit_rows == batch,
               "fit: %d samples for mini-batches of %d and no earlier full mini-batch to complete the step from "
               "(the reference reads unset rows of its batch buffers in this case)", nb, batch);
  *rows = batch;
  return 0;
}

// x_dev / t_dev receive the rows of the latest full mini-batch when a staging buffer holds them
static int fit_rows_to_fixed(b200_net *net) {
  if (net->fit_last < 0) return 0;
  const int batch = net->fit_rows;  // a staging buffer only ever holds a full mini-batch of the last step
  const size_t in_dim = net->layers.front().in_dim, out_dim = net->layers.back().out_dim;
  cudaStream_t st = net->ctx->stream;
  B200_CUDA(cudaMemcpyAsync(net->x_dev, net->x_stage[net->fit_last], in_dim * batch * sizeof(float),
                            cudaMemcpyDeviceToDevice, st));
  B200_CUDA(cudaMemcpyAsync(net->t_dev, net->t_stage[net->fit_last], out_dim * batch * sizeof(float),
                            cudaMemcpyDeviceToDevice, st));
  // the next upload into that staging buffer must come after these copies, not only after its step
  B200_CUDA(cudaEventRecord(net->stage_free[net->fit_last], st));
  net->fit_last = -1;
  return 0;
}

extern "C" {

int b200_net_train_step(b200_net *net, const float *x, const float *t, int batch, int loss_kind,
                        int opt_kind, const b200_opt_hyper *h) {
  B200_TRY(check_net(net));
  B200_REQUIRE(x && t && h, "net_train_step: NULL argument");
  B200_REQUIRE(batch >= 1 && batch <= net->max_batch, "net_train_step: batch %d outside 1..%d",
               batch, net->max_batch);
  B200_TRY(ensure_powers(net, opt_kind, h));
  int r = run_captured(net, 0, step_key(net, x, t, batch, loss_kind, opt_kind, h), [&]() {
    return step_eager(net, x, t, batch, loss_kind, opt_kind, h);
  });
  net->cur_batch = batch;
  net->cur_x = x;
  return r;
}

int b200_net_forward_backward(b200_net *net, const float *x, const float *t, int batch,
                              int loss_kind) {
  B200_TRY(check_net(net));
  B200_REQUIRE(x && t, "net_forward_backward: NULL argument");
  B200_REQUIRE(batch >= 1 && batch <= net->max_batch,
               "net_forward_backward: batch %d outside 1..%d", batch, net->max_batch);
  int r = run_captured(net, 1, step_key(net, x, t, batch, loss_kind, -1, nullptr), [&]() {
    B200_TRY(net_forward_impl(net, x, batch));
    return net_backward_impl(net, t, loss_kind);
  });
  net->cur_batch = batch;
  net->cur_x = x;
  return r;
}

int b200_net_train_step_host(b200_net *net, const float *x_host, const float *t_host, int batch,
                             int loss_kind, int opt_kind, const b200_opt_hyper *h,
                             float *out_host) {
  B200_TRY(check_net(net));
  B200_REQUIRE(x_host && t_host && h, "net_train_step_host: NULL argument");
  B200_REQUIRE(batch >= 1 && batch <= net->max_batch,
               "net_train_step_host: batch %d outside 1..%d", batch, net->max_batch);
  cudaStream_t st = net->ctx->stream;
  size_t in_dim = net->layers.front().in_dim, out_dim = net->layers.back().out_dim;
  B200_CUDA(cudaMemcpyAsync(net->x_dev, x_host, in_dim * batch * sizeof(float),
                            cudaMemcpyHostToDevice, st));
  B200_CUDA(cudaMemcpyAsync(net->t_dev, t_host, out_dim * batch * sizeof(float),
                            cudaMemcpyHostToDevice, st));
  B200_TRY(b200_net_train_step(net, net->x_dev, net->t_dev, batch, loss_kind, opt_kind, h));
  net->fit_rows = batch;
  if (out_host)
    B200_CUDA(cudaMemcpyAsync(out_host, net->layers.back().out, out_dim * batch * sizeof(float),
                              cudaMemcpyDeviceToHost, st));
  B200_CUDA(cudaStreamSynchronize(st));
  return 0;
}

int b200_net_fit_host_wait(b200_net *net) {
  B200_TRY(check_net(net));
  if (net->copy_stream) B200_CUDA(cudaStreamSynchronize(net->copy_stream));
  B200_CUDA(cudaStreamSynchronize(net->ctx->stream));
  if (net->d2h_stream) B200_CUDA(cudaStreamSynchronize(net->d2h_stream));
  return 0;
}

int b200_net_fit_host(b200_net *net, const float *x_host, const float *t_host, long long n_samples,
                      int batch, int epochs, int loss_kind, int opt_kind, const b200_opt_hyper *h,
                      float *out_host) {
  const int rc = b200_net_fit_host_enqueue(net, x_host, t_host, n_samples, batch, epochs, loss_kind, opt_kind, h, out_host);
  if (rc != 0) {  // what was queued before the failure still reads the caller's arrays
    if (net && net->ctx) cudaStreamSynchronize(net->ctx->stream);
    return rc;
  }
  return b200_net_fit_host_wait(net);
}

int b200_net_fit_host_enqueue(b200_net *net, const float *x_host, const float *t_host, long long n_samples,
                              int batch, int epochs, int loss_kind, int opt_kind, const b200_opt_hyper *h,
                              float *out_host) {
  B200_TRY(check_net(net));
  B200_REQUIRE(x_host && t_host && h, "net_fit_host: NULL argument");
  B200_REQUIRE(batch >= 1 && batch <= net->max_batch, "net_fit_host: batch %d outside 1..%d", batch,
               net->max_batch);
  B200_REQUIRE(n_samples >= 0 && epochs >= 0, "net_fit_host: negative count");
  cudaStream_t st = net->ctx->stream;
  const size_t in_dim = net->layers.front().in_dim, out_dim = net->layers.back().out_dim;
  if (!net->copy_stream) {
    B200_CUDA(cudaStreamCreateWithFlags(&net->copy_stream, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
      B200_TRY(net_alloc((void **)&net->x_stage[i], in_dim * net->max_batch * sizeof(float)));
      B200_TRY(net_alloc((void **)&net->t_stage[i], out_dim * net->max_batch * sizeof(float)));
      B200_CUDA(cudaEventCreateWithFlags(&net->up_done[i], cudaEventDisableTiming));
      B200_CUDA(cudaEventCreateWithFlags(&net->stage_free[i], cudaEventDisableTiming));
    }
  }
  if (!net->d2h_stream) {
    B200_CUDA(cudaStreamCreateWithFlags(&net->d2h_stream, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
      B200_TRY(net_alloc((void **)&net->out_stage[i], out_dim * net->max_batch * sizeof(float)));
      B200_CUDA(cudaEventCreateWithFlags(&net->step_done[i], cudaEventDisableTiming));
      B200_CUDA(cudaEventCreateWithFlags(&net->d2h_done[i], cudaEventDisableTiming));
    }
  }
  // A full mini-batch runs where its upload left it (the library keeps one captured step per input
  // address, so two staging buffers mean two graphs) and its output is fetched by a third stream
  // from a copy the step makes: the compute stream carries graph after graph.  A short last
  // mini-batch goes through x_dev / t_dev, which first receive the rows of the latest full one.
  for (int e = 0; e < epochs; ++e) {
    for (long long i = 0; i < n_samples; i += batch) {
      const int nb = (int)((n_samples - i) < batch ? (n_samples - i) : batch);  // new rows of this step
      int run_nb = 0;
      B200_TRY(fit_step_rows(net, nb, batch, &run_nb));
      const int buf = (int)(net->fit_toggle++ & 1u);
      if (net->stage_used[buf]) B200_CUDA(cudaStreamWaitEvent(net->copy_stream, net->stage_free[buf], 0));
      net->stage_used[buf] = true;
      B200_CUDA(cudaMemcpyAsync(net->x_stage[buf], x_host + (size_t)i * in_dim, in_dim * nb * sizeof(float),
                                cudaMemcpyHostToDevice, net->copy_stream));
      B200_CUDA(cudaMemcpyAsync(net->t_stage[buf], t_host + (size_t)i * out_dim, out_dim * nb * sizeof(float),
                                cudaMemcpyHostToDevice, net->copy_stream));
      B200_CUDA(cudaEventRecord(net->up_done[buf], net->copy_stream));
      B200_CUDA(cudaStreamWaitEvent(st, net->up_done[buf], 0));
      if (nb == batch) {
        if (out_host && net->out_stage_used[buf]) B200_CUDA(cudaStreamWaitEvent(st, net->d2h_done[buf], 0));
        net->fit_out_copy = out_host ? net->out_stage[buf] : nullptr;
        int rc = b200_net_train_step(net, net->x_stage[buf], net->t_stage[buf], batch, loss_kind, opt_kind, h);
        net->fit_out_copy = nullptr;
        B200_TRY(rc);
        B200_CUDA(cudaEventRecord(net->stage_free[buf], st));  // the step reads its input to the end (first layer's dW)
        if (out_host) {
          net->out_stage_used[buf] = true;
          B200_CUDA(cudaStreamWaitEvent(net->d2h_stream, net->stage_free[buf], 0));
          B200_CUDA(cudaMemcpyAsync(out_host + (size_t)i * out_dim, net->out_stage[buf], out_dim * nb * sizeof(float),
                                    cudaMemcpyDeviceToHost, net->d2h_stream));
          B200_CUDA(cudaEventRecord(net->d2h_done[buf], net->d2h_stream));
        }
        net->fit_last = buf;
      } else {
        B200_TRY(fit_rows_to_fixed(net));
        B200_CUDA(cudaMemcpyAsync(net->x_dev, net->x_stage[buf], in_dim * nb * sizeof(float),
                                  cudaMemcpyDeviceToDevice, st));
        B200_CUDA(cudaMemcpyAsync(net->t_dev, net->t_stage[buf], out_dim * nb * sizeof(float),
                                  cudaMemcpyDeviceToDevice, st));
        B200_CUDA(cudaEventRecord(net->stage_free[buf], st));
        B200_TRY(b200_net_train_step(net, net->x_dev, net->t_dev, run_nb, loss_kind, opt_kind, h));
        if (out_host)
          B200_CUDA(cudaMemcpyAsync(out_host + (size_t)i * out_dim, net->layers.back().out,
                                    out_dim * nb * sizeof(float), cudaMemcpyDeviceToHost, st));
      }
      net->fit_rows = run_nb;
    }
  }
  return 0;
}

int b200_net_fit_u8_host(b200_net *net, const b200_image_desc *d, const uint8_t *images_host,
                         const uint8_t *labels_host, long long n_samples, int batch, int epochs, float target_min,
                         float target_max, int loss_kind, int opt_kind, const b200_opt_hyper *h, float *out_host) {
  B200_TRY(check_net(net));
  B200_TRY(check_image_desc(d));
  B200_REQUIRE(images_host && labels_host && h, "net_fit_u8_host: NULL argument");
  B200_REQUIRE(batch >= 1 && batch <= net->max_batch, "net_fit_u8_host: batch %d outside 1..%d", batch,
               net->max_batch);
  B200_REQUIRE(n_samples >= 0 && epochs >= 0, "net_fit_u8_host: negative count");
  const size_t in_dim = net->layers.front().in_dim, out_dim = net->layers.back().out_dim;
  const size_t img_bytes = image_in_len(d);
  B200_REQUIRE(image_out_len(d) == in_dim, "net_fit_u8_host: padded images have %zu values, the network reads %zu",
               image_out_len(d), in_dim);
  for (long long i = 0; i < n_samples; ++i)
    B200_REQUIRE(labels_host[i] < out_dim, "net_fit_u8_host: label %d of sample %lld outside the %zu network outputs",
                 (int)labels_host[i], i, out_dim);
  cudaStream_t st = net->ctx->stream;
  if (!net->copy_stream) {
    B200_CUDA(cudaStreamCreateWithFlags(&net->copy_stream, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
      B200_TRY(net_alloc((void **)&net->x_stage[i], in_dim * net->max_batch * sizeof(float)));
      B200_TRY(net_alloc((void **)&net->t_stage[i], out_dim * net->max_batch * sizeof(float)));
      B200_CUDA(cudaEventCreateWithFlags(&net->up_done[i], cudaEventDisableTiming));
      B200_CUDA(cudaEventCreateWithFlags(&net->stage_free[i], cudaEventDisableTiming));
    }
  }
  if (net->u8_stage_bytes < img_bytes * net->max_batch) {
    B200_CUDA(cudaStreamSynchronize(st));
    for (int i = 0; i < 2; ++i) {
      cudaFree(net->u8_stage[i]);
      cudaFree(net->label_stage[i]);
      net->u8_stage[i] = net->label_stage[i] = nullptr;
      B200_TRY(net_alloc((void **)&net->u8_stage[i], img_bytes * net->max_batch));
      B200_TRY(net_alloc((void **)&net->label_stage[i], (size_t)net->max_batch));
    }
    net->u8_stage_bytes = img_bytes * net->max_batch;
  }
  long long step = 0;
  for (int e = 0; e < epochs; ++e) {
    for (long long i = 0; i < n_samples; i += batch, ++step) {
      const int nb = (int)((n_samples - i) < batch ? (n_samples - i) : batch);
      int run_nb = 0;
      B200_TRY(fit_step_rows(net, nb, batch, &run_nb));
      const int buf = (int)(step & 1);
      if (step >= 2) B200_CUDA(cudaStreamWaitEvent(net->copy_stream, net->stage_free[buf], 0));
      B200_CUDA(cudaMemcpyAsync(net->u8_stage[buf], images_host + (size_t)i * img_bytes, img_bytes * nb,
                                cudaMemcpyHostToDevice, net->copy_stream));
      B200_CUDA(cudaMemcpyAsync(net->label_stage[buf], labels_host + i, (size_t)nb, cudaMemcpyHostToDevice,
                                net->copy_stream));
      B200_CUDA(cudaEventRecord(net->up_done[buf], net->copy_stream));
      B200_CUDA(cudaStreamWaitEvent(st, net->up_done[buf], 0));
      B200_TRY(fit_rows_to_fixed(net));
      // scale / pad the bytes into the step's fixed input rows, labels into its target rows
      B200_TRY(images_u8_to_float(net->ctx, d, net->u8_stage[buf], nb, net->x_dev));
      B200_TRY(labels_to_targets(net->ctx, net->label_stage[buf], nb, (int)out_dim, target_min, target_max,
                                 net->t_dev));
      B200_CUDA(cudaEventRecord(net->stage_free[buf], st));
      B200_TRY(b200_net_train_step(net, net->x_dev, net->t_dev, run_nb, loss_kind, opt_kind, h));
      net->fit_rows = run_nb;
      if (out_host)
        B200_CUDA(cudaMemcpyAsync(out_host + (size_t)i * out_dim, net->layers.back().out,
                                  out_dim * nb * sizeof(float), cudaMemcpyDeviceToHost, st));
    }
  }
  B200_CUDA(cudaStreamSynchronize(net->copy_stream));
  B200_CUDA(cudaStreamSynchronize(st));
  return 0;
}

}  // extern "C"
