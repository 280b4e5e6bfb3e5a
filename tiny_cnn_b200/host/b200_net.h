// b200_net.h -- network<sequential>::fit on the device-resident step.
//
// The patched network.h (make_overlay.py) calls b200_fit_hook from network::fit
// (tiny_dnn/network.h:840-879) right after the set-up that fit itself does
// (set_netphase, net_.setup, optimizer.reset).  When every layer of the network
// is on the path -- convolutional / fully-connected / max-pooling layers with
// engine backend_t::b200, average pooling, relu / tanh / softmax in between --
// the loss is mse / cross_entropy / cross_entropy_multiclass and the optimizer
// is one of the reference's seven (adagrad, adam, momentum, RMSprop, adamax,
// gradient_descent, nesterov_momentum), the hook replaces the loop over mini-batches:
//
// (the public fit / train overloads call b200_fit_hook_rows even earlier, before they copy the
// whole data set into tensors)
//
//   layers   -> b200_layer_spec[]            (b200_net_create, cached in the network object)
//   weights  -> flat parameter buffer        (layer::weights(): W before b, layer order)
//   adam     -> b200_net_set_adam_powers     (continues from the object's b1_t / b2_t)
//   batches  -> b200_net_fit_host, one call per epoch from page-locked staging
//              (replaces train_once / train_onebatch, network.h:883-926)
//   weights, optimizer state and adam's powers go back into the host objects after every
//   epoch, before on_epoch_enumerate runs (which typically calls net.test()).
//
// Otherwise the hook returns false and fit carries on with the reference's own loop,
// whose b200 layers then run operator by operator through b200_glue.h.
//
// Differences from the reference's loop, by construction: on_batch_enumerate is called
// once per mini-batch AFTER the epoch's mini-batches have run (the device does not stop
// between them), and stop_ongoing_training() takes effect at the next epoch boundary.
#pragma once

#include <atomic>
#include <cstring>
#include <fstream>
#include <functional>
#include <memory>
#include <string>
#include <thread>
#include <type_traits>
#include <vector>

#include "tiny_dnn/activations/elu_layer.h"
#include "tiny_dnn/activations/leaky_relu_layer.h"
#include "tiny_dnn/activations/relu_layer.h"
#include "tiny_dnn/activations/sigmoid_layer.h"
#include "tiny_dnn/activations/softmax_layer.h"
#include "tiny_dnn/activations/tanh_layer.h"
#include "tiny_dnn/core/kernels/b200_glue.h"
#include "tiny_dnn/layers/average_pooling_layer.h"
#include "tiny_dnn/layers/batch_normalization_layer.h"
#include "tiny_dnn/layers/convolutional_layer.h"
#include "tiny_dnn/layers/fully_connected_layer.h"
#include "tiny_dnn/layers/max_pooling_layer.h"
#include "tiny_dnn/lossfunctions/loss_function.h"
#include "tiny_dnn/optimizers/optimizer.h"

namespace tiny_dnn {
namespace b200 {

template <typename E>
struct loss_kind {
  static const int value = -1;
};
template <>
struct loss_kind<mse> {
  static const int value = B200_LOSS_MSE;
};
template <>
struct loss_kind<cross_entropy> {
  static const int value = B200_LOSS_CROSS_ENTROPY;
};
template <>
struct loss_kind<cross_entropy_multiclass> {
  static const int value = B200_LOSS_CROSS_ENTROPY_MULTICLASS;
};

// how often the hook took a fit (tests and benchmarks read it)
inline unsigned long long &device_fit_count() {
  static unsigned long long n = 0;
  return n;
}

// page-locked staging buffer
struct pinned_buffer {
  float *p = nullptr;
  size_t n = 0;
  void reserve(size_t floats) {
    if (floats <= n) return;
    release();
    void *q = nullptr;
    check(b200_host_alloc(floats * sizeof(float), &q));
    p = static_cast<float *>(q);
    n = floats;
  }
  void release() {
    if (p) b200_host_free(p);
    p = nullptr;
    n = 0;
  }
  ~pinned_buffer() { release(); }
};

// Data-parallel replicas of a C++ program: one process per GPU (B200_DEVICE selects it), every process
// builds the same network from the same seed and calls fit() on its own shard of the data with the
// per-GPU batch size; the device-resident step then sums the gradients over the processes (no 1/N,
// as edge::merge_grads sums the samples of one mini-batch) before every update, so the replicas stay
// bit-identical and equal one process training on the concatenated mini-batches.  The launcher fills
// this in before the first fit: its rank, the number of processes, and `exchange`, which sends this
// process's 64-byte buffer handle and returns every process's, in rank order, over whatever channel
// the launcher has (pipes, MPI, a file).  Every process must make the same number of steps.
struct replica_group {
  int rank = 0, world = 1;
  std::function<void(const unsigned char *own, unsigned char *all)> exchange;
  int timeout_ms = 0;  // bound of every wait for another process (0: the library's 10 s)
};
inline replica_group &replicas() {
  static replica_group g;
  return g;
}

// the device twin of one network<sequential>, kept in the network object
struct device_twin {
  void *peer_own = nullptr;            // this process's exchange buffer
  std::vector<void *> peer_opened;     // the other processes' buffers as mapped here
  b200_net *net = nullptr;
  std::vector<const layer *> layers;          // identity of the network it was built for
  std::vector<std::vector<size_t>> shapes;    // weight tensor lengths per layer
  int max_batch = 0;
  std::vector<std::vector<uint8_t>> tables;   // connection tables the specs point into
  pinned_buffer x, t;
  ~device_twin() {
    if (net) b200_net_destroy(net);
    for (void *q : peer_opened) b200_peer_buffer_close(ctx(), q);
    // peer_own stays allocated: another process may still have it mapped; it goes with the process
  }
};

// maps every replica's exchange buffer and switches the twin's step to the summed gradients
inline void join_replicas(device_twin &tw) {
  replica_group &g = replicas();
  if (g.world <= 1) return;
  if (!g.exchange) throw nn_error("b200: replicas().exchange is not set");
  const size_t bytes = b200_net_peer_reduce_bytes(tw.net, g.world);
  unsigned char own[B200_PEER_HANDLE_BYTES];
  check(b200_peer_buffer_create(ctx(), bytes, &tw.peer_own, own));
  std::vector<unsigned char> all(static_cast<size_t>(g.world) * B200_PEER_HANDLE_BYTES);
  g.exchange(own, all.data());
  std::vector<unsigned long long> bases(g.world);
  for (int r = 0; r < g.world; ++r) {
    if (r == g.rank) {
      bases[r] = reinterpret_cast<unsigned long long>(tw.peer_own);
      continue;
    }
    void *q = nullptr;
    check(b200_peer_buffer_open(ctx(), all.data() + static_cast<size_t>(r) * B200_PEER_HANDLE_BYTES, &q));
    tw.peer_opened.push_back(q);
    bases[r] = reinterpret_cast<unsigned long long>(q);
  }
  check(b200_net_peer_reduce_init(tw.net, g.rank, g.world, bases.data(), g.timeout_ms));
}

// b200_layer_spec of one layer, or false when the layer is not on the path
inline bool spec_of(layer *l, b200_layer_spec &s, std::vector<uint8_t> &tbl) {
  std::memset(&s, 0, sizeof(s));
  if (auto *c = dynamic_cast<convolutional_layer *>(l)) {
    if (c->engine() != core::backend_t::b200) return false;
    s.kind = B200_LAYER_CONV;
    s.conv = conv_desc(c->b200_params(), tbl);
    s.conv.input_is_padded = 0;  // the net pads on the device
    return true;
  }
  if (auto *f = dynamic_cast<fully_connected_layer *>(l)) {
    if (f->engine() != core::backend_t::b200) return false;
    const core::fully_params &p = f->b200_params();
    s.kind = B200_LAYER_FC;
    s.fc_in = static_cast<int32_t>(p.in_size_);
    s.fc_out = static_cast<int32_t>(p.out_size_);
    s.fc_has_bias = p.has_bias_ ? 1 : 0;
    return true;
  }
  if (auto *m = dynamic_cast<max_pooling_layer *>(l)) {
    if (m->engine() != core::backend_t::b200) return false;
    s.kind = B200_LAYER_MAXPOOL;
    s.pool = pool_desc(m->b200_params());
    return true;
  }
  if (auto *a = dynamic_cast<average_pooling_layer *>(l)) {
    s.kind = B200_LAYER_AVGPOOL;
    s.pool = a->b200_pool_desc();
    return true;
  }
  if (dynamic_cast<relu_layer *>(l)) {
    s.kind = B200_LAYER_RELU;
    return true;
  }
  if (dynamic_cast<tanh_layer *>(l)) {
    s.kind = B200_LAYER_TANH;
    return true;
  }
  if (dynamic_cast<softmax_layer *>(l)) {
    s.kind = B200_LAYER_SOFTMAX;
    return true;
  }
  if (dynamic_cast<sigmoid_layer *>(l)) {
    s.kind = B200_LAYER_SIGMOID;
    return true;
  }
  if (auto *k = dynamic_cast<leaky_relu_layer *>(l)) {
    s.kind = B200_LAYER_LEAKY_RELU;
    s.act_param = static_cast<float>(k->epsilon_);
    return true;
  }
  if (auto *e = dynamic_cast<elu_layer *>(l)) {
    s.kind = B200_LAYER_ELU;
    s.act_param = static_cast<float>(e->alpha_);
    return true;
  }
  if (auto *bn = dynamic_cast<batch_normalization_layer *>(l)) {
    s.kind = B200_LAYER_BATCHNORM;
    s.bn_channels = static_cast<int32_t>(bn->b200_channels());
    s.bn_spatial = static_cast<int32_t>(bn->b200_spatial());
    s.bn_eps = static_cast<float>(bn->epsilon());
    s.bn_momentum = static_cast<float>(bn->momentum());
    return true;
  }
  return false;
}

struct opt_choice {
  int kind = -1;
  b200_opt_hyper h{};
  int n_state = 0;  // state vectors the optimizer keeps per weight tensor
  // adam / adamax: the object's running powers b1_t (and b2_t), advanced once per update call
  float_t *pow1 = nullptr, *pow2 = nullptr;
  std::unordered_map<const vec_t *, vec_t> *maps = nullptr;
};

// The reference's optimizers by RTTI (it identifies node types the same way, nodes.h:134-146);
// eps is a private member there and constant 1e-8 (optimizer.h:58,83,110,151)
inline opt_choice choose_optimizer(optimizer *o) {
  opt_choice c;
  c.h.eps = 1e-8f;
  if (auto *a = dynamic_cast<adagrad *>(o)) {
    c.kind = B200_OPT_ADAGRAD;
    c.h.alpha = a->alpha;
    c.n_state = 1;
    c.maps = a->b200_maps();
  } else if (auto *a = dynamic_cast<adam *>(o)) {
    c.kind = B200_OPT_ADAM;
    c.h.alpha = a->alpha;
    c.h.b1 = a->b1;
    c.h.b2 = a->b2;
    c.h.b1_t = a->b1_t;
    c.h.b2_t = a->b2_t;
    c.n_state = 2;
    c.pow1 = &a->b1_t;
    c.pow2 = &a->b2_t;
    c.maps = a->b200_maps();
  } else if (auto *a = dynamic_cast<adamax *>(o)) {
    c.kind = B200_OPT_ADAMAX;
    c.h.alpha = a->alpha;
    c.h.b1 = a->b1;
    c.h.b2 = a->b2;
    c.h.b1_t = a->b1_t;
    c.h.b2_t = a->b2;  // adamax keeps no second power
    c.n_state = 2;
    c.pow1 = &a->b1_t;
    c.maps = a->b200_maps();
  } else if (auto *m = dynamic_cast<nesterov_momentum *>(o)) {
    c.kind = B200_OPT_NESTEROV_MOMENTUM;
    c.h.alpha = m->alpha;
    c.h.mu = m->mu;
    c.h.lambda = m->lambda;
    c.n_state = 1;
    c.maps = m->b200_maps();
  } else if (auto *m = dynamic_cast<momentum *>(o)) {
    c.kind = B200_OPT_MOMENTUM;
    c.h.alpha = m->alpha;
    c.h.mu = m->mu;
    c.h.lambda = m->lambda;
    c.n_state = 1;
    c.maps = m->b200_maps();
  } else if (auto *r = dynamic_cast<RMSprop *>(o)) {
    c.kind = B200_OPT_RMSPROP;
    c.h.alpha = r->alpha;
    c.h.mu = r->mu;
    c.n_state = 1;
    c.maps = r->b200_maps();
  } else if (auto *g = dynamic_cast<gradient_descent *>(o)) {
    c.kind = B200_OPT_GRADIENT_DESCENT;
    c.h.alpha = g->alpha;
    c.h.lambda = g->lambda;
  }
  return c;
}

template <typename Net>
std::shared_ptr<device_twin> twin_for(Net &nn, int batch) {
  const size_t depth = nn.depth();
  std::vector<const layer *> ids(depth);
  std::vector<std::vector<size_t>> shapes(depth);
  for (size_t i = 0; i < depth; ++i) {
    ids[i] = nn[i];
    for (auto *w : nn[i]->weights()) shapes[i].push_back(w->size());
  }
  auto cached = std::static_pointer_cast<device_twin>(nn.b200_twin_);
  if (cached && cached->layers == ids && cached->shapes == shapes && cached->max_batch >= batch) return cached;
  auto tw = std::make_shared<device_twin>();
  std::vector<b200_layer_spec> specs(depth);
  tw->tables.resize(depth);
  for (size_t i = 0; i < depth; ++i)
    if (!spec_of(nn[i], specs[i], tw->tables[i])) return nullptr;
  for (size_t i = 0; i < depth; ++i)  // the tables moved with the vector of vectors: point again
    if (specs[i].kind == B200_LAYER_CONV && specs[i].conv.tbl) specs[i].conv.tbl = tw->tables[i].data();
  // a shape the library declines (b200_net_create says why) leaves the reference loop in charge
  if (b200_net_create(ctx(), specs.data(), static_cast<int>(depth), batch, &tw->net) != 0) return nullptr;
  join_replicas(*tw);
  tw->layers = ids;
  tw->shapes = shapes;
  tw->max_batch = batch;
  nn.b200_twin_ = tw;
  return tw;
}

template <typename Net>
void weights_to_device(Net &nn, device_twin &tw) {
  std::vector<float> flat(b200_net_param_count(tw.net));
  size_t off = 0;
  for (size_t i = 0; i < nn.depth(); ++i)
    for (auto *w : nn[i]->weights()) {
      std::copy(w->begin(), w->end(), flat.begin() + off);
      off += w->size();
    }
  check(b200_net_set_params(tw.net, flat.data()));
  // batch normalization: the layers' moving averages; the fit runs in the train phase
  for (size_t i = 0; i < nn.depth(); ++i)
    if (auto *bn = dynamic_cast<batch_normalization_layer *>(nn[i])) {
      std::vector<float> m(bn->b200_mean().begin(), bn->b200_mean().end()),
        v(bn->b200_variance().begin(), bn->b200_variance().end());
      check(b200_net_bn_stats(tw.net, static_cast<int>(i), m.data(), v.data(), 1));
    }
  check(b200_net_set_phase(tw.net, 1));
}

// weights, optimizer state (stateful_optimizer::E_, keyed by the weight vector's address) and
// adam's powers back into the host objects
template <typename Net>
void state_to_host(Net &nn, device_twin &tw, opt_choice &oc, long long steps_done) {
  const size_t n = b200_net_param_count(tw.net);
  std::vector<float> flat(n);
  check(b200_net_get_params(tw.net, flat.data()));
  size_t off = 0;
  for (size_t i = 0; i < nn.depth(); ++i)
    for (auto *w : nn[i]->weights()) {
      std::copy(flat.begin() + off, flat.begin() + off + w->size(), w->begin());
      off += w->size();
    }
  for (size_t i = 0; i < nn.depth(); ++i)
    if (auto *bn = dynamic_cast<batch_normalization_layer *>(nn[i])) {
      std::vector<float> m(bn->b200_channels()), v(bn->b200_channels());
      check(b200_net_bn_stats(tw.net, static_cast<int>(i), m.data(), v.data(), 0));
      bn->b200_mean().assign(m.begin(), m.end());
      bn->b200_variance().assign(v.begin(), v.end());
    }
  for (int k = 0; k < oc.n_state; ++k) {
    check(b200_net_get_opt_state(tw.net, k, flat.data()));
    off = 0;
    for (size_t i = 0; i < nn.depth(); ++i)
      for (auto *w : nn[i]->weights()) {
        vec_t &e = oc.maps[k][w];
        e.assign(flat.begin() + off, flat.begin() + off + w->size());
        off += w->size();
      }
  }
  if (oc.pow1) {
    // adam::update / adamax::update multiply the powers once per call: tensors x steps sequential
    // float products (optimizer.h:125-126,165); the device table did the same multiplications
    const long long calls = steps_done * static_cast<long long>(b200_net_tensor_count(tw.net));
    for (long long c = 0; c < calls; ++c) {
      *oc.pow1 *= oc.h.b1;
      if (oc.pow2) *oc.pow2 *= oc.h.b2;
    }
  }
}

// rows of the reference's containers: a sample is a vec_t, or a tensor_t holding one vec_t
inline const vec_t *input_row(const vec_t &v) { return &v; }
inline const vec_t *input_row(const tensor_t &t) { return t.size() == 1 ? &t[0] : nullptr; }

// writes one target row; class labels become nodes::label2vec rows (nodes.h:180-189) in the output
// range of the network's last layer (nodes.h:147-156)
struct target_writer {
  size_t out_dim;
  float lo, hi;
  bool write(const vec_t &v, float *dst) const {
    if (v.size() != out_dim) return false;
    std::copy(v.begin(), v.end(), dst);
    return true;
  }
  bool write(const tensor_t &t, float *dst) const { return t.size() == 1 && write(t[0], dst); }
  bool write(label_t l, float *dst) const {
    if (static_cast<size_t>(l) >= out_dim) return false;
    std::fill(dst, dst + out_dim, lo);
    dst[l] = hi;
    return true;
  }
};

// The loop over mini-batches of network::fit on the device.  `preamble`: also do what fit does
// before its loop (network.h:852-857) -- for the hooks that run before fit's own set-up; nothing
// of the network or the optimizer is touched until the whole fit is known to be on the path.
template <typename Error, typename Optimizer, typename In, typename Tg, typename OnBatch, typename OnEpoch>
bool fit_sequential(network<sequential> &nn, Optimizer &opt, const std::vector<In> &inputs,
                    const std::vector<Tg> &targets, size_t batch_size, int epoch, OnBatch on_batch_enumerate,
                    OnEpoch on_epoch_enumerate, bool preamble, bool reset_weights, bool *stop) {
  const int loss = loss_kind<Error>::value;
  if (loss < 0 || inputs.empty() || batch_size == 0 || nn.depth() == 0 || targets.size() != inputs.size()) return false;
  opt_choice oc = choose_optimizer(static_cast<optimizer *>(&opt));
  if (oc.kind < 0) return false;
  bool any_b200 = false;
  for (size_t i = 0; i < nn.depth(); ++i) any_b200 = any_b200 || nn[i]->engine() == core::backend_t::b200;
  if (!any_b200) return false;
  const size_t N = inputs.size();
  if (N < batch_size && N != 1) return false;  // the reference's batch buffers would hold unset rows
  const int batch = static_cast<int>(std::min(batch_size, N));
  std::shared_ptr<device_twin> tw = twin_for(nn, batch);
  if (!tw) return false;
  const size_t in_dim = static_cast<size_t>(b200_net_in_dim(tw->net));
  const size_t out_dim = static_cast<size_t>(b200_net_out_dim(tw->net));
  const std::pair<float_t, float_t> range = nn[nn.depth() - 1]->out_value_range();
  const target_writer tgt{out_dim, static_cast<float>(range.first), static_cast<float>(range.second)};
  std::vector<float> probe(out_dim);
  for (size_t s = 0; s < N; ++s) {
    const vec_t *r = input_row(inputs[s]);
    if (!r || r->size() != in_dim) return false;
  }
  if (!tgt.write(targets[0], probe.data())) return false;

  if (preamble) {
    nn.set_netphase(net_phase::train);
    for (size_t i = 0; i < nn.depth(); ++i) nn[i]->setup(reset_weights);
    for (size_t i = 0; i < nn.depth(); ++i) nn[i]->set_parallelize(true);
    opt.reset();
    *stop = false;
  }
  tw->x.reserve(N * in_dim);
  tw->t.reserve(N * out_dim);
  // The reference keeps one heap vector per sample; the device wants rows back to back in
  // page-locked memory.  Rows [s0, s1) are packed by a few threads, and during the first epoch the
  // packing of the next run of mini-batches overlaps the device's work on the current one.
  float *xp = tw->x.p, *tp = tw->t.p;
  std::atomic<bool> bad_row(false);
  auto pack = [&inputs, &targets, &tgt, &bad_row, xp, tp, in_dim, out_dim](size_t s0, size_t s1) {
    unsigned nt = std::thread::hardware_concurrency();
    nt = nt == 0 ? 1 : nt > 4 ? 4 : nt;
    if (const char *e = std::getenv("B200_PACK_THREADS")) nt = std::max(1, std::atoi(e));
    if (s1 - s0 < 64) nt = 1;
    auto part = [&](size_t a, size_t b) {
      for (size_t s = a; s < b; ++s) {
        const vec_t *r = input_row(inputs[s]);
        std::copy(r->begin(), r->end(), xp + s * in_dim);
        if (!tgt.write(targets[s], tp + s * out_dim)) bad_row = true;
      }
    };
    std::vector<std::thread> helpers;
    const size_t per = (s1 - s0 + nt - 1) / nt;
    for (unsigned k = 1; k < nt; ++k) {
      const size_t a = s0 + k * per, b = std::min(s1, a + per);
      if (a < b) helpers.emplace_back(part, a, b);
    }
    part(s0, std::min(s1, s0 + per));
    for (auto &h : helpers) h.join();
  };
  weights_to_device(nn, *tw);
  // fit() calls optimizer.reset() before its loop: the state maps are empty, adam's powers carry on
  check(b200_net_opt_reset(tw->net, 1));
  if (oc.pow1) check(b200_net_set_adam_powers(tw->net, oc.h.b1, oc.h.b2, *oc.pow1, oc.pow2 ? *oc.pow2 : oc.h.b2));
  const long long steps_per_epoch = static_cast<long long>((N + batch - 1) / batch);
  for (int iter = 0; iter < epoch && !*stop; ++iter) {
    if (iter == 0) {
      // a packer thread runs ahead mini-batch by mini-batch and publishes how far it is; every library
      // call takes the whole mini-batches packed so far, so the device starts after one of them and the
      // calls grow as the packer gains on it
      std::atomic<size_t> packed(0);
      std::thread packer([&] {
        for (size_t s = 0; s < N && !bad_row; s += static_cast<size_t>(batch)) {
          const size_t e = std::min(N, s + static_cast<size_t>(batch));
          pack(s, e);
          packed.store(e, std::memory_order_release);
        }
        packed.store(N, std::memory_order_release);  // also ends the wait below after a bad row
      });
      int rc = 0;
      for (size_t s0 = 0; s0 < N && rc == 0 && !bad_row;) {
        const size_t want = std::min(N, s0 + static_cast<size_t>(batch));
        size_t have;
        while ((have = packed.load(std::memory_order_acquire)) < want) std::this_thread::yield();
        if (bad_row) break;
        const size_t s1 = have == N ? N : s0 + (have - s0) / batch * batch;
        // queued, not waited for: the device goes from one run to the next without draining
        rc = b200_net_fit_host_enqueue(tw->net, xp + s0 * in_dim, tp + s0 * out_dim, static_cast<long long>(s1 - s0),
                                       batch, 1, loss, oc.kind, &oc.h, nullptr);
        s0 = s1;
      }
      packer.join();
      const int rc_wait = b200_net_fit_host_wait(tw->net);
      if (rc == 0) rc = rc_wait;
      if (bad_row) throw nn_error("b200: a target row does not fit the network's output (size or class id)");
      check(rc);
    } else {
      check(b200_net_fit_host(tw->net, xp, tp, static_cast<long long>(N), batch, 1, loss, oc.kind, &oc.h, nullptr));
    }
    check(b200_ctx_sync(ctx()));
    state_to_host(nn, *tw, oc, steps_per_epoch);
    for (long long b = 0; b < steps_per_epoch; ++b) on_batch_enumerate();
    on_epoch_enumerate();
  }
  nn.set_netphase(net_phase::test);
  ++device_fit_count();
  return true;
}

// ---- training straight from the dataset's bytes ----------------------------------------------
//
// parse_cifar10 / parse_mnist_images (tiny_dnn/io/cifar10_parser.h, mnist_parser.h) turn every
// pixel byte into a float on the host, and network::train then uploads 4 bytes per pixel.  The
// loaders below keep the bytes; train_u8 uploads them as they are and the device applies the
// parser's own scaling (bit for bit) and builds the target rows (nodes::label2vec) per mini-batch.
struct u8_dataset {
  std::vector<uint8_t> images;  // n records of channels * height * width bytes, planar
  std::vector<uint8_t> labels;  // n class ids
  b200_image_desc desc{};
  size_t size() const { return labels.size(); }
};

// the records of a CIFAR-10 binary file (1 label byte + 3 x 32 x 32 pixel bytes each), appended to
// `data`; scale / padding as parse_cifar10's arguments (cifar10_parser.h:36-46)
inline void load_cifar10_u8(const std::string &filename, u8_dataset *data, float_t scale_min, float_t scale_max,
                            int x_padding, int y_padding) {
  if (x_padding < 0 || y_padding < 0) throw nn_error("padding size must not be negative");
  if (scale_min >= scale_max) throw nn_error("scale_max must be greater than scale_min");
  std::ifstream ifs(filename.c_str(), std::ios::in | std::ios::binary);
  if (ifs.fail() || ifs.bad()) throw nn_error("failed to open file:" + filename);
  data->desc.mode = B200_IMAGE_CIFAR10;
  data->desc.channels = 3;
  data->desc.height = data->desc.width = 32;
  data->desc.x_padding = x_padding;
  data->desc.y_padding = y_padding;
  data->desc.scale_min = scale_min;
  data->desc.scale_max = scale_max;
  uint8_t label;
  std::vector<char> buf(3 * 32 * 32);
  while (ifs.read(reinterpret_cast<char *>(&label), 1)) {
    if (!ifs.read(buf.data(), buf.size())) break;
    data->labels.push_back(label);
    data->images.insert(data->images.end(), buf.begin(), buf.end());
  }
}

// the images of an MNIST idx3-ubyte file and the labels of the matching idx1-ubyte file
// (mnist_parser.h:88-157: big-endian headers, magic numbers 0x803 / 0x801)
inline void load_mnist_u8(const std::string &image_file, const std::string &label_file, u8_dataset *data,
                          float_t scale_min, float_t scale_max, int x_padding, int y_padding) {
  if (x_padding < 0 || y_padding < 0) throw nn_error("padding size must not be negative");
  if (scale_min >= scale_max) throw nn_error("scale_max must be greater than scale_min");
  auto be32 = [](std::ifstream &f) {
    unsigned char b[4] = {0, 0, 0, 0};
    f.read(reinterpret_cast<char *>(b), 4);
    return (uint32_t(b[0]) << 24) | (uint32_t(b[1]) << 16) | (uint32_t(b[2]) << 8) | uint32_t(b[3]);
  };
  std::ifstream fi(image_file.c_str(), std::ios::in | std::ios::binary);
  if (fi.bad() || fi.fail()) throw nn_error("failed to open file:" + image_file);
  const uint32_t magic = be32(fi), n = be32(fi), rows = be32(fi), cols = be32(fi);
  if (magic != 0x00000803 || n == 0) throw nn_error("MNIST label-file format error");
  if (fi.fail() || fi.bad()) throw nn_error("file error");
  std::ifstream fl(label_file.c_str(), std::ios::in | std::ios::binary);
  if (fl.bad() || fl.fail()) throw nn_error("failed to open file:" + label_file);
  const uint32_t lmagic = be32(fl), ln = be32(fl);
  if (lmagic != 0x00000801 || ln != n) throw nn_error("MNIST label-file format error");
  data->desc.mode = B200_IMAGE_MNIST;
  data->desc.channels = 1;
  data->desc.height = static_cast<int32_t>(rows);
  data->desc.width = static_cast<int32_t>(cols);
  data->desc.x_padding = x_padding;
  data->desc.y_padding = y_padding;
  data->desc.scale_min = scale_min;
  data->desc.scale_max = scale_max;
  const size_t off = data->images.size(), loff = data->labels.size();
  data->images.resize(off + size_t(n) * rows * cols);
  fi.read(reinterpret_cast<char *>(data->images.data() + off), std::streamsize(size_t(n) * rows * cols));
  data->labels.resize(loff + n);
  fl.read(reinterpret_cast<char *>(data->labels.data() + loff), n);
  if (fi.fail() || fl.fail()) throw nn_error("file error");
}

// network::train<Error>(optimizer, images, labels, batch, epochs, callbacks) (network.h:268-307)
// from the raw bytes.  Throws when the network is not wholly on the path: this entry has no host
// form to fall back to (parse with the reference's parsers and call nn.train for that).
template <typename Error, typename Optimizer, typename OnBatch, typename OnEpoch>
bool train_u8(network<sequential> &nn, Optimizer &opt, const u8_dataset &data, size_t batch_size, int epoch,
              OnBatch on_batch_enumerate, OnEpoch on_epoch_enumerate, bool reset_weights = false) {
  const int loss = loss_kind<Error>::value;
  if (loss < 0) throw nn_error("b200::train_u8: loss function is not on the path");
  opt_choice oc = choose_optimizer(static_cast<optimizer *>(&opt));
  if (oc.kind < 0) throw nn_error("b200::train_u8: optimizer is not adagrad, adam or momentum");
  const size_t N = data.size();
  if (N < batch_size || batch_size == 0) return false;  // as network::train (network.h:297-299)
  // what fit() does before its loop (network.h:852-857)
  nn.set_netphase(net_phase::train);
  for (size_t i = 0; i < nn.depth(); ++i) nn[i]->setup(reset_weights);
  for (size_t i = 0; i < nn.depth(); ++i) nn[i]->set_parallelize(true);
  opt.reset();
  const int batch = static_cast<int>(batch_size);
  std::shared_ptr<device_twin> tw = twin_for(nn, batch);
  if (!tw) throw nn_error(std::string("b200::train_u8: the network is not wholly on the B200 path: ") + b200_last_error());
  const std::pair<float_t, float_t> range = nn[nn.depth() - 1]->out_value_range();  // nodes.h:147-156
  // page-locked copies of the bytes, so that uploads overlap the steps
  const size_t img_bytes = data.images.size();
  tw->x.reserve((img_bytes + 3) / 4);
  tw->t.reserve((N + 3) / 4);
  uint8_t *ip = reinterpret_cast<uint8_t *>(tw->x.p), *lp = reinterpret_cast<uint8_t *>(tw->t.p);
  std::memcpy(ip, data.images.data(), img_bytes);
  std::memcpy(lp, data.labels.data(), N);
  weights_to_device(nn, *tw);
  check(b200_net_opt_reset(tw->net, 1));
  if (oc.pow1) check(b200_net_set_adam_powers(tw->net, oc.h.b1, oc.h.b2, *oc.pow1, oc.pow2 ? *oc.pow2 : oc.h.b2));
  const long long steps_per_epoch = static_cast<long long>((N + batch - 1) / batch);
  for (int iter = 0; iter < epoch; ++iter) {
    check(b200_net_fit_u8_host(tw->net, &data.desc, ip, lp, static_cast<long long>(N), batch, 1, range.first,
                               range.second, loss, oc.kind, &oc.h, nullptr));
    check(b200_ctx_sync(ctx()));
    state_to_host(nn, *tw, oc, steps_per_epoch);
    for (long long b = 0; b < steps_per_epoch; ++b) on_batch_enumerate();
    on_epoch_enumerate();
  }
  nn.set_netphase(net_phase::test);
  ++device_fit_count();
  return true;
}

template <typename Error, typename Optimizer>
bool train_u8(network<sequential> &nn, Optimizer &opt, const u8_dataset &data, size_t batch_size = 1, int epoch = 1) {
  return train_u8<Error>(nn, opt, data, batch_size, epoch, nop, nop);
}

template <typename Error, typename Net, typename Optimizer, typename In, typename Tg, typename OnBatch,
          typename OnEpoch>
bool fit_dispatch(std::false_type, Net &, Optimizer &, const std::vector<In> &, const std::vector<Tg> &, size_t, int,
                  OnBatch, OnEpoch, bool, bool, bool *) {
  return false;  // graph networks keep the reference loop
}
template <typename Error, typename Net, typename Optimizer, typename In, typename Tg, typename OnBatch,
          typename OnEpoch>
bool fit_dispatch(std::true_type, Net &nn, Optimizer &opt, const std::vector<In> &inputs,
                  const std::vector<Tg> &targets, size_t batch_size, int epoch, OnBatch on_batch, OnEpoch on_epoch,
                  bool preamble, bool reset_weights, bool *stop) {
  return fit_sequential<Error>(nn, opt, inputs, targets, batch_size, epoch, on_batch, on_epoch, preamble,
                               reset_weights, stop);
}

}  // namespace b200

// Declared in the patched network.h.  b200_fit_hook is called from the private network::fit after
// its own set-up (for callers that hand over std::vector<tensor_t>); b200_fit_hook_rows from the
// public fit / train overloads before they copy the whole data set into tensors
// (normalize_tensor, network.h:1085-1098), which the device path has no use for.
template <typename Error, typename Net, typename Optimizer, typename OnBatch, typename OnEpoch>
bool b200_fit_hook(Net &nn, Optimizer &opt, const std::vector<tensor_t> &inputs,
                   const std::vector<tensor_t> &desired_outputs, size_t batch_size, int epoch, OnBatch on_batch,
                   OnEpoch on_epoch, const std::vector<tensor_t> &t_cost, bool *stop) {
  if (!t_cost.empty()) return false;
  return b200::fit_dispatch<Error>(std::is_same<Net, network<sequential>>(), nn, opt, inputs, desired_outputs,
                                   batch_size, epoch, on_batch, on_epoch, false, false, stop);
}

template <typename Error, typename Net, typename Optimizer, typename In, typename Tg, typename OnBatch,
          typename OnEpoch>
bool b200_fit_hook_rows(Net &nn, Optimizer &opt, const std::vector<In> &inputs, const std::vector<Tg> &targets,
                        size_t batch_size, int epoch, OnBatch on_batch, OnEpoch on_epoch, bool reset_weights,
                        bool *stop) {
  return b200::fit_dispatch<Error>(std::is_same<Net, network<sequential>>(), nn, opt, inputs, targets, batch_size,
                                   epoch, on_batch, on_epoch, true, reset_weights, stop);
}

}  // namespace tiny_dnn
