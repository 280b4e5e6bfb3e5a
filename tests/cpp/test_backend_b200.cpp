// A/B test of the engine core::backend_t::b200 inside tiny-dnn itself.
//
// Compiled against the overlay produced by tiny_cnn_b200/host/make_overlay.py
// placed before the tiny-dnn tree on the include path, and linked with
// libtinycnn_b200.so.  The same layer objects and networks are run with
// backend_t::internal (the reference's CPU kernels) and with backend_t::b200,
// following the reference's own engine A/B tests
// (test/test_convolutional_layer.h:257-497).  Tolerances: forward 1e-4,
// gradients and weights 1e-3, relative to the largest magnitude; the
// quantized layer is compared bit for bit.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>

#include "tiny_dnn/tiny_dnn.h"

using namespace tiny_dnn;

static int g_fail = 0;

static unsigned long long device_fit_count_now() { return b200::device_fit_count(); }
static void expect_ok(bool ok, const char *what) {
  printf(ok ? "ok   %s\n" : "FAIL %s\n", what);
  if (!ok) ++g_fail;
}

static double max_abs(const vec_t &v) {
  double m = 0;
  for (auto x : v) m = std::max(m, (double)std::fabs(x));
  return m;
}

static bool close_vec(const vec_t &a, const vec_t &b, double tol, const char *what) {
  if (a.size() != b.size()) {
    printf("FAIL %s: size %zu vs %zu\n", what, a.size(), b.size());
    ++g_fail;
    return false;
  }
  double scale = std::max(max_abs(b), 1e-30), worst = 0;
  size_t bad = 0, at = 0;
  for (size_t i = 0; i < a.size(); ++i) {
    double err = std::fabs((double)a[i] - (double)b[i]);
    if (err > tol * (std::fabs((double)b[i]) + scale)) ++bad;
    if (err / scale > worst) {
      worst = err / scale;
      at = i;
    }
  }
  if (bad) {
    printf("FAIL %s: %zu of %zu beyond %g; worst [%zu] got %.9g want %.9g (max rel err %.2e, scale %g)\n", what, bad,
           a.size(), tol, at, a[at], b[at], worst, scale);
    ++g_fail;
    return false;
  }
  printf("ok   %s (max rel err %.2e)\n", what, worst);
  return true;
}

static vec_t sum_rows(const tensor_t &t) {
  vec_t s(t[0].size(), 0);
  for (auto &r : t)
    for (size_t i = 0; i < s.size(); ++i) s[i] += r[i];
  return s;
}

static void fill_normal(tensor_t &t, std::mt19937 &g) {
  std::normal_distribution<float> d(0.f, 1.f);
  for (auto &r : t)
    for (auto &x : r) x = d(g);
}
static void fill_uniform(vec_t &v, std::mt19937 &g, float lo, float hi) {
  std::uniform_real_distribution<float> d(lo, hi);
  for (auto &x : v) x = d(g);
}

// Run one layer forward + backward on B samples with the engine given.
struct LayerRun {
  tensor_t out, din, dW, db;
};

template <typename L>
static LayerRun run_layer(L &l, core::backend_t engine, const tensor_t &x, const vec_t &W, const vec_t &b,
                          const tensor_t &dy, bool has_weights) {
  const size_t B = x.size();
  l.set_backend_type(engine);
  tensor_t tx = x, tW(1, W), tb(1, b), tout(B, vec_t(l.out_shape()[0].size()));
  tensor_t gx(B, vec_t(x[0].size())), gW(B, vec_t(W.size())), gb(B, vec_t(b.size())), gout = dy;
  std::vector<tensor_t *> ins = {&tx}, outs = {&tout}, gins = {&gx}, gouts = {&gout};
  if (has_weights) {
    ins.push_back(&tW);
    ins.push_back(&tb);
    gins.push_back(&gW);
    gins.push_back(&gb);
  }
  l.setup(false);
  l.set_sample_count(B);
  l.set_parallelize(true);
  l.forward_propagation(ins, outs);
  l.back_propagation(ins, outs, gouts, gins);
  return {tout, gx, gW, gb};
}

static vec_t flat(const tensor_t &t) {
  vec_t f;
  for (auto &r : t) f.insert(f.end(), r.begin(), r.end());
  return f;
}

template <typename L>
static void ab_layer(const char *name, L &l, size_t B, bool has_weights, unsigned seed) {
  std::mt19937 g(seed);
  tensor_t x(B, vec_t(l.in_shape()[0].size())), dy(B, vec_t(l.out_shape()[0].size()));
  fill_normal(x, g);
  fill_normal(dy, g);
  vec_t W(has_weights ? l.in_shape()[1].size() : 0), b(has_weights ? l.in_shape()[2].size() : 0);
  fill_uniform(W, g, -0.5f, 0.5f);
  fill_uniform(b, g, -0.1f, 0.1f);
  LayerRun a = run_layer(l, core::backend_t::internal, x, W, b, dy, has_weights);
  LayerRun c = run_layer(l, core::backend_t::b200, x, W, b, dy, has_weights);
  char what[128];
  snprintf(what, sizeof(what), "%s forward", name);
  close_vec(flat(c.out), flat(a.out), 1e-4, what);
  snprintf(what, sizeof(what), "%s dX", name);
  close_vec(flat(c.din), flat(a.din), 1e-3, what);
  if (has_weights) {
    snprintf(what, sizeof(what), "%s dW (merged)", name);
    close_vec(sum_rows(c.dW), sum_rows(a.dW), 1e-3, what);
    snprintf(what, sizeof(what), "%s db (merged)", name);
    close_vec(sum_rows(c.db), sum_rows(a.db), 1e-3, what);
  }
}

// lrn_layer has no backward pass in the reference (it throws): forward only
static void ab_lrn() {
  std::mt19937 g(41);
  const size_t B = 3;
  lrn_layer l(6, 5, 5, 8, float_t(1e-4), float_t(0.75));
  tensor_t x(B, vec_t(6 * 5 * 8)), ya(B, vec_t(6 * 5 * 8)), yc = ya;
  fill_normal(x, g);
  std::vector<tensor_t *> ins = {&x}, outs_a = {&ya}, outs_c = {&yc};
  l.set_backend_type(core::backend_t::internal);
  l.forward_propagation(ins, outs_a);
  l.set_backend_type(core::backend_t::b200);
  l.forward_propagation(ins, outs_c);
  close_vec(flat(yc), flat(ya), 1e-4, "lrn across channels forward (set_backend_type)");
}

// batch normalization in the test phase: the moving averages are read, not this batch's moments
static void ab_batchnorm_test_phase() {
  std::mt19937 g(42);
  const size_t B = 4, C = 5, S = 9;
  batch_normalization_layer l(S, C, float_t(1e-5), float_t(0.999), net_phase::test);
  vec_t m(C), v(C);
  fill_uniform(m, g, -1.f, 1.f);
  fill_uniform(v, g, 0.5f, 2.f);
  l.set_mean(m);
  l.set_variance(v);
  tensor_t x(B, vec_t(C * S)), ya(B, vec_t(C * S)), yc = ya;
  fill_normal(x, g);
  std::vector<tensor_t *> ins = {&x}, outs_a = {&ya}, outs_c = {&yc};
  l.set_backend_type(core::backend_t::internal);
  l.forward_propagation(ins, outs_a);
  l.set_backend_type(core::backend_t::b200);
  l.forward_propagation(ins, outs_c);
  close_vec(flat(yc), flat(ya), 1e-4, "batch normalization, test phase forward (set_backend_type)");
}

static void build_net(network<sequential> &nn, core::backend_t e) {
  using conv = convolutional_layer;
  using pool = max_pooling_layer;
  using fc = fully_connected_layer;
  nn << conv(16, 16, 5, 3, 8, padding::same, true, 1, 1, 1, 1, e) << relu_layer()
     << pool(16, 16, 8, 2, false, e)
     << conv(8, 8, 3, 8, 12, padding::valid, true, 1, 1, 1, 1, e) << tanh_layer()
     << pool(6, 6, 12, 2, false, e) << fc(3 * 3 * 12, 10, true, e) << softmax_layer(10);
}

// the remaining optimizers through the device-resident fit: same small network, a few steps each
template <typename Opt>
static void ab_optimizer(const char *name, int n_state) {
  network<sequential> a, c;
  build_net(a, core::backend_t::internal);
  build_net(c, core::backend_t::b200);
  set_random_seed(7);
  a.init_weight();
  c.init_weight();
  for (size_t i = 0; i < a.depth(); ++i) {
    auto wa = a[i]->weights();
    auto wc = c[i]->weights();
    for (size_t k = 0; k < wa.size(); ++k) *wc[k] = *wa[k];
  }
  std::mt19937 g(13);
  const size_t B = 8, steps = 4;
  std::vector<vec_t> x(B * steps, vec_t(16 * 16 * 3)), t(B * steps, vec_t(10, 0.f));
  std::normal_distribution<float> nd(0.f, 1.f);
  for (auto &v : x)
    for (auto &e : v) e = nd(g);
  for (auto &v : t) v[g() % 10] = 1.f;
  Opt oa, oc;
  const unsigned long long fits = device_fit_count_now();
  a.fit<cross_entropy>(oa, x, t, B, 1);
  c.fit<cross_entropy>(oc, x, t, B, 1);
  char what[160];
  snprintf(what, sizeof(what), "%s: network::fit ran as the device-resident step", name);
  expect_ok(device_fit_count_now() == fits + 1, what);
  for (size_t i = 0; i < a.depth(); ++i) {
    auto wa = a[i]->weights();
    auto wc = c[i]->weights();
    for (size_t k = 0; k < wa.size(); ++k) {
      snprintf(what, sizeof(what), "%s fit: layer %zu tensor %zu after %zu steps", name, i, k, steps);
      close_vec(*wc[k], *wa[k], 1e-3, what);
    }
  }
  (void)n_state;
}

static void ab_network() {
  network<sequential> a, c;
  build_net(a, core::backend_t::internal);
  build_net(c, core::backend_t::b200);
  set_random_seed(7);
  a.init_weight();
  // same starting weights
  for (size_t i = 0; i < a.depth(); ++i) {
    auto wa = a[i]->weights();
    auto wc = c[i]->weights();
    for (size_t k = 0; k < wa.size(); ++k) *wc[k] = *wa[k];
  }
  c.init_weight();  // marks layers initialised; restore the weights afterwards
  for (size_t i = 0; i < a.depth(); ++i) {
    auto wa = a[i]->weights();
    auto wc = c[i]->weights();
    for (size_t k = 0; k < wa.size(); ++k) *wc[k] = *wa[k];
  }
  std::mt19937 g(11);
  const size_t B = 8, steps = 3;
  std::vector<vec_t> x(B * steps, vec_t(16 * 16 * 3)), t(B * steps, vec_t(10, 0.f));
  std::normal_distribution<float> nd(0.f, 1.f);
  for (auto &v : x)
    for (auto &e : v) e = nd(g);
  for (auto &v : t) v[g() % 10] = 1.f;
  adam oa, oc;
  a.fit<cross_entropy>(oa, x, t, B, 1);
  c.fit<cross_entropy>(oc, x, t, B, 1);
  for (size_t i = 0; i < a.depth(); ++i) {
    auto wa = a[i]->weights();
    auto wc = c[i]->weights();
    for (size_t k = 0; k < wa.size(); ++k) {
      char what[128];
      snprintf(what, sizeof(what), "network fit: layer %zu tensor %zu after %zu adam steps", i, k, steps);
      close_vec(*wc[k], *wa[k], 1e-3, what);
    }
  }
  vec_t pa = a.predict(x[0]), pc = c.predict(x[0]);
  close_vec(pc, pa, 1e-4, "network predict");
}

static void expect(bool ok, const char *what) {
  printf(ok ? "ok   %s\n" : "FAIL %s\n", what);
  if (!ok) ++g_fail;
}

// same starting weights in two structurally identical networks
static void same_weights(network<sequential> &a, network<sequential> &c, unsigned seed) {
  set_random_seed(seed);
  a.init_weight();
  c.init_weight();  // marks the layers initialised
  for (size_t i = 0; i < a.depth(); ++i) {
    auto wa = a[i]->weights();
    auto wc = c[i]->weights();
    for (size_t k = 0; k < wa.size(); ++k) *wc[k] = *wa[k];
  }
}

// The bias of a layer that feeds a batch normalization layer has a gradient of exactly zero in exact
// arithmetic (the normalization subtracts the channel mean, so a constant added to a channel changes
// nothing): what both runs hold there is rounding noise of the sums, amplified by the optimizer, and
// the network's function does not depend on it.  Such a tensor is checked to be noise (small), not to
// match noise.
static void compare_nets(network<sequential> &a, network<sequential> &c, double tol, const char *label) {
  for (size_t i = 0; i < a.depth(); ++i) {
    auto wa = a[i]->weights();
    auto wc = c[i]->weights();
    const bool feeds_bn = i + 1 < a.depth() && a[i + 1]->layer_type() == "batch-norm";
    for (size_t k = 0; k < wa.size(); ++k) {
      char what[160];
      snprintf(what, sizeof(what), "%s: layer %zu tensor %zu", label, i, k);
      if (feeds_bn && k == 1) {
        snprintf(what, sizeof(what), "%s: layer %zu bias before batch normalization stays at rounding noise", label, i);
        expect(max_abs(*wc[k]) <= 1e-4 && max_abs(*wa[k]) <= 1e-4, what);
        continue;
      }
      close_vec(*wc[k], *wa[k], tol, what);
    }
  }
}

// Whole-net comparison at a large batch under adam.  Two fp32 evaluation orders agree on the forward
// pass to ~1e-6, which is enough for a relu gate or a max-pooling winner to be decided differently
// once in a few million positions; the gradient of that output channel then differs by that
// position's whole contribution, adam turns any gradient difference into a weight difference of
// up to one learning rate per step, and from the next step on that channel's activations differ at
// the 1e-3 level and many more decisions with them: the two trajectories separate the way the
// reference's own internal and AVX engines separate from each other on such a run (after six adam
// steps at batch 256 only ~65 % of their first-layer weights still agree to 1e-3, the worst by
// 1.6e-2 of the largest; after three steps all do).  So: at least `min_frac` of every tensor within
// 1e-3, and no entry further away than half of what adam can have moved it (one adam step moves a
// weight by up to alpha in the direction of its gradient's sign, so two runs whose gradients for a
// weight differ in sign separate by up to 2*alpha a step; the reference's own two CPU engines end
// 1.6e-2 of the largest weight apart on this case).
static void compare_nets_large_batch(network<sequential> &a, network<sequential> &c, double alpha, int steps,
                                     double min_frac, const char *label) {
  for (size_t i = 0; i < a.depth(); ++i) {
    auto wa = a[i]->weights();
    auto wc = c[i]->weights();
    for (size_t k = 0; k < wa.size(); ++k) {
      const vec_t &x = *wc[k], &y = *wa[k];
      const double scale = std::max(max_abs(y), 1e-30);
      size_t within = 0;
      double worst = 0;
      for (size_t j = 0; j < y.size(); ++j) {
        const double err = std::fabs((double)x[j] - (double)y[j]);
        if (err <= 1e-3 * scale) ++within;
        worst = std::max(worst, err);
      }
      const double frac = (double)within / (double)y.size();
      char what[200];
      const double bound = 0.5 * alpha * steps;
      snprintf(what, sizeof(what), "%s: layer %zu tensor %zu: %.1f%% within 1e-3, largest difference %.2e (bound %.2e)",
               label, i, k, 100.0 * frac, worst, bound);
      expect(frac >= min_frac && worst <= bound, what);
    }
  }
}

template <typename Opt>
static void compare_state(network<sequential> &a, network<sequential> &c, Opt &oa, Opt &oc, int n_state,
                          const char *label) {
  // the optimizer state the device-resident fit wrote back (stateful_optimizer::E_) against the CPU run's
  for (int k = 0; k < n_state; ++k)
    for (size_t i = 0; i < a.depth(); ++i) {
      auto wa = a[i]->weights();
      auto wc = c[i]->weights();
      for (size_t j = 0; j < wa.size(); ++j) {
        char what[160];
        snprintf(what, sizeof(what), "%s: optimizer state %d of layer %zu tensor %zu", label, k, i, j);
        close_vec(oc.b200_maps()[k][wc[j]], oa.b200_maps()[k][wa[j]], 1e-3, what);
      }
    }
}

// BASELINE configuration 2: the CIFAR-10 net at batch 256, adam, through network::fit.  With every
// layer on engine b200 the fit runs as the device-resident step (b200_net_fit_host).
static void build_cifar(network<sequential> &nn, core::backend_t e) {
  using conv = convolutional_layer;
  using pool = max_pooling_layer;
  using fc = fully_connected_layer;
  nn << conv(32, 32, 5, 3, 32, padding::same, true, 1, 1, 1, 1, e) << relu_layer() << pool(32, 32, 32, 2, false, e)
     << conv(16, 16, 5, 32, 32, padding::same, true, 1, 1, 1, 1, e) << relu_layer() << pool(16, 16, 32, 2, false, e)
     << conv(8, 8, 5, 32, 64, padding::same, true, 1, 1, 1, 1, e) << relu_layer() << pool(8, 8, 64, 2, false, e)
     << fc(4 * 4 * 64, 64, true, e) << relu_layer() << fc(64, 10, true, e) << softmax_layer(10);
}

static void ab_cifar_fit(size_t B, bool strict) {
  network<sequential> a, c;
  build_cifar(a, core::backend_t::internal);
  build_cifar(c, core::backend_t::b200);
  same_weights(a, c, 42);
  std::mt19937 g(1002);
  const size_t steps = 3;
  std::vector<vec_t> x(B * steps, vec_t(3 * 32 * 32)), t(B * steps, vec_t(10, 0.f));
  std::normal_distribution<float> nd(0.f, 1.f);
  for (auto &v : x)
    for (auto &e : v) e = nd(g);
  for (auto &v : t) v[g() % 10] = 1.f;
  adam oa, oc;
  char label[160];
  const unsigned long long fits = b200::device_fit_count();
  int batches = 0, epochs = 0;
  a.fit<cross_entropy>(oa, x, t, B, 1);
  c.fit<cross_entropy>(oc, x, t, B, 1, [&]() { ++batches; }, [&]() { ++epochs; });
  expect(b200::device_fit_count() == fits + 1, "CIFAR net: network::fit ran as the device-resident step");
  expect(batches == (int)steps && epochs == 1, "CIFAR net: per-batch and per-epoch callbacks were called");
  snprintf(label, sizeof(label), "CIFAR net batch %zu, 3 adam steps via network::fit", B);
  if (strict) {
    compare_nets(a, c, 1e-3, label);
    compare_state(a, c, oa, oc, 2, label);
  } else {
    compare_nets_large_batch(a, c, oa.alpha, (int)steps, 0.95, label);
  }
  expect(oa.b1_t == oc.b1_t && oa.b2_t == oc.b2_t, "CIFAR net: adam powers written back equal the CPU object's");
  // a second fit continues from the written-back powers (fit resets the state maps, not the powers)
  a.fit<cross_entropy>(oa, x, t, B, 1);
  c.fit<cross_entropy>(oc, x, t, B, 1);
  snprintf(label, sizeof(label), "CIFAR net batch %zu, second fit call", B);
  if (strict)
    compare_nets(a, c, 1e-3, label);
  else
    compare_nets_large_batch(a, c, oa.alpha, 2 * (int)steps, 0.0, label);
  expect(oa.b1_t == oc.b1_t && oa.b2_t == oc.b2_t, "CIFAR net: adam powers after the second fit");
  vec_t pa = a.predict(x[0]), pc = c.predict(x[0]);
  close_vec(pc, pa, strict ? 1e-4 : 2e-2, "CIFAR net predict after fit");
}

// BASELINE configuration 1: LeNet-5 (average pooling with trainable scale, tanh, connection table),
// mse on +-1 targets, adagrad, batch 16
static void build_lenet(network<sequential> &nn, core::backend_t e) {
  using conv = convolutional_layer;
  using ave = average_pooling_layer;
  using fc = fully_connected_layer;
#define O true
#define X false
  static const bool tbl[] = {O, X, X, X, O, O, O, X, X, O, O, O, O, X, O, O, O, O, X, X, X, O, O, O, X, X, O, O, O, O, X, O,
                             O, O, O, X, X, X, O, O, O, X, X, O, X, O, O, O, X, O, O, O, X, X, O, O, O, O, X, X, O, X, O, O,
                             X, X, O, O, O, X, X, O, O, O, O, X, O, O, X, O, X, X, X, O, O, O, X, X, O, O, O, O, X, O, O, O};
#undef O
#undef X
  nn << conv(32, 32, 5, 1, 6, padding::valid, true, 1, 1, 1, 1, e) << tanh_layer() << ave(28, 28, 6, 2) << tanh_layer()
     << conv(14, 14, 5, 6, 16, core::connection_table(tbl, 6, 16), padding::valid, true, 1, 1, 1, 1, e) << tanh_layer()
     << ave(10, 10, 16, 2) << tanh_layer() << conv(5, 5, 5, 16, 120, padding::valid, true, 1, 1, 1, 1, e)
     << tanh_layer() << fc(120, 10, true, e) << tanh_layer();
}

static void ab_lenet_fit() {
  network<sequential> a, c;
  build_lenet(a, core::backend_t::internal);
  build_lenet(c, core::backend_t::b200);
  same_weights(a, c, 9);
  std::mt19937 g(1001);
  const size_t B = 16, steps = 10;
  std::vector<vec_t> x(B * steps + 5, vec_t(32 * 32)), t(B * steps + 5, vec_t(10, -1.f));  // ragged last batch
  std::uniform_real_distribution<float> ud(-1.f, 1.f);
  for (auto &v : x)
    for (auto &e : v) e = ud(g);
  for (auto &v : t) v[g() % 10] = 1.f;
  adagrad oa, oc;
  const unsigned long long fits = b200::device_fit_count();
  a.fit<mse>(oa, x, t, B, 2);
  c.fit<mse>(oc, x, t, B, 2);
  expect(b200::device_fit_count() == fits + 1, "LeNet-5: network::fit ran as the device-resident step");
  compare_nets(a, c, 1e-3, "LeNet-5 batch 16, 2 epochs of 11 adagrad steps via network::fit");
  compare_state(a, c, oa, oc, 1, "LeNet-5");
}

// a layer that is not on the path (softsign) keeps the reference's loop: its b200 layers then run
// operator by operator; momentum
static void ab_operator_path() {
  auto build = [](network<sequential> &nn, core::backend_t e) {
    nn << convolutional_layer(12, 12, 3, 2, 4, padding::same, true, 1, 1, 1, 1, e) << softsign_layer()
       << max_pooling_layer(12, 12, 4, 2, false, e) << fully_connected_layer(6 * 6 * 4, 5, true, e) << softmax_layer(5);
  };
  network<sequential> a, c;
  build(a, core::backend_t::internal);
  build(c, core::backend_t::b200);
  same_weights(a, c, 21);
  std::mt19937 g(22);
  const size_t B = 6, steps = 3;
  std::vector<vec_t> x(B * steps, vec_t(12 * 12 * 2)), t(B * steps, vec_t(5, 0.f));
  std::normal_distribution<float> nd(0.f, 1.f);
  for (auto &v : x)
    for (auto &e : v) e = nd(g);
  for (auto &v : t) v[g() % 5] = 1.f;
  momentum oa, oc;
  const unsigned long long fits = b200::device_fit_count();
  a.fit<cross_entropy_multiclass>(oa, x, t, B, 1);
  c.fit<cross_entropy_multiclass>(oc, x, t, B, 1);
  expect(b200::device_fit_count() == fits, "a network with a layer off the path keeps the reference's loop");
  compare_nets(a, c, 1e-3, "operator-by-operator fit (softsign in the net), 3 momentum steps");
  // under engine b200 the weight-gradient tensors are not grown to one row per sample
  expect(c[0]->weights_grads()[0]->size() == 1 && a[0]->weights_grads()[0]->size() == B,
         "weight-gradient tensors stay at one row under engine b200 (B rows under internal)");
}

// leaky relu / elu / sigmoid (constructor parameters other than the defaults) between the hot
// operators: the whole fit runs as the device-resident step; RMSprop, mse
static void ab_parameter_activations_fit() {
  auto build = [](network<sequential> &nn, core::backend_t e) {
    nn << convolutional_layer(12, 12, 3, 2, 4, padding::same, true, 1, 1, 1, 1, e) << leaky_relu_layer(float_t(0.1))
       << max_pooling_layer(12, 12, 4, 2, false, e) << convolutional_layer(6, 6, 3, 4, 5, padding::valid, true, 1, 1, 1, 1, e)
       << elu_layer(float_t(0.8)) << fully_connected_layer(80, 6, true, e) << sigmoid_layer();
  };
  network<sequential> a, c;
  build(a, core::backend_t::internal);
  build(c, core::backend_t::b200);
  same_weights(a, c, 31);
  std::mt19937 g(32);
  const size_t B = 6, steps = 4;
  std::vector<vec_t> x(B * steps, vec_t(12 * 12 * 2)), t(B * steps, vec_t(6, 0.f));
  std::normal_distribution<float> nd(0.f, 1.f);
  for (auto &v : x)
    for (auto &e : v) e = nd(g);
  for (auto &v : t) v[g() % 6] = 1.f;
  RMSprop oa, oc;
  const unsigned long long fits = b200::device_fit_count();
  a.fit<mse>(oa, x, t, B, 1);
  c.fit<mse>(oc, x, t, B, 1);
  expect(b200::device_fit_count() == fits + 1, "leaky relu / elu / sigmoid net trains as the device-resident step");
  compare_nets(a, c, 1e-3, "leaky relu(0.1) / elu(0.8) / sigmoid net, 4 RMSprop steps");
}

// batch normalization between the hot operators: the fit runs as the device-resident step in the train
// phase, the moving averages come back into the layer objects, and predict (test phase, operator by
// operator) then agrees with the CPU network's
static void ab_batchnorm_fit() {
  auto build = [](network<sequential> &nn, core::backend_t e) {
    nn << convolutional_layer(12, 12, 3, 2, 4, padding::same, true, 1, 1, 1, 1, e) << batch_normalization_layer(144, 4)
       << relu_layer() << max_pooling_layer(12, 12, 4, 2, false, e)
       << convolutional_layer(6, 6, 3, 4, 5, padding::valid, true, 1, 1, 1, 1, e)
       << batch_normalization_layer(16, 5, float_t(1e-3), float_t(0.9)) << tanh_layer()
       << fully_connected_layer(80, 6, true, e) << softmax_layer(6);
  };
  network<sequential> a, c;
  build(a, core::backend_t::internal);
  build(c, core::backend_t::b200);
  same_weights(a, c, 51);
  std::mt19937 g(52);
  const size_t B = 6, steps = 4;
  std::vector<vec_t> x(B * steps, vec_t(12 * 12 * 2)), t(B * steps, vec_t(6, 0.f));
  std::normal_distribution<float> nd(0.f, 1.f);
  for (auto &v : x)
    for (auto &e : v) e = nd(g);
  for (auto &v : t) v[g() % 6] = 1.f;
  adam oa, oc;
  const unsigned long long fits = b200::device_fit_count();
  a.fit<cross_entropy>(oa, x, t, B, 1);
  c.fit<cross_entropy>(oc, x, t, B, 1);
  expect(b200::device_fit_count() == fits + 1, "a net with batch normalization trains as the device-resident step");
  compare_nets(a, c, 1e-3, "net with batch normalization, 4 adam steps");
  for (size_t i : {size_t(1), size_t(5)}) {
    auto *ba = dynamic_cast<batch_normalization_layer *>(a[i]);
    auto *bc = dynamic_cast<batch_normalization_layer *>(c[i]);
    char what[96];
    snprintf(what, sizeof(what), "moving mean of batch normalization layer %zu", i);
    close_vec(bc->b200_mean(), ba->b200_mean(), 1e-3, what);
    snprintf(what, sizeof(what), "moving variance of batch normalization layer %zu", i);
    close_vec(bc->b200_variance(), ba->b200_variance(), 1e-3, what);
  }
  vec_t pa = a.predict(x[0]), pc = c.predict(x[0]);
  close_vec(pc, pa, 1e-3, "predict after the fit (test phase: moving averages)");
}

// examples/cifar10/train.cpp's data path: parse_cifar10 -> train<cross_entropy> on the CPU against
// load_cifar10_u8 -> b200::train_u8 (raw bytes uploaded, scaled on the device), on a synthetic file
// in the CIFAR-10 binary format
static void ab_train_from_dataset_bytes() {
  const char *path = "/tmp/b200_synthetic_cifar10.bin";
  const size_t N = 50, B = 16;  // ragged last mini-batch
  {
    std::mt19937 g(77);
    FILE *f = fopen(path, "wb");
    if (!f) throw nn_error("cannot write the synthetic dataset file");
    for (size_t i = 0; i < N; ++i) {
      unsigned char rec[1 + 3072];
      rec[0] = (unsigned char)(g() % 10);
      for (size_t k = 0; k < 3072; ++k) rec[1 + k] = (unsigned char)(g() & 255);
      fwrite(rec, 1, sizeof(rec), f);
    }
    fclose(f);
  }
  std::vector<vec_t> images;
  std::vector<label_t> labels;
  parse_cifar10(path, &images, &labels, -1.0f, 1.0f, 0, 0);
  b200::u8_dataset data;
  b200::load_cifar10_u8(path, &data, -1.0f, 1.0f, 0, 0);
  expect(data.size() == N && images.size() == N, "synthetic CIFAR-10 file: both loaders read every record");
  network<sequential> a, c;
  build_cifar(a, core::backend_t::internal);
  build_cifar(c, core::backend_t::b200);
  same_weights(a, c, 5);
  adam oa, oc;
  a.train<cross_entropy>(oa, images, labels, B, 2);
  const unsigned long long fits = b200::device_fit_count();
  b200::train_u8<cross_entropy>(c, oc, data, B, 2);
  expect(b200::device_fit_count() == fits + 1, "train_u8 ran on the device");
  compare_nets(a, c, 1e-3, "train from dataset bytes, 2 epochs of 4 adam steps");
  expect(oa.b1_t == oc.b1_t && oa.b2_t == oc.b2_t, "train_u8: adam powers equal the CPU object's");
  remove(path);
}

static void ab_quantized() {
  std::mt19937 g(3);
  const size_t B = 3;
  quantized_convolutional_layer qa(12, 12, 5, 5, 4, 6, padding::valid, true, 1, 1, core::backend_t::internal);
  quantized_convolutional_layer qc(12, 12, 5, 5, 4, 6, padding::valid, true, 1, 1, core::backend_t::b200);
  tensor_t x(B, vec_t(4 * 12 * 12)), W(1, vec_t(6 * 4 * 25)), b(1, vec_t(6));
  for (auto &r : x) fill_uniform(r, g, -1.f, 1.f);
  fill_uniform(W[0], g, -0.5f, 0.5f);
  fill_uniform(b[0], g, -0.1f, 0.1f);
  tensor_t oa(B, vec_t(6 * 8 * 8)), oc(B, vec_t(6 * 8 * 8));
  std::vector<tensor_t *> ins = {&x, &W, &b}, outa = {&oa}, outc = {&oc};
  qa.set_parallelize(true);
  qa.forward_propagation(ins, outa);
  qc.forward_propagation(ins, outc);
  bool same = true;
  for (size_t s = 0; s < B; ++s) same = same && std::memcmp(oa[s].data(), oc[s].data(), oa[s].size() * sizeof(float)) == 0;
  if (same) {
    printf("ok   quantized convolution bit-exact\n");
  } else {
    printf("FAIL quantized convolution differs\n");
    ++g_fail;
  }
}

// conv2d_eq / fully_eq of core::backend, called on the backend objects themselves: every constructor of
// the quantized layers declares three inputs, so no layer of the tree reaches the six-input forms
static void ab_quantized_eq() {
  std::mt19937 g(5);
  const size_t B = 3;
  quantized_convolutional_layer owner(12, 12, 5, 5, 4, 6, padding::valid, true, 1, 1, core::backend_t::internal);
  owner.set_parallelize(true);
  core::conv_params p;
  p.in = shape3d(12, 12, 4);
  p.in_padded = p.in;
  p.out = shape3d(8, 8, 6);
  p.weight = shape3d(5, 5, 4 * 6);
  p.has_bias = true;
  p.pad_type = padding::valid;
  p.w_stride = p.h_stride = 1;
  p.w_dilation = p.h_dilation = 1;
  core::conv_layer_worker_specific_storage store;
  auto pad = [&](const tensor_t &in) {
    store.prev_out_padded_.resize(in.size());
    for (size_t s = 0; s < in.size(); ++s) store.prev_out_padded_[s] = &in[s];
  };
  core::tiny_backend cpu(&p, pad, [](const tensor_t &, tensor_t &) {},
                         [](const tensor_t &, const tensor_t &, tensor_t &) {}, &store);
  cpu.set_layer(&owner);
  core::b200_backend dev(&p, pad, &store);
  std::uniform_int_distribution<int> u8(0, 255);
  tensor_t x(B, vec_t(p.in.size())), W(1, vec_t(p.weight.size())), b(1, vec_t(6)), xr(B, vec_t(2));
  tensor_t Wr(1, vec_t{-0.5f, 0.5f}), br(1, vec_t{-0.1f, 0.1f});
  for (size_t s = 0; s < B; ++s) {
    for (auto &v : x[s]) v = static_cast<float>(u8(g));
    xr[s][0] = -1.f - 0.25f * s;
    xr[s][1] = 1.f + 0.125f * s;
  }
  for (auto &v : W[0]) v = static_cast<float>(u8(g));
  for (auto &v : b[0]) v = static_cast<float>(u8(g));
  tensor_t oa(B, vec_t(p.out.size())), oc(B, vec_t(p.out.size())), ra(B, vec_t(2)), rc(B, vec_t(2));
  std::vector<tensor_t *> ins = {&x, &W, &b, &xr, &Wr, &br}, outa = {&oa, &ra}, outc = {&oc, &rc};
  cpu.conv2d_eq(ins, outa);
  dev.conv2d_eq(ins, outc);
  bool same = true;
  for (size_t s = 0; s < B; ++s)
    same = same && std::memcmp(oa[s].data(), oc[s].data(), oa[s].size() * sizeof(float)) == 0 &&
           std::memcmp(ra[s].data(), rc[s].data(), 2 * sizeof(float)) == 0;
  expect(same, "conv2d_eq (uint8 values and ranges in and out) bit-exact against tiny_backend");

  // fully_eq: tiny_backend's needs gemmlowp (backend_tiny.h:321-345), so only the call shape is
  // exercised here; the values are pinned bit for bit by the library's own tests
  core::fully_params fp;
  fp.in_size_ = 40;
  fp.out_size_ = 7;
  fp.has_bias_ = true;
  core::b200_backend devf(&fp);
  tensor_t fx(B, vec_t(40)), fW(1, vec_t(40 * 7)), fb(1, vec_t(7)), fo(B, vec_t(7)), fr(B, vec_t(2));
  for (auto &r : fx)
    for (auto &v : r) v = static_cast<float>(u8(g));
  for (auto &v : fW[0]) v = static_cast<float>(u8(g));
  for (auto &v : fb[0]) v = static_cast<float>(u8(g));
  std::vector<tensor_t *> fins = {&fx, &fW, &fb, &xr, &Wr, &br}, fouts = {&fo, &fr};
  devf.fully_eq(fins, fouts);
  bool sane = true;
  for (size_t s = 0; s < B; ++s) {
    sane = sane && fr[s][0] < fr[s][1];
    for (float v : fo[s]) sane = sane && v >= 0.f && v <= 255.f && v == std::floor(v);
  }
  expect(sane, "fully_eq returns uint8 values and an ordered range");
}

int main() {
  try {
    {
      convolutional_layer l(12, 10, 5, 5, 2, 6, padding::same, true, 1, 1, 1, 1, core::backend_t::internal);
      ab_layer("conv 5x5 same", l, 3, true, 1);
    }
    {
      convolutional_layer l(9, 9, 3, 3, 2, 3, padding::valid, true, 2, 2, 1, 1, core::backend_t::internal);
      ab_layer("conv 3x3 stride 2", l, 2, true, 2);
    }
    {
      bool tbl[] = {true, false, true, true, true, false, false, true, true, true, true, false};  // 3 in x 4 out
      convolutional_layer l(10, 10, 5, 3, 4, core::connection_table(tbl, 3, 4), padding::valid, true, 1, 1, 1, 1,
                            core::backend_t::internal);
      ab_layer("conv 5x5 connection table", l, 3, true, 3);
    }
    {
      fully_connected_layer l(130, 67, true, core::backend_t::internal);
      ab_layer("fully connected", l, 5, true, 4);
    }
    {
      max_pooling_layer l(8, 8, 3, 2, 2, false, core::backend_t::internal);
      ab_layer("max pool 2x2", l, 3, false, 5);
    }
    {
      max_pooling_layer l(7, 7, 2, 3, 3, 2, 2, false, padding::valid, core::backend_t::internal);
      ab_layer("max pool 3x3 stride 2", l, 2, false, 6);
    }
    {
      relu_layer l(37);
      ab_layer("relu (set_backend_type)", l, 4, false, 7);
    }
    {
      tanh_layer l(37);
      ab_layer("tanh (set_backend_type)", l, 4, false, 8);
    }
    {
      softmax_layer l(10);
      ab_layer("softmax (set_backend_type)", l, 6, false, 9);
    }
    {
      sigmoid_layer l(37);
      ab_layer("sigmoid (set_backend_type)", l, 4, false, 11);
    }
    {
      leaky_relu_layer l(37, float_t(0.2));
      ab_layer("leaky relu 0.2 (set_backend_type)", l, 4, false, 12);
    }
    {
      elu_layer l(37, float_t(0.7));
      ab_layer("elu 0.7 (set_backend_type)", l, 4, false, 13);
    }
    {
      batch_normalization_layer l(49, 6);
      ab_layer("batch normalization, train phase (set_backend_type)", l, 5, false, 14);
    }
    ab_batchnorm_test_phase();
    ab_lrn();
    {
      average_pooling_layer l(28, 28, 6, 2);
      ab_layer("average pooling 2x2 (set_backend_type)", l, 4, true, 10);
    }
    ab_network();
    ab_optimizer<RMSprop>("RMSprop", 1);
    ab_optimizer<adamax>("adamax", 2);
    ab_optimizer<gradient_descent>("gradient_descent", 0);
    ab_optimizer<nesterov_momentum>("nesterov_momentum", 1);
    ab_optimizer<momentum>("momentum", 1);
    ab_optimizer<adagrad>("adagrad", 1);
    ab_operator_path();
    ab_parameter_activations_fit();
    ab_batchnorm_fit();
    ab_lenet_fit();
    ab_cifar_fit(16, true);    // optimizer hand-off held to 1e-3 where decision flips are improbable
    ab_cifar_fit(256, false);  // the benchmarked batch
    ab_train_from_dataset_bytes();
    ab_quantized();
    ab_quantized_eq();
    std::ostringstream os;
    os << core::backend_t::b200;
    if (os.str() != "B200") {
      printf("FAIL operator<< gives %s\n", os.str().c_str());
      ++g_fail;
    }
  } catch (const std::exception &e) {
    printf("FAIL exception: %s\n", e.what());
    return 2;
  }
  printf(g_fail ? "RESULT: %d FAILED\n" : "RESULT: all passed\n", g_fail);
  return g_fail ? 1 : 0;
}
