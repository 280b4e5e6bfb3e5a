// bench_fit.cpp -- network<sequential>::fit of the CIFAR-10 net under engine backend_t::b200,
// timed end to end from the C++ side: std::vector<vec_t> inputs in pageable host memory go in,
// trained weights in the layer objects come out.  Compiled against the overlay of
// make_overlay.py and the tiny-dnn tree (oracle/build_oracle.py); bench.py runs the binary and
// reports its figure as `e2e_cpp`.
//
//   bench_fit_b200 [steps] [batch]      prints one JSON line
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>

#include "tiny_dnn/tiny_dnn.h"

using namespace tiny_dnn;

int main(int argc, char **argv) {
  const size_t steps = argc > 1 ? (size_t)atoi(argv[1]) : 200;
  const size_t B = argc > 2 ? (size_t)atoi(argv[2]) : 256;
  const core::backend_t e = core::backend_t::b200;
  try {
    network<sequential> nn;
    using conv = convolutional_layer;
    using pool = max_pooling_layer;
    using fc = fully_connected_layer;
    // examples/cifar10/train.cpp:26-42 in conv-relu-pool order
    nn << conv(32, 32, 5, 3, 32, padding::same, true, 1, 1, 1, 1, e) << relu_layer() << pool(32, 32, 32, 2, false, e)
       << conv(16, 16, 5, 32, 32, padding::same, true, 1, 1, 1, 1, e) << relu_layer() << pool(16, 16, 32, 2, false, e)
       << conv(8, 8, 5, 32, 64, padding::same, true, 1, 1, 1, 1, e) << relu_layer() << pool(8, 8, 64, 2, false, e)
       << fc(4 * 4 * 64, 64, true, e) << relu_layer() << fc(64, 10, true, e) << softmax_layer(10);
    set_random_seed(42);
    nn.init_weight();
    std::mt19937 g(1000);
    std::normal_distribution<float> nd(0.f, 1.f);
    const size_t N = steps * B;
    std::vector<vec_t> x(N, vec_t(3 * 32 * 32)), t(N, vec_t(10, 0.f));
    // eight distinct mini-batches repeated: the same rotation bench.py uses
    for (size_t s = 0; s < std::min(N, 8 * B); ++s) {
      for (auto &v : x[s]) v = nd(g);
      t[s][g() % 10] = 1.f;
    }
    for (size_t s = 8 * B; s < N; ++s) {
      x[s] = x[s % (8 * B)];
      t[s] = t[s % (8 * B)];
    }
    adam opt;
    // warm-up over the same data: builds the device twin, captures the step's graph and sizes the
    // page-locked staging, as the first epoch of a real run does once
    nn.fit<cross_entropy>(opt, x, t, B, 1);
    const unsigned long long fits = b200::device_fit_count();
    auto t0 = std::chrono::steady_clock::now();
    nn.fit<cross_entropy>(opt, x, t, B, 1);
    auto t1 = std::chrono::steady_clock::now();
    const double secs = std::chrono::duration<double>(t1 - t0).count();
    printf("{\"samples_per_s\": %.1f, \"ms_per_step\": %.4f, \"steps\": %zu, \"batch\": %zu, \"device_fit\": %s, "
           "\"kernels_launched\": %llu}\n",
           N / secs, 1e3 * secs / steps, steps, B, b200::device_fit_count() == fits + 1 ? "true" : "false",
           b200_launch_count());
  } catch (const std::exception &ex) {
    fprintf(stderr, "bench_fit_b200: %s\n", ex.what());
    return 1;
  }
  return 0;
}
