// Data-parallel network<sequential>::fit from C++: one process per GPU, no framework.
//
// The parent forks `world` children before anything touches CUDA and serves as the hub of the
// buffer-handle exchange (two pipes per child).  Child r selects GPU r (B200_DEVICE), builds the
// CIFAR-10-style net on backend_t::b200 from a fixed seed, fills tiny_dnn::b200::replicas() and
// calls fit<cross_entropy> with adam on ITS shard of the data.  Checks:
//   * every child: its weights against backend_t::internal training in one process on the
//     concatenated mini-batches (gradients are summed over samples, tiny_dnn/layers/layer.h:663-673,
//     so `world` shards of B samples are one mini-batch of world * B), at 1e-3 of a tensor's
//     largest weight;
//   * the parent: the children's weights agree bit for bit.
// usage: test_dp_b200 [world = 2]
#include <sys/types.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "tiny_dnn/tiny_dnn.h"

using namespace tiny_dnn;
using namespace tiny_dnn::activation;
using namespace tiny_dnn::layers;

static bool read_all(int fd, void *buf, size_t n) {
  char *p = static_cast<char *>(buf);
  while (n) {
    ssize_t k = read(fd, p, n);
    if (k <= 0) return false;
    p += k;
    n -= static_cast<size_t>(k);
  }
  return true;
}

static bool write_all(int fd, const void *buf, size_t n) {
  const char *p = static_cast<const char *>(buf);
  while (n) {
    ssize_t k = write(fd, p, n);
    if (k <= 0) return false;
    p += k;
    n -= static_cast<size_t>(k);
  }
  return true;
}

static void build_cifar(network<sequential> &nn, core::backend_t e) {
  using conv = convolutional_layer;
  using pool = max_pooling_layer;
  using fc = fully_connected_layer;
  nn << conv(32, 32, 5, 3, 32, padding::same, true, 1, 1, 1, 1, e) << relu_layer() << pool(32, 32, 32, 2, false, e)
     << conv(16, 16, 5, 32, 32, padding::same, true, 1, 1, 1, 1, e) << relu_layer() << pool(16, 16, 32, 2, false, e)
     << conv(8, 8, 5, 32, 64, padding::same, true, 1, 1, 1, 1, e) << relu_layer() << pool(8, 8, 64, 2, false, e)
     << fc(4 * 4 * 64, 64, true, e) << relu_layer() << fc(64, 10, true, e) << softmax_layer(10);
}

static std::vector<float> flat_weights(network<sequential> &nn) {
  std::vector<float> f;
  for (size_t i = 0; i < nn.depth(); ++i)
    for (auto *w : nn[i]->weights()) f.insert(f.end(), w->begin(), w->end());
  return f;
}

// the child of rank `rank`: returns 0 when its checks passed
static int child(int rank, int world, int up, int down, int result) {
  char dev[16];
  snprintf(dev, sizeof(dev), "%d", rank);
  setenv("B200_DEVICE", dev, 1);
  const size_t B = 8, steps = 3;
  int fail = 0;
  try {
    // the same data in every process: step s of rank r is rows [(s * world + r) * B, +B) of the whole
    std::mt19937 g(2024);
    std::normal_distribution<float> nd(0.f, 1.f);
    std::vector<vec_t> x(B * steps * world, vec_t(3 * 32 * 32)), t(B * steps * world, vec_t(10, 0.f));
    for (auto &v : x)
      for (auto &e : v) e = nd(g);
    for (auto &v : t) v[g() % 10] = 1.f;
    std::vector<vec_t> xs, ts;
    for (size_t s = 0; s < steps; ++s)
      for (size_t i = 0; i < B; ++i) {
        xs.push_back(x[(s * world + rank) * B + i]);
        ts.push_back(t[(s * world + rank) * B + i]);
      }

    network<sequential> a, c;
    build_cifar(a, core::backend_t::internal);
    build_cifar(c, core::backend_t::b200);
    set_random_seed(42);
    a.init_weight();
    c.init_weight();
    for (size_t i = 0; i < a.depth(); ++i) {
      auto wa = a[i]->weights();
      auto wc = c[i]->weights();
      for (size_t k = 0; k < wa.size(); ++k) *wc[k] = *wa[k];
    }

    b200::replica_group &grp = b200::replicas();
    grp.rank = rank;
    grp.world = world;
    grp.timeout_ms = 5000;
    grp.exchange = [&](const unsigned char *own, unsigned char *all) {
      if (!write_all(up, own, B200_PEER_HANDLE_BYTES) ||
          !read_all(down, all, static_cast<size_t>(world) * B200_PEER_HANDLE_BYTES))
        throw nn_error("handle exchange with the launcher failed");
    };

    adam oa, oc;
    const unsigned long long fits = b200::device_fit_count();
    c.fit<cross_entropy>(oc, xs, ts, B, 1);                  // this rank's shard, B samples a step
    if (b200::device_fit_count() != fits + 1) {
      printf("FAIL rank %d: fit did not run as the device-resident step\n", rank);
      ++fail;
    }
    a.fit<cross_entropy>(oa, x, t, B * world, 1);            // one process, the concatenated mini-batches

    double worst = 0;
    for (size_t i = 0; i < a.depth(); ++i) {
      auto wa = a[i]->weights();
      auto wc = c[i]->weights();
      for (size_t k = 0; k < wa.size(); ++k) {
        double big = 0, diff = 0;
        for (size_t j = 0; j < wa[k]->size(); ++j) {
          big = std::max(big, static_cast<double>(std::fabs((*wa[k])[j])));
          diff = std::max(diff, static_cast<double>(std::fabs((*wa[k])[j] - (*wc[k])[j])));
        }
        worst = std::max(worst, diff / std::max(big, 1e-30));
      }
    }
    const bool near = worst <= 1e-3;
    printf("%s rank %d: weights after %zu data-parallel adam steps vs one process on the concatenated batches: worst %.2e\n",
           near ? "ok  " : "FAIL", rank, steps, worst);
    if (!near) ++fail;
    if (oa.b1_t != oc.b1_t || oa.b2_t != oc.b2_t) {
      printf("FAIL rank %d: adam powers differ from the single-process object's\n", rank);
      ++fail;
    }
    // end the handle exchange first: the launcher reads the results only after its hub loop has seen
    // this end of the pipe close, and the weights do not fit a pipe's buffer
    close(up);
    close(down);
    up = down = -1;
    std::vector<float> f = flat_weights(c);
    unsigned long long n = f.size();
    if (!write_all(result, &n, sizeof(n)) || !write_all(result, f.data(), n * sizeof(float))) ++fail;
  } catch (const std::exception &e) {
    printf("FAIL rank %d: %s\n", rank, e.what());
    ++fail;
  }
  fflush(stdout);
  if (up >= 0) close(up);
  if (down >= 0) close(down);
  close(result);
  return fail ? 1 : 0;
}

int main(int argc, char **argv) {
  const int world = argc > 1 ? atoi(argv[1]) : 2;
  if (world < 2 || world > 8) {
    printf("usage: %s [world 2..8]\n", argv[0]);
    return 2;
  }
  std::vector<int> up_r(world), down_w(world), res_r(world);
  std::vector<pid_t> pids(world);
  std::vector<std::vector<int>> parent_fds;
  for (int r = 0; r < world; ++r) {
    int up[2], down[2], res[2];
    if (pipe(up) || pipe(down) || pipe(res)) return 2;
    fflush(stdout);
    pid_t pid = fork();
    if (pid < 0) return 2;
    if (pid == 0) {
      close(up[0]);
      close(down[1]);
      close(res[0]);
      for (int q = 0; q < r; ++q) {  // the parent's ends towards the earlier children
        close(up_r[q]);
        close(down_w[q]);
        close(res_r[q]);
      }
      _exit(child(r, world, up[1], down[0], res[1]));
    }
    close(up[1]);
    close(down[0]);
    close(res[1]);
    pids[r] = pid;
    up_r[r] = up[0];
    down_w[r] = down[1];
    res_r[r] = res[0];
  }
  // hub: a round = one handle from every child, then all handles to every child; until a child ends
  std::vector<unsigned char> all(static_cast<size_t>(world) * B200_PEER_HANDLE_BYTES);
  int rounds = 0;
  for (;;) {
    bool ok = true;
    for (int r = 0; r < world && ok; ++r) ok = read_all(up_r[r], all.data() + static_cast<size_t>(r) * B200_PEER_HANDLE_BYTES, B200_PEER_HANDLE_BYTES);
    if (!ok) break;
    for (int r = 0; r < world; ++r) write_all(down_w[r], all.data(), all.size());
    ++rounds;
  }
  int fail = 0;
  std::vector<std::vector<float>> weights(world);
  for (int r = 0; r < world; ++r) {
    unsigned long long n = 0;
    if (read_all(res_r[r], &n, sizeof(n)) && n < (1ull << 28)) {
      weights[r].resize(n);
      if (!read_all(res_r[r], weights[r].data(), n * sizeof(float))) weights[r].clear();
    }
  }
  for (int r = 0; r < world; ++r) {
    int st = 0;
    waitpid(pids[r], &st, 0);
    if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) {
      printf("FAIL rank %d ended with status %d\n", r, st);
      ++fail;
    }
  }
  bool same = !weights[0].empty();
  for (int r = 1; r < world && same; ++r)
    same = weights[r].size() == weights[0].size() &&
           std::memcmp(weights[r].data(), weights[0].data(), weights[0].size() * sizeof(float)) == 0;
  printf("%s the %d replicas hold bit-identical weights (%zu floats, %d handle exchange%s)\n", same ? "ok  " : "FAIL", world,
         weights[0].size(), rounds, rounds == 1 ? "" : "s");
  if (!same) ++fail;
  printf(fail ? "RESULT: %d failed\n" : "RESULT: all passed\n", fail);
  return fail ? 1 : 0;
}
