// Context, error text, memory helpers and descriptor helpers of the C ABI.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace b200 {

static thread_local char g_err[1024] = "";
std::atomic<unsigned long long> g_launches{0};

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
void clear_error() { g_err[0] = 0; }

static int grow(b200_ctx *ctx, void **buf, size_t *have, size_t need, bool pinned_host) {
  if (need <= *have) return 0;
  // The old buffer may still be read by work queued on the stream.
  B200_CUDA(cudaStreamSynchronize(ctx->stream));
  if (*buf) {
    if (pinned_host)
      B200_CUDA(cudaFreeHost(*buf));
    else
      B200_CUDA(cudaFree(*buf));
    *buf = nullptr;
    *have = 0;
  }
  size_t want = align_up(need + need / 4, 1 << 20);
  if (pinned_host)
    B200_CUDA(cudaMallocHost(buf, want));
  else
    B200_CUDA(cudaMalloc(buf, want));
  *have = want;
  return 0;
}

int ctx_scratch(b200_ctx *ctx, size_t bytes, void **out) {
  B200_TRY(grow(ctx, &ctx->scratch, &ctx->scratch_bytes, bytes, false));
  *out = ctx->scratch;
  return 0;
}
int ctx_arena(b200_ctx *ctx, size_t bytes, void **out) {
  B200_TRY(grow(ctx, &ctx->arena, &ctx->arena_bytes, bytes, false));
  *out = ctx->arena;
  return 0;
}
int ctx_pinned(b200_ctx *ctx, size_t bytes, void **out) {
  B200_TRY(grow(ctx, &ctx->pinned, &ctx->pinned_bytes, bytes, true));
  *out = ctx->pinned;
  return 0;
}

int ctx_device_table(b200_ctx *ctx, const uint8_t *host_tbl, size_t n, const uint8_t **out) {
  if (!host_tbl) {
    *out = nullptr;
    return 0;
  }
  std::string key(reinterpret_cast<const char *>(host_tbl), n);
  auto it = ctx->tbl_cache.find(key);
  if (it != ctx->tbl_cache.end()) {
    *out = it->second;
    return 0;
  }
  uint8_t *dev = nullptr;
  B200_CUDA(cudaMalloc(&dev, n));
  B200_CUDA(cudaMemcpy(dev, host_tbl, n, cudaMemcpyHostToDevice));
  ctx->tbl_cache[key] = dev;
  *out = dev;
  return 0;
}

void ctx_remember_tile(b200_ctx *ctx, const std::string &key, const TileChoice &c) {
  ctx->tile_cache[key] = c;
  if (const char *path = getenv("B200_TUNE_CACHE")) {
    if (FILE *f = fopen(path, "a")) {
      fprintf(f, "%s|%d %d %d %d %d %d\n", key.c_str(), c.OCT, c.OCB, c.TH, c.TWG, c.NSB, c.ICB);
      fclose(f);
    }
  }
}

static void ctx_load_tiles(b200_ctx *ctx) {
  const char *path = getenv("B200_TUNE_CACHE");
  if (!path) return;
  FILE *f = fopen(path, "r");
  if (!f) return;
  char line[512];
  while (fgets(line, sizeof(line), f)) {
    char *bar = strchr(line, '|');
    if (!bar) continue;
    *bar = 0;
    TileChoice c{};
    if (sscanf(bar + 1, "%d %d %d %d %d %d", &c.OCT, &c.OCB, &c.TH, &c.TWG, &c.NSB, &c.ICB) == 6)
      ctx->tile_cache[line] = c;
  }
  fclose(f);
}

int conv_geom_from_desc(b200_ctx *ctx, const b200_conv_desc *d, ConvGeom *g) {
  B200_REQUIRE(d != nullptr, "conv descriptor is NULL");
  B200_REQUIRE(d->in_w > 0 && d->in_h > 0 && d->in_c > 0 && d->out_c > 0 && d->k_w > 0 &&
                 d->k_h > 0 && d->out_w > 0 && d->out_h > 0,
               "conv descriptor has a non-positive extent");
  B200_REQUIRE(d->stride_w > 0 && d->stride_h > 0 && d->dil_w > 0 && d->dil_h > 0,
               "conv descriptor has a non-positive stride or dilation");
  bool padded_buffers = d->input_is_padded || !d->pad_same;
  g->C = d->in_c;
  g->HI = padded_buffers ? d->inp_h : d->in_h;
  g->WI = padded_buffers ? d->inp_w : d->in_w;
  g->OC = d->out_c;
  g->OH = d->out_h;
  g->OW = d->out_w;
  g->KH = d->k_h;
  g->KW = d->k_w;
  g->SH = d->stride_h;
  g->SW = d->stride_w;
  g->DH = d->dil_h;
  g->DW = d->dil_w;
  g->pad_t = padded_buffers ? 0 : d->k_h / 2;
  g->pad_l = padded_buffers ? 0 : d->k_w / 2;
  g->has_bias = d->has_bias;
  // the last window must stay inside the (logically padded) input
  int hp = d->inp_h, wp = d->inp_w;
  B200_REQUIRE((d->out_h - 1) * d->stride_h + (d->k_h - 1) * d->dil_h < hp &&
                 (d->out_w - 1) * d->stride_w + (d->k_w - 1) * d->dil_w < wp,
               "conv descriptor: window leaves the padded input (%dx%d in, %dx%d out)", wp, hp,
               d->out_w, d->out_h);
  B200_TRY(ctx_device_table(ctx, d->tbl, (size_t)d->in_c * d->out_c, &g->tbl));
  return 0;
}

size_t conv_weight_len(const ConvGeom &g) { return (size_t)g.OC * g.C * g.KH * g.KW; }

}  // namespace b200

using namespace b200;

extern "C" {

const char *b200_version(void) { return "0.1"; }
const char *b200_last_error(void) { return b200::g_err; }
unsigned long long b200_launch_count(void) { return g_launches.load(); }

int b200_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int b200_ctx_create(int device, void *stream, b200_ctx **out) {
  B200_REQUIRE(out != nullptr, "b200_ctx_create: out is NULL");
  int n = b200_device_count();
  B200_REQUIRE(n > 0, "b200_ctx_create: no CUDA device is visible; this library has no CPU path");
  B200_REQUIRE(device >= 0 && device < n, "b200_ctx_create: device %d out of range (%d visible)",
               device, n);
  B200_CUDA(cudaSetDevice(device));
  b200_ctx *c = new b200_ctx();
  c->device = device;
  cudaDeviceProp prop;
  B200_CUDA(cudaGetDeviceProperties(&prop, device));
  c->sm_count = prop.multiProcessorCount;
  c->smem_optin = prop.sharedMemPerBlockOptin;
  if (stream) {
    c->stream = (cudaStream_t)stream;
    c->own_stream = false;
  } else {
    // above the default priority: a net's side branch runs at the default one and yields to this stream
    B200_CUDA(cudaStreamCreateWithPriority(&c->stream, cudaStreamNonBlocking, -1));
    c->own_stream = true;
  }
  ctx_load_tiles(c);
  B200_CUDA(cudaMalloc(&c->dev_err, sizeof(int)));
  B200_CUDA(cudaMemset(c->dev_err, 0, sizeof(int)));
  *out = c;
  return 0;
}

// ---------------------------------------------------------------- exchange buffers across processes
static_assert(sizeof(cudaIpcMemHandle_t) <= B200_PEER_HANDLE_BYTES, "handle does not fit its ABI size");

int b200_peer_buffer_create(b200_ctx *ctx, size_t bytes, void **dev, unsigned char *handle) {
  B200_REQUIRE(ctx && dev && handle, "peer_buffer_create: NULL argument");
  B200_REQUIRE(bytes > 0, "peer_buffer_create: empty buffer");
  B200_CUDA(cudaSetDevice(ctx->device));
  void *p = nullptr;
  // a plain cudaMalloc: memory of a stream-ordered pool cannot be exported
  B200_CUDA(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    B200_CUDA(e);
  }
  memset(handle, 0, B200_PEER_HANDLE_BYTES);
  memcpy(handle, &h, sizeof(h));
  *dev = p;
  return 0;
}

int b200_peer_buffer_open(b200_ctx *ctx, const unsigned char *handle, void **dev) {
  B200_REQUIRE(ctx && dev && handle, "peer_buffer_open: NULL argument");
  B200_CUDA(cudaSetDevice(ctx->device));
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void *p = nullptr;
  B200_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *dev = p;
  return 0;
}

int b200_peer_buffer_close(b200_ctx *ctx, void *dev) {
  B200_REQUIRE(ctx != nullptr, "peer_buffer_close: NULL context");
  if (!dev) return 0;
  B200_CUDA(cudaSetDevice(ctx->device));
  B200_CUDA(cudaIpcCloseMemHandle(dev));
  return 0;
}

int b200_peer_buffer_destroy(b200_ctx *ctx, void *dev) {
  B200_REQUIRE(ctx != nullptr, "peer_buffer_destroy: NULL context");
  if (!dev) return 0;
  B200_CUDA(cudaSetDevice(ctx->device));
  B200_CUDA(cudaFree(dev));
  return 0;
}

int b200_ctx_destroy(b200_ctx *ctx) {
  if (!ctx) return 0;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->arena) cudaFree(ctx->arena);
  if (ctx->pinned) cudaFreeHost(ctx->pinned);
  if (ctx->dev_err) cudaFree(ctx->dev_err);
  for (auto &kv : ctx->tbl_cache) cudaFree(kv.second);
  if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
  return 0;
}

int b200_ctx_set_stream(b200_ctx *ctx, void *stream) {
  B200_REQUIRE(ctx != nullptr, "ctx is NULL");
  B200_CUDA(cudaStreamSynchronize(ctx->stream));
  if (ctx->own_stream) {
    cudaStreamDestroy(ctx->stream);
    ctx->own_stream = false;
  }
  ctx->stream = (cudaStream_t)stream;
  return 0;
}

int b200_ctx_set_option(b200_ctx *ctx, const char *name, int value) {
  B200_REQUIRE(ctx != nullptr && name != nullptr, "ctx_set_option: NULL argument");
  if (strcmp(name, "fc_tensor_cores") == 0) {
    B200_REQUIRE(value >= 0 && value <= 2, "fc_tensor_cores must be 0, 1 or 2");
    ctx->fc_tensor_cores = value;
    return 0;
  }
  if (strcmp(name, "conv_tensor_cores") == 0) {
    B200_REQUIRE(value >= 0 && value <= 2, "conv_tensor_cores must be 0, 1 or 2");
    ctx->conv_tensor_cores = value;
    return 0;
  }
  B200_REQUIRE(false, "ctx_set_option: unknown option '%s'", name);
  return 0;
}

void *b200_ctx_stream(b200_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

int b200_ctx_sync(b200_ctx *ctx) {
  B200_REQUIRE(ctx != nullptr, "ctx is NULL");
  B200_CUDA(cudaStreamSynchronize(ctx->stream));
  if (ctx->dev_err) {
    int flag = 0;
    B200_CUDA(cudaMemcpy(&flag, ctx->dev_err, sizeof(int), cudaMemcpyDeviceToHost));
    if (flag != 0) {
      cudaMemset(ctx->dev_err, 0, sizeof(int));
      B200_REQUIRE(false, "a kernel gave up a bounded wait (code %d: %s)", flag,
                   flag == 7 ? "the sum of the gradients over the replicas timed out waiting for another rank; this rank "
                               "skipped the update, the replicas differ from now on"
                             : "an asynchronous copy or tensor-core operation did not complete");
    }
  }
  return 0;
}

int b200_host_alloc(size_t bytes, void **out) {
  B200_REQUIRE(out != nullptr, "b200_host_alloc: NULL argument");
  B200_CUDA(cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocPortable));
  return 0;
}
int b200_host_free(void *ptr) {
  if (ptr) B200_CUDA(cudaFreeHost(ptr));
  return 0;
}

int b200_malloc(b200_ctx *ctx, size_t bytes, void **out) {
  B200_REQUIRE(ctx != nullptr && out != nullptr, "b200_malloc: NULL argument");
  B200_CUDA(cudaSetDevice(ctx->device));
  B200_CUDA(cudaMalloc(out, bytes ? bytes : 1));
  return 0;
}
int b200_free(b200_ctx *ctx, void *ptr) {
  B200_REQUIRE(ctx != nullptr, "ctx is NULL");
  B200_CUDA(cudaStreamSynchronize(ctx->stream));
  B200_CUDA(cudaFree(ptr));
  return 0;
}
int b200_memcpy_h2d(b200_ctx *ctx, void *dst, const void *src, size_t bytes) {
  B200_REQUIRE(ctx != nullptr, "ctx is NULL");
  B200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  B200_CUDA(cudaStreamSynchronize(ctx->stream));
  return 0;
}
int b200_memcpy_d2h(b200_ctx *ctx, void *dst, const void *src, size_t bytes) {
  B200_REQUIRE(ctx != nullptr, "ctx is NULL");
  B200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  B200_CUDA(cudaStreamSynchronize(ctx->stream));
  return 0;
}
int b200_memset(b200_ctx *ctx, void *dst, int value, size_t bytes) {
  B200_REQUIRE(ctx != nullptr, "ctx is NULL");
  B200_CUDA(cudaMemsetAsync(dst, value, bytes, ctx->stream));
  return 0;
}

// conv_out_length (tiny_dnn/util/util.h:329-344)
static int conv_out_len(int in, int k, int stride, int dil, int pad_same) {
  int len = pad_same ? in : in - dil * k + dil;
  return (len + stride - 1) / stride;
}

int b200_conv_desc_init(b200_conv_desc *d, int in_w, int in_h, int in_c, int k_w, int k_h,
                        int out_c, int pad_same, int has_bias, int stride_w, int stride_h,
                        int dil_w, int dil_h) {
  B200_REQUIRE(d != nullptr, "b200_conv_desc_init: d is NULL");
  B200_REQUIRE(in_w > 0 && in_h > 0 && in_c > 0 && k_w > 0 && k_h > 0 && out_c > 0 &&
                 stride_w > 0 && stride_h > 0 && dil_w > 0 && dil_h > 0,
               "b200_conv_desc_init: non-positive argument");
  memset(d, 0, sizeof(*d));
  d->in_w = in_w;
  d->in_h = in_h;
  d->in_c = in_c;
  d->inp_w = pad_same ? in_w + k_w - 1 : in_w;
  d->inp_h = pad_same ? in_h + k_h - 1 : in_h;
  d->out_w = conv_out_len(in_w, k_w, stride_w, dil_w, pad_same);
  d->out_h = conv_out_len(in_h, k_h, stride_h, dil_h, pad_same);
  d->out_c = out_c;
  d->k_w = k_w;
  d->k_h = k_h;
  d->stride_w = stride_w;
  d->stride_h = stride_h;
  d->dil_w = dil_w;
  d->dil_h = dil_h;
  d->has_bias = has_bias;
  d->pad_same = pad_same;
  B200_REQUIRE(d->out_w > 0 && d->out_h > 0, "b200_conv_desc_init: empty output");
  return 0;
}

// pool_out_length (tiny_dnn/util/util.h:346-363)
static int pool_out_len(int in, int win, int stride, int ceil_mode, int pad_same) {
  int len = pad_same ? in : in - win + 1;
  float tmp = static_cast<float>(len + stride - 1) / stride;
  return static_cast<int>(ceil_mode ? ceilf(tmp) : floorf(tmp));
}

int b200_pool_desc_init(b200_pool_desc *d, int in_w, int in_h, int in_c, int pool_w, int pool_h,
                        int stride_w, int stride_h, int ceil_mode, int pad_same) {
  B200_REQUIRE(d != nullptr, "b200_pool_desc_init: d is NULL");
  B200_REQUIRE(in_w > 0 && in_h > 0 && in_c > 0 && pool_w > 0 && pool_h > 0 && stride_w > 0 &&
                 stride_h > 0,
               "b200_pool_desc_init: non-positive argument");
  d->in_w = in_w;
  d->in_h = in_h;
  d->in_c = in_c;
  d->pool_w = pool_w;
  d->pool_h = pool_h;
  d->stride_w = stride_w;
  d->stride_h = stride_h;
  d->out_w = pool_out_len(in_w, pool_w, stride_w, ceil_mode, pad_same);
  d->out_h = pool_out_len(in_h, pool_h, stride_h, ceil_mode, pad_same);
  B200_REQUIRE(d->out_w > 0 && d->out_h > 0, "b200_pool_desc_init: empty output");
  return 0;
}

}  // extern "C"
