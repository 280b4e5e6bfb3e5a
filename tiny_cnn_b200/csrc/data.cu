// The callers' data formats, converted on the device: raw uint8 images (the records of a CIFAR-10
// binary file, the pixels of an MNIST idx3 file) are uploaded as they are -- a quarter of the bytes
// of the float rows the reference's parsers produce -- and scaled / padded into the float rows the
// first layer reads; class labels become the target rows network::train builds.
//
//   parse_cifar10        tiny_dnn/io/cifar10_parser.h:26-86
//       v = scale_min + (scale_max - scale_min) * c / 255        (padding filled with scale_min)
//   parse_mnist_images   tiny_dnn/io/mnist_parser.h:43-68,130-157
//       v = (c / 255) * (scale_max - scale_min) + scale_min      (padding filled with scale_min)
//   label2vec            tiny_dnn/nodes.h:180-189
//       t[j] = target_value_min, t[label] = target_value_max
//
// Each formula is evaluated with the reference's operation order in explicit round-to-nearest
// float operations (no fused multiply-add), once per byte value into a 256-entry table in shared
// memory, so the device rows equal the parser's bit for bit.  The kernels are bound by HBM:
// 1 byte read and 4 bytes written per pixel.
#include "common.cuh"
#include "device_utils.cuh"

namespace b200 {

namespace {

__device__ __forceinline__ float scale_byte(int mode, int c, float smin, float smax) {
  const float range = __fsub_rn(smax, smin);
  if (mode == B200_IMAGE_CIFAR10) return __fadd_rn(smin, __fdiv_rn(__fmul_rn(range, (float)c), 255.f));
  return __fadd_rn(__fmul_rn(__fdiv_rn((float)c, 255.f), range), smin);
}

// one block converts `rows_per_block` rows of W pixels of one (image, channel) plane
__global__ void __launch_bounds__(256) images_u8_to_float_kernel(const uint8_t *__restrict__ src, float *__restrict__ dst,
                                                                 int mode, long long planes, int H, int W, int xp,
                                                                 int yp, float smin, float smax) {
  __shared__ float lut[256];
  lut[threadIdx.x] = scale_byte(mode, threadIdx.x, smin, smax);
  __syncthreads();
  const int Wo = W + 2 * xp, Ho = H + 2 * yp;
  const long long out_plane = (long long)Wo * Ho, in_plane = (long long)W * H;
  const long long total = planes * out_plane;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long p = i / out_plane;
    const int r = (int)(i - p * out_plane);
    const int yo = r / Wo, xo = r - yo * Wo;
    const int y = yo - yp, x = xo - xp;
    float v = smin;
    if (y >= 0 && y < H && x >= 0 && x < W) v = lut[src[p * in_plane + (long long)y * W + x]];
    dst[i] = v;
  }
}

__global__ void labels_to_targets_kernel(const uint8_t *__restrict__ labels, float *__restrict__ dst, long long n,
                                         int out_dim, float tmin, float tmax) {
  const long long total = n * out_dim;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long s = i / out_dim;
    const int j = (int)(i - s * out_dim);
    dst[i] = (int)labels[s] == j ? tmax : tmin;
  }
}

int grid_for(long long total, int sm_count) {
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sm_count * 16;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace

int check_image_desc(const b200_image_desc *d) {
  B200_REQUIRE(d != nullptr, "image descriptor is NULL");
  B200_REQUIRE(d->mode == B200_IMAGE_CIFAR10 || d->mode == B200_IMAGE_MNIST, "image descriptor: unknown mode %d", d->mode);
  B200_REQUIRE(d->channels > 0 && d->height > 0 && d->width > 0, "image descriptor: empty image");
  // the reference's parsers throw on these (cifar10_parser.h:43-46, mnist_parser.h:136-139)
  B200_REQUIRE(d->x_padding >= 0 && d->y_padding >= 0, "padding size must not be negative");
  B200_REQUIRE(d->scale_min < d->scale_max, "scale_max must be greater than scale_min");
  return 0;
}

size_t image_in_len(const b200_image_desc *d) { return (size_t)d->channels * d->height * d->width; }
size_t image_out_len(const b200_image_desc *d) {
  return (size_t)d->channels * (d->height + 2 * d->y_padding) * (d->width + 2 * d->x_padding);
}

int images_u8_to_float(b200_ctx *ctx, const b200_image_desc *d, const uint8_t *src, long long n, float *dst) {
  if (n <= 0) return 0;
  const long long planes = n * d->channels;
  const long long total = planes * (d->height + 2 * d->y_padding) * (d->width + 2 * d->x_padding);
  images_u8_to_float_kernel<<<grid_for(total, ctx->sm_count), 256, 0, ctx->stream>>>(
    src, dst, d->mode, planes, d->height, d->width, d->x_padding, d->y_padding, d->scale_min, d->scale_max);
  B200_LAUNCHED();
  return 0;
}

int labels_to_targets(b200_ctx *ctx, const uint8_t *labels, long long n, int out_dim, float tmin, float tmax,
                      float *dst) {
  if (n <= 0) return 0;
  labels_to_targets_kernel<<<grid_for(n * out_dim, ctx->sm_count), 256, 0, ctx->stream>>>(labels, dst, n, out_dim,
                                                                                        tmin, tmax);
  B200_LAUNCHED();
  return 0;
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_images_u8_to_float(b200_ctx *ctx, const b200_image_desc *d, const uint8_t *src, long long n, float *dst) {
  B200_REQUIRE(ctx != nullptr, "ctx is NULL");
  B200_CUDA(cudaSetDevice(ctx->device));
  B200_TRY(check_image_desc(d));
  B200_REQUIRE(n >= 0 && (n == 0 || (src && dst)), "images_u8_to_float: bad argument");
  return images_u8_to_float(ctx, d, src, n, dst);
}

int b200_labels_to_targets(b200_ctx *ctx, const uint8_t *labels, long long n, int out_dim, float target_min,
                           float target_max, float *dst) {
  B200_REQUIRE(ctx != nullptr, "ctx is NULL");
  B200_CUDA(cudaSetDevice(ctx->device));
  B200_REQUIRE(n >= 0 && out_dim > 0 && (n == 0 || (labels && dst)), "labels_to_targets: bad argument");
  return labels_to_targets(ctx, labels, n, out_dim, target_min, target_max, dst);
}

}  // extern "C"
