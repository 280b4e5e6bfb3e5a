// Stride-1 convolution on the 5th-generation tensor cores (tcgen05), fp32-accurate
// through the 3xTF32 split (x = hi + lo; lo*hi + hi*lo + hi*hi accumulated in fp32 in
// tensor memory).  Replaces the loops of kernels::conv2d_op_internal and
// kernels::conv2d_grad_op_internal (tiny_dnn/core/kernels/conv2d_op_internal.h:13-74,
// :91-127 dX, :130-169 dW, :172-179 db) for layers with enough channels to feed the
// tensor pipe; the FFMA kernels of conv_tiled.cu keep the rest.
//
// Operand layout ("tall" pixel-major split tensors, made by to_tall_kernel):
//   P[hi|lo][t][x][c]   c < Cp (channels padded to 32: one 128-byte row per pixel),
//   t = b*period + y    every image is followed by `period - H` rows of zeros, which serve
//                       as the bottom padding of image b and the top padding of image b+1;
//                       left/right padding and the rows before the first image come from
//                       the zero fill of out-of-range TMA coordinates.
//
// Forward / dX (conv_tc_kernel): implicit GEMM, M = 128 output pixels (16 tall rows x 8
//   columns), N = output channels, K = 32 input channels per filter tap.  One TMA load
//   brings the haloed input tile (16+KH-1 rows x 16 columns x 32 channels) into shared
//   memory once; every tap's A operand is the same tile addressed at a row offset
//   (ky*16 + kx rows) -- the 128-byte swizzle is a function of the absolute address, so
//   no im2col copy is made.  Filters stream through a ring of per-tap tiles.
// dW (conv_dw_tc_kernel): K = pixels.  Both operands are MN-major (rows = pixels):
//   A = dY with the kx shifts stacked along M (blocks one pixel row = 128 bytes apart),
//   B = X with the ky shifts stacked along N (blocks one tile row apart), so one MMA chain
//   computes 4 x KH taps of a 32 x 32 channel block.  The batch is cut into slices whose
//   partial sums are merged in fixed order (the device form of edge::merge_grads).
// Warp roles in both kernels: warps 0-3 epilogue (one TMEM lane per thread), warp 4 TMEM
// allocation + TMA producer, warp 5 MMA issuer.  Every load is CTA-local; every wait is bounded and a
// timeout sets the context's error word, frees tensor memory and returns.
#include <float.h>
#include <stdlib.h>

#include "tc_utils.cuh"

namespace b200 {

namespace {

constexpr int TCV_THREADS = 192;
constexpr int TCV_TILE_ROWS = 16;  // tall rows per output tile
constexpr int TCV_TILE_COLS = 8;   // columns per output tile (one group of 8 MMA rows)
constexpr int TCV_HALO_W = 16;     // most columns a haloed tile has in shared memory (8 + KW - 1, KW <= 8 ... 9)

// geometry of the tall tensors of one convolution
struct TallGeom {
  int pad_b, pad_r;        // implied bottom / right padding
  int period;              // tall rows per image
  int Cp, OCp;             // channels padded to 32
  long long rows;          // B * period
};

TallGeom tall_geom(const ConvGeom &g, int B) {
  TallGeom t;
  t.pad_b = g.OH + g.KH - 1 - g.pad_t - g.HI;
  t.pad_r = g.OW + g.KW - 1 - g.pad_l - g.WI;
  int pv = g.pad_t > t.pad_b ? g.pad_t : t.pad_b;
  if (pv < 0) pv = 0;
  t.period = g.HI + pv;
  t.Cp = (g.C + 31) / 32 * 32;
  t.OCp = (g.OC + 31) / 32 * 32;
  t.rows = (long long)B * t.period;
  return t;
}

// rows per image of the tall form of dY as the dX pass needs it (padding KH-1-pad on each side)
int dy_period(const ConvGeom &g) {
  TallGeom t = tall_geom(g, 1);
  int a = g.KH - 1 - g.pad_t, b = g.KH - 1 - t.pad_b;
  int pv = a > b ? a : b;
  if (pv < 0) pv = 0;
  return g.OH + pv;
}

// ---- CHW rows -> tall split tensors ---------------------------------------------------

// Where the CHW values to convert come from.  mode 0: a CHW tensor.  mode 1: the 2x2/2 max-pool of
// `a` (planes in_h x in_w = 2H x 2W): the pooled values and their argmax are also written, CHW, as
// maxpool2x2_fwd_kernel would (strict '>' in window order).  mode 2: the gradient of a 2x2/2
// max-pool (pooled gradient `a`, argmax `am`), masked by the relu before the pooling layer when
// `pooled_y` (the pooling layer's forward output: the relu's output at each window's winner) is
// given; the CHW gradient is also written to `out_chw`.
struct TallSrc {
  int mode;
  const float *a;
  const int32_t *am;
  const float *pooled_y;
  float *out_chw;
  int32_t *out_am;
};

// one 2x2 window as maxpool2x2_fwd_kernel takes it: strict '>' in window order from -FLT_MAX, the
// index of the winner in the sample's CHW numbering (0 when nothing exceeds -FLT_MAX)
__device__ __forceinline__ void pool_window(float a, float b, float c, float d, int base, int in_w, float &best,
                                            int &idx) {
  best = -FLT_MAX;
  int code = -1;
  if (a > best) { best = a; code = 0; }
  if (b > best) { best = b; code = 1; }
  if (c > best) { best = c; code = 2; }
  if (d > best) { best = d; code = 3; }
  idx = code < 0 ? 0 : base + (code & 1) + (code >> 1) * in_w;
}

// One block converts `rb` tall rows of one image: src[b][c][y][x] -> hi/lo[t][x][c],
// zero for padded channels and for the rows between images.  With `bsum` the block also
// writes the per-channel sum of what it read (bias gradient partials, fixed order).
// Shared tile [c][pixel] with an odd pitch: scalar, coalesced loads along x; 16-byte
// stores of four channels of one pixel.
template <int MODE, int MINB>
__global__ void __launch_bounds__(256, MINB) to_tall_kernel(const TallSrc src, int C, int H, int W, int Cp, int period,
                                                      int rb, int pitch, float *__restrict__ hi,
                                                      float *__restrict__ lo, float *__restrict__ bsum) {
  extern __shared__ float tile[];  // [C][pitch]
  const int chunks = (period + rb - 1) / rb;
  const int b = blockIdx.x / chunks, r0 = (blockIdx.x % chunks) * rb;
  const int nr = min(rb, period - r0);
  const int npx = nr * W;
  const int valid_px = max(0, min(nr, H - r0)) * W;
  const size_t plane = (size_t)H * W;
  // phase 1: one warp per channel (channels w, w+8, ...), lanes along the pixels of the chunk
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (MODE == 0) {
    const float *img = src.a + ((size_t)b * C * H + r0) * W;
    for (int c = warp; c < C; c += 8) {
      const float *ch = img + c * plane;
      float *trow = tile + c * pitch;
#pragma unroll 4
      for (int p = lane; p < npx; p += 32) trow[p] = p < valid_px ? ch[p] : 0.f;
    }
  } else if (MODE == 1) {
    // two pooled pixels per lane: 16-byte loads of the two input rows, 8-byte stores.  Two channels
    // per pass, so that four loads are in flight per lane; the pair's place in the chunk does not
    // depend on the channel.
    const int in_w = 2 * W, in_h = 2 * H, W2 = W >> 1, nq = npx >> 1;
    const int w2s = (W2 & (W2 - 1)) == 0 ? 31 - __clz(W2) : -1;
    const size_t iplane = (size_t)in_h * in_w;
    for (int q = lane; q < nq; q += 32) {
      const int ry = w2s >= 0 ? q >> w2s : q / W2, x = (q - ry * W2) * 2, y = r0 + ry, pp = ry * W + x;
      const bool live = pp < valid_px;
      const size_t ioff = (size_t)(2 * y) * in_w + 2 * x, ooff = (size_t)y * W + x;
      for (int c = warp; c < C; c += 16) {
        const int c2 = c + 8;
        const bool two = c2 < C;
        float b00 = 0.f, b01 = 0.f, b10 = 0.f, b11 = 0.f;
        if (live) {
          const float *ip0 = src.a + ((size_t)b * C + c) * iplane + ioff;
          const float *ip1 = src.a + ((size_t)b * C + (two ? c2 : c)) * iplane + ioff;
          const float4 u0 = *reinterpret_cast<const float4 *>(ip0);
          const float4 v0 = *reinterpret_cast<const float4 *>(ip0 + in_w);
          const float4 u1 = *reinterpret_cast<const float4 *>(ip1);
          const float4 v1 = *reinterpret_cast<const float4 *>(ip1 + in_w);
          int i00, i01, i10, i11;
          pool_window(u0.x, u0.y, v0.x, v0.y, (in_h * c + 2 * y) * in_w + 2 * x, in_w, b00, i00);
          pool_window(u0.z, u0.w, v0.z, v0.w, (in_h * c + 2 * y) * in_w + 2 * x + 2, in_w, b01, i01);
          const size_t o0 = ((size_t)b * C + c) * plane + ooff;
          *reinterpret_cast<float2 *>(src.out_chw + o0) = make_float2(b00, b01);
          *reinterpret_cast<int2 *>(src.out_am + o0) = make_int2(i00, i01);
          if (two) {
            pool_window(u1.x, u1.y, v1.x, v1.y, (in_h * c2 + 2 * y) * in_w + 2 * x, in_w, b10, i10);
            pool_window(u1.z, u1.w, v1.z, v1.w, (in_h * c2 + 2 * y) * in_w + 2 * x + 2, in_w, b11, i11);
            const size_t o1 = ((size_t)b * C + c2) * plane + ooff;
            *reinterpret_cast<float2 *>(src.out_chw + o1) = make_float2(b10, b11);
            *reinterpret_cast<int2 *>(src.out_am + o1) = make_int2(i10, i11);
          }
        }
        tile[c * pitch + pp] = b00;
        tile[c * pitch + pp + 1] = b01;
        if (two) {
          tile[c2 * pitch + pp] = b10;
          tile[c2 * pitch + pp + 1] = b11;
        }
      }
    }
  } else {
    // one pooled pixel of one channel per thread: its gradient goes to the one input position
    // argmax names.  (channel, pixel) pairs are spread over the whole block, so that narrow images
    // (a handful of pooled pixels per chunk) still fill the lanes; consecutive threads read
    // consecutive pooled pixels, and consecutive channel planes are neighbours in memory.
    const int pw = W >> 1, ph = H >> 1;
    if ((W & 3) == 0) {
      // two pooled pixels of one channel per thread: 8-byte loads of the pooled gradient and the
      // winners, 16-byte loads / stores of the two input rows they cover
      const int pw2 = pw >> 1, nq = ((nr + 1) >> 1) * pw2;
      const int pws = (pw2 & (pw2 - 1)) == 0 ? 31 - __clz(pw2) : -1;
      for (int it = threadIdx.x; it < C * nq; it += 256) {
        const int c = it / nq, q = it - c * nq;
        const int pry = pws >= 0 ? q >> pws : q / pw2, prx = (q - pry * pw2) * 2, ry = 2 * pry, x = 2 * prx,
                  y = r0 + ry;
        const int pp = ry * W + x;
        float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
        if (y < H) {
          const size_t po = ((size_t)b * C + c) * ph * pw + (size_t)(y >> 1) * pw + prx;
          const size_t o = ((size_t)b * C + c) * plane + (size_t)y * W + x;
          float2 gv = *reinterpret_cast<const float2 *>(src.a + po);
          const int2 am = *reinterpret_cast<const int2 *>(src.am + po);
          if (src.pooled_y != nullptr) {  // relu mask: the relu's output at a winner is the pooled value
            const float2 py = *reinterpret_cast<const float2 *>(src.pooled_y + po);
            gv.x = py.x > 0.f ? gv.x : 0.f;
            gv.y = py.y > 0.f ? gv.y : 0.f;
          }
          const int base0 = (H * c + y) * W + x;
          const int a0 = am.x - base0, a1 = am.y - (base0 + 2);  // offset inside the window: 0, 1, W, W+1
          v0.x = a0 == 0 ? gv.x : 0.f;
          v0.y = a0 == 1 ? gv.x : 0.f;
          v0.z = a1 == 0 ? gv.y : 0.f;
          v0.w = a1 == 1 ? gv.y : 0.f;
          v1.x = a0 == W ? gv.x : 0.f;
          v1.y = a0 == W + 1 ? gv.x : 0.f;
          v1.z = a1 == W ? gv.y : 0.f;
          v1.w = a1 == W + 1 ? gv.y : 0.f;
          if (src.out_chw != nullptr) {
            *reinterpret_cast<float4 *>(src.out_chw + o) = v0;
            *reinterpret_cast<float4 *>(src.out_chw + o + W) = v1;
          }
        }
        float *trow = tile + c * pitch + pp;
        trow[0] = v0.x;
        trow[1] = v0.y;
        trow[2] = v0.z;
        trow[3] = v0.w;
        if (ry + 1 < nr) {
          trow[W] = v1.x;
          trow[W + 1] = v1.y;
          trow[W + 2] = v1.z;
          trow[W + 3] = v1.w;
        }
      }
    } else {
    const int nq = ((nr + 1) >> 1) * pw;
    const int pws = (pw & (pw - 1)) == 0 ? 31 - __clz(pw) : -1;
    for (int it = threadIdx.x; it < C * nq; it += 256) {
      const int c = it / nq, q = it - c * nq;
      const int pry = pws >= 0 ? q >> pws : q / pw, prx = q - pry * pw, ry = 2 * pry, x = 2 * prx, y = r0 + ry;
      const int pp = ry * W + x;
      float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
      if (y < H) {
        const size_t po = ((size_t)b * C + c) * ph * pw + (size_t)(y >> 1) * pw + prx;
        const size_t o = ((size_t)b * C + c) * plane + (size_t)y * W + x;
        float gval = src.a[po];
        const int am = src.am[po] - ((H * c + y) * W + x);  // offset inside the window: 0, 1, W, W+1
        if (src.pooled_y != nullptr && !(src.pooled_y[po] > 0.f)) gval = 0.f;
        v0 = am == 0 ? gval : 0.f;
        v1 = am == 1 ? gval : 0.f;
        v2 = am == W ? gval : 0.f;
        v3 = am == W + 1 ? gval : 0.f;
        if (src.out_chw != nullptr) {
          *reinterpret_cast<float2 *>(src.out_chw + o) = make_float2(v0, v1);
          *reinterpret_cast<float2 *>(src.out_chw + o + W) = make_float2(v2, v3);
        }
      }
      float *trow = tile + c * pitch;
      trow[pp] = v0;
      trow[pp + 1] = v1;
      if (ry + 1 < nr) {
        trow[pp + W] = v2;
        trow[pp + W + 1] = v3;
      }
    }
    }
  }
  __syncthreads();
  const size_t base = ((size_t)b * period + r0) * W * Cp;
  const int Cq = Cp >> 2, total2 = npx * Cq;
  float4 *hi4 = reinterpret_cast<float4 *>(hi + base), *lo4 = reinterpret_cast<float4 *>(lo + base);
  if (256 % Cq == 0) {
    // the channel quad of a thread is the same for every pixel it stores: no division per item
    const int c = (threadIdx.x % Cq) * 4, pstep = 256 / Cq;
    const float *t0 = tile + c * pitch;
    const bool k0 = c < C, k1 = c + 1 < C, k2 = c + 2 < C, k3 = c + 3 < C;
    int i = threadIdx.x;
#pragma unroll 4
    for (int p = threadIdx.x / Cq; p < npx; p += pstep, i += 256) {
      float h[4], l[4];
      split_tf32_rn(k0 ? t0[p] : 0.f, h[0], l[0]);
      split_tf32_rn(k1 ? t0[pitch + p] : 0.f, h[1], l[1]);
      split_tf32_rn(k2 ? t0[2 * pitch + p] : 0.f, h[2], l[2]);
      split_tf32_rn(k3 ? t0[3 * pitch + p] : 0.f, h[3], l[3]);
      hi4[i] = make_float4(h[0], h[1], h[2], h[3]);
      lo4[i] = make_float4(l[0], l[1], l[2], l[3]);
    }
  } else {
#pragma unroll 4
    for (int i = threadIdx.x; i < total2; i += 256) {
      int p = i / Cq, c = (i - p * Cq) * 4;
      float h[4], l[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        h[j] = l[j] = 0.f;
        if (c + j < C) split_tf32_rn(tile[(c + j) * pitch + p], h[j], l[j]);
      }
      hi4[i] = make_float4(h[0], h[1], h[2], h[3]);
      lo4[i] = make_float4(l[0], l[1], l[2], l[3]);
    }
  }
  if (bsum != nullptr) {
    for (int c = warp; c < C; c += 8) {
      float s = 0.f;
      for (int p = lane; p < valid_px; p += 32) s += tile[c * pitch + p];
      s = warp_sum(s);
      if (lane == 0) bsum[(size_t)blockIdx.x * C + c] = s;
    }
  }
}

// ---- filter matrices ----------------------------------------------------------------------

// One tile per (slab, kx, group): rows n = ky*gs + j (j < gs output channels of the group),
// 32 floats (the slab's contracted channels) each.
// Forward: F[slab][kx][grp][ky][j][k] = W[o = grp*gs + j][inc = slab*32 + k][ky][kx]
// dX:      F[slab][kx][grp][ky][j][k] = W[o = slab*32 + k][inc = grp*gs + j][KH-1-ky][KW-1-kx]
// zero beyond the real channels and for unconnected pairs.
struct FilterPrepOne {
  int gs, groups, slabs, for_dx;
  float *hi, *lo;
};

// blockIdx.y selects the matrix set: both the forward and the dX matrices of a layer in one launch
__global__ void tc_filter_prep_kernel(const float *__restrict__ W, const uint8_t *__restrict__ tbl, int C,
                                      int OC, int KH, int KW, const FilterPrepOne m0, const FilterPrepOne m1) {
  const FilterPrepOne m = blockIdx.y == 0 ? m0 : m1;
  const int gs = m.gs, groups = m.groups, slabs = m.slabs, for_dx = m.for_dx;
  float *__restrict__ hi = m.hi, *__restrict__ lo = m.lo;
  const long long total = (long long)slabs * KW * groups * KH * gs * 32;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int k = (int)(i % 32);
    long long r = i / 32;
    int j = (int)(r % gs);
    r /= gs;
    int ky = (int)(r % KH);
    r /= KH;
    int grp = (int)(r % groups);
    r /= groups;
    int kx = (int)(r % KW);
    int slab = (int)(r / KW);
    int o, inc;
    if (for_dx) {
      o = slab * 32 + k;
      inc = grp * gs + j;
      ky = KH - 1 - ky;
      kx = KW - 1 - kx;
    } else {
      o = grp * gs + j;
      inc = slab * 32 + k;
    }
    float h = 0.f, l = 0.f;
    if (o < OC && inc < C && (tbl == nullptr || tbl[inc * OC + o]))
      split_tf32_rn(W[((size_t)(o * C + inc) * KH + ky) * KW + kx], h, l);
    hi[i] = h;
    lo[i] = l;
  }
}

}  // namespace

// ---- forward / dX: implicit GEMM with the window rows stacked along N -------------------------
//
// For a tile of 16 tall input rows r and 8 columns x the tensor cores compute
//   D[(r, x)][(ky, o)] = sum over kx, c of  X[r][x + kx - pad_l][c] * W[o][c][ky][kx]
// (M = 128 pixels, N = KH * channels of the group, K = 32 channels per kx step; the kx shift is a
// row offset into the haloed tile in shared memory), and the epilogue adds the KH row-shifted
// column blocks:  out[t][x][o] = sum over ky of D[(t + ky - pad_t, x)][(ky, o)], which yields
// 16 - (KH-1) output rows per tile.  Stacking ky along N makes every MMA instruction KH times
// wider; an instruction narrower than about 128 columns runs at a fixed cost.

namespace {

constexpr int TCV_EPI_FLOATS = 2 * 128 * 16;  // row exchange buffer of the epilogue (two halves)

struct TcConvArgs {
  float *out;          // [B][N][OH][OW]
  const float *bias;   // N values or nullptr
  int *err;
  int B, period;       // images, tall rows per image (input and output share the row index)
  int OH, OW, N;       // output extent and channels
  int slabs;           // 32-channel slabs of the input
  int groups, gs;      // output-channel groups, channels per group (multiple of 16)
  int KH, KW, pad_t, pad_l;
  int tiles_x, ntiles;
  int act;
  int hw;              // columns of the haloed tile in shared memory: 8 + KW - 1
  int nh;              // haloed-tile buffers (1 or 2)
  int nf;              // filter ring stages
  int nb;              // accumulator buffers in tensor memory (1 or 2)
  int tmem_cols;       // allocated columns (power of two >= nb * groups * KH * gs)
  // Image-aligned tiles (images whose height H divides the 16 tile rows and equals the output
  // height): a tile holds the H rows of 16 / H whole images, loaded through a 4D tensor map that
  // skips the zero rows between images, and the epilogue leaves out the window rows that fall
  // outside the image instead of reading zeros.  Every one of the 16 tile rows is then an output
  // row -- no tile overlap, no padding rows through the tensor cores.
  int aligned;         // 0: tiles of 16 - (KH-1) output rows that overlap by KH-1 input rows
  int img_h, ipt;      // aligned: rows per image, images per tile
  long long *dbg;      // [grid][8] cycle counters in a build with -DB200_TC_TIMING, else nullptr
};

__global__ void __launch_bounds__(TCV_THREADS, 1)
  conv_tc_kernel(const __grid_constant__ CUtensorMap in_hi, const __grid_constant__ CUtensorMap in_lo,
                 const __grid_constant__ CUtensorMap f_hi, const __grid_constant__ CUtensorMap f_lo,
                 const TcConvArgs a) {
  const long long t_entry = tc_clock();  // 0 unless built with -DB200_TC_TIMING
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t HB = (uint32_t)a.hw * TCV_TILE_ROWS * 128u;  // one haloed tile (hi or lo): 24 KiB for a 5-wide window
  const int Ng = a.KH * a.gs;                                 // MMA width
  const uint32_t FB = (uint32_t)Ng * 128u;                    // one filter tile (hi or lo)
  const int CB = Ng;                                          // accumulator columns per buffer
  const int nunits = a.ntiles * a.groups;                     // work unit = (pixel tile, channel group)
  uint8_t *halo = smem;                                       // [nh][hi | lo]
  uint8_t *filt = halo + (size_t)a.nh * 2 * HB;               // [nf] filter tiles (hi and lo alternate)
  float *xch = reinterpret_cast<float *>(filt + (size_t)a.nf * FB);
  uint64_t *halo_full = reinterpret_cast<uint64_t *>(xch + TCV_EPI_FLOATS);
  uint64_t *halo_empty = halo_full + 2;
  uint64_t *acc_full = halo_empty + 2;
  uint64_t *acc_empty = acc_full + 2;
  uint64_t *filt_full = acc_empty + 2;
  uint64_t *filt_empty = filt_full + a.nf;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(filt_empty + a.nf);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&halo_full[i], 1);
      mbar_init(&halo_empty[i], 1);
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);
    }
    for (int i = 0; i < a.nf; ++i) {
      mbar_init(&filt_full[i], 1);
      mbar_init(&filt_empty[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == 4) tmem_alloc(tmem_slot, (uint32_t)a.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int TR = TCV_TILE_ROWS - (a.KH - 1);  // output rows per tile
  bool failed = false;

  if (warp == 4 && lane == 0) {
    // ---- TMA producer -----------------------------------------------------------------
    uint32_t u = 0, f = 0;
    for (int unit = blockIdx.x; unit < nunits && !failed; unit += gridDim.x) {
      const int tile = unit / a.groups, grp = unit - tile * a.groups;
      const int x0 = (tile % a.tiles_x) * TCV_TILE_COLS, r0 = (tile / a.tiles_x) * TR - a.pad_t;
      const int img0 = (tile / a.tiles_x) * a.ipt;  // aligned tiles: first image of the tile
      for (int slab = 0; slab < a.slabs && !failed; ++slab, ++u) {
        const uint32_t hb = u % a.nh, use = u / a.nh;
        if (use > 0 && !mbar_wait_bounded(&halo_empty[hb], (use - 1) & 1)) {
          failed = true;
          break;
        }
        uint8_t *h = halo + (size_t)hb * 2 * HB;
        mbar_expect_tx(&halo_full[hb], 2 * HB);
        if (a.aligned) {
          tma_load_4d(h, &in_hi, slab * 32, x0 - a.pad_l, 0, img0, &halo_full[hb]);
          tma_load_4d(h + HB, &in_lo, slab * 32, x0 - a.pad_l, 0, img0, &halo_full[hb]);
        } else {
          tma_load_3d(h, &in_hi, slab * 32, x0 - a.pad_l, r0, &halo_full[hb]);
          tma_load_3d(h + HB, &in_lo, slab * 32, x0 - a.pad_l, r0, &halo_full[hb]);
        }
        for (int s = 0; s < 2 * a.KW; ++s, ++f) {  // per kx: the hi tile, then the lo tile
          const uint32_t fs = f % a.nf, fuse = f / a.nf;
          if (fuse > 0 && !mbar_wait_bounded(&filt_empty[fs], (fuse - 1) & 1)) {
            failed = true;
            break;
          }
          const int row = ((slab * a.KW + (s >> 1)) * a.groups + grp) * Ng;
          mbar_expect_tx(&filt_full[fs], FB);
          tma_load_2d(filt + (size_t)fs * FB, (s & 1) ? &f_lo : &f_hi, 0, row, &filt_full[fs]);
        }
      }
    }
  } else if (warp == 5 && lane == 0) {
    // ---- MMA issuer -----------------------------------------------------------------------
    const uint32_t idesc = umma_idesc_tf32(128, Ng);
    uint32_t u = 0, f = 0, it = 0;
    long long w_acc = 0, w_halo = 0, w_filt = 0, t_begin = tc_clock(), tq, t_first = 0;
    for (int unit = blockIdx.x; unit < nunits && !failed; unit += gridDim.x, ++it) {
      const uint32_t ab = it % a.nb, ause = it / a.nb;
      tq = tc_clock();
      if (ause > 0 && !mbar_wait_bounded(&acc_empty[ab], (ause - 1) & 1)) {
        failed = true;
        break;
      }
      w_acc += tc_clock() - tq;
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + ab * (uint32_t)CB;
      for (int slab = 0; slab < a.slabs && !failed; ++slab, ++u) {
        const uint32_t hb = u % a.nh;
        tq = tc_clock();
        if (!mbar_wait_bounded(&halo_full[hb], (u / a.nh) & 1)) {
          failed = true;
          break;
        }
        w_halo += tc_clock() - tq;
        if (t_first == 0) t_first = tc_clock() - t_entry;  // kernel entry -> first operand tile in place
        tc_fence_after();
        const uint32_t hbase = smem_u32(halo + (size_t)hb * 2 * HB);
        for (int kx = 0; kx < a.KW && !failed; ++kx) {
          {
            // A: the haloed tile addressed kx pixels (rows of 128 bytes) further on
            const uint32_t abase = hbase + (uint32_t)kx * 128u;
            const uint32_t d = tmem_d;
            for (int part = 0; part < 2; ++part, ++f) {  // the hi filter tile, then the lo tile
              const uint32_t fs = f % a.nf;
              tq = tc_clock();
              if (!mbar_wait_bounded(&filt_full[fs], (f / a.nf) & 1)) {
                failed = true;
                break;
              }
              w_filt += tc_clock() - tq;
              tc_fence_after();
              const uint32_t bbase = smem_u32(filt + (size_t)fs * FB);
#pragma unroll
              for (int k4 = 0; k4 < 4; ++k4) {
                const uint64_t ahi = umma_desc(abase + k4 * 32, 16, a.hw * 128, 2);
                const uint64_t b = umma_desc(bbase + k4 * 32, 16, 1024, 2);
                if (part == 0) {
                  const uint64_t alo = umma_desc(abase + HB + k4 * 32, 16, a.hw * 128, 2);
                  umma_tf32(d, alo, b, idesc, (slab | kx | k4) != 0);
                  umma_tf32(d, ahi, b, idesc, 1);
                } else {
                  umma_tf32(d, ahi, b, idesc, 1);
                }
              }
              umma_commit(&filt_empty[fs]);
            }
          }
        }
        if (!failed) umma_commit(&halo_empty[hb]);
      }
      if (!failed) umma_commit(&acc_full[ab]);
    }
    if (a.dbg) {
      long long *d = a.dbg + (size_t)blockIdx.x * 8;
      d[0] = tc_clock() - t_begin;
      d[1] = w_acc;
      d[2] = w_halo;
      d[3] = w_filt;
      d[6] = t_first;
    }
  } else if (warp < 4) {
    // ---- epilogue: sum the KH row-shifted column blocks, bias, activation, store -------------
    uint32_t it = 0;
    const int m = warp * 32 + lane, r = m >> 3, dx = m & 7;
    const size_t plane = (size_t)a.OH * a.OW;
    uint32_t half = 0;  // exchange buffer half in use
    long long w_full = 0, t_begin = tc_clock(), tq;
    for (int unit = blockIdx.x; unit < nunits; unit += gridDim.x, ++it) {
      const int tile = unit / a.groups, grp = unit - tile * a.groups;
      const uint32_t ab = it % a.nb;
      tq = tc_clock();
      if (!mbar_wait_bounded(&acc_full[ab], (it / a.nb) & 1)) failed = true;
      w_full += tc_clock() - tq;
      // every epilogue thread takes part in the named barriers below, so leave together
      {
        int any;
        asm volatile(
          "{\n .reg .pred p, q;\n setp.ne.b32 p, %1, 0;\n bar.red.or.pred q, 1, 128, p;\n selp.u32 %0, 1, 0, q;\n}\n"
          : "=r"(any)
          : "r"((int)failed)
          : "memory");
        if (any) {
          failed = true;
          break;
        }
      }
      tc_fence_after();
      const int x = (tile % a.tiles_x) * TCV_TILE_COLS + dx;
      // the output row this thread owns, and the tile rows [row_lo, row_hi) whose window-row
      // blocks may be added to it
      int b, y, row_lo, row_hi, ky_own;
      bool valid;
      if (a.aligned) {
        const int bi = r / a.img_h;
        y = r - bi * a.img_h;
        b = (tile / a.tiles_x) * a.ipt + bi;
        valid = b < a.B && x < a.OW;
        row_lo = bi * a.img_h;          // rows of other images (or outside the image) are not read:
        row_hi = row_lo + a.img_h;      // they stand for the zero padding above and below
        ky_own = a.pad_t;               // input row r itself carries window row pad_t of output row r
      } else {
        const int t = (tile / a.tiles_x) * TR + r;  // output tall row (if r < TR)
        b = t / a.period;
        y = t - b * a.period;
        valid = r < TR && b < a.B && y < a.OH && x < a.OW;
        row_lo = 0;
        row_hi = TCV_TILE_ROWS;
        ky_own = 0;
      }
      float *obase = a.out + ((size_t)b * a.N * a.OH + y) * a.OW + x;
      const uint32_t tbase = tmem_base + ((uint32_t)(warp * 32) << 16) + ab * (uint32_t)CB;
      {
        for (int c0 = 0; c0 < a.gs; c0 += 16) {
          float acc[16];
          tmem_ld16(tbase + (uint32_t)(ky_own * a.gs + c0), acc);
          for (int ky = 0; ky < a.KH; ++ky) {
            if (ky == ky_own) continue;
            float v[16];
            tmem_ld16(tbase + (uint32_t)(ky * a.gs + c0), v);
            // hand the block to the thread that owns the output row it belongs to (ky - ky_own rows
            // up): 64-byte rows, 16-byte chunks swizzled
            float4 *row = reinterpret_cast<float4 *>(xch + half * (TCV_EPI_FLOATS / 2) + m * 16);
            const int sw = (m >> 1) & 3;
#pragma unroll
            for (int q = 0; q < 4; ++q)
              row[q ^ sw] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            const int srow = r + ky - ky_own;
            if (srow >= row_lo && srow < row_hi) {
              const int src = m + 8 * (ky - ky_own);
              const float4 *srow4 =
                reinterpret_cast<const float4 *>(xch + half * (TCV_EPI_FLOATS / 2) + src * 16);
              const int ssw = (src >> 1) & 3;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                float4 w = srow4[q ^ ssw];
                acc[4 * q] += w.x;
                acc[4 * q + 1] += w.y;
                acc[4 * q + 2] += w.z;
                acc[4 * q + 3] += w.w;
              }
            }
            half ^= 1;
          }
          if (valid) {
            // bias first, all at once: loads interleaved with the stores would wait on each of them
            float bv[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int oc = grp * a.gs + c0 + j;
              bv[j] = (a.bias != nullptr && oc < a.N) ? __ldg(a.bias + oc) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int oc = grp * a.gs + c0 + j;
              if (oc < a.N) obase[oc * plane] = apply_act(acc[j] + bv[j], a.act);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[ab]);
    }
    if (a.dbg && tid == 0) {
      long long *d = a.dbg + (size_t)blockIdx.x * 8;
      d[4] = tc_clock() - t_begin;
      d[5] = w_full;
      d[7] = tc_clock() - t_entry;  // kernel entry -> end of the last epilogue
    }
  }
  if (failed && a.err) atomicExch(a.err, 3);
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, (uint32_t)a.tmem_cols);
}

}  // namespace

// ---- dW: pixels are the contraction ----------------------------------------------------------

namespace {

constexpr int TCW_ROWS = 16;    // tall rows per stage
constexpr int TCW_STAGES = 2;

struct TcDwArgs {
  float *part;            // [ksplits][row_stride] partial weight gradients, reference order
  int *err;
  int KH, KW, pad_t, pad_l, C, OC;
  int groups_x;           // groups of 8 input columns
  int nstages;            // row blocks x column groups
  int ic_slabs;
  int ksplits;
  int tmem_cols;
  long long row_stride;
  long long *dbg;  // [blocks][8] cycle counters in a build with -DB200_TC_TIMING, else nullptr
};

// dW[o][inc][ky][kx] = sum over pixels u of X dY[t][u + pad_l - kx] * X[t + ky - pad_t][u]
__global__ void __launch_bounds__(TCV_THREADS, 1)
  conv_dw_tc_kernel(const __grid_constant__ CUtensorMap dy_hi, const __grid_constant__ CUtensorMap dy_lo,
                    const __grid_constant__ CUtensorMap x_hi, const __grid_constant__ CUtensorMap x_lo,
                    const TcDwArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t DYB = 16u * TCW_ROWS * 128u;                 // dY tile: 16 columns x rows (hi or lo)
  const uint32_t XB = 8u * (TCW_ROWS + a.KH - 1) * 128u;      // X tile: 8 columns x (rows + KH-1)
  const uint32_t STAGE = 2 * DYB + 2 * XB;
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + TCW_STAGES * STAGE);
  uint64_t *empty = full + TCW_STAGES;
  uint64_t *accum = empty + TCW_STAGES;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(accum + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ocs = blockIdx.y / a.ic_slabs, ics = blockIdx.y % a.ic_slabs;
  const int s_begin = (int)((long long)blockIdx.x * a.nstages / a.ksplits);
  const int s_end = (int)((long long)(blockIdx.x + 1) * a.nstages / a.ksplits);
  const int chunks = (a.KW + 3) / 4;
  const int N = a.KH * 32;

  if (tid == 0) {
    for (int s = 0; s < TCW_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum, 1);
    mbar_fence_init();
  }
  if (warp == 4) tmem_alloc(tmem_slot, (uint32_t)a.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool failed = false;
  long long t_begin = 0, t_acc = 0;

  if (warp == 4 && lane == 0) {
    for (int s = s_begin; s < s_end; ++s) {
      const uint32_t i = s - s_begin, st = i % TCW_STAGES, use = i / TCW_STAGES;
      if (use > 0 && !mbar_wait_bounded(&empty[st], (use - 1) & 1)) {
        failed = true;
        break;
      }
      const int t0 = (s / a.groups_x) * TCW_ROWS, u0 = (s % a.groups_x) * 8;
      uint8_t *p = smem + st * STAGE;
      mbar_expect_tx(&full[st], STAGE);
      tma_load_3d(p, &dy_hi, ocs * 32, u0 + a.pad_l - (a.KW - 1), t0, &full[st]);
      tma_load_3d(p + DYB, &dy_lo, ocs * 32, u0 + a.pad_l - (a.KW - 1), t0, &full[st]);
      tma_load_3d(p + 2 * DYB, &x_hi, ics * 32, u0, t0 - a.pad_t, &full[st]);
      tma_load_3d(p + 2 * DYB + XB, &x_lo, ics * 32, u0, t0 - a.pad_t, &full[st]);
    }
  } else if (warp == 5 && lane == 0) {
    const uint32_t idesc = umma_idesc_tf32_major(128, N, 1, 1);
    uint32_t accumulate = 0;
    long long w_full = 0, t_begin = tc_clock(), tq;
    for (int s = s_begin; s < s_end && !failed; ++s) {
      const uint32_t i = s - s_begin, st = i % TCW_STAGES;
      tq = tc_clock();
      if (!mbar_wait_bounded(&full[st], (i / TCW_STAGES) & 1)) {
        failed = true;
        break;
      }
      w_full += tc_clock() - tq;
      tc_fence_after();
      const uint32_t base = smem_u32(smem + st * STAGE);
      for (int r = 0; r < TCW_ROWS; ++r) {
        // B: X rows r .. r+KH-1 of this 8-column strip, one 32 x 8-pixel block per ky
        const uint32_t xb = base + 2 * DYB + (uint32_t)r * 1024u;
        const uint64_t bhi = umma_desc(xb, 1024, 512, 1);
        const uint64_t blo = umma_desc(xb + XB, 1024, 512, 1);
        for (int ch = 0; ch < chunks; ++ch) {
          // A: dY pixels shifted by j = 4*ch .. 4*ch+3 columns (kx = KW-1-j), one block per shift
          const uint32_t ab = base + (uint32_t)(r * 16 + ch * 4) * 128u;
          const uint64_t ahi = umma_desc(ab, 128, 512, 1);
          const uint64_t alo = umma_desc(ab + DYB, 128, 512, 1);
          const uint32_t d = tmem_base + (uint32_t)(ch * N);
          umma_tf32(d, alo, bhi, idesc, accumulate);
          umma_tf32(d, ahi, blo, idesc, 1);
          umma_tf32(d, ahi, bhi, idesc, 1);
        }
        accumulate = 1;
      }
      umma_commit(&empty[st]);
    }
    if (!failed) umma_commit(accum);
    if (a.dbg) {
      long long *d = a.dbg + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 8;
      d[0] = tc_clock() - t_begin;
      d[1] = w_full;
      d[2] = s_end - s_begin;
    }
  } else if (warp < 4) {
    // partial row in the kernel's own order [unit][j][ky][inc][o] (o fastest: one 128-byte line per
    // store instruction); conv_tc_dw_finish sums the rows and reorders to the reference layout
    float *row = a.part + (size_t)blockIdx.x * a.row_stride + (size_t)blockIdx.y * a.KW * N * 32;
    t_begin = tc_clock();
    if (s_end > s_begin) {
      if (!mbar_wait_bounded(accum, 0)) failed = true;
      tc_fence_after();
    }
    t_acc = tc_clock();
    if (!failed) {
      for (int ch = 0; ch < chunks; ++ch) {
        const int j = ch * 4 + warp;
        for (int c0 = 0; c0 < N; c0 += 32) {
          float v[32];
          if (s_end > s_begin) {
            tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(ch * N + c0), v);
          } else {
#pragma unroll
            for (int q = 0; q < 32; ++q) v[q] = 0.f;
          }
          if (j < a.KW) {
            float *dst = row + ((size_t)j * N + c0) * 32 + lane;
#pragma unroll
            for (int q = 0; q < 32; ++q) dst[q * 32] = v[q];
          }
        }
      }
    }
  }
  if (a.dbg && tid == 0) {
    long long *d = a.dbg + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 8;
    d[3] = t_acc - t_begin;
    d[4] = tc_clock() - t_acc;
  }
  if (failed && a.err) atomicExch(a.err, 4);
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, (uint32_t)a.tmem_cols);
}

}  // namespace

// ---- host side -----------------------------------------------------------------------------

namespace {

int pow2_at_least(int v) {
  int p = 32;
  while (p < v) p <<= 1;
  return p;
}

int pad16(int n) { return (n + 15) / 16 * 16; }

// tiling of the forward / dX kernel for a window height and an output channel count
struct TcPlan {
  bool ok;
  int groups, gs;   // output-channel groups and channels per group
  int nh, nf, nb;   // haloed-tile buffers, filter ring stages, accumulator buffers
  int hw;           // columns of the haloed tile in shared memory
  int tmem_cols;
  size_t smem;
};

// `KW` decides how wide the haloed tile is (8 output columns + KW - 1); groups / gs do not depend on it
TcPlan conv_tc_plan(const b200_ctx *ctx, int KH, int n_out, int KW = 8) {
  TcPlan p = {};
  p.hw = 8 + KW - 1 < TCV_HALO_W ? 8 + KW - 1 : TCV_HALO_W;
  const int c16 = pad16(n_out);
  const int gmax = 256 / KH / 16 * 16;
  if (gmax < 16) return p;
  p.groups = (c16 + gmax - 1) / gmax;
  p.gs = pad16((c16 + p.groups - 1) / p.groups);
  const int CB = KH * p.gs;  // accumulator columns of one (tile, group) unit
  p.nb = 2 * CB <= 512 ? 2 : 1;
  p.tmem_cols = pow2_at_least(p.nb * CB);
  const size_t HB = (size_t)p.hw * TCV_TILE_ROWS * 128, stage = (size_t)KH * p.gs * 128;
  const size_t fixed = 1024 + (size_t)TCV_EPI_FLOATS * 4 + 512;
  for (p.nh = 2; p.nh >= 1; --p.nh) {
    size_t need = fixed + (size_t)p.nh * 2 * HB;
    if (ctx->smem_optin < need + 2 * stage) continue;
    size_t nf = (ctx->smem_optin - need) / stage;
    p.nf = (int)(nf > 12 ? 12 : nf);  // measured on the CIFAR layers: 3, 4 and 5 stages run the same
    p.smem = need + (size_t)p.nf * stage;
    p.ok = true;
    return p;
  }
  return p;
}

size_t dw_tc_smem(int KH) {
  size_t st = 2 * (16 * TCW_ROWS * 128) + 2 * (8 * (TCW_ROWS + KH - 1) * 128);
  return 1024 + TCW_STAGES * st + (2 * TCW_STAGES + 1) * 8 + 16;
}

int make_map_rows(CUtensorMap *m, const float *base, uint64_t rows, uint32_t box_rows) {
  return make_map_2d(m, base, 32, rows, 32, box_rows);
}

// rows of one image a conversion block takes
int to_tall_rows(int C, int W, int period) {
  int px = 4096 / (C > 0 ? C : 1);  // about 16 KiB of tile: several blocks per SM
  if (px > 512) px = 512;
  int rb = px / W;
  if (rb < 1) rb = 1;
  if (rb > period) rb = period;
  // even out the chunks of one image
  int chunks = ceil_div(period, rb);
  rb = ceil_div(period, chunks);
  if ((rb & 1) && rb < period) ++rb;  // even chunks: the pooling gradient is produced two rows at a time
  return rb;
}

int to_tall_blocks(int C, int W, int period, int B) {
  return B * ceil_div(period, to_tall_rows(C, W, period));
}

int to_tall(b200_ctx *ctx, const TallSrc &src, int C, int H, int W, int Cp, int period, int B, float *dst,
            float *bsum) {
  const int rb = to_tall_rows(C, W, period);
  B200_REQUIRE(src.mode != 2 || (((rb & 1) == 0 || rb == period) && (H & 1) == 0),
               "tall conversion: the pooling gradient needs even row counts");
  const int pitch = ((rb * W + 7) & ~7) + 1;
  size_t smem = (size_t)C * pitch * sizeof(float);
  int chunks = ceil_div(period, rb);
  size_t one = (size_t)B * period * W * Cp;
  // one instantiation per source, so that the plain and the pooling-gradient conversions do not
  // carry the registers of the pooling one
  auto launch = [&](auto kernel) -> int {
    if (smem > 48 * 1024)
      B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<B * chunks, 256, smem, ctx->stream>>>(src, C, H, W, Cp, period, rb, pitch, dst, dst + one, bsum);
    B200_LAUNCHED();
    return 0;
  };
  // resident blocks per SM the compiler is held to: six spill the pooling source's registers
  // (measured 15.3 against 12.5 µs), five do not
  if (src.mode == 0) return launch(to_tall_kernel<0, 6>);
  if (src.mode == 1) return launch(to_tall_kernel<1, 5>);
  return launch(to_tall_kernel<2, 6>);
}

// shared launcher of the forward and dX passes
// `Hin` = rows per image of the tall tensor (its images are `period` rows apart)
int launch_conv_tc(b200_ctx *ctx, const float *tall, int Cp, int Win, int Hin, long long rows, int period,
                   const float *wt, int KH, int KW, int pad_t, int pad_l, int N, float *out, int OH, int OW,
                   const float *bias, int act, int B) {
  const TcPlan p = conv_tc_plan(ctx, KH, N, KW);
  B200_REQUIRE(p.ok, "tensor-core convolution: tiles do not fit (window height %d, %d channels)", KH, N);
  const int slabs = Cp / 32, Ng = KH * p.gs;
  CUtensorMap in_hi, in_lo, f_hi, f_lo;
  const size_t one = (size_t)rows * Win * Cp;
  // image-aligned tiles: whole images per tile (see TcConvArgs)
  static const bool no_aligned = getenv("B200_CONV_TC_NO_ALIGNED") != nullptr;
  const bool aligned = !no_aligned && Hin == OH && Hin >= 1 && TCV_TILE_ROWS % Hin == 0 && pad_t <= KH - 1;
  const int ipt = aligned ? TCV_TILE_ROWS / Hin : 1;
  if (aligned) {
    B200_TRY(make_map_4d(&in_hi, tall, Cp, Win, Hin, B, (uint64_t)period * Win * Cp, 32, p.hw, Hin, ipt,
                         CU_TENSOR_MAP_SWIZZLE_128B));
    B200_TRY(make_map_4d(&in_lo, tall + one, Cp, Win, Hin, B, (uint64_t)period * Win * Cp, 32, p.hw, Hin,
                         ipt, CU_TENSOR_MAP_SWIZZLE_128B));
  } else {
    B200_TRY(make_map_3d(&in_hi, tall, Cp, Win, rows, 32, p.hw, TCV_TILE_ROWS,
                         CU_TENSOR_MAP_SWIZZLE_128B));
    B200_TRY(make_map_3d(&in_lo, tall + one, Cp, Win, rows, 32, p.hw, TCV_TILE_ROWS,
                         CU_TENSOR_MAP_SWIZZLE_128B));
  }
  const size_t frows = (size_t)slabs * KW * p.groups * Ng;
  B200_TRY(make_map_rows(&f_hi, wt, frows, Ng));
  B200_TRY(make_map_rows(&f_lo, wt + frows * 32, frows, Ng));
  TcConvArgs a;
  a.out = out;
  a.bias = bias;
  a.err = ctx->dev_err;
  a.B = B;
  a.period = period;
  a.OH = OH;
  a.OW = OW;
  a.N = N;
  a.slabs = slabs;
  a.groups = p.groups;
  a.gs = p.gs;
  a.KH = KH;
  a.KW = KW;
  a.pad_t = pad_t;
  a.pad_l = pad_l;
  const int TR = TCV_TILE_ROWS - (KH - 1);
  a.tiles_x = ceil_div(OW, TCV_TILE_COLS);
  a.ntiles = a.tiles_x * (aligned ? ceil_div(B, ipt) : (int)((rows + TR - 1) / TR));
  a.aligned = aligned ? 1 : 0;
  a.img_h = Hin;
  a.ipt = ipt;
  a.act = act;
  a.nh = p.nh;
  a.nf = p.nf;
  a.nb = p.nb;
  a.hw = p.hw;
  a.tmem_cols = p.tmem_cols;
  a.dbg = nullptr;
  B200_CUDA(cudaFuncSetAttribute(conv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem));
  const int units = a.ntiles * a.groups;
  int grid = units < ctx->sm_count ? units : ctx->sm_count;
#ifdef B200_TC_TIMING
  static const bool timing = getenv("B200_TC_TIMING") != nullptr;
  if (timing) B200_CUDA(cudaMalloc(&a.dbg, (size_t)grid * 8 * sizeof(long long)));
#endif
  conv_tc_kernel<<<grid, TCV_THREADS, p.smem, ctx->stream>>>(in_hi, in_lo, f_hi, f_lo, a);
  B200_LAUNCHED();
#ifdef B200_TC_TIMING
  if (timing) {  // diagnostic: where the MMA and epilogue roles spent their cycles, averaged over blocks
    std::vector<long long> h((size_t)grid * 8);
    B200_CUDA(cudaStreamSynchronize(ctx->stream));
    B200_CUDA(cudaMemcpy(h.data(), a.dbg, h.size() * sizeof(long long), cudaMemcpyDeviceToHost));
    B200_CUDA(cudaFree(a.dbg));
    double s[8] = {0};
    for (int i = 0; i < grid; ++i)
      for (int k = 0; k < 8; ++k) s[k] += (double)h[(size_t)i * 8 + k] / grid;
    fprintf(stderr,
            "[tc-timing] tiles %d grid %d N %d: mma total %.0f clk, waits acc %.0f halo %.0f filt %.0f | "
            "epilogue total %.0f, wait full %.0f | entry -> first tile in place %.0f, entry -> last epilogue done %.0f\n",
            a.ntiles, grid, KH * p.gs, s[0], s[1], s[2], s[3], s[4], s[5], s[6], s[7]);
  }
#endif
  return 0;
}

FilterPrepOne filter_prep_one(const b200_ctx *ctx, const ConvGeom &g, int for_dx, float *wt, long long *total) {
  TallGeom t = tall_geom(g, 1);
  const TcPlan p = conv_tc_plan(ctx, g.KH, for_dx ? g.C : g.OC);
  FilterPrepOne m;
  m.gs = p.gs;
  m.groups = p.groups;
  m.slabs = (for_dx ? t.OCp : t.Cp) / 32;
  m.for_dx = for_dx;
  *total = (long long)m.slabs * g.KW * p.groups * g.KH * p.gs * 32;
  m.hi = wt;
  m.lo = wt + *total;
  return m;
}

}  // namespace

// filter matrices of the forward pass (wt_fwd) and / or of the dX pass (wt_dx) in one launch
int conv_tc_prep(b200_ctx *ctx, const ConvGeom &g, const float *W, float *wt_fwd, float *wt_dx) {
  if (!wt_fwd && !wt_dx) return 0;
  long long t0 = 0, t1 = 0;
  FilterPrepOne m0 = filter_prep_one(ctx, g, wt_fwd ? 0 : 1, wt_fwd ? wt_fwd : wt_dx, &t0);
  FilterPrepOne m1 = m0;
  int sets = 1;
  if (wt_fwd && wt_dx) {
    m1 = filter_prep_one(ctx, g, 1, wt_dx, &t1);
    sets = 2;
  }
  long long total = t0 > t1 ? t0 : t1;
  int blocks = (int)((total + 255) / 256);
  if (blocks > ctx->sm_count * 8) blocks = ctx->sm_count * 8;
  tc_filter_prep_kernel<<<dim3(blocks, sets), 256, 0, ctx->stream>>>(W, g.tbl, g.C, g.OC, g.KH, g.KW, m0, m1);
  B200_LAUNCHED();
  return 0;
}

namespace {

// One block of the finishing pass of a tensor-core dW kernel (DwFinishArgs): 8 row lanes per
// element, lane k adds rows k, k+8, ... in order, lanes combined in order.
__device__ __forceinline__ void dw_finish_block(const DwFinishArgs &a, const int block) {
  constexpr int RL = 8;  // row lanes
  __shared__ float lanes[RL][33];
  __shared__ float tree[256];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int wblocks = (a.row_w + 31) / 32;
  if (block >= wblocks) {
    // bias gradient: one block per output channel; its many short partial rows are spread over
    // all 256 threads (thread k adds rows k, k+256, ... in order), combined by a fixed tree
    const int o = block - wblocks, t = ty * 32 + tx;
    if (a.db == nullptr || o >= a.OC) return;
    const float *src = a.bsrc + a.bs_off + o;
    float s = 0.f;
    for (int r = t; r < a.bs_rows; r += 256) s += src[(size_t)r * a.bs_stride];
    tree[t] = s;
    __syncthreads();
#pragma unroll
    for (int w = 128; w > 0; w >>= 1) {
      if (t < w) tree[t] += tree[t + w];
      __syncthreads();
    }
    if (t == 0) a.db[o] = a.accumulate ? a.db[o] + tree[0] : tree[0];
    return;
  }
  const int e = block * 32 + tx;
  float s0 = 0.f, s1 = 0.f;
  if (e < a.row_w) {
    const float *src = a.part + e;
    int r = ty;
    for (; r + RL < a.splits; r += 2 * RL) {
      s0 += src[(size_t)r * a.part_stride];
      s1 += src[(size_t)(r + RL) * a.part_stride];
    }
    if (r < a.splits) s0 += src[(size_t)r * a.part_stride];
  }
  lanes[ty][tx] = s0 + s1;
  __syncthreads();
  if (ty == 0 && e < a.row_w) {
    float s = lanes[0][tx];
#pragma unroll
    for (int k = 1; k < RL; ++k) s += lanes[k][tx];
    int o, inc, ky, kx;
    if (a.layout == 0) {
      int r = e;
      const int ol = r & 31;
      r >>= 5;
      const int il = r & 31;
      r >>= 5;
      ky = r % a.KH;
      r /= a.KH;
      const int j = r % a.KW, unit = r / a.KW;
      kx = a.KW - 1 - j;
      o = (unit / a.ic_slabs) * 32 + ol;
      inc = (unit % a.ic_slabs) * 32 + il;
    } else {
      const int k = e / a.OCp, KK = a.KH * a.KW;
      o = e - k * a.OCp;
      inc = k / KK;
      const int t = k - inc * KK;
      ky = t / a.KW;
      kx = t - ky * a.KW;
    }
    if (o < a.OC && inc < a.C) {
      if (a.tbl && !a.tbl[inc * a.OC + o]) s = 0.f;
      float *d = a.dW + (((size_t)o * a.C + inc) * a.KH + ky) * a.KW + kx;
      *d = a.accumulate ? *d + s : s;
    }
  }
}

__global__ void __launch_bounds__(256) dw_finish_kernel(const DwFinishArgs a) { dw_finish_block(a, (int)blockIdx.x); }

// several layers' finishing passes as one launch: block ranges [first[i], first[i + 1]) belong to layer i
struct DwFinishBatch {
  int n;
  int first[DW_FINISH_MAX + 1];
  DwFinishArgs a[DW_FINISH_MAX];
};

__global__ void __launch_bounds__(256) dw_finish_multi_kernel(const DwFinishBatch b) {
  int i = 0;
  while (i + 1 < b.n && (int)blockIdx.x >= b.first[i + 1]) ++i;
  dw_finish_block(b.a[i], (int)blockIdx.x - b.first[i]);
}

int dw_finish_blocks(const DwFinishArgs &a) { return (a.row_w + 31) / 32 + (a.db != nullptr ? a.OC : 0); }

int launch_dw_finish(b200_ctx *ctx, const DwFinishArgs &a) {
  dw_finish_kernel<<<dw_finish_blocks(a), dim3(32, 8), 0, ctx->stream>>>(a);
  B200_LAUNCHED();
  return 0;
}

}  // namespace

bool conv_tc_ok(const b200_ctx *ctx, const ConvGeom &g) {
  if (g.SH != 1 || g.SW != 1 || g.DH != 1 || g.DW != 1) return false;
  if (g.KH > 8 || g.KW > 8 || g.OC > 256 || g.C > 256) return false;
  TallGeom t = tall_geom(g, 1);
  if (g.pad_t < 0 || g.pad_l < 0 || t.pad_b < 0 || t.pad_r < 0) return false;
  if (g.pad_t > g.KH - 1 || t.pad_b > g.KH - 1 || g.pad_l > g.KW - 1 || t.pad_r > g.KW - 1) return false;
  if (g.WI > 256 || g.OW > 256) return false;
  if (!conv_tc_plan(ctx, g.KH, g.OC).ok || !conv_tc_plan(ctx, g.KH, g.C).ok) return false;
  if (dw_tc_smem(g.KH) > ctx->smem_optin) return false;
  size_t tall_smem = (size_t)((g.WI > g.OW ? g.WI : g.OW) + 9) * (g.C > g.OC ? g.C : g.OC) * 4;
  return tall_smem <= ctx->smem_optin;
}

ConvTcUse conv_tc_use(const b200_ctx *ctx, const ConvGeom &g, int algo) {
  ConvTcUse u = {false, false, false, false, false};
  if (algo == 1 || algo == 2) return u;
  if (algo != 3 && ctx->conv_tensor_cores == 0) return u;
  if (conv_tc_ok(ctx, g)) {
    if (algo == 3 || ctx->conv_tensor_cores >= 2) {
      u.fwd = u.dx = u.dw = true;
    } else {
      // a pass pays off when both channel counts fill a good part of a 32-wide slab / MMA width
      u.fwd = u.dx = u.dw = g.C >= 16 && g.OC >= 16;
    }
    if (algo != 3) {
      if (const char *e = getenv("B200_CONV_TC")) {  // bit 0 forward, bit 1 dX, bit 2 dW
        int m = atoi(e);
        u.fwd = (m & 1) != 0;
        u.dx = (m & 2) != 0;
        u.dw = (m & 4) != 0;
      }
    }
  }
  // few input channels: the im2col form of dW instead of the slab form
  if (conv_dw_small_ok(ctx, g) && (!u.dw || g.C < 16)) {
    bool want = true;
    if (const char *e = getenv("B200_CONV_TC")) want = algo == 3 || (atoi(e) & 8) != 0;
    if (want) {
      u.dw = false;
      u.dw_small = true;
    }
  }
  // and the im2col form of the forward pass (bit 4 of B200_CONV_TC)
  if (conv_fwd_small_ok(ctx, g) && (!u.fwd || g.C < 16)) {
    bool want = true;
    if (const char *e = getenv("B200_CONV_TC")) want = algo == 3 || (atoi(e) & 16) != 0;
    if (want) {
      u.fwd = false;
      u.fwd_small = true;
    }
  }
  return u;
}

// floats of the tall split form (hi + lo) of the input (which = 0) or of dY (which = 1)
size_t conv_tc_tall_floats(const ConvGeom &g, int B, int which) {
  TallGeom t = tall_geom(g, B);
  if (which == 0) return (size_t)2 * t.rows * g.WI * t.Cp;
  return (size_t)2 * B * dy_period(g) * g.OW * t.OCp;
}

size_t conv_tc_filter_floats(const b200_ctx *ctx, const ConvGeom &g, int for_dx) {
  TallGeom t = tall_geom(g, 1);
  const TcPlan p = conv_tc_plan(ctx, g.KH, for_dx ? g.C : g.OC);
  int slabs = (for_dx ? t.OCp : t.Cp) / 32;
  return (size_t)2 * slabs * g.KW * p.groups * g.KH * p.gs * 32;
}

// rows of per-block bias-gradient partials the dY conversion writes
int conv_tc_bsum_rows(const ConvGeom &g, int B) {
  TallGeom t = tall_geom(g, 1);
  return to_tall_blocks(g.OC, g.OW, dy_period(g), B);
}

int conv_tc_dw_splits(const b200_ctx *ctx, const ConvGeom &g, int B) {
  TallGeom t = tall_geom(g, B);
  int units = (t.Cp / 32) * (t.OCp / 32);
  long long nstages = (t.rows + TCW_ROWS - 1) / TCW_ROWS * ceil_div(g.WI, 8);
  int k = ctx->sm_count / units;
  if (k < 1) k = 1;
  if (k > nstages) k = (int)nstages;
  return k;
}

// floats of one partial row of the dW kernel (its own order, channels padded to 32)
static size_t dw_tc_row(const ConvGeom &g) {
  TallGeom t = tall_geom(g, 1);
  return (size_t)(t.Cp / 32) * (t.OCp / 32) * g.KW * g.KH * 32 * 32;
}

// floats of scratch of the dW pass: the partial rows and their sum
size_t conv_tc_dw_floats(const b200_ctx *ctx, const ConvGeom &g, int B) {
  return ((size_t)conv_tc_dw_splits(ctx, g, B) + 1) * dw_tc_row(g);
}

// sum the partial rows conv_tc_dw wrote (fixed order) and store them in the reference layout; with
// `bsum` (the per-block channel sums of conv_tc_tall_dy) and `db` also the bias gradient
int dw_finish_many(b200_ctx *ctx, const DwFinishArgs *list, int n) {
  for (int i0 = 0; i0 < n; i0 += DW_FINISH_MAX) {
    const int m = n - i0 < DW_FINISH_MAX ? n - i0 : DW_FINISH_MAX;
    if (m == 1) {
      B200_TRY(launch_dw_finish(ctx, list[i0]));
      continue;
    }
    DwFinishBatch b;
    b.n = m;
    b.first[0] = 0;
    for (int i = 0; i < m; ++i) {
      b.a[i] = list[i0 + i];
      b.first[i + 1] = b.first[i] + dw_finish_blocks(list[i0 + i]);
    }
    dw_finish_multi_kernel<<<b.first[m], dim3(32, 8), 0, ctx->stream>>>(b);
    B200_LAUNCHED();
  }
  return 0;
}

int conv_tc_dw_finish(b200_ctx *ctx, const ConvGeom &g, float *part, int splits, float *dW, int accumulate,
                      const float *bsum, int B, float *db, DwFinishArgs *defer) {
  TallGeom t = tall_geom(g, 1);
  DwFinishArgs a;
  a.part = part;
  a.part_stride = (long long)dw_tc_row(g);
  a.splits = splits;
  a.bsrc = bsum;
  a.bs_stride = g.OC;
  a.bs_off = 0;
  a.bs_rows = bsum ? conv_tc_bsum_rows(g, B) : 0;
  a.dW = dW;
  a.db = (bsum && g.has_bias) ? db : nullptr;
  a.layout = 0;
  a.row_w = (int)dw_tc_row(g);
  a.C = g.C;
  a.OC = g.OC;
  a.OCp = t.OCp;
  a.KH = g.KH;
  a.KW = g.KW;
  a.ic_slabs = t.Cp / 32;
  a.tbl = g.tbl;
  a.accumulate = accumulate;
  if (defer != nullptr) {  // the caller launches it later, with other layers' (dw_finish_many)
    *defer = a;
    return 0;
  }
  return launch_dw_finish(ctx, a);
}

int conv_tc_tall_x(b200_ctx *ctx, const ConvGeom &g, const float *in, int B, float *xs) {
  TallGeom t = tall_geom(g, B);
  const TallSrc src = {0, in, nullptr, nullptr, nullptr, nullptr};
  return to_tall(ctx, src, g.C, g.HI, g.WI, t.Cp, t.period, B, xs, nullptr);
}

// dY -> tall split form; bsum (conv_tc_bsum_rows x OC floats, may be nullptr) receives the
// per-block channel sums whose in-order total is the bias gradient
int conv_tc_tall_dy(b200_ctx *ctx, const ConvGeom &g, const float *dout, int B, float *dys, float *bsum) {
  TallGeom t = tall_geom(g, B);
  const TallSrc src = {0, dout, nullptr, nullptr, nullptr, nullptr};
  return to_tall(ctx, src, g.OC, g.OH, g.OW, t.OCp, dy_period(g), B, dys, bsum);
}

// 2x2/2 max-pooling fused with the conversion: `in` is the pooling layer's input (planes 2*HI x 2*WI),
// `pooled` / `argmax` receive what maxpool_fwd would write, `xs` the tall split copy of the pooled values
int conv_tc_tall_x_pool(b200_ctx *ctx, const ConvGeom &g, const float *in, float *pooled, int32_t *argmax, int B,
                        float *xs) {
  TallGeom t = tall_geom(g, B);
  const TallSrc src = {1, in, nullptr, nullptr, pooled, argmax};
  return to_tall(ctx, src, g.C, g.HI, g.WI, t.Cp, t.period, B, xs, nullptr);
}

// gradient of a 2x2/2 max-pooling layer (pooled gradient `gpool`, its `argmax`) that follows this
// convolution -- through the relu in between when `pooled_y` (the pooling layer's forward output) is
// given -- written as
// the tall split copy of dY, as the CHW gradient `dout_chw` (may be nullptr) and as bias partials
int conv_tc_tall_dy_unpool(b200_ctx *ctx, const ConvGeom &g, const float *gpool, const int32_t *argmax,
                           const float *pooled_y, float *dout_chw, int B, float *dys, float *bsum) {
  TallGeom t = tall_geom(g, B);
  const TallSrc src = {2, gpool, argmax, pooled_y, dout_chw, nullptr};
  return to_tall(ctx, src, g.OC, g.OH, g.OW, t.OCp, dy_period(g), B, dys, bsum);
}

int conv_tc_fwd(b200_ctx *ctx, const ConvGeom &g, const float *xs, const float *W, const float *bias,
                float *out, int B, int act, float *wt, int prep) {
  TallGeom t = tall_geom(g, B);
  if (prep) B200_TRY(conv_tc_prep(ctx, g, W, wt, nullptr));
  return launch_conv_tc(ctx, xs, t.Cp, g.WI, g.HI, t.rows, t.period, wt, g.KH, g.KW, g.pad_t, g.pad_l, g.OC, out,
                        g.OH, g.OW, g.has_bias ? bias : nullptr, act, B);
}

int conv_tc_dx(b200_ctx *ctx, const ConvGeom &g, const float *dys, const float *W, float *din, int B,
               float *wt, int prep) {
  TallGeom t = tall_geom(g, B);
  const int period = dy_period(g);
  if (prep) B200_TRY(conv_tc_prep(ctx, g, W, nullptr, wt));
  return launch_conv_tc(ctx, dys, t.OCp, g.OW, g.OH, (long long)B * period, period, wt, g.KH, g.KW,
                        g.KH - 1 - g.pad_t, g.KW - 1 - g.pad_l, g.C, din, g.HI, g.WI, nullptr, B200_ACT_NONE,
                        B);
}

// partial weight gradients: *splits rows in `part` (conv_tc_dw_floats floats), finished by conv_tc_dw_finish
int conv_tc_dw(b200_ctx *ctx, const ConvGeom &g, const float *xs, const float *dys, int B, float *part,
               int *splits) {
  TallGeom t = tall_geom(g, B);
  B200_REQUIRE(dy_period(g) == t.period, "tensor-core dW: input and gradient row periods differ");
  CUtensorMap dy_hi, dy_lo, x_hi, x_lo;
  const size_t one_dy = (size_t)t.rows * g.OW * t.OCp, one_x = (size_t)t.rows * g.WI * t.Cp;
  const CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
  B200_TRY(make_map_3d(&dy_hi, dys, t.OCp, g.OW, t.rows, 32, 16, TCW_ROWS, swz));
  B200_TRY(make_map_3d(&dy_lo, dys + one_dy, t.OCp, g.OW, t.rows, 32, 16, TCW_ROWS, swz));
  B200_TRY(make_map_3d(&x_hi, xs, t.Cp, g.WI, t.rows, 32, 8, TCW_ROWS + g.KH - 1, swz));
  B200_TRY(make_map_3d(&x_lo, xs + one_x, t.Cp, g.WI, t.rows, 32, 8, TCW_ROWS + g.KH - 1, swz));
  TcDwArgs a;
  a.part = part;
  a.err = ctx->dev_err;
  a.KH = g.KH;
  a.KW = g.KW;
  a.pad_t = g.pad_t;
  a.pad_l = g.pad_l;
  a.C = g.C;
  a.OC = g.OC;
  a.groups_x = ceil_div(g.WI, 8);
  a.nstages = (int)((t.rows + TCW_ROWS - 1) / TCW_ROWS) * a.groups_x;
  a.ic_slabs = t.Cp / 32;
  a.ksplits = conv_tc_dw_splits(ctx, g, B);
  a.tmem_cols = pow2_at_least(((g.KW + 3) / 4) * g.KH * 32);
  a.row_stride = (long long)dw_tc_row(g);
  const size_t smem = dw_tc_smem(g.KH);
  B200_CUDA(cudaFuncSetAttribute(conv_dw_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(a.ksplits, a.ic_slabs * (t.OCp / 32));
  a.dbg = nullptr;
  const int nblk = (int)(grid.x * grid.y);
#ifdef B200_TC_TIMING
  static const bool timing = getenv("B200_TC_TIMING") != nullptr;
  if (timing) B200_CUDA(cudaMalloc(&a.dbg, (size_t)nblk * 8 * sizeof(long long)));
#endif
  conv_dw_tc_kernel<<<grid, TCV_THREADS, smem, ctx->stream>>>(dy_hi, dy_lo, x_hi, x_lo, a);
  B200_LAUNCHED();
#ifdef B200_TC_TIMING
  if (timing) {  // diagnostic: cycles of the MMA role and of the epilogue, averaged over blocks
    std::vector<long long> h((size_t)nblk * 8);
    B200_CUDA(cudaStreamSynchronize(ctx->stream));
    B200_CUDA(cudaMemcpy(h.data(), a.dbg, h.size() * sizeof(long long), cudaMemcpyDeviceToHost));
    B200_CUDA(cudaFree(a.dbg));
    double s[8] = {0};
    for (int i = 0; i < nblk; ++i)
      for (int k = 0; k < 8; ++k) s[k] += (double)h[(size_t)i * 8 + k] / nblk;
    fprintf(stderr,
            "[tc-timing] dW blocks %d stages/block %.2f: mma total %.0f clk, wait full %.0f | epilogue wait %.0f, "
            "store %.0f\n",
            nblk, s[2], s[0], s[1], s[3], s[4]);
  }
#endif
  *splits = a.ksplits;
  return 0;
}

// ---- dW of layers with few input channels: explicit transposed im2col operand -----------------
//
// When in_c * KH * KW <= 128 (the first layer of a network: 3 x 5 x 5 = 75) a 32-channel slab would
// be almost all padding.  Here the contraction still runs over pixels, but both operands are
// K-major with 32 consecutive pixels of one output row per 128-byte row:
//   B[o][p]  = dY[b][o][y][x0 + p]                  a TMA tile straight from the CHW gradient
//   A[k][p]  = Xpad[b][c][y + ky][x0 + p + kx]      k = (c*KH + ky)*KW + kx: a converter thread owns
//              tap k, gathers its pixels from the raw input rows (one TMA tile), splits them and
//              writes hi / lo into TMEM lane k (tcgen05.st); the MMAs take A from tensor memory, so
//              the im2col rows never pass through shared memory
//   D[k][o] += A * B^T                              M = 128 (k padded), N = out channels, 4 k-steps
// so dW needs 8 MMAs per 32 pixels.  The converter warps also split B into hi / lo in place and
// keep the bias-gradient sums.  Per-CTA partial results are merged in fixed order afterwards.

namespace {

constexpr int TCS_MAX_STAGES = 4;     // gradient tile + raw input rows per stage: a few KB each
constexpr int TCS_PX = 32;          // pixels per step (one 128-byte operand row)
constexpr int TCS_GROUPS = 2;       // converter groups; group g converts the steps i with i % 2 == g
constexpr int TCS_GROUP_WARPS = 8;
static_assert(TCS_GROUPS <= 2, "a group's first step must be the first use of its stage: stages >= groups");
constexpr int TCS_CONV_WARPS = TCS_GROUPS * TCS_GROUP_WARPS;  // then one TMA warp and one MMA warp
constexpr int TCS_THREADS = (TCS_CONV_WARPS + 2) * 32;

struct TcDwSmallArgs {
  float *part;          // [ksplits][row] with row = 128 * OCp (D[k][o]) + OCp (bias sums)
  int *err;
  int C, OC, OCp, KH, KW, pad_t, pad_l;
  int OH, OW, nxb;      // output extent, 32-pixel blocks per output row
  int Kreal;            // C * KH * KW
  int bw;               // floats per raw input row in shared memory
  int nsteps, ksplits;
  int nst;              // pipeline stages
  int tmem_cols;        // accumulator 2*OCp, then two A buffers of 32 hi + 32 lo columns
  long long row;
  long long *dbg;       // [blocks][8] cycle counters in a build with -DB200_TC_TIMING, else nullptr
};

__global__ void __launch_bounds__(TCS_THREADS, 1)
  conv_dw_small_tc_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap dy_map,
                          const TcDwSmallArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t BB = (uint32_t)a.OCp * 128u;           // B tile (hi or lo)
  const uint32_t XB = ((uint32_t)(a.C * a.KH * a.bw * 4) + 1023u) & ~1023u;  // raw input rows
  const uint32_t STAGE = 2 * BB + XB;
  uint64_t *tma_full = reinterpret_cast<uint64_t *>(smem + (size_t)a.nst * STAGE);
  uint64_t *op_full = tma_full + TCS_MAX_STAGES;
  uint64_t *op_empty = op_full + TCS_MAX_STAGES;
  uint64_t *a_empty = op_empty + TCS_MAX_STAGES;   // [2] A buffers in tensor memory, one per converter group
  uint64_t *accum = a_empty + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(accum + 1);
  float *bsum_s = reinterpret_cast<float *>(tmem_slot + 4);   // [group][8 pixel quads][OCp] bias partials

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int s_begin = (int)((long long)blockIdx.x * a.nsteps / a.ksplits);
  const int s_end = (int)((long long)(blockIdx.x + 1) * a.nsteps / a.ksplits);
  if (tid == 0) {
    for (int s = 0; s < a.nst; ++s) {
      mbar_init(&tma_full[s], 1);
      mbar_init(&op_full[s], TCS_CONV_WARPS);
      mbar_init(&op_empty[s], 1);
    }
    mbar_init(&a_empty[0], 1);
    mbar_init(&a_empty[1], 1);
    mbar_init(accum, 1);
    mbar_fence_init();
  }
  if (warp == TCS_CONV_WARPS) tmem_alloc(tmem_slot, (uint32_t)a.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_a = tmem_base + 2u * (uint32_t)a.OCp;   // A buffer of group g: 64 columns from tmem_a + 64 g
  bool failed = false;

  if (warp == TCS_CONV_WARPS && lane == 0) {
    // ---- TMA producer: raw input rows and the gradient tile of each step ----------------------
    long long w = 0, t0 = tc_clock(), tq;
    for (int s = s_begin; s < s_end; ++s) {
      const uint32_t i = s - s_begin, st = i % a.nst, use = i / a.nst;
      tq = tc_clock();
      if (use > 0 && !mbar_wait_bounded(&op_empty[st], (use - 1) & 1)) {
        failed = true;
        break;
      }
      w += tc_clock() - tq;
      if (a.dbg && s == s_end - 1) {
        a.dbg[blockIdx.x * 8 + 0] = tc_clock() - t0;
        a.dbg[blockIdx.x * 8 + 1] = w;
      }
      const int xb = s % a.nxb, by = s / a.nxb, y = by % a.OH, b = by / a.OH;
      const int x0 = xb * TCS_PX;
      const int xs = (x0 - a.pad_l) & ~3;  // aligned start column of the raw rows (floor to 4)
      uint8_t *p = smem + (size_t)st * STAGE;
      mbar_expect_tx(&tma_full[st], BB + (uint32_t)(a.C * a.KH * a.bw * 4));
      tma_load_4d(p, &dy_map, x0, 0, y, b, &tma_full[st]);
      tma_load_4d(p + 2 * BB, &x_map, xs, y - a.pad_t, 0, b, &tma_full[st]);
    }
  } else if (warp == TCS_CONV_WARPS + 1 && lane == 0) {
    // ---- MMA issuer ---------------------------------------------------------------------------
    // the hi and lo gradient tiles are neighbours in shared memory: A_hi * [B_hi | B_lo] is one
    // instruction of width 2*OCp (columns OCp.. hold the A_hi*B_lo part, added in the epilogue)
    const uint32_t idesc1 = umma_idesc_tf32(128, a.OCp), idesc2 = umma_idesc_tf32(128, 2 * a.OCp);
    long long w = 0, t0 = tc_clock(), tq;
    for (int s = s_begin; s < s_end && !failed; ++s) {
      const uint32_t i = s - s_begin, st = i % a.nst;
      tq = tc_clock();
      if (!mbar_wait_bounded(&op_full[st], (i / a.nst) & 1)) {
        failed = true;
        break;
      }
      w += tc_clock() - tq;
      if (a.dbg && s == s_end - 1) {
        a.dbg[blockIdx.x * 8 + 2] = tc_clock() - t0;
        a.dbg[blockIdx.x * 8 + 3] = w;
      }
      tc_fence_after();
      const uint32_t base = smem_u32(smem + (size_t)st * STAGE);
      const uint32_t ta = tmem_a + (i & 1u) * 64u;
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4) {
        const uint64_t b = umma_desc(base + k4 * 32, 16, 1024, 2);
        umma_tf32_ta(tmem_base, ta + k4 * 8, b, idesc2, (i | k4) != 0);
        umma_tf32_ta(tmem_base, ta + 32 + k4 * 8, b, idesc1, 1);
      }
      umma_commit(&op_empty[st]);
      umma_commit(&a_empty[i & 1u]);
    }
    if (!failed) umma_commit(accum);
  } else if (warp < TCS_CONV_WARPS) {
    // ---- converters: im2col rows and the hi / lo split, then the epilogue ----------------------
    const int KK = a.KH * a.KW;
    const int grp = warp / TCS_GROUP_WARPS, gtid = tid - grp * (TCS_GROUP_WARPS * 32);
    constexpr int NCT = TCS_GROUP_WARPS * 32;  // threads of one group
    // A: this thread owns tap k = its TMEM lane and half of the step's 32 pixels (two warps of a
    // group share a lane quadrant); taps beyond the real ones are written as zeros
    static_assert(TCS_GROUP_WARPS == 8, "two warps per TMEM lane quadrant in every converter group");
    const int k = 32 * (warp & 3) + lane, phalf = ((warp - grp * TCS_GROUP_WARPS) >> 2) * 16;
    int soff = -1;  // floats into the raw rows (without the step's column offset)
    if (k < a.Kreal) {
      const int c = k / KK, r = k - c * KK, ky = r / a.KW, kx = r - ky * a.KW;
      soff = (c * a.KH + ky) * a.bw + kx + phalf;
    }
    const uint32_t ta_thread = tmem_a + (uint32_t)grp * 64u + ((uint32_t)(warp & 3) << 21) + (uint32_t)phalf;
    constexpr int NB = 128 * 8 / NCT;  // at most 128 out channels x 8 quads per step
    float bacc[NB];                    // bias partials of the (o, quad) items this thread owns
#pragma unroll
    for (int q = 0; q < NB; ++q) bacc[q] = 0.f;
    long long w = 0, t0 = tc_clock(), tq;
    // Every converter warp observes every step's barrier, in order, and takes part in the
    // hand-over, although only the step's group converts: a warp that skipped phases of an
    // mbarrier could no longer tell one phase from the one two later (the wait is by parity).
    for (int s = s_begin; s < s_end; ++s) {
      const uint32_t i = s - s_begin, st = i % a.nst;
      tq = tc_clock();
      if (!mbar_wait_bounded(&tma_full[st], (i / a.nst) & 1)) {
        failed = true;
        break;
      }
      w += tc_clock() - tq;
      if ((int)(i % TCS_GROUPS) != grp) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&op_full[st]);
        continue;
      }
      // this group's A buffer was read by the MMAs of its previous step
      if (i >= 2 && !mbar_wait_bounded(&a_empty[grp], ((i >> 1) - 1) & 1)) {
        failed = true;
        break;
      }
      tc_fence_after();
      uint8_t *p = smem + (size_t)st * STAGE;
      const int x0 = (s % a.nxb) * TCS_PX;
      const int d = (x0 - a.pad_l) - ((x0 - a.pad_l) & ~3);  // offset of the first needed column
      const float *xr = reinterpret_cast<const float *>(p + 2 * BB) + d;
      {
        uint32_t h[16], l[16];
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          float hv, lv;
          split_tf32_rn(soff >= 0 ? xr[soff + q] : 0.f, hv, lv);
          h[q] = __float_as_uint(hv);
          l[q] = __float_as_uint(lv);
        }
        tmem_st16(ta_thread, h);
        tmem_st16(ta_thread + 32, l);
      }
      // B: split the gradient tile in place (hi) and into the lo tile; bias partial sums
#pragma unroll
      for (int slot = 0; slot < NB; ++slot) {
        const int it = gtid + NCT * slot;
        if (it < a.OCp * 8) {
          const int o = it >> 3, quad = it & 7;
          const uint32_t off = (uint32_t)o * 128u + (uint32_t)((quad ^ (o & 7)) << 4);
          float4 v = *reinterpret_cast<float4 *>(p + off);
          float h[4], l[4];
          split_tf32_rn(v.x, h[0], l[0]);
          split_tf32_rn(v.y, h[1], l[1]);
          split_tf32_rn(v.z, h[2], l[2]);
          split_tf32_rn(v.w, h[3], l[3]);
          *reinterpret_cast<float4 *>(p + off) = make_float4(h[0], h[1], h[2], h[3]);
          *reinterpret_cast<float4 *>(p + BB + off) = make_float4(l[0], l[1], l[2], l[3]);
          bacc[slot] += (v.x + v.y) + (v.z + v.w);
        }
      }
      // generic-proxy writes -> visible to the tensor core (async proxy); the TMEM stores have
      // landed; then hand over
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&op_full[st]);
    }
    if (a.dbg && tid == 0) {
      a.dbg[blockIdx.x * 8 + 4] = tc_clock() - t0;
      a.dbg[blockIdx.x * 8 + 5] = w;
    }
    // ---- epilogue ------------------------------------------------------------------------------
    float *row = a.part + (size_t)blockIdx.x * a.row;
#pragma unroll
    for (int slot = 0; slot < NB; ++slot) {
      const int it = gtid + NCT * slot;
      if (it < a.OCp * 8) bsum_s[(grp * 8 + (it & 7)) * a.OCp + (it >> 3)] = bacc[slot];
    }
    asm volatile("bar.sync 1, %0;\n" ::"n"(TCS_CONV_WARPS * 32) : "memory");
    for (int o = tid; o < a.OCp; o += TCS_CONV_WARPS * 32) {
      float t = bsum_s[o];
#pragma unroll
      for (int q = 1; q < TCS_GROUPS * 8; ++q) t += bsum_s[q * a.OCp + o];
      row[(size_t)128 * a.OCp + o] = t;
    }
    if (warp < 4 && s_end > s_begin && !failed) {
      if (!mbar_wait_bounded(accum, 0)) failed = true;
      tc_fence_after();
    }
    if (warp < 4 && !failed) {  // one warp per TMEM lane quadrant
      const int k = warp * 32 + lane;
      for (int c0 = 0; c0 < a.OCp; c0 += 16) {
        float v[16];
        if (s_end > s_begin) {
          float w[16];
          tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
          tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(a.OCp + c0), w);
#pragma unroll
          for (int q = 0; q < 16; ++q) v[q] += w[q];
        } else {
#pragma unroll
          for (int q = 0; q < 16; ++q) v[q] = 0.f;
        }
        float4 *dst = reinterpret_cast<float4 *>(row + (size_t)k * a.OCp + c0);
#pragma unroll
        for (int q = 0; q < 4; ++q) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      }
    }
  }
  if (failed && a.err) atomicExch(a.err, 5);
  tc_fence_before();
  __syncthreads();
  if (warp == TCS_CONV_WARPS) tmem_dealloc(tmem_base, (uint32_t)a.tmem_cols);
}

size_t dw_small_stage(const ConvGeom &g, int OCp, int bw) {
  size_t XB = ((size_t)g.C * g.KH * bw * 4 + 1023) & ~(size_t)1023;
  return 2 * (size_t)OCp * 128 + XB;
}

size_t dw_small_fixed(int OCp) {
  return 1024 + (3 * TCS_MAX_STAGES + 3) * 8 + 32 + (size_t)TCS_GROUPS * 8 * OCp * 4 + 64;
}

// pipeline stages that fit (0: the kernel does not fit)
int dw_small_stages(const b200_ctx *ctx, const ConvGeom &g, int OCp, int bw) {
  size_t fixed = dw_small_fixed(OCp), stage = dw_small_stage(g, OCp, bw);
  // at least as many stages as converter groups: a group waiting for the second use of a stage
  // before its first use has happened would see the barrier's parity as already satisfied
  if (ctx->smem_optin < fixed + TCS_GROUPS * stage) return 0;
  size_t n = (ctx->smem_optin - fixed) / stage;
  return (int)(n > TCS_MAX_STAGES ? TCS_MAX_STAGES : n);
}

int dw_small_bw(const ConvGeom &g) { return (TCS_PX + g.KW - 1 + 3 + 3) & ~3; }

}  // namespace

// true when the small-input-channel dW kernel applies
bool conv_dw_small_ok(const b200_ctx *ctx, const ConvGeom &g) {
  if (g.SH != 1 || g.SW != 1 || g.DH != 1 || g.DW != 1) return false;
  if (g.C * g.KH * g.KW > 128 || g.OC > 128) return false;
  if ((g.WI & 3) || (g.OW & 3)) return false;                 // TMA strides are multiples of 16 bytes
  if (((size_t)g.HI * g.WI) & 3 || ((size_t)g.OH * g.OW) & 3) return false;
  TallGeom t = tall_geom(g, 1);
  if (g.pad_t < 0 || g.pad_l < 0 || t.pad_b < 0 || t.pad_r < 0) return false;
  const int OCp = (g.OC + 15) / 16 * 16;
  return dw_small_stages(ctx, g, OCp, dw_small_bw(g)) >= TCS_GROUPS;
}

int conv_dw_small_splits(const b200_ctx *ctx, const ConvGeom &g, int B) {
  long long nsteps = (long long)B * g.OH * ceil_div(g.OW, TCS_PX);
  return (int)(nsteps < ctx->sm_count ? nsteps : ctx->sm_count);
}

size_t conv_dw_small_floats(const b200_ctx *ctx, const ConvGeom &g, int B) {
  const int OCp = (g.OC + 15) / 16 * 16;
  return ((size_t)conv_dw_small_splits(ctx, g, B) + 1) * ((size_t)129 * OCp);
}

// dW (+ db when the layer has a bias) from the CHW input and gradient; `part` holds conv_dw_small_floats
int conv_dw_small(b200_ctx *ctx, const ConvGeom &g, const float *in, const float *dout, int B, float *part,
                  float *dW, float *db, int accumulate, DwFinishArgs *defer) {
  const int OCp = (g.OC + 15) / 16 * 16, bw = dw_small_bw(g);
  EncodeTiledFn fn = encode_fn();
  B200_REQUIRE(fn != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMap x_map, dy_map;
  {
    cuuint64_t dims[4] = {(cuuint64_t)g.WI, (cuuint64_t)g.HI, (cuuint64_t)g.C, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)g.WI * 4, (cuuint64_t)g.HI * g.WI * 4, (cuuint64_t)g.C * g.HI * g.WI * 4};
    cuuint32_t box[4] = {(cuuint32_t)bw, (cuuint32_t)g.KH, (cuuint32_t)g.C, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(&x_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(in), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed (%d) for the input rows", (int)r);
  }
  {
    // dimensions ordered (x, o, y, b) so that one box is the K-major tile [o][32 pixels]
    cuuint64_t dims[4] = {(cuuint64_t)g.OW, (cuuint64_t)g.OC, (cuuint64_t)g.OH, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)g.OH * g.OW * 4, (cuuint64_t)g.OW * 4, (cuuint64_t)g.OC * g.OH * g.OW * 4};
    cuuint32_t box[4] = {TCS_PX, (cuuint32_t)OCp, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(&dy_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(dout), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed (%d) for the gradient tiles", (int)r);
  }
  TcDwSmallArgs a;
  a.part = part;
  a.err = ctx->dev_err;
  a.C = g.C;
  a.OC = g.OC;
  a.OCp = OCp;
  a.KH = g.KH;
  a.KW = g.KW;
  a.pad_t = g.pad_t;
  a.pad_l = g.pad_l;
  a.OH = g.OH;
  a.OW = g.OW;
  a.nxb = ceil_div(g.OW, TCS_PX);
  a.Kreal = g.C * g.KH * g.KW;
  a.bw = bw;
  a.nsteps = B * g.OH * a.nxb;
  a.ksplits = conv_dw_small_splits(ctx, g, B);
  a.nst = dw_small_stages(ctx, g, OCp, bw);
  B200_REQUIRE(a.nst >= TCS_GROUPS, "conv_dw_small: the tiles do not fit shared memory");
  a.tmem_cols = pow2_at_least(2 * OCp + 128);
  a.row = (long long)129 * OCp;
  const size_t smem = dw_small_fixed(OCp) + (size_t)a.nst * dw_small_stage(g, OCp, bw);
  B200_CUDA(cudaFuncSetAttribute(conv_dw_small_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  a.dbg = nullptr;
#ifdef B200_TC_TIMING
  static const bool timing = getenv("B200_TC_TIMING") != nullptr;
  if (timing) B200_CUDA(cudaMalloc(&a.dbg, (size_t)a.ksplits * 8 * sizeof(long long)));
#endif
  conv_dw_small_tc_kernel<<<a.ksplits, TCS_THREADS, smem, ctx->stream>>>(x_map, dy_map, a);
  B200_LAUNCHED();
#ifdef B200_TC_TIMING
  if (timing) {  // diagnostic: cycles of the three roles and of their waits, averaged over blocks
    std::vector<long long> h((size_t)a.ksplits * 8);
    B200_CUDA(cudaStreamSynchronize(ctx->stream));
    B200_CUDA(cudaMemcpy(h.data(), a.dbg, h.size() * sizeof(long long), cudaMemcpyDeviceToHost));
    B200_CUDA(cudaFree(a.dbg));
    double s[8] = {0};
    for (int i = 0; i < a.ksplits; ++i)
      for (int k = 0; k < 8; ++k) s[k] += (double)h[(size_t)i * 8 + k] / a.ksplits;
    fprintf(stderr,
            "[tc-timing] dW small: steps/block %.1f stages %d: producer %.0f clk (wait %.0f), mma %.0f (wait %.0f), "
            "converter group 0 %.0f (wait %.0f)\n",
            (double)a.nsteps / a.ksplits, a.nst, s[0], s[1], s[2], s[3], s[4], s[5]);
  }
#endif
  DwFinishArgs f;
  f.part = part;
  f.part_stride = a.row;
  f.splits = a.ksplits;
  f.bsrc = part;            // the bias sums are the last OCp entries of every partial row
  f.bs_stride = a.row;
  f.bs_off = (long long)128 * OCp;
  f.bs_rows = a.ksplits;
  f.dW = dW;
  f.db = g.has_bias ? db : nullptr;
  f.layout = 1;
  f.row_w = 128 * OCp;
  f.C = g.C;
  f.OC = g.OC;
  f.OCp = OCp;
  f.KH = g.KH;
  f.KW = g.KW;
  f.ic_slabs = 1;
  f.tbl = g.tbl;
  f.accumulate = accumulate;
  if (defer != nullptr) {
    *defer = f;
    return 0;
  }
  B200_TRY(launch_dw_finish(ctx, f));
  return 0;
}

}  // namespace b200
