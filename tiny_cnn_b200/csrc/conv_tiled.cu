// Tiled FP32 convolution kernels for stride 1, dilation 1, 3x3 and 5x5 filters
// (every convolution of the LeNet, CIFAR-10 and 3x3 sweep configurations).
//
//   conv_core_kernel      direct convolution with a register tile of
//                         8 output pixels x 8 output channels per thread,
//                         input tile and re-laid-out filters staged in shared
//                         memory with cp.async, double buffered over input
//                         channel chunks.  Used for the forward pass and, with
//                         flipped/transposed filters and dY as input, for dX.
//   conv_dw_kernel        dW (+db) as a batch-reduced outer product: each
//                         thread owns OCT output channels x all KHxKW taps of
//                         one input channel and streams 8-pixel strips of
//                         (X, dY) from shared memory; the batch is split over
//                         the grid and every block writes one partial sum row.
//
// The math is that of kernels::conv2d_op_internal
// (tiny_dnn/core/kernels/conv2d_op_internal.h:13-74, :91-127, :130-179) with
// zero padding applied by predicated staging instead of a padded copy
// (tiny_dnn/core/params/conv_params.h:106-133).
#include <algorithm>

#include "common.cuh"
#include "device_utils.cuh"

namespace b200 {

// ---------------------------------------------------------------------------
// filter re-layout
// ---------------------------------------------------------------------------

// wt[(ic*KK + tap)*COp + o] = W[(o*C + ic)*KK + tap]   (0 if o >= OC or unconnected)
__global__ void conv_prep_wt_fwd_kernel(const float *__restrict__ W, float *__restrict__ wt,
                                        int C, int OC, int COp, int KK,
                                        const uint8_t *__restrict__ tbl) {
  int total = C * KK * COp;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    int o = i % COp;
    int r = i / COp;
    int tap = r % KK;
    int ic = r / KK;
    float v = 0.f;
    if (o < OC && (!tbl || tbl[ic * OC + o])) v = W[((size_t)o * C + ic) * KK + tap];
    wt[i] = v;
  }
}

// wt[(o*KK + a*KW + b)*Cp + ic] = W[(o*C + ic)*KK + (KH-1-a)*KW + (KW-1-b)]
__global__ void conv_prep_wt_dx_kernel(const float *__restrict__ W, float *__restrict__ wt, int C,
                                       int OC, int Cp, int KH, int KW,
                                       const uint8_t *__restrict__ tbl) {
  int KK = KH * KW;
  int total = OC * KK * Cp;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    int ic = i % Cp;
    int r = i / Cp;
    int tap = r % KK;
    int o = r / KK;
    int a = tap / KW, b = tap % KW;
    float v = 0.f;
    if (ic < C && (!tbl || tbl[ic * OC + o]))
      v = W[((size_t)o * C + ic) * KK + (KH - 1 - a) * KW + (KW - 1 - b)];
    wt[i] = v;
  }
}

// ---------------------------------------------------------------------------
// direct convolution core
// ---------------------------------------------------------------------------

struct CoreCfg {
  // problem: out[n][co][y][x] = bias[co] + sum_{ci,wy,wx} wt[ci][wy][wx][co] *
  //                             in[n][ci][y + wy - pad_t][x + wx - pad_l]
  const float *in;
  const float *wt;    // [CI][KH][KW][COp]
  const float *bias;  // [CO] or nullptr
  float *out;
  int *err;           // set when a bounded wait on a bulk copy runs out
  int B, CI, HI, WI, CO, COp, HO, WO;
  int pad_t, pad_l, act;
  // tiling
  int TH, TWG, NSB, OCB, ICB;
  int THp, PITCH;
  int tiles_x, tiles_y, tiles_oc, tiles_n;
  int in_tile_floats, w_tile_floats, nrows;
  unsigned pitch_magic;
  int log2_ocb4;
  int w_bulk;  // 1: a filter chunk is contiguous in memory and is fetched by one bulk copy
};

// v / d for v*d < 2^32 through one multiply; magic 0 encodes d == 1
__device__ __forceinline__ unsigned fastdiv(unsigned v, unsigned magic) {
  return magic ? __umulhi(v, magic) : v;
}
static unsigned make_magic(unsigned d) {
  return d <= 1 ? 0u : (unsigned)((0x100000000ULL / d) + 1ULL);
}

// Block = one tile of (NSB samples) x (TH rows) x (TWG*8 columns) x (OCB output
// channels); thread = 8 consecutive pixels x OCT output channels.  Input
// channels are consumed in chunks of ICB through a two-stage shared-memory
// pipeline: the input patch arrives by 4-byte cp.async (zero fill outside the
// image = padding), the filter chunk by one bulk asynchronous copy signalled on
// an mbarrier when it is contiguous in memory, else by 16-byte cp.async.
template <int KH, int KW, int OCT>
__global__ void __launch_bounds__(256, 2) conv_core_kernel(const CoreCfg p) {
  extern __shared__ __align__(16) float smem[];
  const int tid = threadIdx.x;
  const int nthreads = blockDim.x;
  constexpr int KK = KH * KW;

  // ---- tile coordinates -------------------------------------------------
  int bid = blockIdx.x;
  const int tx_ = bid % p.tiles_x;
  bid /= p.tiles_x;
  const int ty_ = bid % p.tiles_y;
  bid /= p.tiles_y;
  const int toc = bid % p.tiles_oc;
  const int tn = bid / p.tiles_oc;
  const int x0 = tx_ * p.TWG * 8;
  const int y0 = ty_ * p.TH;
  const int o0 = toc * p.OCB;
  const int n0 = tn * p.NSB;

  // ---- shared memory carve-up --------------------------------------------
  const int stage_floats = p.in_tile_floats + p.w_tile_floats;
  float *stage0 = smem;
  float *stage1 = smem + stage_floats;
  long long *rowoff = reinterpret_cast<long long *>(smem + 2 * stage_floats);
  uint64_t *bars = reinterpret_cast<uint64_t *>(rowoff + p.nrows);  // one per stage
  int *rowic = reinterpret_cast<int *>(bars + 2);

  if (p.w_bulk && tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_fence_init();
  }
  // row table: staged row -> offset of (n, ic, y, x=0) with ic relative to the
  // chunk base, or -1 when the row lies outside the batch / image
  for (int r = tid; r < p.nrows; r += nthreads) {
    int rr = r % p.THp;
    int q = r / p.THp;
    int ic = q % p.ICB;
    int s = q / p.ICB;
    int n = n0 + s;
    int y = y0 + rr - p.pad_t;
    long long off = -1;
    if (n < p.B && y >= 0 && y < p.HI)
      off = (((long long)n * p.CI + ic) * p.HI + y) * (long long)p.WI;
    rowoff[r] = off;
    rowic[r] = ic;
  }
  __syncthreads();

  const int nchunks = (p.CI + p.ICB - 1) / p.ICB;
  const long long chan_stride = (long long)p.HI * p.WI;
  const int ocb4 = p.OCB >> 2;

  auto load_chunk = [&](int chunk, float *stage, uint64_t *bar) {
    const int c0 = chunk * p.ICB;
    float *itile = stage;
    float *wtile = stage + p.in_tile_floats;
    if (p.w_bulk) {
      if (tid == 0) {
        const int icn = min(p.ICB, p.CI - c0);
        const uint32_t bytes = (uint32_t)(icn * KK * p.COp) * 4u;
        mbar_expect_tx(bar, bytes);
        bulk_copy_g2s(wtile, p.wt + (size_t)c0 * KK * p.COp, bytes, bar);
      }
    } else {
      const int nq = p.ICB * KK * ocb4;
      for (int q = tid; q < nq; q += nthreads) {
        int row = q >> p.log2_ocb4;
        int c4 = q & (ocb4 - 1);
        int ic = row / KK;
        int tap = row - ic * KK;
        int oc = o0 + c4 * 4;
        bool ok = (c0 + ic) < p.CI && oc < p.COp;
        const float *src = ok ? p.wt + ((size_t)(c0 + ic) * KK + tap) * p.COp + oc : p.wt;
        cp_async16(wtile + q * 4, src, ok);
      }
    }
    for (int idx = tid; idx < p.in_tile_floats; idx += nthreads) {
      int row = (int)fastdiv((unsigned)idx, p.pitch_magic);
      int j = idx - row * p.PITCH;
      long long off = rowoff[row];
      int ic = rowic[row];
      int x = x0 - p.pad_l + j;
      bool ok = off >= 0 && (c0 + ic) < p.CI && x >= 0 && x < p.WI;
      const float *src = ok ? p.in + off + (long long)c0 * chan_stride + x : p.in;
      cp_async4(itile + idx, src, ok);
    }
  };

  // ---- thread coordinates -------------------------------------------------
  const int nocg = p.OCB / OCT;
  const int ocg = tid % nocg;
  int pg = tid / nocg;
  const int txg = pg % p.TWG;
  pg /= p.TWG;
  const int ty = pg % p.TH;
  const int s = pg / p.TH;

  float acc[OCT][8];  // [oc][px]
#pragma unroll
  for (int o = 0; o < OCT; ++o)
#pragma unroll
    for (int px = 0; px < 8; ++px) acc[o][px] = 0.f;

  load_chunk(0, stage0, &bars[0]);
  cp_async_commit();

  bool failed = false;
  for (int chunk = 0; chunk < nchunks; ++chunk) {
    float *cur = (chunk & 1) ? stage1 : stage0;
    if (chunk + 1 < nchunks) {
      load_chunk(chunk + 1, (chunk & 1) ? stage0 : stage1, &bars[(chunk + 1) & 1]);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    if (p.w_bulk) {
      // stage (chunk & 1) completes for the (chunk >> 1)-th time
      if (!mbar_wait_bounded(&bars[chunk & 1], (uint32_t)((chunk >> 1) & 1))) failed = true;
    }
    failed = __syncthreads_or(failed) != 0;  // every thread takes the same exit
    if (failed) break;

    const float *itile = cur + ((s * p.ICB) * p.THp + ty) * p.PITCH + txg * 8;
    const float *wtile = cur + p.in_tile_floats + ocg * OCT;
    const int icn = min(p.ICB, p.CI - chunk * p.ICB);
    for (int ic = 0; ic < icn; ++ic) {
      const float *irow = itile + ic * p.THp * p.PITCH;
      const float *wrow = wtile + ic * KK * p.OCB;
#pragma unroll
      for (int wy = 0; wy < KH; ++wy) {
        float xin[12];
        {
          const float4 *ip = reinterpret_cast<const float4 *>(irow + wy * p.PITCH);
          float4 a = ip[0], b = ip[1], c = ip[2];
          xin[0] = a.x; xin[1] = a.y; xin[2] = a.z; xin[3] = a.w;
          xin[4] = b.x; xin[5] = b.y; xin[6] = b.z; xin[7] = b.w;
          xin[8] = c.x; xin[9] = c.y; xin[10] = c.z; xin[11] = c.w;
        }
#pragma unroll
        for (int wx = 0; wx < KW; ++wx) {
          const float4 *wp = reinterpret_cast<const float4 *>(wrow + (wy * KW + wx) * p.OCB);
          float w[OCT];
#pragma unroll
          for (int h = 0; h < OCT / 4; ++h) {
            float4 wv = wp[h];
            w[h * 4 + 0] = wv.x;
            w[h * 4 + 1] = wv.y;
            w[h * 4 + 2] = wv.z;
            w[h * 4 + 3] = wv.w;
          }
#pragma unroll
          for (int o = 0; o < OCT; ++o)
#pragma unroll
            for (int px = 0; px < 8; ++px) acc[o][px] = fmaf(w[o], xin[px + wx], acc[o][px]);
        }
      }
    }
    __syncthreads();
  }
  if (failed) {
    // a bulk copy never signalled: report, let the other copies of this block
    // drain, and leave without writing results
    if (p.err) atomicExch(p.err, 1);
    cp_async_wait<0>();
    return;
  }

  // ---- epilogue -------------------------------------------------------------
  const int n = n0 + s;
  const int y = y0 + ty;
  const int xb = x0 + txg * 8;
  if (n >= p.B || y >= p.HO || xb >= p.WO) return;
  const bool vec = ((p.WO & 3) == 0) && (xb + 8 <= p.WO);
#pragma unroll
  for (int o = 0; o < OCT; ++o) {
    int oc = o0 + ocg * OCT + o;
    if (oc >= p.CO) continue;
    float bv = p.bias ? p.bias[oc] : 0.f;
    float *op = p.out + (((size_t)n * p.CO + oc) * p.HO + y) * p.WO + xb;
    float v[8];
#pragma unroll
    for (int px = 0; px < 8; ++px) v[px] = apply_act(acc[o][px] + bv, p.act);
    if (vec) {
      reinterpret_cast<float4 *>(op)[0] = make_float4(v[0], v[1], v[2], v[3]);
      reinterpret_cast<float4 *>(op)[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
#pragma unroll
      for (int px = 0; px < 8; ++px)
        if (xb + px < p.WO) op[px] = v[px];
    }
  }
}

static int ilog2(int v) {
  int l = 0;
  while ((1 << l) < v) ++l;
  return l;
}

bool conv_tiled_ok(const ConvGeom &g) {
  if (g.SH != 1 || g.SW != 1 || g.DH != 1 || g.DW != 1) return false;
  if (!((g.KH == 3 && g.KW == 3) || (g.KH == 5 && g.KW == 5))) return false;
  return true;
}

static int round_up(int a, int b) { return (a + b - 1) / b * b; }

// channel pitch of the re-laid-out filters: output channels padded to a
// multiple of 8 (4 when there are at most 4 of them)
static int padded_channels(int c) { return c <= 4 ? 4 : round_up(c, 8); }

static size_t core_smem_bytes(const CoreCfg &p) {
  return (size_t)2 * (p.in_tile_floats + p.w_tile_floats) * 4 + (size_t)p.nrows * 12 + 16 + 16;
}

static void core_fill_tile(CoreCfg &p, int KH, int KW) {
  p.THp = p.TH + KH - 1;
  p.PITCH = round_up(p.TWG * 8 + KW - 1, 4);
  p.in_tile_floats = p.NSB * p.ICB * p.THp * p.PITCH;
  p.w_tile_floats = p.ICB * KH * KW * p.OCB;
  p.nrows = p.NSB * p.ICB * p.THp;
  p.tiles_x = ceil_div(p.WO, p.TWG * 8);
  p.tiles_y = ceil_div(p.HO, p.TH);
  p.tiles_oc = ceil_div(p.CO, p.OCB);
  p.tiles_n = ceil_div(p.B, p.NSB);
  p.pitch_magic = make_magic((unsigned)p.PITCH);
  p.log2_ocb4 = ilog2(p.OCB / 4);
  p.w_bulk = (p.OCB == p.COp) ? 1 : 0;
}

static void apply_choice(CoreCfg &p, const TileChoice &c, int KH, int KW) {
  p.OCB = c.OCB;
  p.TH = c.TH;
  p.TWG = c.TWG;
  p.NSB = c.NSB;
  p.ICB = c.ICB;
  core_fill_tile(p, KH, KW);
}

// Every legal tile shape with a score from a small model of the launch: blocks
// are spread over the SMs, an SM's time is its number of blocks times the
// instructions of a block (FMAs plus staging plus a fixed cost per chunk),
// discounted when few warps are resident (latency is exposed) and for the 8x4
// thread tile (more shared-memory loads per FMA); blocks that do not all fit on
// the machine at once run in waves.  Sorted best first.
static std::vector<std::pair<double, TileChoice>> core_candidates(const b200_ctx *ctx, CoreCfg p,
                                                                   int KH, int KW) {
  std::vector<std::pair<double, TileChoice>> out;
  p.COp = padded_channels(p.CO);
  const int sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
  const size_t smem_sm = 233472;  // shared memory of one SM
  const int wg = ceil_div(p.WO, 8);
  for (int OCT = 8; OCT >= 4; OCT -= 4) {
    if (OCT == 8 && p.COp < 8) continue;
    // channels per block: all of them when they fit 64 (the filter chunk is then
    // one contiguous bulk copy), else tiles of 64 or 32
    const int ocb_opts[3] = {p.COp <= 64 ? p.COp : 0, 64, 32};
    for (int oi = 0; oi < 3; ++oi) {
      const int OCB = ocb_opts[oi];
      if (OCB <= 0 || OCB > p.COp || OCB % OCT) continue;
      if (oi > 0 && OCB == ocb_opts[0]) continue;
      const int nocg = OCB / OCT;
      for (int tt = 32; tt <= 256; tt <<= 1) {
        int pgs = tt / nocg;
        if (pgs < 1) continue;
        TileChoice c;
        c.OCT = OCT;
        c.OCB = OCB;
        c.TWG = wg <= 8 ? wg : 4;
        if (c.TWG > pgs) c.TWG = pgs;
        c.TH = pgs / c.TWG;
        if (c.TH > p.HO) c.TH = p.HO;
        if (c.TH < 1) c.TH = 1;
        c.NSB = pgs / (c.TWG * c.TH);
        if (c.NSB > p.B) c.NSB = p.B;
        if (c.NSB < 1) c.NSB = 1;
        int threads = nocg * c.TWG * c.TH * c.NSB;
        if (threads > 256) continue;
        for (int icb = 8; icb >= 2; icb >>= 1) {
          c.ICB = p.CI < icb ? p.CI : icb;
          CoreCfg q = p;
          apply_choice(q, c, KH, KW);
          size_t smem = core_smem_bytes(q);
          if (smem > ctx->smem_optin) continue;
          bool dup = false;
          for (auto &o : out)
            if (o.second.OCT == c.OCT && o.second.OCB == c.OCB && o.second.TH == c.TH &&
                o.second.TWG == c.TWG && o.second.NSB == c.NSB && o.second.ICB == c.ICB)
              dup = true;
          if (dup) continue;
          int warps = ceil_div(threads, 32);
          int resident = (int)(smem_sm / (smem + 1024));
          int by_regs = 65536 / (128 * warps * 32);
          if (by_regs < resident) resident = by_regs;
          if (resident > 32) resident = 32;
          if (resident < 1) continue;
          long long blocks = (long long)q.tiles_x * q.tiles_y * q.tiles_oc * q.tiles_n;
          long long per_sm = (blocks + sms - 1) / sms;
          double waves = 1.0;
          long long conc = per_sm;  // blocks an SM runs at the same time
          if (per_sm > resident) {
            waves = (double)((per_sm + resident - 1) / resident);
            conc = resident;
          }
          // warp instructions of one block per chunk
          double fma = 8.0 * OCT * q.ICB * KH * KW;
          double stage_in = 10.0 * q.in_tile_floats / threads;
          double stage_w = q.w_bulk ? 2.0 : 8.0 * q.w_tile_floats / 4.0 / threads;
          double per_chunk = fma * (OCT == 8 ? 1.08 : 1.18) + stage_in + stage_w + 150.0;
          double block_cost = warps * per_chunk * ceil_div(p.CI, q.ICB);
          double occ = 0.45 + 0.55 * (conc * warps >= 8 ? 1.0 : (conc * warps) / 8.0);
          double t = waves * conc * block_cost / occ;
          out.push_back({t, c});
        }
      }
    }
  }
  std::sort(out.begin(), out.end(),
            [](const std::pair<double, TileChoice> &a, const std::pair<double, TileChoice> &b) {
              return a.first < b.first;
            });
  return out;
}

template <int KH, int KW, int OCT>
static int launch_core_t(b200_ctx *ctx, const CoreCfg &p, long long blocks, int threads,
                         size_t smem) {
  B200_CUDA(cudaFuncSetAttribute(conv_core_kernel<KH, KW, OCT>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  conv_core_kernel<KH, KW, OCT><<<(unsigned)blocks, threads, smem, ctx->stream>>>(p);
  B200_LAUNCHED();
  return 0;
}

static int launch_choice(b200_ctx *ctx, CoreCfg p, const TileChoice &c, int KH, int KW) {
  apply_choice(p, c, KH, KW);
  p.err = ctx->dev_err;
  size_t smem = core_smem_bytes(p);
  B200_REQUIRE(smem <= ctx->smem_optin, "conv tile needs %zu bytes of shared memory (limit %zu)",
               smem, ctx->smem_optin);
  int threads = (p.OCB / c.OCT) * p.TWG * p.TH * p.NSB;
  B200_REQUIRE(threads >= 1 && threads <= 256, "conv tile thread count %d out of range", threads);
  long long blocks = (long long)p.tiles_x * p.tiles_y * p.tiles_oc * p.tiles_n;
  B200_REQUIRE(blocks > 0 && blocks < 0x7fffffffLL, "conv grid too large");
  if (KH == 3 && c.OCT == 8) return launch_core_t<3, 3, 8>(ctx, p, blocks, threads, smem);
  if (KH == 3 && c.OCT == 4) return launch_core_t<3, 3, 4>(ctx, p, blocks, threads, smem);
  if (KH == 5 && c.OCT == 8) return launch_core_t<5, 5, 8>(ctx, p, blocks, threads, smem);
  return launch_core_t<5, 5, 4>(ctx, p, blocks, threads, smem);
}

// Tile shape for this problem: remembered per context; on first sight the best
// candidates of the model are each timed with CUDA events on the real buffers
// (every shape computes identical results -- the accumulation order per output
// does not depend on the tiling) and the fastest is kept.  Inside a stream
// capture, or with B200_AUTOTUNE=0, the model's first choice is used.
static int launch_core(b200_ctx *ctx, CoreCfg &p, int KH, int KW) {
  p.COp = padded_channels(p.CO);
  char key[160];
  snprintf(key, sizeof(key), "core %d %d %d %d %d %d %d %d %d %d", KH, p.B, p.CI, p.HI, p.WI, p.CO,
           p.HO, p.WO, p.pad_t, p.pad_l);
  auto it = ctx->tile_cache.find(key);
  if (it != ctx->tile_cache.end()) return launch_choice(ctx, p, it->second, KH, KW);

  auto cands = core_candidates(ctx, p, KH, KW);
  B200_REQUIRE(!cands.empty(), "conv: no tile shape fits shared memory");
  TileChoice pick = cands[0].second;
  if (const char *e = getenv("B200_CONV_TILE")) {
    // tuning override "OCT,OCB,TH,TWG,NSB,ICB" (must be one of the legal shapes)
    int v[6];
    if (sscanf(e, "%d,%d,%d,%d,%d,%d", &v[0], &v[1], &v[2], &v[3], &v[4], &v[5]) == 6)
      for (auto &c : cands)
        if (c.second.OCT == v[0] && c.second.OCB == v[1] && c.second.TH == v[2] &&
            c.second.TWG == v[3] && c.second.NSB == v[4] && c.second.ICB == v[5])
          pick = c.second;
    return launch_choice(ctx, p, pick, KH, KW);
  }
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  B200_CUDA(cudaStreamIsCapturing(ctx->stream, &cap));
  const char *at = getenv("B200_AUTOTUNE");
  bool tune = !(at && at[0] == '0') && cap == cudaStreamCaptureStatusNone && cands.size() > 1;
  if (tune) {
    cudaEvent_t e0, e1;
    B200_CUDA(cudaEventCreate(&e0));
    B200_CUDA(cudaEventCreate(&e1));
    float best_ms = 1e30f;
    size_t ntry = cands.size() < 24 ? cands.size() : 24;
    for (size_t i = 0; i < ntry; ++i) {
      const TileChoice &c = cands[i].second;
      int r = launch_choice(ctx, p, c, KH, KW);  // warm-up (sets the kernel attribute)
      if (r == 0) {
        B200_CUDA(cudaEventRecord(e0, ctx->stream));
        for (int rep = 0; rep < 3 && r == 0; ++rep) r = launch_choice(ctx, p, c, KH, KW);
        B200_CUDA(cudaEventRecord(e1, ctx->stream));
        B200_CUDA(cudaEventSynchronize(e1));
      }
      if (r != 0) {
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        return r;
      }
      float ms = 0.f;
      B200_CUDA(cudaEventElapsedTime(&ms, e0, e1));
      if (ms < best_ms) {
        best_ms = ms;
        pick = c;
      }
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (getenv("B200_TUNE_LOG"))
      fprintf(stderr, "[b200] %s -> OCT %d OCB %d TH %d TWG %d NSB %d ICB %d (%.1f us; model pick OCT %d OCB %d TH %d TWG %d NSB %d ICB %d)\n",
              key, pick.OCT, pick.OCB, pick.TH, pick.TWG, pick.NSB, pick.ICB, best_ms * 1000.f / 3.f,
              cands[0].second.OCT, cands[0].second.OCB, cands[0].second.TH, cands[0].second.TWG,
              cands[0].second.NSB, cands[0].second.ICB);
  }
  if (cap == cudaStreamCaptureStatusNone) ctx_remember_tile(ctx, key, pick);
  return launch_choice(ctx, p, pick, KH, KW);
}

size_t conv_tiled_fwd_scratch(const ConvGeom &g) {
  return (size_t)g.C * g.KH * g.KW * padded_channels(g.OC);
}
size_t conv_tiled_dx_scratch(const ConvGeom &g) {
  return (size_t)g.OC * g.KH * g.KW * padded_channels(g.C);
}

// ---------------------------------------------------------------------------
// direct convolution with at most four input channels (forward of a first layer)
// ---------------------------------------------------------------------------
//
// out[n][co][y][x] = act(bias[co] + sum_{ci,wy,wx} wt[ci][wy][wx][co] * in[n][ci][y+wy-pad_t][x+wx-pad_l])
// A block covers a 32 x 8 output tile of one image for all output channels: thread = (2 x 4 pixel
// patch, group of 8 output channels), 64 accumulators.  The whole input tile (all <= 4 channels)
// is staged once; per input channel a thread reads its (2+KH-1) x (4+KW-1) window into registers
// and applies all taps, fetching the 8 weights of a tap with two broadcast 16-byte loads.

constexpr int FI_TILE_W = 32, FI_TILE_H = 8, FI_PX = 4, FI_PY = 2, FI_OCG = 8;
constexpr int FI_PATCHES = (FI_TILE_W / FI_PX) * (FI_TILE_H / FI_PY);  // 32: one warp per channel group

struct FewInCfg {
  const float *in;    // [B][CI][HI][WI]
  const float *wt;    // [CI][KH*KW][COp]  (COp a multiple of 8)
  const float *bias;  // CO values or nullptr
  float *out;         // [B][CO][HO][WO]
  int CI, HI, WI, CO, COp, HO, WO, pad_t, pad_l, tiles_x, act;
};

template <int KH, int KW>
__global__ void __launch_bounds__(256) conv_fewin_kernel(const FewInCfg p) {
  constexpr int KK = KH * KW;
  constexpr int TH = FI_TILE_H + KH - 1;
  constexpr int PITCH = (FI_TILE_W + KW - 1 + 3) & ~3;
  constexpr int WC = FI_PX + KW - 1, WC4 = (WC + 3) / 4;
  extern __shared__ __align__(16) float fi_smem[];
  float *wsm = fi_smem;                          // [CI][KK][COp]
  float *xs = fi_smem + p.CI * KK * p.COp;       // [CI][TH][PITCH]
  const int tid = threadIdx.x, grp = tid / FI_PATCHES, t = tid - grp * FI_PATCHES, tx = t & 7, ty = t >> 3;
  const int b = blockIdx.y, tile = blockIdx.x;
  const int x0 = (tile % p.tiles_x) * FI_TILE_W, y0 = (tile / p.tiles_x) * FI_TILE_H;
  const int nthreads = blockDim.x;
  for (int i = tid; i < p.CI * KK * p.COp / 4; i += nthreads)
    reinterpret_cast<float4 *>(wsm)[i] = reinterpret_cast<const float4 *>(p.wt)[i];
  const float *img = p.in + (size_t)b * p.CI * p.HI * p.WI;
  for (int i = tid; i < p.CI * TH * PITCH; i += nthreads) {
    const int col = i % PITCH, r = i / PITCH, row = r % TH, c = r / TH;
    const int gy = y0 + row - p.pad_t, gx = x0 + col - p.pad_l;
    const bool ok = gy >= 0 && gy < p.HI && gx >= 0 && gx < p.WI;
    cp_async4(xs + i, ok ? img + ((size_t)c * p.HI + gy) * p.WI + gx : img, ok);
  }
  cp_async_commit();
  float acc[FI_OCG][FI_PY][FI_PX];
#pragma unroll
  for (int n = 0; n < FI_OCG; ++n)
#pragma unroll
    for (int i = 0; i < FI_PY; ++i)
#pragma unroll
      for (int j = 0; j < FI_PX; ++j) acc[n][i][j] = 0.f;
  cp_async_wait<0>();
  __syncthreads();
  // one (input channel, window row) per iteration: a loop body of KW * 64 FFMAs stays in the
  // instruction cache, which the fully unrolled KH*KW body does not
#pragma unroll 1
  for (int it = 0; it < p.CI * KH; ++it) {
    const int ci = it / KH, wy = it - ci * KH;
    float win[FI_PY][WC4 * 4];
    const float *wp = xs + ((size_t)ci * TH + ty * FI_PY + wy) * PITCH + tx * FI_PX;
#pragma unroll
    for (int r = 0; r < FI_PY; ++r)
#pragma unroll
      for (int q = 0; q < WC4; ++q) {
        const float4 v = *reinterpret_cast<const float4 *>(wp + r * PITCH + 4 * q);
        win[r][4 * q] = v.x;
        win[r][4 * q + 1] = v.y;
        win[r][4 * q + 2] = v.z;
        win[r][4 * q + 3] = v.w;
      }
    const float *wc = wsm + ((size_t)ci * KK + wy * KW) * p.COp + grp * FI_OCG;
#pragma unroll
    for (int wx = 0; wx < KW; ++wx) {
      const float4 wa = *reinterpret_cast<const float4 *>(wc + wx * p.COp);
      const float4 wb = *reinterpret_cast<const float4 *>(wc + wx * p.COp + 4);
      const float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
      for (int n = 0; n < FI_OCG; ++n)
#pragma unroll
        for (int i = 0; i < FI_PY; ++i)
#pragma unroll
          for (int j = 0; j < FI_PX; ++j) acc[n][i][j] = fmaf(w[n], win[i][j + wx], acc[n][i][j]);
    }
  }
  const int ox = x0 + tx * FI_PX, oy = y0 + ty * FI_PY;
#pragma unroll
  for (int n = 0; n < FI_OCG; ++n) {
    const int co = grp * FI_OCG + n;
    if (co >= p.CO) break;
    const float bv = p.bias ? __ldg(p.bias + co) : 0.f;
#pragma unroll
    for (int i = 0; i < FI_PY; ++i) {
      if (oy + i >= p.HO) continue;
      float *o = p.out + (((size_t)b * p.CO + co) * p.HO + oy + i) * p.WO + ox;
      float v[FI_PX];
#pragma unroll
      for (int j = 0; j < FI_PX; ++j) v[j] = apply_act(acc[n][i][j] + bv, p.act);
      if (ox + FI_PX <= p.WO && (p.WO & 3) == 0) {
        *reinterpret_cast<float4 *>(o) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
#pragma unroll
        for (int j = 0; j < FI_PX; ++j)
          if (ox + j < p.WO) o[j] = v[j];
      }
    }
  }
}

static size_t fewin_smem(int CI, int COp, int KH, int KW) {
  size_t TH = FI_TILE_H + KH - 1, PITCH = (FI_TILE_W + KW - 1 + 3) & ~3;
  return ((size_t)CI * KH * KW * COp + (size_t)CI * TH * PITCH) * 4;
}

template <int KH, int KW>
static int launch_fewin(b200_ctx *ctx, const FewInCfg &p, int B) {
  size_t smem = fewin_smem(p.CI, p.COp, KH, KW);
  dim3 grid(p.tiles_x * ceil_div(p.HO, FI_TILE_H), B);
  B200_CUDA(cudaFuncSetAttribute(conv_fewin_kernel<KH, KW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  conv_fewin_kernel<KH, KW><<<grid, FI_PATCHES * (p.COp / FI_OCG), smem, ctx->stream>>>(p);
  B200_LAUNCHED();
  return 0;
}

int conv_tiled_fwd(b200_ctx *ctx, const ConvGeom &g, const float *in, const float *W,
                   const float *bias, float *out, int B, int act, float *scratch) {
  if (B == 0) return 0;
  int KK = g.KH * g.KW;
  int COp = padded_channels(g.OC);
  int total = g.C * KK * COp;
  conv_prep_wt_fwd_kernel<<<ceil_div(total, 256), 256, 0, ctx->stream>>>(W, scratch, g.C, g.OC,
                                                                        COp, KK, g.tbl);
  B200_LAUNCHED();
  if (g.C <= 4 && COp % 8 == 0 && COp <= 64 && fewin_smem(g.C, COp, g.KH, g.KW) <= ctx->smem_optin) {
    FewInCfg f{};
    f.in = in;
    f.wt = scratch;
    f.bias = g.has_bias ? bias : nullptr;
    f.out = out;
    f.CI = g.C;
    f.HI = g.HI;
    f.WI = g.WI;
    f.CO = g.OC;
    f.COp = COp;
    f.HO = g.OH;
    f.WO = g.OW;
    f.pad_t = g.pad_t;
    f.pad_l = g.pad_l;
    f.tiles_x = ceil_div(g.OW, FI_TILE_W);
    f.act = act;
    if (g.KH == 5 && g.KW == 5) return launch_fewin<5, 5>(ctx, f, B);
    if (g.KH == 3 && g.KW == 3) return launch_fewin<3, 3>(ctx, f, B);
  }
  CoreCfg p{};
  p.in = in;
  p.wt = scratch;
  p.bias = g.has_bias ? bias : nullptr;
  p.out = out;
  p.B = B;
  p.CI = g.C;
  p.HI = g.HI;
  p.WI = g.WI;
  p.CO = g.OC;
  p.HO = g.OH;
  p.WO = g.OW;
  p.pad_t = g.pad_t;
  p.pad_l = g.pad_l;
  p.act = act;
  return launch_core(ctx, p, g.KH, g.KW);
}

// ---------------------------------------------------------------------------
// direct convolution with at most four output channels (dX of a first layer)
// ---------------------------------------------------------------------------
//
// out[n][co][y][x] = sum_{ci,wy,wx} wt[ci][wy][wx][co(4)] * in[n][ci][y + wy - pad_t][x + wx - pad_l]
// With so few output channels a thread cannot reuse an input value across channels, so it reuses
// it across the window instead: each thread owns a 2 x 4 pixel patch for all NOUT channels, reads
// its (2+KH-1) x (4+KW-1) input window of one input channel into registers (16-byte loads) and
// applies all KH*KW taps to it; the NOUT weights of a tap come from shared memory in one
// broadcast load.  A block covers a 32 x 8 output tile of one image; input channels are staged
// four at a time with zero-filled cp.async, double buffered, and each of the four thread groups
// of a block takes one of them (more warps in flight); the groups' sums are added in group order.

constexpr int FO_TILE = 32, FO_TILE_H = 8, FO_PX = 4, FO_PY = 2, FO_ICB = 4;  // 32 x 8 output tile: many small blocks
constexpr int FO_PATCHES = (FO_TILE / FO_PX) * (FO_TILE_H / FO_PY);  // 8 x 4 patches of 4 x 2 pixels
constexpr int FO_THREADS = FO_PATCHES * FO_ICB;       // one thread group per staged input channel

struct FewOutCfg {
  const float *in;   // [B][CI][HI][WI]
  const float *wt;   // [CI][KH*KW][4]
  float *out;        // [B][CO][HO][WO]
  int CI, HI, WI, CO, HO, WO, pad_t, pad_l, tiles_x;
};

template <int KH, int KW, int NOUT>
__global__ void __launch_bounds__(FO_THREADS) conv_fewout_kernel(const FewOutCfg p) {
  constexpr int KK = KH * KW;
  constexpr int TH = FO_TILE_H + KH - 1;               // staged rows
  constexpr int PITCH = (FO_TILE + KW - 1 + 3) & ~3;   // staged row pitch (floats, 16-byte rows)
  constexpr int WC = FO_PX + KW - 1;                   // register window columns
  constexpr int WC4 = (WC + 3) / 4;                    // 16-byte loads per window row
  extern __shared__ __align__(16) float fo_smem[];
  float *wsm = fo_smem;                                // [CI][KK][4]
  float *xs = fo_smem + ((p.CI * KK * 4 + 3) & ~3);     // [2][FO_ICB][TH][PITCH]
  const int tid = threadIdx.x, z = tid / FO_PATCHES, t = tid - z * FO_PATCHES, tx = t & 7, ty = t >> 3;
  const int b = blockIdx.y, tile = blockIdx.x;
  const int x0 = (tile % p.tiles_x) * FO_TILE, y0 = (tile / p.tiles_x) * FO_TILE_H;
  for (int i = tid; i < p.CI * KK; i += FO_THREADS)
    reinterpret_cast<float4 *>(wsm)[i] = reinterpret_cast<const float4 *>(p.wt)[i];
  const float *img = p.in + (size_t)b * p.CI * p.HI * p.WI;
  const int nchunks = (p.CI + FO_ICB - 1) / FO_ICB;
  // The elements a thread stages are at the same tile positions in every chunk: their source
  // offsets (relative to the chunk's first channel) and validity are computed once.
  constexpr int NEL = FO_ICB * TH * PITCH;
  constexpr int NST = (NEL + FO_THREADS - 1) / FO_THREADS;
  int soff[NST];       // float offset from the first channel of the chunk, -1: padding (zero fill)
  int schan[NST];      // channel within the chunk
#pragma unroll
  for (int k = 0; k < NST; ++k) {
    const int i = tid + k * FO_THREADS;
    const int col = i % PITCH, r = i / PITCH, row = r % TH, c = r / TH;
    const int gy = y0 + row - p.pad_t, gx = x0 + col - p.pad_l;
    const bool ok = i < NEL && gy >= 0 && gy < p.HI && gx >= 0 && gx < p.WI;
    soff[k] = ok ? (c * p.HI + gy) * p.WI + gx : -1;
    schan[k] = i < NEL ? c : FO_ICB;
  }
  auto stage = [&](int chunk, int buf) {
    float *dst = xs + (size_t)buf * NEL;
    const int c0 = chunk * FO_ICB;
    const float *src = img + (size_t)c0 * p.HI * p.WI;
#pragma unroll
    for (int k = 0; k < NST; ++k) {
      if (schan[k] < FO_ICB) {
        const bool ok = soff[k] >= 0 && c0 + schan[k] < p.CI;
        cp_async4(dst + tid + k * FO_THREADS, ok ? src + soff[k] : img, ok);
      }
    }
    cp_async_commit();
  };
  float acc[NOUT][FO_PY][FO_PX];
#pragma unroll
  for (int n = 0; n < NOUT; ++n)
#pragma unroll
    for (int i = 0; i < FO_PY; ++i)
#pragma unroll
      for (int j = 0; j < FO_PX; ++j) acc[n][i][j] = 0.f;
  stage(0, 0);
  for (int chunk = 0; chunk < nchunks; ++chunk) {
    if (chunk + 1 < nchunks) {
      stage(chunk + 1, (chunk + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float *xb = xs + (size_t)(chunk & 1) * FO_ICB * TH * PITCH;
    {
      const int c = z, ci = chunk * FO_ICB + c;
      if (ci < p.CI) {
      const float4 *wc = reinterpret_cast<const float4 *>(wsm) + (size_t)ci * KK;
      // one window row per iteration keeps the loop body inside the instruction cache
#pragma unroll 1
      for (int wy = 0; wy < KH; ++wy) {
        float win[FO_PY][WC4 * 4];
        const float *wp = xb + ((size_t)c * TH + ty * FO_PY + wy) * PITCH + tx * FO_PX;
#pragma unroll
        for (int r = 0; r < FO_PY; ++r)
#pragma unroll
          for (int q = 0; q < WC4; ++q) {
            const float4 v = *reinterpret_cast<const float4 *>(wp + r * PITCH + 4 * q);
            win[r][4 * q] = v.x;
            win[r][4 * q + 1] = v.y;
            win[r][4 * q + 2] = v.z;
            win[r][4 * q + 3] = v.w;
          }
#pragma unroll
        for (int wx = 0; wx < KW; ++wx) {
          const float4 w4 = wc[wy * KW + wx];
          const float w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
          for (int n = 0; n < NOUT; ++n)
#pragma unroll
            for (int i = 0; i < FO_PY; ++i)
#pragma unroll
              for (int j = 0; j < FO_PX; ++j) acc[n][i][j] = fmaf(w[n], win[i][j + wx], acc[n][i][j]);
        }
      }
    }
    }
    __syncthreads();
  }
  // add the groups' partial sums in group order (the staging buffers are free now)
  float *red = xs;  // [FO_ICB - 1][NOUT * FO_PY * FO_PX][FO_PATCHES]
  if (z > 0) {
#pragma unroll
    for (int n = 0; n < NOUT; ++n)
#pragma unroll
      for (int i = 0; i < FO_PY; ++i)
#pragma unroll
        for (int j = 0; j < FO_PX; ++j)
          red[((size_t)(z - 1) * NOUT * FO_PY * FO_PX + (n * FO_PY + i) * FO_PX + j) * FO_PATCHES + t] = acc[n][i][j];
  }
  __syncthreads();
  if (z > 0) return;
#pragma unroll
  for (int g = 0; g < FO_ICB - 1; ++g)
#pragma unroll
    for (int n = 0; n < NOUT; ++n)
#pragma unroll
      for (int i = 0; i < FO_PY; ++i)
#pragma unroll
        for (int j = 0; j < FO_PX; ++j)
          acc[n][i][j] += red[((size_t)g * NOUT * FO_PY * FO_PX + (n * FO_PY + i) * FO_PX + j) * FO_PATCHES + t];
  const int ox = x0 + tx * FO_PX, oy = y0 + ty * FO_PY;
#pragma unroll
  for (int n = 0; n < NOUT; ++n) {
    if (n >= p.CO) break;
#pragma unroll
    for (int i = 0; i < FO_PY; ++i) {
      if (oy + i >= p.HO) continue;
      float *o = p.out + (((size_t)b * p.CO + n) * p.HO + oy + i) * p.WO + ox;
      if (ox + FO_PX <= p.WO && (p.WO & 3) == 0) {
        *reinterpret_cast<float4 *>(o) = make_float4(acc[n][i][0], acc[n][i][1], acc[n][i][2], acc[n][i][3]);
      } else {
#pragma unroll
        for (int j = 0; j < FO_PX; ++j)
          if (ox + j < p.WO) o[j] = acc[n][i][j];
      }
    }
  }
}

static size_t fewout_smem(int CI, int KH, int KW) {
  size_t TH = FO_TILE_H + KH - 1, PITCH = (FO_TILE + KW - 1 + 3) & ~3;
  size_t stages = 2 * FO_ICB * TH * PITCH * 4, red = (size_t)(FO_ICB - 1) * 4 * FO_PY * FO_PX * FO_PATCHES * 4;
  return (((size_t)CI * KH * KW * 4 + 3) & ~(size_t)3) * 4 + (stages > red ? stages : red);
}

template <int KH, int KW>
static int launch_fewout(b200_ctx *ctx, const FewOutCfg &p, int B) {
  size_t smem = fewout_smem(p.CI, KH, KW);
  dim3 grid(p.tiles_x * ceil_div(p.HO, FO_TILE_H), B);
#define B200_FEWOUT(N)                                                                                   \
  do {                                                                                                   \
    B200_CUDA(cudaFuncSetAttribute(conv_fewout_kernel<KH, KW, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                   (int)smem));                                                          \
    conv_fewout_kernel<KH, KW, N><<<grid, FO_THREADS, smem, ctx->stream>>>(p);                           \
  } while (0)
  if (p.CO == 1) B200_FEWOUT(1);
  else if (p.CO == 2) B200_FEWOUT(2);
  else if (p.CO == 3) B200_FEWOUT(3);
  else B200_FEWOUT(4);
#undef B200_FEWOUT
  B200_LAUNCHED();
  return 0;
}

// the flipped, transposed filter copy the dX kernels read; depends on the weights only
int conv_tiled_dx_prep(b200_ctx *ctx, const ConvGeom &g, const float *W, float *scratch) {
  int KK = g.KH * g.KW;
  int Cp = padded_channels(g.C);
  int total = g.OC * KK * Cp;
  conv_prep_wt_dx_kernel<<<ceil_div(total, 256), 256, 0, ctx->stream>>>(W, scratch, g.C, g.OC, Cp,
                                                                       g.KH, g.KW, g.tbl);
  B200_LAUNCHED();
  return 0;
}

// `prep` = 0: `scratch` already holds the filter copy of these weights (conv_tiled_dx_prep)
int conv_tiled_dx(b200_ctx *ctx, const ConvGeom &g, const float *W, const float *dout,
                  float *din, int B, float *scratch, int prep) {
  if (B == 0) return 0;
  int Cp = padded_channels(g.C);
  if (prep) B200_TRY(conv_tiled_dx_prep(ctx, g, W, scratch));
  if (g.C <= 4 && Cp == 4 && fewout_smem(g.OC, g.KH, g.KW) <= ctx->smem_optin) {
    // few input channels: dX is a convolution with few OUTPUT channels
    FewOutCfg f{};
    f.in = dout;
    f.wt = scratch;
    f.out = din;
    f.CI = g.OC;
    f.HI = g.OH;
    f.WI = g.OW;
    f.CO = g.C;
    f.HO = g.HI;
    f.WO = g.WI;
    f.pad_t = g.KH - 1 - g.pad_t;
    f.pad_l = g.KW - 1 - g.pad_l;
    f.tiles_x = ceil_div(g.WI, FO_TILE);
    if (g.KH == 5 && g.KW == 5) return launch_fewout<5, 5>(ctx, f, B);
    if (g.KH == 3 && g.KW == 3) return launch_fewout<3, 3>(ctx, f, B);
  }
  CoreCfg p{};
  p.in = dout;
  p.wt = scratch;
  p.bias = nullptr;
  p.out = din;
  p.B = B;
  p.CI = g.OC;
  p.HI = g.OH;
  p.WI = g.OW;
  p.CO = g.C;
  p.HO = g.HI;
  p.WO = g.WI;
  p.pad_t = g.KH - 1 - g.pad_t;
  p.pad_l = g.KW - 1 - g.pad_l;
  p.act = 0;
  return launch_core(ctx, p, g.KH, g.KW);
}

// ---------------------------------------------------------------------------
// dW / db
// ---------------------------------------------------------------------------

struct DwCfg {
  const float *in;    // [B][C][HI][WI]
  const float *dout;  // [B][OC][OH][OW]
  float *partial;     // [splits][lenW + OC]
  int B, C, HI, WI, OC, OH, OW, pad_t, pad_l, has_bias;
  int OCB, ICT, SL;   // block tile: OCB out channels x ICT in channels, SL strip lanes
  int TH, TWG, TWp;   // band rows, strips per row, staged dY row length
  int THp, PITCHX, PSX;  // staged X rows, row pitch, plane stride
  int OCBp;           // dY tile channel pitch
  int tiles_oc, tiles_ic, splits, bands;
  int x_tile_floats, dy_tile_floats;
  unsigned magic_pitchx, magic_thp, magic_twp, magic_th;
  size_t row_len;     // lenW + OC
};

template <int KH, int KW, int OCT>
__global__ void __launch_bounds__(256) conv_dw_kernel(const DwCfg p) {
  extern __shared__ __align__(16) float smem[];
  const int tid = threadIdx.x;
  const int nthreads = blockDim.x;
  constexpr int KK = KH * KW;

  int bid = blockIdx.x;
  const int toc = bid % p.tiles_oc;
  bid /= p.tiles_oc;
  const int tic = bid % p.tiles_ic;
  const int split = bid / p.tiles_ic;
  const int o0 = toc * p.OCB;
  const int c0 = tic * p.ICT;

  const int stage_floats = p.x_tile_floats + p.dy_tile_floats;
  float *stage0 = smem;
  float *stage1 = smem + stage_floats;

  const int units = p.B * p.bands;

  auto load_unit = [&](int u, float *stage) {
    const int n = u / p.bands;
    const int y0 = (u - n * p.bands) * p.TH;
    float *xt = stage;
    float *dyt = stage + p.x_tile_floats;
    // X tile: [ICT][THp][PITCHX] with plane stride PSX, zero outside the image
    const int xcount = p.ICT * p.THp * p.PITCHX;
    for (int idx = tid; idx < xcount; idx += nthreads) {
      int row = (int)fastdiv((unsigned)idx, p.magic_pitchx);
      int j = idx - row * p.PITCHX;
      int ic = (int)fastdiv((unsigned)row, p.magic_thp);
      int r = row - ic * p.THp;
      int y = y0 + r - p.pad_t;
      int x = j - p.pad_l;
      int c = c0 + ic;
      bool ok = c < p.C && y >= 0 && y < p.HI && x >= 0 && x < p.WI;
      const float *src =
        ok ? p.in + (((size_t)n * p.C + c) * p.HI + y) * (size_t)p.WI + x : p.in;
      cp_async4(xt + ic * p.PSX + r * p.PITCHX + j, src, ok);
    }
    // dY tile, channel-fastest: [TH][TWp][OCBp]
    const int dcount = p.OCB * p.TH * p.TWp;
    for (int idx = tid; idx < dcount; idx += nthreads) {
      int row = (int)fastdiv((unsigned)idx, p.magic_twp);
      int x = idx - row * p.TWp;
      int oc = (int)fastdiv((unsigned)row, p.magic_th);
      int r = row - oc * p.TH;
      int y = y0 + r;
      int o = o0 + oc;
      bool ok = o < p.OC && y < p.OH && x < p.OW;
      const float *src =
        ok ? p.dout + (((size_t)n * p.OC + o) * p.OH + y) * (size_t)p.OW + x : p.dout;
      cp_async4(dyt + (r * p.TWp + x) * p.OCBp + oc, src, ok);
    }
  };

  // thread -> (output channel group, input channel, strip lane)
  const int nocg = p.OCB / OCT;
  const int ocg = tid % nocg;
  int q = tid / nocg;
  const int icl = q % p.ICT;
  const int sl = q / p.ICT;
  const bool do_db = p.has_bias && tic == 0 && icl == 0;

  float acc[OCT][KK];
  float dbacc[OCT];
#pragma unroll
  for (int o = 0; o < OCT; ++o) {
    dbacc[o] = 0.f;
#pragma unroll
    for (int t = 0; t < KK; ++t) acc[o][t] = 0.f;
  }

  const int nstrips = p.TH * p.TWG;
  int u = split;
  if (u < units) {
    load_unit(u, stage0);
  }
  cp_async_commit();
  int it = 0;
  for (; u < units; u += p.splits, ++it) {
    float *cur = (it & 1) ? stage1 : stage0;
    int un = u + p.splits;
    if (un < units) load_unit(un, (it & 1) ? stage0 : stage1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    const float *xt = cur + icl * p.PSX;
    const float *dyt = cur + p.x_tile_floats + ocg * OCT;
    for (int strip = sl; strip < nstrips; strip += p.SL) {
      int y = strip / p.TWG;
      int xg = strip - y * p.TWG;
      float dy[OCT][8];
#pragma unroll
      for (int px = 0; px < 8; ++px) {
        const float4 *dp =
          reinterpret_cast<const float4 *>(dyt + (y * p.TWp + xg * 8 + px) * p.OCBp);
#pragma unroll
        for (int h = 0; h < OCT / 4; ++h) {
          float4 v = dp[h];
          dy[h * 4 + 0][px] = v.x;
          dy[h * 4 + 1][px] = v.y;
          dy[h * 4 + 2][px] = v.z;
          dy[h * 4 + 3][px] = v.w;
        }
      }
#pragma unroll
      for (int wy = 0; wy < KH; ++wy) {
        const float4 *ip = reinterpret_cast<const float4 *>(xt + (y + wy) * p.PITCHX + xg * 8);
        float4 a = ip[0], b = ip[1], c = ip[2];
        float xin[12] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w, c.x, c.y, c.z, c.w};
#pragma unroll
        for (int wx = 0; wx < KW; ++wx)
#pragma unroll
          for (int o = 0; o < OCT; ++o)
#pragma unroll
            for (int px = 0; px < 8; ++px)
              acc[o][wy * KW + wx] = fmaf(dy[o][px], xin[px + wx], acc[o][wy * KW + wx]);
      }
      if (do_db) {
#pragma unroll
        for (int o = 0; o < OCT; ++o)
#pragma unroll
          for (int px = 0; px < 8; ++px) dbacc[o] += dy[o][px];
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- reduce the strip lanes through shared memory (fixed order) ----------
  constexpr int NACC = OCT * KK + OCT;
  if (p.SL > 1) {
    const int ntask = nocg * p.ICT;
    const int task = icl * nocg + ocg;
    float *red = smem;  // [SL][ntask][NACC]
    float *mine = red + ((size_t)sl * ntask + task) * NACC;
#pragma unroll
    for (int o = 0; o < OCT; ++o) {
#pragma unroll
      for (int t = 0; t < KK; ++t) mine[o * KK + t] = acc[o][t];
      mine[OCT * KK + o] = dbacc[o];
    }
    __syncthreads();
    if (sl == 0) {
      for (int l = 1; l < p.SL; ++l) {
        const float *other = red + ((size_t)l * ntask + task) * NACC;
#pragma unroll
        for (int o = 0; o < OCT; ++o) {
#pragma unroll
          for (int t = 0; t < KK; ++t) acc[o][t] += other[o * KK + t];
          dbacc[o] += other[OCT * KK + o];
        }
      }
    }
  }
  if (sl != 0) return;

  // ---- write this block's partial row ----------------------------------------
  float *prow = p.partial + (size_t)split * p.row_len;
  const int c = c0 + icl;
  if (c < p.C) {
#pragma unroll
    for (int o = 0; o < OCT; ++o) {
      int oc = o0 + ocg * OCT + o;
      if (oc >= p.OC) continue;
      float *wp = prow + ((size_t)oc * p.C + c) * KK;
#pragma unroll
      for (int t = 0; t < KK; ++t) wp[t] = acc[o][t];
    }
  }
  if (do_db) {
    size_t lenW = (size_t)p.OC * p.C * KK;
#pragma unroll
    for (int o = 0; o < OCT; ++o) {
      int oc = o0 + ocg * OCT + o;
      if (oc < p.OC) prow[lenW + oc] = dbacc[o];
    }
  }
}

static size_t dw_smem_bytes(const DwCfg &p, int KH, int KW, int OCT) {
  const int NACC = OCT * KH * KW + OCT;
  size_t stage = (size_t)(p.x_tile_floats + p.dy_tile_floats) * 4;
  size_t red = (size_t)p.SL * (p.OCB / OCT) * p.ICT * NACC * 4;
  return 2 * stage > red ? 2 * stage : red;
}

// Fill the tiling for a band height `th` and `splits` batch slices (0 = defaults:
// the tallest band that fits shared memory, one slice per SM).
static void dw_tiling(const b200_ctx *ctx, DwCfg &p, int KH, int KW, int OCT, int th = 0,
                      int splits = 0) {
  int oc_r = round_up(p.OC, OCT);
  p.OCB = oc_r < 32 ? oc_r : 32;
  int nocg = p.OCB / OCT;
  p.ICT = 256 / nocg;
  if (p.ICT > p.C) p.ICT = p.C;
  p.SL = 256 / (nocg * p.ICT);
  if (p.SL < 1) p.SL = 1;
  if (p.SL > 8) p.SL = 8;
  p.TWG = ceil_div(p.OW, 8);
  p.TWp = p.TWG * 8;
  p.PITCHX = round_up(p.TWp + KW - 1, 4);
  p.OCBp = p.OCB + 4;
  // the register tile (100+ accumulators) already limits an SM to one block,
  // so a block may take nearly all shared memory
  size_t limit = ctx->smem_optin;
  auto need = [&](int h) {
    p.TH = h;
    p.THp = h + KH - 1;
    int plane = p.THp * p.PITCHX;
    // plane stride with (PSX/4) odd keeps 8 consecutive channels on distinct banks
    int ps = round_up(plane, 4);
    if (((ps / 4) & 1) == 0) ps += 4;
    p.PSX = ps;
    p.x_tile_floats = p.ICT * p.PSX;
    p.dy_tile_floats = round_up(p.TH * p.TWp * p.OCBp, 4);
    return dw_smem_bytes(p, KH, KW, OCT);
  };
  if (th <= 0 || th > p.OH) th = p.OH;
  while (th > 1 && need(th) > limit) --th;
  need(th);
  p.bands = ceil_div(p.OH, p.TH);
  p.tiles_oc = ceil_div(p.OC, p.OCB);
  p.tiles_ic = ceil_div(p.C, p.ICT);
  int units = p.B * p.bands;
  int tiles = p.tiles_oc * p.tiles_ic;
  if (splits <= 0) splits = ctx->sm_count / tiles;
  if (splits > units) splits = units;
  if (splits < 1) splits = 1;
  p.splits = splits;
  p.magic_pitchx = make_magic((unsigned)p.PITCHX);
  p.magic_thp = make_magic((unsigned)p.THp);
  p.magic_twp = make_magic((unsigned)p.TWp);
  p.magic_th = make_magic((unsigned)p.TH);
}

static void dw_fill(DwCfg &p, const ConvGeom &g, int B) {
  p.B = B;
  p.C = g.C;
  p.HI = g.HI;
  p.WI = g.WI;
  p.OC = g.OC;
  p.OH = g.OH;
  p.OW = g.OW;
  p.pad_t = g.pad_t;
  p.pad_l = g.pad_l;
  p.has_bias = g.has_bias;
  p.row_len = conv_weight_len(g) + g.OC;
}

// Upper bound of the partial rows any choice of (band height, slices) writes.
size_t conv_tiled_dw_scratch(const b200_ctx *ctx, const ConvGeom &g, int B) {
  (void)B;
  size_t row = conv_weight_len(g) + g.OC;
  return (size_t)2 * ctx->sm_count * row;
}

static int dw_launch(b200_ctx *ctx, const DwCfg &p, int KH, int KW, int OCT) {
  size_t smem = dw_smem_bytes(p, KH, KW, OCT);
  B200_REQUIRE(smem <= ctx->smem_optin, "conv dW tile needs %zu bytes of shared memory (limit %zu)",
               smem, ctx->smem_optin);
  int threads = (p.OCB / OCT) * p.ICT * p.SL;
  B200_REQUIRE(threads >= 1 && threads <= 256, "conv dW thread count %d out of range", threads);
  int blocks = p.tiles_oc * p.tiles_ic * p.splits;
  // blocks that own no unit still write zeros, so every partial row is defined
  if (KH == 3) {
    B200_CUDA(cudaFuncSetAttribute(conv_dw_kernel<3, 3, 8>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    conv_dw_kernel<3, 3, 8><<<blocks, threads, smem, ctx->stream>>>(p);
  } else {
    B200_CUDA(cudaFuncSetAttribute(conv_dw_kernel<5, 5, 4>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    conv_dw_kernel<5, 5, 4><<<blocks, threads, smem, ctx->stream>>>(p);
  }
  B200_LAUNCHED();
  return 0;
}

// Band height and slice count regroup the partial sums, so they decide the fp32
// summation order of dW.  By default they are a fixed function of the problem
// and the SM count (tallest band, one slice per SM and tile): the same inputs
// give the same bits in every process.  With B200_AUTOTUNE=1 a few choices are
// timed with CUDA events on first sight (shorter bands give more, finer units
// to balance over the SMs at the price of more halo rows; more slices mean more
// partial rows to merge), the fastest is kept per context and, through
// B200_TUNE_CACHE, across processes; results are then reproducible only for
// one tuning outcome.
int conv_tiled_dw_partials(b200_ctx *ctx, const ConvGeom &g, const float *in, const float *dout,
                           int B, float *scratch, int *splits) {
  B200_REQUIRE(B > 0, "conv_tiled_dw_partials: empty batch");
  B200_REQUIRE(g.OW <= 64, "conv_tiled_dw_partials: output width %d > 64", g.OW);
  const int OCT = g.KH == 3 ? 8 : 4;
  DwCfg base{};
  dw_fill(base, g, B);
  base.in = in;
  base.dout = dout;
  base.partial = scratch;
  char key[160];
  snprintf(key, sizeof(key), "dw %d %d %d %d %d %d %d %d %d %d", g.KH, B, g.C, g.HI, g.WI, g.OC,
           g.OH, g.OW, g.pad_t, g.pad_l);
  int th = 0, sp = 0;
  auto it = ctx->tile_cache.find(key);
  if (it != ctx->tile_cache.end()) {
    // an entry read from a tuning file may come from another GPU or an edited file: the scratch
    // holds 2 * sm_count partial rows, a band cannot be taller than the output
    th = it->second.TH < 0 ? 0 : it->second.TH > g.OH ? g.OH : it->second.TH;
    sp = it->second.NSB < 0 ? 0 : it->second.NSB > 2 * ctx->sm_count ? 2 * ctx->sm_count : it->second.NSB;
  } else {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    B200_CUDA(cudaStreamIsCapturing(ctx->stream, &cap));
    const char *at = getenv("B200_AUTOTUNE");
    bool tune = at && at[0] == '1' && cap == cudaStreamCaptureStatusNone;
    if (tune) {
      DwCfg t0 = base;
      dw_tiling(ctx, t0, g.KH, g.KW, OCT);
      const int th_max = t0.TH;
      const int tiles = t0.tiles_oc * t0.tiles_ic;
      std::vector<std::pair<int, int>> cands;
      for (int h = th_max; h >= 1; h = h > 1 ? (h + 1) / 2 : 0)
        for (int mult = 1; mult <= 2; ++mult) {
          int s = mult * ctx->sm_count / tiles;
          if (s < 1) s = 1;
          bool dup = false;
          for (auto &c : cands) dup = dup || (c.first == h && c.second == s);
          if (!dup) cands.push_back({h, s});
        }
      cudaEvent_t e0, e1;
      B200_CUDA(cudaEventCreate(&e0));
      B200_CUDA(cudaEventCreate(&e1));
      float best_ms = 1e30f;
      for (auto &c : cands) {
        DwCfg t = base;
        dw_tiling(ctx, t, g.KH, g.KW, OCT, c.first, c.second);
        int r = dw_launch(ctx, t, g.KH, g.KW, OCT);
        if (r == 0) {
          B200_CUDA(cudaEventRecord(e0, ctx->stream));
          for (int rep = 0; rep < 3 && r == 0; ++rep) r = dw_launch(ctx, t, g.KH, g.KW, OCT);
          B200_CUDA(cudaEventRecord(e1, ctx->stream));
          B200_CUDA(cudaEventSynchronize(e1));
        }
        if (r != 0) {
          cudaEventDestroy(e0);
          cudaEventDestroy(e1);
          return r;
        }
        float ms = 0.f;
        B200_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        // the rows still have to be merged: charge them at a nominal 3 TB/s
        ms += 3.f * (float)((double)t.splits * t.row_len * 4.0 / 3e12 * 1e3);
        if (ms < best_ms) {
          best_ms = ms;
          th = t.TH;
          sp = t.splits;
        }
      }
      cudaEventDestroy(e0);
      cudaEventDestroy(e1);
      if (getenv("B200_TUNE_LOG"))
        fprintf(stderr, "[b200] %s -> band %d rows, %d slices (%.1f us incl. merge estimate)\n", key,
                th, sp, best_ms * 1000.f / 3.f);
    }
    if (cap == cudaStreamCaptureStatusNone) {
      TileChoice c{};
      c.TH = th;
      c.NSB = sp;
      ctx_remember_tile(ctx, key, c);
    }
  }
  DwCfg p = base;
  dw_tiling(ctx, p, g.KH, g.KW, OCT, th, sp);
  B200_TRY(dw_launch(ctx, p, g.KH, g.KW, OCT));
  *splits = p.splits;
  return 0;
}

// ---------------------------------------------------------------------------
// merging partial rows
// ---------------------------------------------------------------------------

__global__ void merge_rows_kernel(const float *__restrict__ src, int rows, size_t stride,
                                  float *__restrict__ dst, size_t len, int accumulate,
                                  const uint8_t *__restrict__ tbl, int C, int OC, int KK,
                                  size_t lenW, int in_order = 0) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < len; i += step) {
    // four interleaved running sums (rows r, r+4, ...) combined at the end: a
    // fixed order, with four independent load/add chains in flight
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    int r = 0;
    if (in_order) {  // rows added one after the other, as edge::merge_grads does
      s0 = src[i];
      for (r = 1; r < rows; ++r) s0 += src[(size_t)r * stride + i];
    }
    for (; r + 4 <= rows; r += 4) {
      s0 += src[(size_t)(r + 0) * stride + i];
      s1 += src[(size_t)(r + 1) * stride + i];
      s2 += src[(size_t)(r + 2) * stride + i];
      s3 += src[(size_t)(r + 3) * stride + i];
    }
    for (; r < rows; ++r) s0 += src[(size_t)r * stride + i];
    float s = (s0 + s1) + (s2 + s3);
    if (tbl && i < lenW) {
      // unconnected (o, inc) pairs get no gradient (conv2d_op_internal.h:132)
      size_t pair = i / KK;
      int inc = (int)(pair % C);
      int o = (int)(pair / C);
      if (!tbl[inc * OC + o]) s = 0.f;
    }
    dst[i] = accumulate ? dst[i] + s : s;
  }
}

// Same sum for many partial rows: 8 row lanes per output element (lane k adds rows k, k+8, ...
// in order, two chains in flight), combined in lane order -- a fixed order, 8x the loads in flight.
__global__ void __launch_bounds__(256)
  merge_rows_lanes_kernel(const float *__restrict__ src, int rows, size_t stride, float *__restrict__ dst,
                          size_t len, int accumulate, const uint8_t *__restrict__ tbl, int C, int OC, int KK,
                          size_t lenW) {
  __shared__ float part[8][33];
  const int tx = threadIdx.x, ty = threadIdx.y;
  for (size_t base = (size_t)blockIdx.x * 32; base < len; base += (size_t)gridDim.x * 32) {
    const size_t i = base + tx;
    float s0 = 0.f, s1 = 0.f;
    if (i < len) {
      int r = ty;
      for (; r + 8 < rows; r += 16) {
        s0 += src[(size_t)r * stride + i];
        s1 += src[(size_t)(r + 8) * stride + i];
      }
      if (r < rows) s0 += src[(size_t)r * stride + i];
    }
    part[ty][tx] = s0 + s1;
    __syncthreads();
    if (ty == 0 && i < len) {
      float s = part[0][tx];
#pragma unroll
      for (int k = 1; k < 8; ++k) s += part[k][tx];
      if (tbl && i < lenW) {
        size_t pair = i / KK;
        int inc = (int)(pair % C);
        int o = (int)(pair / C);
        if (!tbl[inc * OC + o]) s = 0.f;
      }
      dst[i] = accumulate ? dst[i] + s : s;
    }
    __syncthreads();
  }
}

int merge_rows(b200_ctx *ctx, const float *src, int rows, size_t stride, float *dst, size_t len,
               int accumulate, const ConvGeom *mask, int in_order) {
  if (len == 0) return 0;
  B200_REQUIRE(rows >= 1, "merge_rows: rows must be >= 1");
  size_t blocks = ceil_div_sz(len, 256);
  size_t cap = (size_t)ctx->sm_count * 8;
  if (blocks > cap) blocks = cap;
  const uint8_t *tbl = mask ? mask->tbl : nullptr;
  if (!in_order && rows >= 16) {
    size_t lb = ceil_div_sz(len, 32);
    if (lb > cap * 4) lb = cap * 4;
    merge_rows_lanes_kernel<<<(unsigned)lb, dim3(32, 8), 0, ctx->stream>>>(
      src, rows, stride, dst, len, accumulate, tbl, mask ? mask->C : 1, mask ? mask->OC : 1,
      mask ? mask->KH * mask->KW : 1, mask ? conv_weight_len(*mask) : 0);
    B200_LAUNCHED();
    return 0;
  }
  merge_rows_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(
    src, rows, stride, dst, len, accumulate, tbl, mask ? mask->C : 1, mask ? mask->OC : 1,
    mask ? mask->KH * mask->KW : 1, mask ? conv_weight_len(*mask) : 0, in_order);
  B200_LAUNCHED();
  return 0;
}

// ---------------------------------------------------------------------------
// weight gradient for callers that must not allocate
// ---------------------------------------------------------------------------

// Fixed scratch for b200_conv2d_dw_noalloc: 4 Mi floats (16 MiB) of partial-sum
// rows.  It is part of the library image, so every GPU that loads the library
// holds it from load to exit whether or not the entry point is ever called.
constexpr size_t kNoAllocScratchFloats = (size_t)4 << 20;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];

constexpr int kNoAllocMaxDevices = 64;
struct NoAllocDevice {
  bool ready = false;
  float *scratch = nullptr;  // device address of g_noalloc_scratch on this GPU
  int sm_count = 0;
  size_t smem_optin = 0;
};
static NoAllocDevice g_noalloc_dev[kNoAllocMaxDevices];
static std::atomic_flag g_noalloc_lock = ATOMIC_FLAG_INIT;

// One-time set-up for the CURRENT device.  `g_noalloc_scratch` used as a value
// in host code is only the host-side shadow of the symbol; the address a kernel
// can dereference has to be asked for with cudaGetSymbolAddress.
static int noalloc_setup(int dev, NoAllocDevice **out) {
  B200_REQUIRE(dev >= 0 && dev < kNoAllocMaxDevices, "conv2d_dw_noalloc: device %d not supported",
               dev);
  while (g_noalloc_lock.test_and_set(std::memory_order_acquire)) {
  }
  NoAllocDevice &nd = g_noalloc_dev[dev];
  int rc = 0;
  if (!nd.ready) {
    void *addr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&addr, g_noalloc_scratch);
    int sms = 0, smem = 0;
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess)
      e = cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (e != cudaSuccess || addr == nullptr) {
      set_error("conv2d_dw_noalloc: set-up on device %d failed: %s", dev, cudaGetErrorString(e));
      rc = 1;
    } else {
      nd.scratch = static_cast<float *>(addr);
      nd.sm_count = sms;
      nd.smem_optin = (size_t)smem;
      nd.ready = true;
    }
  }
  g_noalloc_lock.clear(std::memory_order_release);
  *out = &nd;
  return rc;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_conv2d_dw_noalloc(void *stream, const b200_conv_desc *d, const float *in,
                                      const float *dout, float *dW, float *db, int accumulate,
                                      int batch) {
  B200_REQUIRE(d != nullptr, "conv2d_dw_noalloc: descriptor is NULL");
  B200_REQUIRE(batch >= 0, "conv2d_dw_noalloc: negative batch");
  B200_REQUIRE(d->tbl == nullptr,
               "conv2d_dw_noalloc: connection tables are not supported (they need a device copy)");
  int dev = -1;
  B200_CUDA(cudaGetDevice(&dev));
  NoAllocDevice *nd = nullptr;
  B200_TRY(noalloc_setup(dev, &nd));
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  // geometry through the same routine as every other entry point; with no
  // table it touches nothing but the descriptor
  b200_ctx shell;
  shell.device = dev;
  shell.sm_count = nd->sm_count;
  shell.smem_optin = nd->smem_optin;
  shell.stream = st;
  ConvGeom g;
  B200_TRY(conv_geom_from_desc(&shell, d, &g));
  B200_REQUIRE(dW && (db || !g.has_bias), "conv2d_dw_noalloc: NULL gradient buffer");
  const size_t lenW = conv_weight_len(g);
  if (batch == 0) {
    if (!accumulate) {
      B200_CUDA(cudaMemsetAsync(dW, 0, lenW * sizeof(float), st));
      if (g.has_bias) B200_CUDA(cudaMemsetAsync(db, 0, g.OC * sizeof(float), st));
    }
    return 0;
  }
  B200_REQUIRE(in && dout, "conv2d_dw_noalloc: NULL input buffer");
  B200_REQUIRE(conv_tiled_ok(g) && g.OW <= 64,
               "conv2d_dw_noalloc: only stride 1, dilation 1, 3x3 or 5x5 windows and output width "
               "<= 64 are supported");

  DwCfg p{};
  dw_fill(p, g, batch);
  const int OCT = g.KH == 3 ? 8 : 4;
  dw_tiling(&shell, p, g.KH, g.KW, OCT);
  // the partial rows must fit the fixed array: fewer, longer batch slices if needed
  const size_t max_rows = kNoAllocScratchFloats / p.row_len;
  B200_REQUIRE(max_rows >= 1,
               "conv2d_dw_noalloc: one partial row needs %zu floats but the fixed scratch holds %zu; "
               "use b200_conv2d_bwd for filters this large",
               p.row_len, kNoAllocScratchFloats);
  if ((size_t)p.splits > max_rows) p.splits = (int)max_rows;
  p.in = in;
  p.dout = dout;
  p.partial = nd->scratch;
  size_t smem = dw_smem_bytes(p, g.KH, g.KW, OCT);
  B200_REQUIRE(smem <= nd->smem_optin,
               "conv2d_dw_noalloc: tile needs %zu bytes of shared memory (limit %zu)", smem,
               nd->smem_optin);
  int threads = (p.OCB / OCT) * p.ICT * p.SL;
  B200_REQUIRE(threads >= 1 && threads <= 256, "conv2d_dw_noalloc: thread count %d out of range", threads);
  int blocks = p.tiles_oc * p.tiles_ic * p.splits;
  // Every block overwrites its whole tile of its row, so nothing left in the
  // array by an earlier call is ever read: no clearing is needed.
  if (g.KH == 3) {
    B200_CUDA(cudaFuncSetAttribute(conv_dw_kernel<3, 3, 8>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    conv_dw_kernel<3, 3, 8><<<blocks, threads, smem, st>>>(p);
  } else {
    B200_CUDA(cudaFuncSetAttribute(conv_dw_kernel<5, 5, 4>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    conv_dw_kernel<5, 5, 4><<<blocks, threads, smem, st>>>(p);
  }
  B200_LAUNCHED();
  const int mblocks = (int)((lenW + 255) / 256 < (size_t)nd->sm_count * 8 ? (lenW + 255) / 256
                                                                          : (size_t)nd->sm_count * 8);
  merge_rows_kernel<<<mblocks, 256, 0, st>>>(nd->scratch, p.splits, p.row_len, dW, lenW, accumulate,
                                             nullptr, 1, 1, 1, 0);
  B200_LAUNCHED();
  if (g.has_bias) {
    merge_rows_kernel<<<(g.OC + 255) / 256, 256, 0, st>>>(nd->scratch + lenW, p.splits, p.row_len,
                                                         db, (size_t)g.OC, accumulate, nullptr, 1, 1,
                                                         1, 0);
    B200_LAUNCHED();
  }
  return 0;
}
