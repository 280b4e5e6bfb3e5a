// Forward convolution of layers with few input channels on the 5th-generation tensor cores
// (tcgen05), fp32-accurate through the 3xTF32 split.  Replaces the loops of
// kernels::conv2d_op_internal (tiny_dnn/core/kernels/conv2d_op_internal.h:13-74) for the first layer
// of a network (3 x 5 x 5 = 75 taps), where a 32-channel slab per tap would be almost all padding.
//
// GEMM form: D[pixel][o] = sum_k A[pixel][k] * W[o][k], k = (c*KH + ky)*KW + kx -- the reference's
// own weight order, so the filter needs no reordering, only the hi / lo split.
//   M = 128 pixels: 4 output rows x 32 columns of one image
//   N = out channels (padded to 16); hi and lo rows of the filter are neighbours in shared memory,
//       so A_hi x [W_hi | W_lo] is one instruction of width 2N; A_lo x W_hi is the second
//   K = taps in steps of 8; the filter K-major with the 128-byte swizzle, 32 taps per row
// A (the im2col rows of the tile) exists only in tensor memory: one TMA load brings the raw
// (4 + KH - 1) input rows of every channel (zero filled outside the image) into shared memory,
// sixteen converter warps gather each pixel's taps from them, split them and write the hi / lo
// values into the pixel's TMEM lane (tcgen05.st), from where the MMAs take their A operand -- the
// im2col matrix never passes through shared memory, whose bandwidth bounded the first form of this
// kernel.  The filter is split once per CTA and stays resident in shared memory.
// Warp roles: 0-7 epilogue (one TMEM lane = one pixel per thread, two warps share a lane quadrant and
// split the channels), 8-23 converters, 24 TMA producer + TMEM allocation, 25 MMA issuer.  Accumulators and A buffers are double buffered in tensor memory.
// Every load is CTA-local; every wait is bounded and a timeout sets the context's error word,
// frees tensor memory and returns.
#include <stdio.h>
#include <stdlib.h>

#include <vector>

#include "tc_utils.cuh"

namespace b200 {

namespace {

constexpr int TFS_ROWS = 4;          // output rows per step
constexpr int TFS_PX = 32;           // output columns per step
constexpr int TFS_CONV_WARPS = 16;         // four warps per tile row: each takes every fourth quad of taps
constexpr int TFS_EPI_WARPS = 8;           // two per TMEM lane quadrant: each takes every other 16 channels
constexpr int TFS_THREADS = (TFS_EPI_WARPS + TFS_CONV_WARPS + 2) * 32;
constexpr int TFS_STAGES = 4;        // raw input tiles in flight
constexpr int TFS_MAX_KB = 3;        // 128-byte K blocks (32 taps each): 96 taps at most
constexpr size_t TFS_MIN_SMEM = 120 * 1024;  // ask for more than half an SM's shared memory: the kernel
                                             // takes all 512 TMEM columns, a second CTA would only wait

struct TcFwdSmallArgs {
  const float *W, *bias;
  const uint8_t *tbl;
  float *out;
  int *err;
  int C, OC, OCp, KH, KW, pad_t, pad_l;
  int OH, OW, nxb, nyb;
  int Kreal;    // C * KH * KW
  int ksteps;   // MMA steps of 8 taps
  int nkb;      // K blocks of 32 taps
  int bw, rows; // raw tile: floats per row, rows per channel
  int nsteps, nblocks;
  int act;
  int tmem_cols;
  long long *dbg;  // optional [blocks][12] cycle counters (B200_TC_TIMING=1), else nullptr
};

// four consecutive TMEM columns of the warp's 32 lanes
__device__ __forceinline__ void tmem_st4(uint32_t taddr, float a, float b, float c, float d) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(taddr),
               "r"(__float_as_uint(a)), "r"(__float_as_uint(b)), "r"(__float_as_uint(c)), "r"(__float_as_uint(d))
               : "memory");
}

// tile coordinates of consecutive steps without a division per step
struct StepPos {
  int xb, yb, b;
  __device__ __forceinline__ void init(int s, int nxb, int nyb) {
    xb = s % nxb;
    const int t = s / nxb;
    yb = t % nyb;
    b = t / nyb;
  }
  __device__ __forceinline__ void next(int nxb, int nyb) {
    if (++xb == nxb) {
      xb = 0;
      if (++yb == nyb) {
        yb = 0;
        ++b;
      }
    }
  }
};

// 16 channels of one pixel: hi + lo parts, bias, activation, one store per channel plane
template <int ACT>
__device__ __forceinline__ void store16(float *dst, size_t plane, int n, const uint32_t *v, const uint32_t *w,
                                        const float *bv) {
#pragma unroll
  for (int q = 0; q < 16; ++q) {
    float r = (__uint_as_float(v[q]) + __uint_as_float(w[q])) + bv[q];
    if (ACT == B200_ACT_RELU) r = fmaxf(0.f, r);
    if (ACT == B200_ACT_TANH) r = tanhf(r);
    if (q < n) dst[(size_t)q * plane] = r;
  }
}

__global__ void __launch_bounds__(TFS_THREADS, 1)
  conv_fwd_small_tc_kernel(const __grid_constant__ CUtensorMap x_map, const TcFwdSmallArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t WT = 2u * (uint32_t)a.OCp * 128u;               // one K block of the filter: hi rows, lo rows
  const uint32_t XBYTES = (uint32_t)(a.C * a.rows * a.bw * 4);
  const uint32_t XB = (XBYTES + 1023u) & ~1023u;
  const uint32_t STAGE = XB;                                     // one raw input tile
  uint8_t *wt = smem;                                            // [nkb][2*OCp][128 B]
  uint8_t *stage0 = smem + (size_t)a.nkb * WT;
  int *koff = reinterpret_cast<int *>(stage0 + (size_t)TFS_STAGES * STAGE);  // [ksteps*8]
  uint64_t *tma_full = reinterpret_cast<uint64_t *>(koff + TFS_MAX_KB * 32);
  uint64_t *raw_empty = tma_full + TFS_STAGES;
  uint64_t *a_full = raw_empty + TFS_STAGES;   // [2] A buffers in tensor memory
  uint64_t *a_empty = a_full + 2;
  uint64_t *acc_full = a_empty + 2;
  uint64_t *acc_empty = acc_full + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
  float *bias_s = reinterpret_cast<float *>(tmem_slot + 4);      // [OCp], zeros without a bias

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int s_begin = (int)((long long)blockIdx.x * a.nsteps / a.nblocks);
  const int s_end = (int)((long long)(blockIdx.x + 1) * a.nsteps / a.nblocks);
  constexpr int W_TMA = TFS_EPI_WARPS + TFS_CONV_WARPS, W_MMA = W_TMA + 1;
  if (tid == 0) {
    for (int s = 0; s < TFS_STAGES; ++s) {
      mbar_init(&tma_full[s], 1);
      mbar_init(&raw_empty[s], TFS_CONV_WARPS);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&a_full[s], TFS_CONV_WARPS);
      mbar_init(&a_empty[s], 1);
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], TFS_EPI_WARPS);
    }
    mbar_fence_init();
  }
  for (int o = tid; o < a.OCp; o += TFS_THREADS) bias_s[o] = (a.bias && o < a.OC) ? a.bias[o] : 0.f;
  if (warp == W_TMA) tmem_alloc(tmem_slot, (uint32_t)a.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // tensor memory columns: two accumulators of 2*OCp, then two A buffers of (hi | lo) x Kp
  const uint32_t Kp = (uint32_t)a.ksteps * 8u, tmem_a = tmem_base + 4u * (uint32_t)a.OCp;
  bool failed = false;

  if (warp == W_TMA && lane == 0) {
    // ---- TMA producer: the raw input rows of each step -------------------------------------------
    long long w = 0, t0 = tc_clock(), tq;
    StepPos pos;
    pos.init(s_begin, a.nxb, a.nyb);
    for (int s = s_begin; s < s_end; ++s, pos.next(a.nxb, a.nyb)) {
      const uint32_t i = s - s_begin, st = i % TFS_STAGES, use = i / TFS_STAGES;
      tq = tc_clock();
      if (use > 0 && !mbar_wait_bounded(&raw_empty[st], (use - 1) & 1)) {
        failed = true;
        break;
      }
      w += tc_clock() - tq;
      if (a.dbg && s == s_end - 1) {
        a.dbg[blockIdx.x * 12 + 0] = tc_clock() - t0;
        a.dbg[blockIdx.x * 12 + 1] = w;
      }
      const int xs = (pos.xb * TFS_PX - a.pad_l) & ~3;  // aligned start column (floor to a multiple of 4)
      mbar_expect_tx(&tma_full[st], XBYTES);
      tma_load_4d(stage0 + (size_t)st * STAGE, &x_map, xs, pos.yb * TFS_ROWS - a.pad_t, 0, pos.b,
                  &tma_full[st]);
    }
  } else if (warp == W_MMA && lane == 0) {
    // ---- MMA issuer ------------------------------------------------------------------------------
    const uint32_t idesc1 = umma_idesc_tf32(128, a.OCp), idesc2 = umma_idesc_tf32(128, 2 * a.OCp);
    const uint64_t b0 = umma_desc(smem_u32(wt), 16, 1024, 2);
    long long w = 0, w2 = 0, t0 = tc_clock(), tq;
    for (int s = s_begin; s < s_end; ++s) {
      const uint32_t i = s - s_begin, ab = i & 1;
      tq = tc_clock();
      if (!mbar_wait_bounded(&a_full[ab], (i >> 1) & 1)) {
        failed = true;
        break;
      }
      w += tc_clock() - tq;
      tq = tc_clock();
      if (i >= 2 && !mbar_wait_bounded(&acc_empty[ab], ((i >> 1) - 1) & 1)) {
        failed = true;
        break;
      }
      w2 += tc_clock() - tq;
      if (a.dbg && s == s_end - 1) {
        a.dbg[blockIdx.x * 12 + 2] = tc_clock() - t0;
        a.dbg[blockIdx.x * 12 + 3] = w;
        a.dbg[blockIdx.x * 12 + 4] = w2;
      }
      tc_fence_after();
      const uint32_t acc = tmem_base + ab * 2u * (uint32_t)a.OCp;
      const uint32_t ahi = tmem_a + ab * 2u * Kp, alo = ahi + Kp;
      // the descriptor of K step ks is the first one plus its byte offset / 16 in the address field
#pragma unroll 4
      for (int ks = 0; ks < a.ksteps; ++ks) {
        const uint64_t b = b0 + (uint64_t)(((uint32_t)(ks >> 2) * WT + (uint32_t)(ks & 3) * 32u) >> 4);
        umma_tf32_ta(acc, ahi + ks * 8, b, idesc2, ks != 0);
        umma_tf32_ta(acc, alo + ks * 8, b, idesc1, 1);
      }
      umma_commit(&a_empty[ab]);
      umma_commit(&acc_full[ab]);
    }
  } else if (warp >= TFS_EPI_WARPS && warp < W_TMA) {
    // ---- converters ------------------------------------------------------------------------------
    const int ct = tid - TFS_EPI_WARPS * 32;
    constexpr int NCT = TFS_CONV_WARPS * 32;
    const int KK = a.KH * a.KW, nk = a.ksteps * 8;
    // tap -> offset in the raw tile (-1: padding tap)
    for (int k = ct; k < nk; k += NCT) {
      int off = -1;
      if (k < a.Kreal) {
        const int c = k / KK, r = k - c * KK, ky = r / a.KW, kx = r - ky * a.KW;
        off = (c * a.rows + ky) * a.bw + kx;
      }
      koff[k] = off;
    }
    // the filter: W[o][k] split into hi rows and lo rows of every K block
    for (int idx = ct; idx < a.OCp * a.nkb * 32; idx += NCT) {
      const int o = idx / (a.nkb * 32), k = idx - o * (a.nkb * 32);
      float v = 0.f;
      if (o < a.OC && k < a.Kreal && (!a.tbl || a.tbl[(k / KK) * a.OC + o])) v = a.W[(size_t)o * a.Kreal + k];
      float h, l;
      split_tf32_rn(v, h, l);
      const uint32_t kb = k >> 5, kk = k & 31;
      const uint32_t rh = o, rl = a.OCp + o;
      uint8_t *tile = wt + (size_t)kb * WT;
      *reinterpret_cast<float *>(tile + rh * 128u + (((kk >> 2) ^ (rh & 7)) << 4) + (kk & 3) * 4u) = h;
      *reinterpret_cast<float *>(tile + rl * 128u + (((kk >> 2) ^ (rl & 7)) << 4) + (kk & 3) * 4u) = l;
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    asm volatile("bar.sync 1, %0;\n" ::"n"(NCT) : "memory");
    const int p = ct & 127, part = ct >> 7;                // pixel of the tile, which share of the tap quads
    const int pixoff = (p >> 5) * a.bw + (p & 31);
    const uint32_t lane_base = (uint32_t)(warp & 3) << 21;   // this warp's TMEM lanes: 32 * (warp % 4), in bits 16..
    const int nkq = a.ksteps * 2, nfull = a.Kreal >> 2;
    constexpr int NPART = TFS_CONV_WARPS / 4, NQ = (TFS_MAX_KB * 8 + NPART - 1) / NPART;
    int4 ko[NQ];  // raw-tile offsets of the tap quads this thread converts, the same in every step
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
      const int kq = part + j * NPART;
      ko[j] = kq < nkq ? *reinterpret_cast<const int4 *>(koff + kq * 4) : make_int4(-1, -1, -1, -1);
    }
    long long w = 0, w2 = 0, t0 = tc_clock(), tq;
    int xb = s_begin % a.nxb;
    for (int s = s_begin; s < s_end; ++s, xb = (xb + 1 == a.nxb) ? 0 : xb + 1) {
      const uint32_t i = s - s_begin, st = i % TFS_STAGES, use = i / TFS_STAGES, ab = i & 1;
      tq = tc_clock();
      if (!mbar_wait_bounded(&tma_full[st], use & 1)) {
        failed = true;
        break;
      }
      w += tc_clock() - tq;
      tq = tc_clock();
      if (i >= 2 && !mbar_wait_bounded(&a_empty[ab], ((i >> 1) - 1) & 1)) {
        failed = true;
        break;
      }
      w2 += tc_clock() - tq;
      tc_fence_after();
      uint8_t *sp = stage0 + (size_t)st * STAGE;
      const int x0 = xb * TFS_PX;
      const int d = (x0 - a.pad_l) - ((x0 - a.pad_l) & ~3);
      const float *xr = reinterpret_cast<const float *>(sp) + d + pixoff;
      const uint32_t thi = tmem_a + ab * 2u * Kp + lane_base, tlo = thi + Kp;
#pragma unroll
      for (int j = 0; j < NQ; ++j) {
        const int kq = part + j * NPART;
        if (kq < nkq) {
          const int4 o4 = ko[j];
          float h[4], l[4];
          if (kq < nfull) {  // all four taps exist (uniform over the warp)
            split_tf32_rn(xr[o4.x], h[0], l[0]);
            split_tf32_rn(xr[o4.y], h[1], l[1]);
            split_tf32_rn(xr[o4.z], h[2], l[2]);
            split_tf32_rn(xr[o4.w], h[3], l[3]);
          } else {
            split_tf32_rn(o4.x >= 0 ? xr[o4.x] : 0.f, h[0], l[0]);
            split_tf32_rn(o4.y >= 0 ? xr[o4.y] : 0.f, h[1], l[1]);
            split_tf32_rn(o4.z >= 0 ? xr[o4.z] : 0.f, h[2], l[2]);
            split_tf32_rn(o4.w >= 0 ? xr[o4.w] : 0.f, h[3], l[3]);
          }
          tmem_st4(thi + (uint32_t)kq * 4u, h[0], h[1], h[2], h[3]);
          tmem_st4(tlo + (uint32_t)kq * 4u, l[0], l[1], l[2], l[3]);
        }
      }
      // the stores have landed in tensor memory: hand the A buffer over, give the raw tile back
      asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&a_full[ab]);
        mbar_arrive(&raw_empty[st]);
      }
    }
    if (a.dbg && ct == 0) {
      a.dbg[blockIdx.x * 12 + 5] = tc_clock() - t0;
      a.dbg[blockIdx.x * 12 + 6] = w;
      a.dbg[blockIdx.x * 12 + 7] = w2;
    }
  } else if (warp < TFS_EPI_WARPS) {
    // ---- epilogue: hi + lo parts, bias, activation, store ------------------------------------------
    const size_t plane = (size_t)a.OH * a.OW;
    long long w = 0, wl = 0, t0 = tc_clock(), tq;
    StepPos pos;
    pos.init(s_begin, a.nxb, a.nyb);
    for (int s = s_begin; s < s_end; ++s, pos.next(a.nxb, a.nyb)) {
      const uint32_t i = s - s_begin, ab = i & 1;
      tq = tc_clock();
      if (!mbar_wait_bounded(&acc_full[ab], (i >> 1) & 1)) {
        failed = true;
        break;
      }
      w += tc_clock() - tq;
      if (a.dbg && tid == 0 && s == s_end - 1) {
        a.dbg[blockIdx.x * 12 + 8] = tc_clock() - t0;
        a.dbg[blockIdx.x * 12 + 9] = w;
      }
      tc_fence_after();
      const int b = pos.b;
      const int y = pos.yb * TFS_ROWS + (warp & 3), x = pos.xb * TFS_PX + lane;
      const bool inside = y < a.OH && x < a.OW;
      float *obase = a.out + (size_t)b * a.OC * plane + (size_t)y * a.OW + x;
      const uint32_t tacc = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + ab * 2u * (uint32_t)a.OCp;
      const int cfirst = (warp >> 2) * 16;
      if (cfirst >= a.OCp) {  // no channels for this warp: it only keeps step with the barrier
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[ab]);
      }
      for (int c0 = cfirst; c0 < a.OCp; c0 += 32) {
        uint32_t v[16], w[16];
        tq = tc_clock();
        tmem_ld16_nowait(tacc + (uint32_t)c0, v);
        tmem_ld16_nowait(tacc + (uint32_t)(a.OCp + c0), w);
        tmem_ld_wait();
        if (c0 + 32 >= a.OCp) {  // the buffer is read: the next step but one may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[ab]);
        }
        wl += tc_clock() - tq;
        float bv[16];
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<float4 *>(bv + 4 * q) = *reinterpret_cast<const float4 *>(bias_s + c0 + 4 * q);
        if (inside) {  // one branch on the activation per 16 channels, not per element
          float *dst = obase + (size_t)c0 * plane;
          const int n = a.OC - c0;
          if (a.act == B200_ACT_RELU)
            store16<B200_ACT_RELU>(dst, plane, n, v, w, bv);
          else if (a.act == B200_ACT_TANH)
            store16<B200_ACT_TANH>(dst, plane, n, v, w, bv);
          else
            store16<B200_ACT_NONE>(dst, plane, n, v, w, bv);
        }
      }
      if (a.dbg && tid == 0 && s == s_end - 1) a.dbg[blockIdx.x * 12 + 10] = wl;
    }
  }
  if (failed && a.err) atomicExch(a.err, 6);
  tc_fence_before();
  __syncthreads();
  if (warp == W_TMA) tmem_dealloc(tmem_base, (uint32_t)a.tmem_cols);
}

int fwd_small_bw(const ConvGeom &g) { return (TFS_PX + g.KW - 1 + 3 + 3) & ~3; }

size_t fwd_small_smem(const ConvGeom &g, int OCp) {
  const int K = g.C * g.KH * g.KW, nkb = (K + 31) / 32;
  const size_t XB = ((size_t)g.C * (TFS_ROWS + g.KH - 1) * fwd_small_bw(g) * 4 + 1023) & ~(size_t)1023;
  const size_t need = 1024 + (size_t)nkb * 2 * OCp * 128 + TFS_STAGES * XB + TFS_MAX_KB * 32 * 4 +
                      (2 * TFS_STAGES + 8) * 8 + 16 + (size_t)OCp * 4 + 64;
  return need > TFS_MIN_SMEM ? need : TFS_MIN_SMEM;
}

// tensor memory columns: two accumulators (hi | lo parts) and two A buffers (hi | lo)
int fwd_small_tmem(const ConvGeom &g, int OCp) {
  const int Kp = (g.C * g.KH * g.KW + 7) / 8 * 8;
  return 4 * OCp + 4 * Kp;
}

int pow2_cols(int v) {
  int p = 32;
  while (p < v) p <<= 1;
  return p;
}

}  // namespace

// true when the im2col tensor-core forward kernel applies
bool conv_fwd_small_ok(const b200_ctx *ctx, const ConvGeom &g) {
  if (g.SH != 1 || g.SW != 1 || g.DH != 1 || g.DW != 1) return false;
  const int K = g.C * g.KH * g.KW;
  if (K > TFS_MAX_KB * 32 || g.OC > 64) return false;
  if (g.WI & 3) return false;                               // TMA strides are multiples of 16 bytes
  if (((size_t)g.HI * g.WI) & 3) return false;
  if (g.pad_t < 0 || g.pad_l < 0) return false;
  const int OCp = (g.OC + 15) / 16 * 16;
  if (fwd_small_tmem(g, OCp) > 512) return false;
  return fwd_small_smem(g, OCp) <= (size_t)ctx->smem_optin;
}

// forward (+ bias, activation) from the CHW input; no scratch
int conv_fwd_small(b200_ctx *ctx, const ConvGeom &g, const float *in, const float *W, const float *bias, float *out,
                   int B, int act) {
  if (B == 0) return 0;
  const int OCp = (g.OC + 15) / 16 * 16, bw = fwd_small_bw(g);
  EncodeTiledFn fn = encode_fn();
  B200_REQUIRE(fn != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
  TcFwdSmallArgs a;
  a.rows = TFS_ROWS + g.KH - 1;
  CUtensorMap x_map;
  {
    cuuint64_t dims[4] = {(cuuint64_t)g.WI, (cuuint64_t)g.HI, (cuuint64_t)g.C, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)g.WI * 4, (cuuint64_t)g.HI * g.WI * 4, (cuuint64_t)g.C * g.HI * g.WI * 4};
    cuuint32_t box[4] = {(cuuint32_t)bw, (cuuint32_t)a.rows, (cuuint32_t)g.C, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(&x_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(in), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed (%d) for the input rows", (int)r);
  }
  a.W = W;
  a.bias = g.has_bias ? bias : nullptr;
  a.tbl = g.tbl;
  a.out = out;
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
  a.nxb = ceil_div(g.OW, TFS_PX);
  a.nyb = ceil_div(g.OH, TFS_ROWS);
  a.Kreal = g.C * g.KH * g.KW;
  a.ksteps = (a.Kreal + 7) / 8;
  a.nkb = (a.Kreal + 31) / 32;
  a.bw = bw;
  a.nsteps = B * a.nyb * a.nxb;
  a.nblocks = a.nsteps < ctx->sm_count ? a.nsteps : ctx->sm_count;
  a.act = act;
  a.tmem_cols = pow2_cols(fwd_small_tmem(g, OCp));
  const size_t smem = fwd_small_smem(g, OCp);
  B200_REQUIRE(smem <= (size_t)ctx->smem_optin, "conv_fwd_small: the tiles do not fit shared memory");
  B200_CUDA(cudaFuncSetAttribute(conv_fwd_small_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  a.dbg = nullptr;
#ifdef B200_TC_TIMING
  static const bool timing = getenv("B200_TC_TIMING") != nullptr;
  if (timing) B200_CUDA(cudaMalloc(&a.dbg, (size_t)a.nblocks * 12 * sizeof(long long)));
#endif
  conv_fwd_small_tc_kernel<<<a.nblocks, TFS_THREADS, smem, ctx->stream>>>(x_map, a);
  B200_LAUNCHED();
#ifdef B200_TC_TIMING
  if (timing) {  // diagnostic: cycles of the four roles and of their waits, averaged over blocks
    std::vector<long long> h((size_t)a.nblocks * 12);
    B200_CUDA(cudaStreamSynchronize(ctx->stream));
    B200_CUDA(cudaMemcpy(h.data(), a.dbg, h.size() * sizeof(long long), cudaMemcpyDeviceToHost));
    B200_CUDA(cudaFree(a.dbg));
    double s[12] = {0};
    for (int i = 0; i < a.nblocks; ++i)
      for (int k = 0; k < 12; ++k) s[k] += (double)h[(size_t)i * 12 + k] / a.nblocks;
    fprintf(stderr,
            "[tc-timing] fwd small: steps/block %.1f: producer %.0f clk (wait raw %.0f), mma %.0f (wait operands %.0f, "
            "accumulator %.0f), converter %.0f (wait tma %.0f, tile free %.0f), epilogue %.0f (wait %.0f, tmem loads %.0f)\n",
            (double)a.nsteps / a.nblocks, s[0], s[1], s[2], s[3], s[4], s[5], s[6], s[7], s[8], s[9], s[10]);
  }
#endif
  return 0;
}

}  // namespace b200
