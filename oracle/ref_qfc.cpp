// ref_qfc.cpp -- door into the reference's quantized fully-connected kernel.
//
// TEST INFRASTRUCTURE ONLY.  quantized_fully_connected_layer cannot be built in
// this snapshot of the reference (its backend wiring refers to a member that is
// commented out), but the arithmetic lives in the free function
// core::kernels::tiny_quantized_fully_connected_kernel
// (tiny_dnn/core/kernels/tiny_quantized_fully_connected_kernel.h:22-128), which
// is compiled here unmodified and called once per sample the way
// tiny_backend::fully_q would (tiny_dnn/core/backend_tiny.h:306-311).  The
// include path puts oracle/ref_stub first so the gemmlowp wrapper resolves to a
// stub for the kernel's dead `use_gemm` branch.
#include <cstddef>
#include <cstdint>
#include <vector>

#include "tiny_dnn/config.h"
#include "tiny_dnn/util/util.h"
#include "tiny_dnn/core/params/fully_params.h"

#define CNN_USE_GEMMLOWP 1
#include "tiny_dnn/core/kernels/tiny_quantized_fully_connected_kernel.h"

using namespace tiny_dnn;

extern "C" __attribute__((visibility("default"))) int ref_qfc_fwd(int in_size, int out_size,
                                                                   const float *in, const float *W,
                                                                   const float *bias, float *out,
                                                                   int B) {
  core::fully_params p;
  p.in_size_ = in_size;
  p.out_size_ = out_size;
  p.has_bias_ = bias != nullptr;
  vec_t vW(W, W + (size_t)in_size * out_size);
  vec_t vb;
  if (bias) vb.assign(bias, bias + out_size);
  for (int n = 0; n < B; ++n) {
    vec_t vin(in + (size_t)n * in_size, in + (size_t)(n + 1) * in_size);
    vec_t vout(out_size, 0.f);
    core::kernels::tiny_quantized_fully_connected_kernel(p, vin, vW, vb, vout, true);
    std::copy(vout.begin(), vout.end(), out + (size_t)n * out_size);
  }
  return 0;
}

// The eleven-argument overload (:269-370): operands are uint8 values held in floats with their
// ranges, the result leaves the same way; called once per sample the way tiny_backend::fully_eq
// would (tiny_dnn/core/backend_tiny.h:321-345).  in_r / out_r: [B][2], W_r / b_r: [2].
extern "C" __attribute__((visibility("default"))) int ref_qfc_eq_fwd(int in_size, int out_size, const float *in,
                                                                      const float *W, const float *bias,
                                                                      const float *in_r, const float *W_r,
                                                                      const float *b_r, float *out, float *out_r,
                                                                      int B) {
  core::fully_params p;
  p.in_size_ = in_size;
  p.out_size_ = out_size;
  p.has_bias_ = bias != nullptr;
  vec_t vW(W, W + (size_t)in_size * out_size), vWr(W_r, W_r + 2), vbr(b_r, b_r + 2);
  vec_t vb;
  if (bias) vb.assign(bias, bias + out_size);
  for (int n = 0; n < B; ++n) {
    vec_t vin(in + (size_t)n * in_size, in + (size_t)(n + 1) * in_size), vinr(in_r + 2 * n, in_r + 2 * n + 2);
    vec_t vout(out_size, 0.f), voutr(2, 0.f);
    core::kernels::tiny_quantized_fully_connected_kernel(p, vin, vW, vb, vinr, vWr, vbr, vout, voutr, true);
    std::copy(vout.begin(), vout.end(), out + (size_t)n * out_size);
    out_r[2 * n] = voutr[0];
    out_r[2 * n + 1] = voutr[1];
  }
  return 0;
}
