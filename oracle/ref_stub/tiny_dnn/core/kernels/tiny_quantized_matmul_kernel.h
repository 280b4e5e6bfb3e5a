// Stand-in for the reference header of the same name, placed FIRST on the
// include path of ref_qfc.cpp only.  The reference's
// tiny_quantized_fully_connected_kernel includes its gemmlowp matmul wrapper,
// which does not compile in this snapshot, but only calls it from a branch
// guarded by `bool use_gemm = false`
// (tiny_dnn/core/kernels/tiny_quantized_fully_connected_kernel.h:89-99).
// This declaration satisfies the compiler for that dead branch; it is never
// executed.
#pragma once

#include <cstdint>
#include <cstdlib>
#include <vector>

#include "tiny_dnn/core/kernels/tiny_quantization_kernel.h"

namespace tiny_dnn {
namespace core {
namespace kernels {

template <class T1, class T2, class Toutput>
void tiny_quantized_matmul(const std::vector<T1> &, const std::vector<T2> &, std::vector<Toutput> &,
                           const std::vector<size_t>, const int32_t, const int32_t, const int32_t,
                           const int32_t, const int32_t) {
  std::abort();  // unreachable: use_gemm is a constant false in the caller
}

}  // namespace kernels
}  // namespace core
}  // namespace tiny_dnn
