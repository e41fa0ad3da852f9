// Tensor-core GEMM path (tcgen05 + TMEM + TMA).  Placeholder until the kernels land:
// every shape is declined, so tl::gemm falls through to the FFMA tiles.
#include "tl_kernels.h"
namespace tl {
template <class T> bool gemm_tensor_core(const GemmDesc<T> &) { return false; }
template bool gemm_tensor_core<float>(const GemmDesc<float> &);
template bool gemm_tensor_core<__half>(const GemmDesc<__half> &);
}
