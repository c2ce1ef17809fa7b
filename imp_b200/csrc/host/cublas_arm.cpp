// The library arm of the matrix products: cuBLASLt, loaded at run time, for IMP_B200_GEMM=cublas.
// It exists as a yardstick (the reference's engine sends its T>1 products to cublasLtMatmul,
// src/compute/gemm.cu:303-445); the default path never comes here.
#include "ops.hpp"

namespace imp {

bool library_gemm_bf16(Runtime&, Tensor, const Tensor&, const Tensor&) { return false; }

}  // namespace imp
