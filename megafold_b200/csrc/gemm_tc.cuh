// Interface of the general tensor-core GEMM (gemm_tc.cu).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace mf {

// C[M, N] = sum_r A(m, r) B(n, r), fp32 accumulation, 16-bit operands of one dtype.
//   a_mn = 0: A stored [M, R] row-major;  a_mn = 1: stored [R, M].   Same for B with N.
//   out_kind 0: C stored in the operand dtype; 1: fp32; 2: fp32 with the reduction split over CTAs and summed by
//   TMA add-reductions (C is zeroed first unless `accumulate` is set - a caller that feeds the reduction in several row
//   ranges; summation order, and so the last bits, vary from run to run).
struct GemmTcArgs {
  const void* a; const void* b; void* c;
  int64_t M, N, R;
  int dtype, a_mn, b_mn, out_kind;
  int accumulate = 0;
};
bool gemm_tc_ok(const GemmTcArgs& g);
int gemm_tc(const GemmTcArgs& g, cudaStream_t st);

}  // namespace mf
