// CUDA-core GEMM skeleton with functor operands, fp32 accumulation.
//
//   C(m, n) = sum_{k in split z} A(m, k) * B(k, n)
//
// A and B are functors returning fp32 (they do bounds checks themselves and fuse LayerNorm,
// transposes or SwiGLU into the load); the epilogue functor receives one output row segment of
// four consecutive columns.  blockIdx.z selects a slice of the reduction dimension so that tall
// reductions (weight gradients over M) can be split and summed in a fixed order afterwards.
#pragma once
#include "common.cuh"

namespace mf {

constexpr int kGemmBM = 64, kGemmBN = 64, kGemmBK = 16;

// A_M_CONTIG: consecutive m are adjacent in memory (else consecutive k are).
// B_K_CONTIG: consecutive k are adjacent in memory (else consecutive n are).
template <bool A_M_CONTIG, bool B_K_CONTIG, class ALoad, class BLoad, class Epi>
__global__ void __launch_bounds__(256) gemm_simt_kernel(int64_t M, int N, int64_t K, int64_t k_per_split,
                                                        ALoad A, BLoad Bm, Epi epi) {
  __shared__ float As[kGemmBK][kGemmBM + 4];
  __shared__ float Bs[kGemmBK][kGemmBN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int64_t m0 = (int64_t)blockIdx.x * kGemmBM;
  const int n0 = blockIdx.y * kGemmBN;
  const int z = blockIdx.z;
  const int64_t kbeg = (int64_t)z * k_per_split;
  const int64_t kend = kbeg + k_per_split < K ? kbeg + k_per_split : K;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int64_t k0 = kbeg; k0 < kend; k0 += kGemmBK) {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      int mm, kk;
      if (A_M_CONTIG) { mm = tid & 63; kk = (tid >> 6) + 4 * t; }
      else            { kk = tid & 15; mm = (tid >> 4) + 16 * t; }
      const int64_t m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < M && k < kend) ? A(m, k) : 0.f;
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      int nn, kk;
      if (B_K_CONTIG) { kk = tid & 15; nn = (tid >> 4) + 16 * t; }
      else            { nn = tid & 63; kk = (tid >> 6) + 4 * t; }
      const int n = n0 + nn; const int64_t k = k0 + kk;
      Bs[kk][nn] = (n < N && k < kend) ? Bm(k, n) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kGemmBK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m < M) epi(m, n0 + tx * 4, acc[i], z);
  }
}

template <bool A_M_CONTIG, bool B_K_CONTIG, class ALoad, class BLoad, class Epi>
int launch_gemm_simt(const char* name, int64_t M, int N, int64_t K, int splits, ALoad A, BLoad B, Epi epi,
                     cudaStream_t st) {
  if (M <= 0 || N <= 0) return MF_OK;
  int64_t kps = (K + splits - 1) / splits;
  kps = (kps + kGemmBK - 1) / kGemmBK * kGemmBK;
  dim3 grid((unsigned)((M + kGemmBM - 1) / kGemmBM), (unsigned)((N + kGemmBN - 1) / kGemmBN), (unsigned)splits);
  gemm_simt_kernel<A_M_CONTIG, B_K_CONTIG><<<grid, 256, 0, st>>>(M, N, K, kps, A, B, epi);
  return after_launch(name);
}

// number of slices of a reduction of length `red` for an output of `tiles` 64x64 tiles
inline int pick_splits(int64_t tiles, int64_t red) {
  int64_t s = (592 + tiles - 1) / tiles;
  int64_t cap = red / 256; if (cap < 1) cap = 1;
  if (s > cap) s = cap;
  if (s > 128) s = 128;
  if (s < 1) s = 1;
  // every slice must be non-empty after rounding to kGemmBK
  while (s > 1) {
    int64_t kps = ((red + s - 1) / s + kGemmBK - 1) / kGemmBK * kGemmBK;
    if (kps * (s - 1) < red) break;
    --s;
  }
  return (int)s;
}

}  // namespace mf
