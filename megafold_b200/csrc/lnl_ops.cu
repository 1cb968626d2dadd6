// LayernormLinear, SwiGLU and Transition: launch plans, and the CUDA-core kernels (fp32 arithmetic).
//
// The forward entry points named *_simt and every kernel in this file run on CUDA cores and take every shape and dtype.
// lnl_bwd and transition_bwd are the backward launch plans: they choose, per call, between the tensor-core GEMMs
// (gemm_tc.cuh, transition_bwd_tc.cu) for the 16-bit hot shapes and the CUDA-core GEMMs (gemm_simt.cuh) for the rest.
// All reductions over rows (weight, gain and bias gradients) are split into slices whose partial sums are added in a
// fixed order, so results are bit-reproducible.
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"

namespace mf {
namespace {

// ---- operand functors ------------------------------------------------------------------------
template <typename T> struct LoadRM {   // f(r, c) = p[r*ld + c]
  const T* p; int64_t ld;
  __device__ float operator()(int64_t r, int64_t c) const { return to_f(p[r * ld + c]); }
};
template <typename T> struct LoadTr {   // f(r, c) = p[c*ld + r]
  const T* p; int64_t ld;
  __device__ float operator()(int64_t r, int64_t c) const { return to_f(p[c * ld + r]); }
};
// LayerNorm applied on the fly; gain == nullptr means "identity" (no LayerNorm)
template <typename T> struct LoadLN {
  const T* x; const T* gain; const T* shift; const float* mean; const float* rstd; int K;
  __device__ float at(int64_t m, int64_t k) const {
    float v = to_f(x[m * K + k]);
    if (gain == nullptr) return v;
    v = (v - mean[m]) * rstd[m] * to_f(gain[k]);
    return shift ? v + to_f(shift[k]) : v;
  }
  __device__ float operator()(int64_t m, int64_t k) const { return at(m, k); }
};
template <typename T> struct LoadLNTr {
  LoadLN<T> ln;
  __device__ float operator()(int64_t k, int64_t m) const { return ln.at(m, k); }
};
// weight [K, 2I] presented with interleaved columns: virtual column 2c -> c, 2c+1 -> I + c
template <typename T> struct LoadW1Interleaved {
  const T* w; int I;
  __device__ float operator()(int64_t k, int64_t n) const {
    return to_f(w[k * (2 * (int64_t)I) + (n >> 1) + (n & 1) * I]);
  }
};
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
// g(m, c) = silu(h[m, I+c]) * h[m, c]
template <typename T> struct LoadSwiGLU {
  const T* h; int I;
  __device__ float operator()(int64_t m, int64_t c) const {
    float a = to_f(h[m * 2 * I + c]), b = to_f(h[m * 2 * I + I + c]);
    return b * sigmoidf_(b) * a;
  }
};

// ---- epilogues ---------------------------------------------------------------------------------
template <typename T> struct EpiStore {
  T* y; int64_t ld; int N; const T* bias;
  __device__ void operator()(int64_t m, int n0, const float (&acc)[4], int) const {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + j;
      if (n < N) y[m * ld + n] = from_f<T>(acc[j] + (bias ? to_f(bias[n]) : 0.f));
    }
  }
};
struct EpiPartial {
  float* part; int64_t MN; int64_t ld; int N;
  __device__ void operator()(int64_t m, int n0, const float (&acc)[4], int z) const {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + j;
      if (n < N) part[z * MN + m * ld + n] = acc[j];
    }
  }
};
template <typename T> struct EpiSwiGLU {   // consumes interleaved (a, gate) column pairs
  T* g; int I;
  __device__ void operator()(int64_t m, int n0, const float (&acc)[4], int) const {
#pragma unroll
    for (int j = 0; j < 4; j += 2) {
      int c = (n0 + j) >> 1;
      if (c < I) g[m * I + c] = from_f<T>(acc[j + 1] * sigmoidf_(acc[j + 1]) * acc[j]);
    }
  }
};
template <typename T> struct EpiSwiGLUBwd {  // acc = dg[m, c]; h -> dh in place
  T* h; int I;
  __device__ void operator()(int64_t m, int n0, const float (&acc)[4], int) const {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int c = n0 + j;
      if (c < I) {
        float a = to_f(h[m * 2 * I + c]), b = to_f(h[m * 2 * I + I + c]);
        float sg = sigmoidf_(b), sl = b * sg;
        h[m * 2 * I + c] = from_f<T>(acc[j] * sl);
        h[m * 2 * I + I + c] = from_f<T>(acc[j] * (sl * (1.f - sg) + sg) * a);
      }
    }
  }
};

// ---- small kernels -----------------------------------------------------------------------------
template <typename T>
__global__ void ln_stats_kernel(const T* __restrict__ x, float* __restrict__ mean, float* __restrict__ rstd,
                                int64_t M, int K, float eps) {
  const int64_t m = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (m >= M) return;
  const int lane = threadIdx.x & 31;
  const T* row = x + m * K;
  float s = 0.f;
  for (int k = lane; k < K; k += 32) s += to_f(row[k]);
  const float mu = warp_sum(s) / K;
  float v = 0.f;
  for (int k = lane; k < K; k += 32) { float d = to_f(row[k]) - mu; v = fmaf(d, d, v); }
  v = warp_sum(v) / K;
  if (lane == 0) { mean[m] = mu; rstd[m] = rsqrtf(v + eps); }
}

// dx = (wdy - (c1*xhat + c2)) * rstd with wdy = dyln*gain, c1 = mean_k(xhat*wdy), c2 = mean_k(wdy)
template <typename T>
__global__ void ln_bwd_rows_kernel(const float* __restrict__ dyln, const T* __restrict__ x, const T* __restrict__ gain,
                                   const float* __restrict__ mean, const float* __restrict__ rstd,
                                   T* __restrict__ dx, int64_t M, int K) {
  const int64_t m = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (m >= M) return;
  const int lane = threadIdx.x & 31;
  const float mu = mean[m], rs = rstd[m];
  float c1 = 0.f, c2 = 0.f;
  for (int k = lane; k < K; k += 32) {
    float xh = (to_f(x[m * K + k]) - mu) * rs;
    float w = dyln[m * K + k] * to_f(gain[k]);
    c1 = fmaf(xh, w, c1); c2 += w;
  }
  c1 = warp_sum(c1) / K; c2 = warp_sum(c2) / K;
  for (int k = lane; k < K; k += 32) {
    float xh = (to_f(x[m * K + k]) - mu) * rs;
    float w = dyln[m * K + k] * to_f(gain[k]);
    dx[m * K + k] = from_f<T>((w - (c1 * xh + c2)) * rs);
  }
}

// Row pass of the tensor-core backward (16-bit T, K % 4 == 0, K <= 128 * KJ): one read of dyln and x gives dx,
// LN(x) in the operand dtype (the A operand of the weight-gradient GEMM) and per-block partial column sums
// of dyln * xhat and dyln.  part is [gridDim.x][2 * K]; the partials are added in a fixed order afterwards.
template <typename T, int KJ>
__global__ void __launch_bounds__(256)
ln_bwd_rows_fused_kernel(const float* __restrict__ dyln, const T* __restrict__ x, const T* __restrict__ gain,
                         const T* __restrict__ shift, const float* __restrict__ mean, const float* __restrict__ rstd,
                         T* __restrict__ dx, T* __restrict__ xln, float* __restrict__ part, int64_t M, int K,
                         int64_t rows_per_block) {
  extern __shared__ float red[];   // [8][2 * K]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t beg = (int64_t)blockIdx.x * rows_per_block;
  const int64_t end = beg + rows_per_block < M ? beg + rows_per_block : M;
  float gn[KJ][4], sh[KJ][4], dgn[KJ][4], dsh[KJ][4];
#pragma unroll
  for (int j = 0; j < KJ; ++j) {
    const int k = j * 128 + lane * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      gn[j][e] = k + e < K ? to_f(gain[k + e]) : 0.f;
      sh[j][e] = (shift && k + e < K) ? to_f(shift[k + e]) : 0.f;
      dgn[j][e] = 0.f; dsh[j][e] = 0.f;
    }
  }
  const float invK = 1.f / K;
  for (int64_t m = beg + warp; m < end; m += 8) {
    const float mu = mean[m], rs = rstd[m];
    float xh[KJ][4], d[KJ][4];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int j = 0; j < KJ; ++j) {
      const int k = j * 128 + lane * 4;
      if (k < K) {
        const uint2 xr = *reinterpret_cast<const uint2*>(x + m * K + k);
        const float4 dr = *reinterpret_cast<const float4*>(dyln + m * K + k);
        const T* xe = reinterpret_cast<const T*>(&xr);
        d[j][0] = dr.x; d[j][1] = dr.y; d[j][2] = dr.z; d[j][3] = dr.w;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          xh[j][e] = (to_f(xe[e]) - mu) * rs;
          const float w = d[j][e] * gn[j][e];
          c1 = fmaf(xh[j][e], w, c1); c2 += w;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) { xh[j][e] = 0.f; d[j][e] = 0.f; }
      }
    }
    c1 = warp_sum(c1) * invK; c2 = warp_sum(c2) * invK;
#pragma unroll
    for (int j = 0; j < KJ; ++j) {
      const int k = j * 128 + lane * 4;
      if (k < K) {
        __align__(8) T o[4]; __align__(8) T l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float w = d[j][e] * gn[j][e];
          o[e] = from_f<T>((w - (c1 * xh[j][e] + c2)) * rs);
          l[e] = from_f<T>(fmaf(xh[j][e], gn[j][e], sh[j][e]));
          dgn[j][e] = fmaf(d[j][e], xh[j][e], dgn[j][e]);
          dsh[j][e] += d[j][e];
        }
        *reinterpret_cast<uint2*>(dx + m * K + k) = *reinterpret_cast<const uint2*>(o);
        if (xln) *reinterpret_cast<uint2*>(xln + m * K + k) = *reinterpret_cast<const uint2*>(l);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < KJ; ++j) {
    const int k = j * 128 + lane * 4;
    if (k < K) {
#pragma unroll
      for (int e = 0; e < 4; ++e) { red[warp * 2 * K + k + e] = dgn[j][e]; red[warp * 2 * K + K + k + e] = dsh[j][e]; }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * K; c += 256) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w * 2 * K + c];
    part[(int64_t)blockIdx.x * 2 * K + c] = t;
  }
}

// xln = LN(x) from saved statistics, four elements per thread (16-bit T, K % 4 == 0)
template <typename T>
__global__ void ln_apply_kernel(const T* __restrict__ x, const T* __restrict__ gain, const T* __restrict__ shift,
                                const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ xln,
                                int64_t M, int K) {
  const int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int kq = K >> 2;
  if (q >= M * kq) return;
  const int64_t m = q / kq; const int k = (int)(q - m * kq) * 4;
  const float mu = mean[m], rs = rstd[m];
  const uint2 xr = *reinterpret_cast<const uint2*>(x + m * K + k);
  const T* xe = reinterpret_cast<const T*>(&xr);
  __align__(8) T o[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float v = (to_f(xe[e]) - mu) * rs * to_f(gain[k + e]);
    o[e] = from_f<T>(shift ? v + to_f(shift[k + e]) : v);
  }
  *reinterpret_cast<uint2*>(xln + m * K + k) = *reinterpret_cast<const uint2*>(o);
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ src, T* __restrict__ dst, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = from_f<T>(src[i]);
}

// partial column sums: part[z, c] = sum over the rows of slice z of f(m, c)
template <class F>
__global__ void colsum_partial_kernel(F f, float* __restrict__ part, int64_t M, int ncols, int64_t rows_per_slice) {
  __shared__ float red[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  const int z = blockIdx.y;
  const int64_t beg = (int64_t)z * rows_per_slice;
  const int64_t end = beg + rows_per_slice < M ? beg + rows_per_slice : M;
  float s = 0.f;
  if (c < ncols)
    for (int64_t m = beg + threadIdx.y; m < end; m += 8) s += f(m, c);
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < ncols) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += red[i][threadIdx.x];
    part[(int64_t)z * ncols + c] = t;
  }
}
__global__ void sum_slices_kernel(const float* __restrict__ part, float* __restrict__ out, int64_t n, int slices) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
  for (int z = 0; z < slices; ++z) s += part[(int64_t)z * n + i];
  out[i] = s;
}

template <typename T> struct ColDyXhat {   // dgain: dyln * xhat
  const float* dyln; const T* x; const float* mean; const float* rstd; int K;
  __device__ float operator()(int64_t m, int c) const {
    return dyln[m * K + c] * (to_f(x[m * K + c]) - mean[m]) * rstd[m];
  }
};
struct ColF32 { const float* p; int ld; __device__ float operator()(int64_t m, int c) const { return p[m * ld + c]; } };
template <typename T> struct ColT { const T* p; int ld; __device__ float operator()(int64_t m, int c) const { return to_f(p[m * ld + c]); } };

constexpr int kColSlices = 64;

template <class F>
int colsum(const char* name, F f, float* out, float* scratch, int64_t M, int ncols, cudaStream_t st) {
  int slices = (int)((M + 255) / 256); if (slices > kColSlices) slices = kColSlices; if (slices < 1) slices = 1;
  int64_t rps = (M + slices - 1) / slices;
  dim3 grid((ncols + 31) / 32, slices), block(32, 8);
  colsum_partial_kernel<<<grid, block, 0, st>>>(f, scratch, M, ncols, rps);
  int r = after_launch(name); if (r) return r;
  sum_slices_kernel<<<(ncols + 255) / 256, 256, 0, st>>>(scratch, out, ncols, slices);
  return after_launch("sum_slices_kernel");
}

// Column sums of a small fp32 matrix [rows, ncols] (the per-block partial sums of a row pass) in one launch and in a fixed
// order: columns [0, split) go to out_a, the others to out_b (which may be NULL).
__global__ void __launch_bounds__(1024)
colsum_small_kernel(const float* __restrict__ p, int rows, int ncols, float* __restrict__ out_a, float* __restrict__ out_b, int split) {
  __shared__ float red[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < ncols)
    for (int m = threadIdx.y; m < rows; m += 32) s += p[(int64_t)m * ncols + c];
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < ncols) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) t += red[i][threadIdx.x];
    if (c < split) out_a[c] = t;
    else if (out_b) out_b[c - split] = t;
  }
}
int colsum_small(const char* name, const float* p, int rows, int ncols, float* out_a, float* out_b, int split, cudaStream_t st) {
  colsum_small_kernel<<<(ncols + 31) / 32, dim3(32, 32), 0, st>>>(p, rows, ncols, out_a, out_b, split);
  return after_launch(name);
}

int sum_slices(const float* part, float* out, int64_t n, int slices, cudaStream_t st) {
  sum_slices_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(part, out, n, slices);
  return after_launch("sum_slices_kernel");
}

template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t total, int I) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  int64_t m = idx / I; int c = idx - m * I;
  float a = to_f(x[m * 2 * I + c]), b = to_f(x[m * 2 * I + I + c]);
  y[idx] = from_f<T>(b * sigmoidf_(b) * a);
}
template <typename T>
__global__ void swiglu_bwd_kernel(const T* x, const T* __restrict__ dy, T* dx,   // dx may alias x
                                  int64_t total, int I) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  int64_t m = idx / I; int c = idx - m * I;
  float a = to_f(x[m * 2 * I + c]), b = to_f(x[m * 2 * I + I + c]), g = to_f(dy[idx]);
  float sg = sigmoidf_(b), sl = b * sg;
  dx[m * 2 * I + c] = from_f<T>(g * sl);
  dx[m * 2 * I + I + c] = from_f<T>(g * (sl * (1.f - sg) + sg) * a);
}

// 16-bit SwiGLU, eight elements per thread (I % 8 == 0): full 16-byte accesses on both halves of the row
template <typename T>
__global__ void swiglu_fwd_vec_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t total8, int I8) {
  const int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= total8) return;
  const int64_t m = q / I8; const int c = (int)(q - m * I8) * 8;
  const int I = I8 * 8;
  const uint4 av = *reinterpret_cast<const uint4*>(x + m * 2 * I + c);
  const uint4 bv = *reinterpret_cast<const uint4*>(x + m * 2 * I + I + c);
  const T* a = reinterpret_cast<const T*>(&av); const T* b = reinterpret_cast<const T*>(&bv);
  __align__(16) T o[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { const float bf = to_f(b[e]); o[e] = from_f<T>(bf * sigmoidf_(bf) * to_f(a[e])); }
  *reinterpret_cast<uint4*>(y + m * I + c) = *reinterpret_cast<const uint4*>(o);
}
template <typename T>
__global__ void swiglu_bwd_vec_kernel(const T* x, const T* __restrict__ dy, T* dx, int64_t total8, int I8) {   // dx may alias x
  const int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= total8) return;
  const int64_t m = q / I8; const int c = (int)(q - m * I8) * 8;
  const int I = I8 * 8;
  const uint4 av = *reinterpret_cast<const uint4*>(x + m * 2 * I + c);
  const uint4 bv = *reinterpret_cast<const uint4*>(x + m * 2 * I + I + c);
  const uint4 gv = *reinterpret_cast<const uint4*>(dy + m * I + c);
  const T* a = reinterpret_cast<const T*>(&av); const T* b = reinterpret_cast<const T*>(&bv);
  const T* g = reinterpret_cast<const T*>(&gv);
  __align__(16) T da[8]; __align__(16) T db[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float bf = to_f(b[e]), gf = to_f(g[e]);
    const float sg = sigmoidf_(bf), sl = bf * sg;
    da[e] = from_f<T>(gf * sl);
    db[e] = from_f<T>(gf * (sl * (1.f - sg) + sg) * to_f(a[e]));
  }
  *reinterpret_cast<uint4*>(dx + m * 2 * I + c) = *reinterpret_cast<const uint4*>(da);
  *reinterpret_cast<uint4*>(dx + m * 2 * I + I + c) = *reinterpret_cast<const uint4*>(db);
}

// Column sums of a 16-bit [M, N] matrix (N % 8 == 0, N <= 2048): thread = (row lane, 8-column chunk), 16-byte loads,
// one partial row of sums per block; part is [gridDim.x][N].
template <typename T>
__global__ void __launch_bounds__(256)
colsum16_partial_kernel(const T* __restrict__ p, float* __restrict__ part, int64_t M, int N, int64_t rows_per_block) {
  extern __shared__ float red[];       // [row lanes][N]
  const int chunks = N >> 3;
  const int lanes = 256 / chunks;      // row lanes per block (chunks <= 256)
  const int rl = threadIdx.x / chunks, ch = threadIdx.x - rl * chunks;
  const int64_t beg = (int64_t)blockIdx.x * rows_per_block;
  const int64_t end = beg + rows_per_block < M ? beg + rows_per_block : M;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (rl < lanes) {
    for (int64_t m = beg + rl; m < end; m += lanes) {
      const uint4 v = *reinterpret_cast<const uint4*>(p + m * N + ch * 8);
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += to_f(e[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) red[rl * N + ch * 8 + i] = acc[i];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < N; c += 256) {
    float t = 0.f;
    for (int l = 0; l < lanes; ++l) t += red[l * N + c];
    part[(int64_t)blockIdx.x * N + c] = t;
  }
}

// workspace carving ------------------------------------------------------------------------------
struct Carver {
  char* base; size_t off = 0;
  explicit Carver(void* p) : base(static_cast<char*>(p)) {}
  template <typename U> U* take(size_t count) {
    U* r = reinterpret_cast<U*>(base + off);
    off += align_up(count * sizeof(U), 256);
    return r;
  }
};

int dw_splits(int K, int N, int64_t M) {
  int64_t tiles = (int64_t)((K + kGemmBM - 1) / kGemmBM) * ((N + kGemmBN - 1) / kGemmBN);
  return pick_splits(tiles, M);
}

constexpr int kRowBlocks = 1184;  // blocks of the fused row pass: eight per SM (64 resident warps), because a warp keeps only one row in
                                  // flight and the pass is bound by memory latency, not bandwidth, with fewer

// Can the backward GEMMs of a LayernormLinear with these sizes run on the tensor cores?
bool lnl_bwd_core_tc_ok(int64_t M, int K, int N, int dtype, bool has_ln, const void* x, const void* w, const void* dy,
                        const void* dx, const void* dw) {
  if (!has_ln || (dtype != MF_BF16 && dtype != MF_F16)) return false;
  if (K % 8 || N % 8 || K > 512 || M < 1) return false;
  const uintptr_t al = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(dy) |
                       reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(dw);
  return (al & 15) == 0;
}

// The fused LayerNorm-backward row pass over M rows; returns the number of blocks (= rows of `part`, [blocks][2 K]).
template <typename T>
int launch_ln_bwd_rows(const float* dyln, const T* x, const T* gain, const T* shift, const float* mean, const float* rstd,
                       T* dx, T* xln, float* part, int64_t M, int K, cudaStream_t st) {
  int blocks = (int)((M + 63) / 64); if (blocks > kRowBlocks) blocks = kRowBlocks;
  const int64_t rpb = (M + blocks - 1) / blocks;
  blocks = (int)((M + rpb - 1) / rpb);
  const size_t sm = sizeof(float) * 8 * 2 * K;
  const int kj = (K + 127) / 128;
#define MF_ROWS(KJ) ln_bwd_rows_fused_kernel<T, KJ><<<blocks, 256, sm, st>>>(dyln, x, gain, shift, mean, rstd, dx, xln, part, M, K, rpb)
  if (kj == 1) MF_ROWS(1); else if (kj == 2) MF_ROWS(2); else if (kj == 3) MF_ROWS(3); else MF_ROWS(4);
#undef MF_ROWS
  MF_LAUNCHED("ln_bwd_rows_fused_kernel");
  return blocks;
}

// Shared tail of LayernormLinear backward: given dy [M,N] computes dx, dw, d_ln_w, d_ln_b, db.
// gain == nullptr: no LayerNorm (dx = dy @ w^T, dw = x^T dy).
// tc: both GEMMs on the tensor cores (gemm_tc), with one fused row pass between them.
template <typename T>
int lnl_bwd_core(int64_t M, int K, int N, const T* x, const T* gain, const T* shift, const T* w, const T* dy,
                 const float* mean, const float* rstd, T* dx, float* dw, float* db, float* d_ln_w, float* d_ln_b,
                 Carver& ws, bool tc, int dtype, cudaStream_t st, const T* xln_ready = nullptr,
                 const float* dyln_ready = nullptr) {
  int r;
  float* col_scratch = ws.take<float>((size_t)kColSlices * (K > N ? K : N));
  if constexpr (sizeof(T) == 2) {
    if (tc) {
      float* dyln = dyln_ready ? const_cast<float*>(dyln_ready) : ws.take<float>((size_t)M * K);
      T* xln = xln_ready ? nullptr : ws.take<T>((size_t)M * K);
      float* part = ws.take<float>((size_t)kRowBlocks * 2 * K);
      if (!dyln_ready) {
        // dyln[M,K] = dy @ w^T  (A = dy [M,N], B = w [K,N], both with the reduction index contiguous)
        r = gemm_tc(GemmTcArgs{dy, w, dyln, M, K, N, dtype, 0, 0, 1}, st);
        if (r) return r;
      }
      const int blocks = launch_ln_bwd_rows<T>(dyln, x, gain, shift, mean, rstd, dx, xln, part, M, K, st);
      r = colsum_small("lnl_bwd_dgain_dshift", part, blocks, 2 * K, d_ln_w, d_ln_b, K, st);
      if (r) return r;
      if (db) {
        if (N <= 2048) {
          int cb = (int)((M + 63) / 64); if (cb > kRowBlocks) cb = kRowBlocks;
          const int64_t rows = (M + cb - 1) / cb;
          cb = (int)((M + rows - 1) / rows);
          float* dpart = ws.take<float>((size_t)kRowBlocks * N);
          const int lanes = 256 / (N / 8);
          colsum16_partial_kernel<T><<<cb, 256, sizeof(float) * lanes * N, st>>>(dy, dpart, M, N, rows);
          MF_LAUNCHED("colsum16_partial_kernel");
          r = colsum_small("lnl_bwd_dbias", dpart, cb, N, db, nullptr, N, st);
        } else {
          r = colsum("lnl_bwd_dbias", ColT<T>{dy, N}, db, col_scratch, M, N, st);
        }
        if (r) return r;
      }
      // dw[K,N] = LN(x)^T @ dy: both operands are given with the reduction index (rows) outermost
      return gemm_tc(GemmTcArgs{xln_ready ? xln_ready : xln, dy, dw, K, N, M, dtype, 1, 1, 2}, st);
    }
  }
  LoadLN<T> ln{x, gain, shift, mean, rstd, K};
  if (gain) {
    float* dyln = ws.take<float>((size_t)M * K);
    // dyln[M,K] = dy @ w^T
    r = launch_gemm_simt<false, true>("lnl_bwd_dyln", M, K, N, 1, LoadRM<T>{dy, N}, LoadTr<T>{w, N},
                                      EpiPartial{dyln, 0, K, K}, st);
    if (r) return r;
    ln_bwd_rows_kernel<T><<<(unsigned)((M + 7) / 8), 256, 0, st>>>(dyln, x, gain, mean, rstd, dx, M, K);
    MF_LAUNCHED("ln_bwd_rows_kernel");
    r = colsum("lnl_bwd_dgain", ColDyXhat<T>{dyln, x, mean, rstd, K}, d_ln_w, col_scratch, M, K, st);
    if (r) return r;
    if (d_ln_b) { r = colsum("lnl_bwd_dshift", ColF32{dyln, K}, d_ln_b, col_scratch, M, K, st); if (r) return r; }
  } else {
    r = launch_gemm_simt<false, true>("lin_bwd_dx", M, K, N, 1, LoadRM<T>{dy, N}, LoadTr<T>{w, N},
                                      EpiStore<T>{dx, K, K, nullptr}, st);
    if (r) return r;
  }
  if (db) { r = colsum("lnl_bwd_dbias", ColT<T>{dy, N}, db, col_scratch, M, N, st); if (r) return r; }
  // dw[K,N] = LN(x)^T @ dy, reduction over M in slices
  const int S = dw_splits(K, N, M);
  float* part = S > 1 ? ws.take<float>((size_t)S * K * N) : dw;
  r = launch_gemm_simt<true, false>("lnl_bwd_dw", K, N, M, S, LoadLNTr<T>{ln}, LoadRM<T>{dy, N},
                                    EpiPartial{part, (int64_t)K * N, N, N}, st);
  if (r) return r;
  if (S > 1) { r = sum_slices(part, dw, (int64_t)K * N, S, st); if (r) return r; }
  return MF_OK;
}

size_t lnl_bwd_core_bytes(int64_t M, int K, int N, bool has_ln, bool tc, int dtype) {
  size_t b = align_up(sizeof(float) * (size_t)kColSlices * (K > N ? K : N), 256);
  if (tc) {
    b += align_up(sizeof(float) * (size_t)M * K, 256) + align_up(dtype_size(dtype) * (size_t)M * K, 256) +
         align_up(sizeof(float) * (size_t)kRowBlocks * 2 * K, 256) + align_up(sizeof(float) * (size_t)kRowBlocks * N, 256);
    return b;
  }
  if (has_ln) b += align_up(sizeof(float) * (size_t)M * K, 256);
  int S = dw_splits(K, N, M);
  if (S > 1) b += align_up(sizeof(float) * (size_t)S * K * N, 256);
  return b;
}

bool lnl_bwd_use_tc(const mf_lnl_bwd_args& a) {
  return !(a.flags & MF_FLAG_FORCE_SIMT) &&
         lnl_bwd_core_tc_ok(a.M, a.K, a.N, a.dtype, a.ln_w != nullptr, a.x, a.w, a.dy, a.dx, a.dw);
}

// The tensor-core Transition backward needs 16-byte aligned rows everywhere.
bool transition_bwd_use_tc(const mf_transition_bwd_args& a) {
  if ((a.flags & MF_FLAG_FORCE_SIMT) || !a.ln_w) return false;
  if (a.inner % 8 || a.dim % 8) return false;
  const uintptr_t al = reinterpret_cast<uintptr_t>(a.w2) | reinterpret_cast<uintptr_t>(a.dw2);
  if (al & 15) return false;
  return lnl_bwd_core_tc_ok(a.M, a.dim, 2 * a.inner, a.dtype, true, a.x, a.w1, a.dy, a.dx, a.dw1);
}

}  // namespace

// ---- LayernormLinear ---------------------------------------------------------------------------
int lnl_fwd_simt(const mf_lnl_fwd_args& a, cudaStream_t st) {
  MF_DISPATCH_FLOAT(a.dtype, T, {
    const T* x = static_cast<const T*>(a.x);
    ln_stats_kernel<T><<<(unsigned)((a.M + 7) / 8), 256, 0, st>>>(x, a.mean, a.rstd, a.M, a.K, a.eps);
    MF_LAUNCHED("ln_stats_kernel");
    LoadLN<T> ln{x, static_cast<const T*>(a.ln_w), static_cast<const T*>(a.ln_b), a.mean, a.rstd, a.K};
    int r = launch_gemm_simt<false, false>("lnl_fwd_gemm", a.M, a.N, a.K, 1, ln,
                                           LoadRM<T>{static_cast<const T*>(a.w), a.N},
                                           EpiStore<T>{static_cast<T*>(a.y), a.N, a.N, static_cast<const T*>(a.b)}, st);
    if (r) return r;
  });
  return MF_OK;
}

size_t lnl_bwd_workspace(const mf_lnl_bwd_args& a) {
  // the larger of the two paths, so that the answer does not depend on pointer alignment
  const size_t simt = lnl_bwd_core_bytes(a.M, a.K, a.N, true, false, a.dtype);
  const size_t tc = lnl_bwd_use_tc(a) ? lnl_bwd_core_bytes(a.M, a.K, a.N, true, true, a.dtype) : 0;
  return simt > tc ? simt : tc;
}
bool lnl_bwd_runs_on_tc(const mf_lnl_bwd_args& a) { return lnl_bwd_use_tc(a); }
bool transition_bwd_runs_on_tc(const mf_transition_bwd_args& a) { return transition_bwd_use_tc(a); }

int lnl_bwd(const mf_lnl_bwd_args& a, cudaStream_t st) {
  Carver ws(a.workspace);
  const bool tc = lnl_bwd_use_tc(a);
  MF_DISPATCH_FLOAT(a.dtype, T, {
    int r = lnl_bwd_core<T>(a.M, a.K, a.N, static_cast<const T*>(a.x), static_cast<const T*>(a.ln_w),
                            static_cast<const T*>(a.ln_b), static_cast<const T*>(a.w), static_cast<const T*>(a.dy),
                            a.mean, a.rstd, static_cast<T*>(a.dx), a.dw, a.db, a.d_ln_w, a.d_ln_b, ws, tc, a.dtype, st);
    if (r) return r;
  });
  return MF_OK;
}

// ---- SwiGLU --------------------------------------------------------------------------------------
int swiglu_fwd(const void* x, void* y, int64_t M, int inner, int dtype, cudaStream_t st) {
  const int64_t total = M * inner;
  if (total == 0) return MF_OK;
  if (dtype != MF_F32 && inner % 8 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0) {
    const int64_t t8 = total / 8;
    if (dtype == MF_BF16)
      swiglu_fwd_vec_kernel<__nv_bfloat16><<<(unsigned)((t8 + 255) / 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), t8, inner / 8);
    else
      swiglu_fwd_vec_kernel<__half><<<(unsigned)((t8 + 255) / 256), 256, 0, st>>>(static_cast<const __half*>(x), static_cast<__half*>(y), t8, inner / 8);
    MF_LAUNCHED("swiglu_fwd_vec_kernel");
    return MF_OK;
  }
  MF_DISPATCH_FLOAT(dtype, T, {
    swiglu_fwd_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(y), total, inner);
    MF_LAUNCHED("swiglu_fwd_kernel");
  });
  return MF_OK;
}
int swiglu_bwd(const void* x, const void* dy, void* dx, int64_t M, int inner, int dtype, cudaStream_t st) {
  const int64_t total = M * inner;
  if (total == 0) return MF_OK;
  if (dtype != MF_F32 && inner % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) & 15) == 0) {
    const int64_t t8 = total / 8;
    if (dtype == MF_BF16)
      swiglu_bwd_vec_kernel<__nv_bfloat16><<<(unsigned)((t8 + 255) / 256), 256, 0, st>>>(
          static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx), t8, inner / 8);
    else
      swiglu_bwd_vec_kernel<__half><<<(unsigned)((t8 + 255) / 256), 256, 0, st>>>(
          static_cast<const __half*>(x), static_cast<const __half*>(dy), static_cast<__half*>(dx), t8, inner / 8);
    MF_LAUNCHED("swiglu_bwd_vec_kernel");
    return MF_OK;
  }
  MF_DISPATCH_FLOAT(dtype, T, {
    swiglu_bwd_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        static_cast<const T*>(x), static_cast<const T*>(dy), static_cast<T*>(dx), total, inner);
    MF_LAUNCHED("swiglu_bwd_kernel");
  });
  return MF_OK;
}

// ---- Transition ------------------------------------------------------------------------------------
size_t transition_fwd_simt_workspace(const mf_transition_fwd_args& a) {
  return align_up((size_t)a.M * a.inner * dtype_size(a.dtype), 256);
}

int transition_fwd_simt(const mf_transition_fwd_args& a, cudaStream_t st) {
  Carver ws(a.workspace);
  const int I = a.inner;
  MF_DISPATCH_FLOAT(a.dtype, T, {
    const T* x = static_cast<const T*>(a.x);
    if (a.ln_w) {
      ln_stats_kernel<T><<<(unsigned)((a.M + 7) / 8), 256, 0, st>>>(x, a.mean, a.rstd, a.M, a.dim, a.eps);
      MF_LAUNCHED("ln_stats_kernel");
    }
    T* g = ws.take<T>((size_t)a.M * I);
    LoadLN<T> ln{x, static_cast<const T*>(a.ln_w), static_cast<const T*>(a.ln_b), a.mean, a.rstd, a.dim};
    int r = launch_gemm_simt<false, false>("transition_fwd_gemm1", a.M, 2 * I, a.dim, 1, ln,
                                           LoadW1Interleaved<T>{static_cast<const T*>(a.w1), I}, EpiSwiGLU<T>{g, I}, st);
    if (r) return r;
    r = launch_gemm_simt<false, true>("transition_fwd_gemm2", a.M, a.dim, I, 1, LoadRM<T>{g, I},
                                      LoadTr<T>{static_cast<const T*>(a.w2), I},
                                      EpiStore<T>{static_cast<T*>(a.y), a.dim, a.dim, nullptr}, st);
    if (r) return r;
  });
  return MF_OK;
}

size_t transition_bwd_fused_bytes(const mf_transition_bwd_args& a);

// Scratch of the path that exactly these arguments take (the choice depends on dtype, sizes and pointer alignment, all of
// which the caller has filled in when it asks).
size_t transition_bwd_workspace(const mf_transition_bwd_args& a) {
  if (transition_bwd_use_tc(a)) {
    if (transition_bwd_fused_ok(a)) return transition_bwd_fused_bytes(a);
    const size_t es = dtype_size(a.dtype);
    return align_up((size_t)a.M * 2 * a.inner * es, 256) + 2 * align_up((size_t)a.M * a.inner * es, 256) +   // h/dh, g, dg
           align_up((size_t)a.M * a.dim * es, 256) +                                                          // LN(x)
           lnl_bwd_core_bytes(a.M, a.dim, 2 * a.inner, true, true, a.dtype);
  }
  size_t simt = align_up((size_t)a.M * 2 * a.inner * dtype_size(a.dtype), 256);     // h, then dh in place
  int S = dw_splits(a.dim, a.inner, a.M);
  if (S > 1) simt += align_up(sizeof(float) * (size_t)S * a.dim * a.inner, 256);     // dw2 slices
  simt += lnl_bwd_core_bytes(a.M, a.dim, 2 * a.inner, a.ln_w != nullptr, false, a.dtype);
  return simt;
}

// Tensor-core composition: xln = LN(x) from the saved statistics; h = xln w1 (recomputed, never saved by forward);
// g = swiglu(h); dw2 = dy^T g; dg = dy w2; dh = swiglu'(h, dg) in place; LayernormLinear backward with dy := dh.
template <typename T>
int transition_bwd_tc(const mf_transition_bwd_args& a, cudaStream_t st) {
  Carver ws(a.workspace);
  const int I = a.inner;
  const int64_t M = a.M;
  T* h = ws.take<T>((size_t)M * 2 * I);
  T* g = ws.take<T>((size_t)M * I);
  T* dg = ws.take<T>((size_t)M * I);
  T* xln = ws.take<T>((size_t)M * a.dim);
  {
    const int64_t quads = M * (a.dim / 4);
    ln_apply_kernel<T><<<(unsigned)((quads + 255) / 256), 256, 0, st>>>(
        static_cast<const T*>(a.x), static_cast<const T*>(a.ln_w), static_cast<const T*>(a.ln_b), a.mean, a.rstd, xln, M, a.dim);
    MF_LAUNCHED("ln_apply_kernel");
  }
  // h[M, 2I] = LN(x) @ w1   (w1 [dim, 2I]: the reduction index is outermost)
  int r = gemm_tc(GemmTcArgs{xln, a.w1, h, M, 2 * I, a.dim, a.dtype, 0, 1, 0}, st);
  if (r) return r;
  r = swiglu_fwd(h, g, M, I, a.dtype, st);
  if (r) return r;
  r = gemm_tc(GemmTcArgs{a.dy, g, a.dw2, a.dim, I, M, a.dtype, 1, 1, 2}, st);
  if (r) return r;
  r = gemm_tc(GemmTcArgs{a.dy, a.w2, dg, M, I, a.dim, a.dtype, 0, 1, 0}, st);
  if (r) return r;
  r = swiglu_bwd(h, dg, h, M, I, a.dtype, st);
  if (r) return r;
  return lnl_bwd_core<T>(M, a.dim, 2 * I, static_cast<const T*>(a.x), static_cast<const T*>(a.ln_w),
                         static_cast<const T*>(a.ln_b), static_cast<const T*>(a.w1), h, a.mean, a.rstd,
                         static_cast<T*>(a.dx), a.dw1, nullptr, a.d_ln_w, a.d_ln_b, ws, true, a.dtype, st, xln);
}

// Fused composition (dim = 128): one kernel recomputes h on chip and leaves g, dh (chunk-ordered columns) and dyln in
// HBM; then the LayerNorm row pass and the two weight-gradient GEMMs.  The rows are processed in ranges of at most
// kTransitionChunkRows so that the scratch (g, dh, dyln, LN(x): 3.8 KB per row at inner = 512) stays below what the
// reference's forward keeps as saved activations; the weight gradients accumulate over the ranges, the partial column
// sums of every range are reduced together at the end.
constexpr int64_t kTransitionChunkRows = 131072;
struct TransitionChunks { int n; int64_t rows; };
TransitionChunks transition_chunks(int64_t M) {
  TransitionChunks c;
  c.n = (int)((M + kTransitionChunkRows - 1) / kTransitionChunkRows);
  if (c.n < 1) c.n = 1;
  c.rows = (((M + c.n - 1) / c.n) + 127) / 128 * 128;
  return c;
}
size_t transition_bwd_fused_bytes(const mf_transition_bwd_args& a) {
  const size_t es = dtype_size(a.dtype);
  const TransitionChunks ch = transition_chunks(a.M);
  const size_t rows = (size_t)(ch.rows < a.M ? ch.rows : a.M);
  return align_up(rows * a.inner * es, 256) + align_up(rows * 2 * a.inner * es, 256) + align_up(sizeof(float) * rows * a.dim, 256) +
         align_up(rows * a.dim * es, 256) + align_up(sizeof(float) * (size_t)a.dim * 2 * a.inner, 256) +
         align_up(sizeof(float) * (size_t)ch.n * kRowBlocks * 2 * a.dim, 256);
}

template <typename T>
int transition_bwd_fused_path(const mf_transition_bwd_args& a, cudaStream_t st) {
  Carver ws(a.workspace);
  const int I = a.inner, K = a.dim;
  const int64_t M = a.M;
  const TransitionChunks ch = transition_chunks(M);
  const size_t rows_max = (size_t)(ch.rows < M ? ch.rows : M);
  T* g = ws.take<T>(rows_max * I);
  T* dh = ws.take<T>(rows_max * 2 * I);
  float* dyln = ws.take<float>(rows_max * K);
  T* xln = ws.take<T>(rows_max * K);
  float* dw1p = ws.take<float>((size_t)K * 2 * I);
  float* part = ws.take<float>((size_t)ch.n * kRowBlocks * 2 * K);
  int part_rows = 0;
  for (int c = 0; c < ch.n; ++c) {
    const int64_t m0 = (int64_t)c * ch.rows, rows = (m0 + ch.rows < M ? ch.rows : M - m0);
    if (rows <= 0) break;
    mf_transition_bwd_args ac = a;
    ac.M = rows;
    ac.x = static_cast<const T*>(a.x) + m0 * K;
    ac.dy = static_cast<const T*>(a.dy) + m0 * K;
    ac.dx = static_cast<T*>(a.dx) + m0 * K;
    ac.mean = a.mean + m0; ac.rstd = a.rstd + m0;
    int r = transition_bwd_fused(ac, g, dh, dyln, st);
    if (r) return r;
    GemmTcArgs g2{ac.dy, g, a.dw2, K, I, rows, a.dtype, 1, 1, 2};
    g2.accumulate = c > 0;
    r = gemm_tc(g2, st);
    if (r) return r;
    part_rows += launch_ln_bwd_rows<T>(dyln, static_cast<const T*>(ac.x), static_cast<const T*>(a.ln_w), static_cast<const T*>(a.ln_b),
                                       ac.mean, ac.rstd, static_cast<T*>(ac.dx), xln, part + (size_t)part_rows * 2 * K, rows, K, st);
    // dw1 (chunk-ordered columns) += LN(x)^T dh
    GemmTcArgs g1{xln, dh, dw1p, K, 2 * I, rows, a.dtype, 1, 1, 2};
    g1.accumulate = c > 0;
    r = gemm_tc(g1, st);
    if (r) return r;
  }
  int r = colsum_small("transition_bwd_dgain_dshift", part, part_rows, 2 * K, a.d_ln_w, a.d_ln_b, K, st);
  if (r) return r;
  return unpermute_dw1(dw1p, a.dw1, K, I, st);
}

int transition_bwd(const mf_transition_bwd_args& a, cudaStream_t st) {
  if (transition_bwd_use_tc(a)) {
    if (transition_bwd_fused_ok(a))
      return a.dtype == MF_BF16 ? transition_bwd_fused_path<__nv_bfloat16>(a, st) : transition_bwd_fused_path<__half>(a, st);
    return a.dtype == MF_BF16 ? transition_bwd_tc<__nv_bfloat16>(a, st) : transition_bwd_tc<__half>(a, st);
  }
  Carver ws(a.workspace);
  const int I = a.inner;
  MF_DISPATCH_FLOAT(a.dtype, T, {
    const T* x = static_cast<const T*>(a.x);
    const T* dy = static_cast<const T*>(a.dy);
    const T* w1 = static_cast<const T*>(a.w1);
    const T* w2 = static_cast<const T*>(a.w2);
    T* h = ws.take<T>((size_t)a.M * 2 * I);
    LoadLN<T> ln{x, static_cast<const T*>(a.ln_w), static_cast<const T*>(a.ln_b), a.mean, a.rstd, a.dim};
    // 1. recompute the pre-activation h = LN(x) @ w1
    int r = launch_gemm_simt<false, false>("transition_bwd_recompute", a.M, 2 * I, a.dim, 1, ln, LoadRM<T>{w1, 2 * I},
                                           EpiStore<T>{h, 2 * I, 2 * I, nullptr}, st);
    if (r) return r;
    // 2. dw2[dim, I] = dy^T @ swiglu(h), sliced over M
    const int S = dw_splits(a.dim, I, a.M);
    float* part = S > 1 ? ws.take<float>((size_t)S * a.dim * I) : a.dw2;
    r = launch_gemm_simt<true, false>("transition_bwd_dw2", a.dim, I, a.M, S, LoadTr<T>{dy, a.dim}, LoadSwiGLU<T>{h, I},
                                      EpiPartial{part, (int64_t)a.dim * I, I, I}, st);
    if (r) return r;
    if (S > 1) { r = sum_slices(part, a.dw2, (int64_t)a.dim * I, S, st); if (r) return r; }
    // 3. dg = dy @ w2, SwiGLU backward applied in the epilogue: h becomes dh
    r = launch_gemm_simt<false, false>("transition_bwd_dg", a.M, I, a.dim, 1, LoadRM<T>{dy, a.dim}, LoadRM<T>{w2, I},
                                       EpiSwiGLUBwd<T>{h, I}, st);
    if (r) return r;
    // 4. LayernormLinear backward with dy := dh
    r = lnl_bwd_core<T>(a.M, a.dim, 2 * I, x, static_cast<const T*>(a.ln_w), static_cast<const T*>(a.ln_b), w1, h,
                        a.mean, a.rstd, static_cast<T*>(a.dx), a.dw1, nullptr, a.d_ln_w, a.d_ln_b, ws, false, a.dtype, st);
    if (r) return r;
  });
  return MF_OK;
}

}  // namespace mf
