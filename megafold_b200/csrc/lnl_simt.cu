// LayernormLinear, SwiGLU and Transition on CUDA cores (fp32 arithmetic).
//
// These kernels take every shape and dtype; the tensor-core kernels cover the bf16 hot shapes.
// All reductions over rows (weight, gain and bias gradients) are split into slices whose partial
// sums are added in a fixed order, so results are bit-reproducible.
#include "gemm_simt.cuh"

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
__global__ void swiglu_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dx,
                                  int64_t total, int I) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  int64_t m = idx / I; int c = idx - m * I;
  float a = to_f(x[m * 2 * I + c]), b = to_f(x[m * 2 * I + I + c]), g = to_f(dy[idx]);
  float sg = sigmoidf_(b), sl = b * sg;
  dx[m * 2 * I + c] = from_f<T>(g * sl);
  dx[m * 2 * I + I + c] = from_f<T>(g * (sl * (1.f - sg) + sg) * a);
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

// Shared tail of LayernormLinear backward: given dy [M,N] computes dx, dw, d_ln_w, d_ln_b, db.
// gain == nullptr: no LayerNorm (dx = dy @ w^T, dw = x^T dy).
template <typename T>
int lnl_bwd_core(int64_t M, int K, int N, const T* x, const T* gain, const T* shift, const T* w, const T* dy,
                 const float* mean, const float* rstd, T* dx, float* dw, float* db, float* d_ln_w, float* d_ln_b,
                 Carver& ws, cudaStream_t st) {
  int r;
  float* col_scratch = ws.take<float>((size_t)kColSlices * (K > N ? K : N));
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

size_t lnl_bwd_core_bytes(int64_t M, int K, int N, bool has_ln) {
  size_t b = align_up(sizeof(float) * (size_t)kColSlices * (K > N ? K : N), 256);
  if (has_ln) b += align_up(sizeof(float) * (size_t)M * K, 256);
  int S = dw_splits(K, N, M);
  if (S > 1) b += align_up(sizeof(float) * (size_t)S * K * N, 256);
  return b;
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

size_t lnl_bwd_simt_workspace(const mf_lnl_bwd_args& a) { return lnl_bwd_core_bytes(a.M, a.K, a.N, true); }

int lnl_bwd_simt(const mf_lnl_bwd_args& a, cudaStream_t st) {
  Carver ws(a.workspace);
  MF_DISPATCH_FLOAT(a.dtype, T, {
    int r = lnl_bwd_core<T>(a.M, a.K, a.N, static_cast<const T*>(a.x), static_cast<const T*>(a.ln_w),
                            static_cast<const T*>(a.ln_b), static_cast<const T*>(a.w), static_cast<const T*>(a.dy),
                            a.mean, a.rstd, static_cast<T*>(a.dx), a.dw, a.db, a.d_ln_w, a.d_ln_b, ws, st);
    if (r) return r;
  });
  return MF_OK;
}

// ---- SwiGLU --------------------------------------------------------------------------------------
int swiglu_fwd(const void* x, void* y, int64_t M, int inner, int dtype, cudaStream_t st) {
  const int64_t total = M * inner;
  if (total == 0) return MF_OK;
  MF_DISPATCH_FLOAT(dtype, T, {
    swiglu_fwd_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(y), total, inner);
    MF_LAUNCHED("swiglu_fwd_kernel");
  });
  return MF_OK;
}
int swiglu_bwd(const void* x, const void* dy, void* dx, int64_t M, int inner, int dtype, cudaStream_t st) {
  const int64_t total = M * inner;
  if (total == 0) return MF_OK;
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

size_t transition_bwd_simt_workspace(const mf_transition_bwd_args& a) {
  size_t b = align_up((size_t)a.M * 2 * a.inner * dtype_size(a.dtype), 256);     // h, then dh in place
  int S = dw_splits(a.dim, a.inner, a.M);
  if (S > 1) b += align_up(sizeof(float) * (size_t)S * a.dim * a.inner, 256);     // dw2 slices
  b += lnl_bwd_core_bytes(a.M, a.dim, 2 * a.inner, a.ln_w != nullptr);
  return b;
}

int transition_bwd_simt(const mf_transition_bwd_args& a, cudaStream_t st) {
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
                        a.mean, a.rstd, static_cast<T*>(a.dx), a.dw1, nullptr, a.d_ln_w, a.d_ln_b, ws, st);
    if (r) return r;
  });
  return MF_OK;
}

}  // namespace mf
