// Pair-biased masked attention on CUDA cores, fp32 arithmetic throughout.
//
// This family serves fp32 storage (where tensor-core input rounding would break the 1e-4 bound),
// head sizes and strides the tcgen05 kernels do not take, and acts as the on-device cross-check of
// the tensor-core kernels.  One warp owns a query (or key) row; the lanes split the opposite
// sequence index, 32 rows of it staged in shared memory at a time.
#include "common.cuh"

namespace mf {
namespace {

constexpr int kWarps = 8;
constexpr int kTile = 32;
constexpr int kRowsPerWarp = 4;   // forward: query rows handled together by one warp

struct EvoP {
  int B, N, L, H, D, DP;
  int bias_dtype, mask_dtype, dbias_dtype;
  float scale;
  const void *q, *k, *v;
  int64_t qs[5], ks[5], vs[5];
  const void* mask; int64_t ms[3];
  const void* bias; int64_t bs[4];
  void* o; float* lse;
  // backward
  const void *oo, *d_o; float* delta;
  void *dq, *dk, *dv; void* d_bias;
};

template <typename T>
__device__ __forceinline__ float ld5(const void* p, const int64_t* s, int b, int n, int l, int h, int d) {
  return to_f(static_cast<const T*>(p)[b * s[0] + n * s[1] + (int64_t)l * s[2] + h * s[3] + d * s[4]]);
}

// Loads rows [row0, row0+32) x [0,DP) of a [.., L, H, D] operand into shared memory as fp32,
// zero-padded outside L and D.  pitch = DP + 1 keeps lane-per-row reads conflict free.
template <typename T>
__device__ __forceinline__ void load_tile(float* dst, const void* src, const int64_t* s, int b, int n, int h,
                                          int row0, int L, int D, int DP) {
  const int pitch = DP + 1;
  for (int idx = threadIdx.x; idx < kTile * DP; idx += blockDim.x) {
    int r = idx / DP, d = idx - r * DP;
    int l = row0 + r;
    dst[r * pitch + d] = (l < L && d < D) ? ld5<T>(src, s, b, n, l, h, d) : 0.f;
  }
}

// ------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------
template <typename T, int DPW>
__global__ void __launch_bounds__(kWarps * 32) evo_fwd_simt_kernel(EvoP p) {
  extern __shared__ float smem[];
  const int DP = DPW * 32, pitch = DP + 1;
  float* Ks = smem;
  float* Vs = Ks + kTile * pitch;
  float* Qs = Vs + kTile * pitch;   // [kWarps][kRowsPerWarp][DP]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, bn = blockIdx.z, b = bn / p.N, n = bn - b * p.N;
  const int row_base = blockIdx.x * (kWarps * kRowsPerWarp) + warp * kRowsPerWarp;
  float* myq = Qs + warp * kRowsPerWarp * DP;

  for (int r = 0; r < kRowsPerWarp; ++r) {
    int i = row_base + r;
    for (int d = lane; d < DP; d += 32)
      myq[r * DP + d] = (i < p.L && d < p.D) ? ld5<T>(p.q, p.qs, b, n, i, h, d) * p.scale : 0.f;
  }
  float acc[kRowsPerWarp][DPW], m[kRowsPerWarp], l[kRowsPerWarp];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
    for (int dd = 0; dd < DPW; ++dd) acc[r][dd] = 0.f;
  }

  for (int j0 = 0; j0 < p.L; j0 += kTile) {
    __syncthreads();
    load_tile<T>(Ks, p.k, p.ks, b, n, h, j0, p.L, p.D, DP);
    load_tile<T>(Vs, p.v, p.vs, b, n, h, j0, p.L, p.D, DP);
    __syncthreads();
    const int j = j0 + lane;
    const bool valid = j < p.L;
    const float mt = valid ? mask_term(p.mask, b * p.ms[0] + n * p.ms[1] + j * p.ms[2], p.mask_dtype) : 0.f;
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const int i = row_base + r;
      if (i >= p.L) continue;
      float s = 0.f;
      for (int d = 0; d < DP; ++d) s = fmaf(myq[r * DP + d], Ks[lane * pitch + d], s);
      if (valid) {
        s += load_rt(p.bias, b * p.bs[0] + h * p.bs[1] + (int64_t)i * p.bs[2] + j * p.bs[3], p.bias_dtype);
        s += mt;
      } else {
        s = -INFINITY;
      }
      const float m_new = fmaxf(m[r], warp_max(s));
      const float corr = expf(m[r] - m_new);
      const float pr = expf(s - m_new);
      l[r] = l[r] * corr + warp_sum(pr);
      m[r] = m_new;
#pragma unroll
      for (int dd = 0; dd < DPW; ++dd) acc[r][dd] *= corr;
      for (int jj = 0; jj < kTile; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, pr, jj);
#pragma unroll
        for (int dd = 0; dd < DPW; ++dd) acc[r][dd] = fmaf(pj, Vs[jj * pitch + lane + 32 * dd], acc[r][dd]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    const int i = row_base + r;
    if (i >= p.L) continue;
    const float inv = 1.f / l[r];
    T* orow = static_cast<T*>(p.o) + ((((int64_t)b * p.N + n) * p.L + i) * p.H + h) * p.D;
#pragma unroll
    for (int dd = 0; dd < DPW; ++dd) {
      int d = lane + 32 * dd;
      if (d < p.D) orow[d] = from_f<T>(acc[r][dd] * inv);
    }
    if (lane == 0) p.lse[(((int64_t)b * p.N + n) * p.H + h) * p.L + i] = m[r] + logf(l[r]);
  }
}

// ------------------------------------------------------------------------------------------
// backward, step 0: delta[b,n,h,i] = sum_d dO * O      (one warp per (b,n,i,h))
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void evo_delta_kernel(const T* __restrict__ o, const T* __restrict__ d_o, float* __restrict__ delta,
                                 int64_t rows, int N, int L, int H, int D) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float s = 0.f;
  for (int d = lane; d < D; d += 32) s = fmaf(to_f(o[row * D + d]), to_f(d_o[row * D + d]), s);
  s = warp_sum(s);
  if (lane == 0) {
    // row = ((b*N+n)*L + i)*H + h  ->  delta index ((b*N+n)*H + h)*L + i
    int h = row % H; int64_t t = row / H; int i = t % L; int64_t bn = t / L;
    delta[(bn * H + h) * L + i] = s;
  }
}

// ------------------------------------------------------------------------------------------
// backward, step 1: dQ and dBias.  A block owns (b, h, 8 query rows); it walks the N rows that
// share the bias in order, so the dBias sum has a fixed order.  dBias row accumulators live in
// shared memory ([kWarps][L]).
// ------------------------------------------------------------------------------------------
template <typename T, int DPW>
__global__ void __launch_bounds__(kWarps * 32) evo_bwd_dq_simt_kernel(EvoP p) {
  extern __shared__ float smem[];
  const int DP = DPW * 32, pitch = DP + 1;
  float* Ks = smem;
  float* Vs = Ks + kTile * pitch;
  float* Qs = Vs + kTile * pitch;         // [kWarps][DP]
  float* Gs = Qs + kWarps * DP;           // dO rows [kWarps][DP]
  float* Bs = Gs + kWarps * DP;           // dBias accumulators [kWarps][L]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int i = blockIdx.x * kWarps + warp;
  const bool row_ok = i < p.L;
  float* myq = Qs + warp * DP;
  float* myg = Gs + warp * DP;
  float* myb = Bs + (size_t)warp * p.L;
  for (int j = lane; j < p.L; j += 32) myb[j] = 0.f;

  for (int n = 0; n < p.N; ++n) {
    float lse = 0.f, dl = 0.f;
    if (row_ok) {
      const int64_t srow = (((int64_t)b * p.N + n) * p.H + h) * p.L + i;
      lse = p.lse[srow]; dl = p.delta[srow];
      const T* grow = static_cast<const T*>(p.d_o) + ((((int64_t)b * p.N + n) * p.L + i) * p.H + h) * p.D;
      for (int d = lane; d < DP; d += 32) {
        myq[d] = d < p.D ? ld5<T>(p.q, p.qs, b, n, i, h, d) * p.scale : 0.f;
        myg[d] = d < p.D ? to_f(grow[d]) : 0.f;
      }
    }
    float accq[DPW];
#pragma unroll
    for (int dd = 0; dd < DPW; ++dd) accq[dd] = 0.f;
    for (int j0 = 0; j0 < p.L; j0 += kTile) {
      __syncthreads();
      load_tile<T>(Ks, p.k, p.ks, b, n, h, j0, p.L, p.D, DP);
      load_tile<T>(Vs, p.v, p.vs, b, n, h, j0, p.L, p.D, DP);
      __syncthreads();
      if (!row_ok) continue;
      const int j = j0 + lane;
      float ds = 0.f;
      if (j < p.L) {
        float s = 0.f, dp = 0.f;
        for (int d = 0; d < DP; ++d) {
          s = fmaf(myq[d], Ks[lane * pitch + d], s);
          dp = fmaf(myg[d], Vs[lane * pitch + d], dp);
        }
        s += load_rt(p.bias, b * p.bs[0] + h * p.bs[1] + (int64_t)i * p.bs[2] + j * p.bs[3], p.bias_dtype);
        const float mt = mask_term(p.mask, b * p.ms[0] + n * p.ms[1] + j * p.ms[2], p.mask_dtype);
        s += mt;
        // a row whose keys are all masked has lse = -FLT_MAX (log l is absorbed): it is uniform over its L keys
        const float pr = lse <= -3e38f ? 1.f / p.L : expf(s - lse);
        // a masked logit is a constant (masked_fill): no gradient flows into q, k or the bias through it,
        // which only matters for a row whose keys are ALL masked (elsewhere pr is exactly 0)
        ds = mt <= -FLT_MAX ? 0.f : pr * (dp - dl);
        myb[j] += ds;
      }
      for (int jj = 0; jj < kTile; ++jj) {
        const float dsj = __shfl_sync(0xffffffffu, ds, jj);
#pragma unroll
        for (int dd = 0; dd < DPW; ++dd) accq[dd] = fmaf(dsj, Ks[jj * pitch + lane + 32 * dd], accq[dd]);
      }
    }
    if (row_ok) {
      T* qrow = static_cast<T*>(p.dq) + ((((int64_t)b * p.N + n) * p.L + i) * p.H + h) * p.D;
#pragma unroll
      for (int dd = 0; dd < DPW; ++dd) {
        int d = lane + 32 * dd;
        if (d < p.D) qrow[d] = from_f<T>(accq[dd] * p.scale);
      }
    }
  }
  if (row_ok) {
    const int64_t base = (((int64_t)b * p.H + h) * p.L + i) * p.L;
    for (int j = lane; j < p.L; j += 32) store_rt(p.d_bias, base + j, p.dbias_dtype, myb[j]);
  }
}

// ------------------------------------------------------------------------------------------
// backward, step 2: dK and dV.  A block owns (b, n, h, 8 key rows) and walks the query tiles.
// ------------------------------------------------------------------------------------------
template <typename T, int DPW>
__global__ void __launch_bounds__(kWarps * 32) evo_bwd_dkv_simt_kernel(EvoP p) {
  extern __shared__ float smem[];
  const int DP = DPW * 32, pitch = DP + 1;
  float* Qt = smem;                        // query tile (scaled)
  float* Gt = Qt + kTile * pitch;          // dO tile
  float* Ks = Gt + kTile * pitch;          // [kWarps][DP]
  float* Vs = Ks + kWarps * DP;            // [kWarps][DP]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, bn = blockIdx.z, b = bn / p.N, n = bn - b * p.N;
  const int j = blockIdx.x * kWarps + warp;
  const bool row_ok = j < p.L;
  float* myk = Ks + warp * DP;
  float* myv = Vs + warp * DP;
  float mt = 0.f;
  if (row_ok) {
    for (int d = lane; d < DP; d += 32) {
      myk[d] = d < p.D ? ld5<T>(p.k, p.ks, b, n, j, h, d) : 0.f;
      myv[d] = d < p.D ? ld5<T>(p.v, p.vs, b, n, j, h, d) : 0.f;
    }
    mt = mask_term(p.mask, b * p.ms[0] + n * p.ms[1] + j * p.ms[2], p.mask_dtype);
  }
  // d_o is contiguous [B,N,L,H,D]
  const int64_t gs[5] = {(int64_t)p.N * p.L * p.H * p.D, (int64_t)p.L * p.H * p.D, (int64_t)p.H * p.D, p.D, 1};
  float acck[DPW], accv[DPW];
#pragma unroll
  for (int dd = 0; dd < DPW; ++dd) { acck[dd] = 0.f; accv[dd] = 0.f; }

  for (int i0 = 0; i0 < p.L; i0 += kTile) {
    __syncthreads();
    load_tile<T>(Qt, p.q, p.qs, b, n, h, i0, p.L, p.D, DP);
    load_tile<T>(Gt, p.d_o, gs, b, n, h, i0, p.L, p.D, DP);
    __syncthreads();
    if (!row_ok) continue;
    const int i = i0 + lane;
    float pr = 0.f, ds = 0.f;
    if (i < p.L) {
      float s = 0.f, dp = 0.f;
      for (int d = 0; d < DP; ++d) {
        s = fmaf(Qt[lane * pitch + d] * p.scale, myk[d], s);
        dp = fmaf(Gt[lane * pitch + d], myv[d], dp);
      }
      const int64_t srow = (((int64_t)b * p.N + n) * p.H + h) * p.L + i;
      s += load_rt(p.bias, b * p.bs[0] + h * p.bs[1] + (int64_t)i * p.bs[2] + j * p.bs[3], p.bias_dtype);
      s += mt;
      const float lse = p.lse[srow];
      pr = lse <= -3e38f ? 1.f / p.L : expf(s - lse);
      ds = mt <= -FLT_MAX ? 0.f : pr * (dp - p.delta[srow]);
    }
    for (int ii = 0; ii < kTile; ++ii) {
      const float pi = __shfl_sync(0xffffffffu, pr, ii);
      const float dsi = __shfl_sync(0xffffffffu, ds, ii);
#pragma unroll
      for (int dd = 0; dd < DPW; ++dd) {
        accv[dd] = fmaf(pi, Gt[ii * pitch + lane + 32 * dd], accv[dd]);
        acck[dd] = fmaf(dsi, Qt[ii * pitch + lane + 32 * dd], acck[dd]);
      }
    }
  }
  if (row_ok) {
    const int64_t off = ((((int64_t)b * p.N + n) * p.L + j) * p.H + h) * p.D;
#pragma unroll
    for (int dd = 0; dd < DPW; ++dd) {
      int d = lane + 32 * dd;
      if (d < p.D) {
        static_cast<T*>(p.dk)[off + d] = from_f<T>(acck[dd] * p.scale);
        static_cast<T*>(p.dv)[off + d] = from_f<T>(accv[dd]);
      }
    }
  }
}

template <typename A>
void fill_common(EvoP& p, const A& a) {
  p.B = a.B; p.N = a.N; p.L = a.L; p.H = a.H; p.D = a.D;
  p.DP = (a.D + 31) / 32 * 32;
  p.bias_dtype = a.bias_dtype; p.mask_dtype = a.mask_dtype;
  p.scale = 1.0f / sqrtf((float)a.D);
  p.q = a.q; p.k = a.k; p.v = a.v;
  for (int i = 0; i < 5; ++i) { p.qs[i] = a.q_strides[i]; p.ks[i] = a.k_strides[i]; p.vs[i] = a.v_strides[i]; }
  p.mask = a.mask; for (int i = 0; i < 3; ++i) p.ms[i] = a.mask_strides[i];
  p.bias = a.bias; for (int i = 0; i < 4; ++i) p.bs[i] = a.bias_strides[i];
}

template <typename K>
int set_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) MF_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return MF_OK;
}

}  // namespace

#define MF_DISPATCH_DPW(DP, W, ...)                   \
  switch ((DP) / 32) {                                \
    case 1: { constexpr int W = 1; __VA_ARGS__; } break; \
    case 2: { constexpr int W = 2; __VA_ARGS__; } break; \
    case 3: case 4: { constexpr int W = 4; __VA_ARGS__; } break; \
    default: return fail(MF_ERR_UNSUPPORTED, "head size %d > 128 is not supported", (DP)); \
  }

int evo_fwd_simt(const mf_evo_fwd_args& a, cudaStream_t st) {
  EvoP p{};
  fill_common(p, a);
  p.o = a.o; p.lse = a.lse;
  MF_DISPATCH_FLOAT(a.dtype, T, MF_DISPATCH_DPW(p.DP, W, {
    const int DP = W * 32;
    size_t smem = sizeof(float) * (2 * kTile * (DP + 1) + kWarps * kRowsPerWarp * DP);
    auto kern = evo_fwd_simt_kernel<T, W>;
    int r = set_smem(kern, smem); if (r) return r;
    dim3 grid((a.L + kWarps * kRowsPerWarp - 1) / (kWarps * kRowsPerWarp), a.H, a.B * a.N);
    kern<<<grid, kWarps * 32, smem, st>>>(p);
    MF_LAUNCHED("evo_fwd_simt_kernel");
  }));
  return MF_OK;
}

size_t evo_bwd_simt_workspace(const mf_evo_bwd_args& a) {
  return align_up(sizeof(float) * (size_t)a.B * a.N * a.H * a.L, 256);
}

int evo_bwd_simt(const mf_evo_bwd_args& a, cudaStream_t st) {
  EvoP p{};
  fill_common(p, a);
  p.lse = const_cast<float*>(a.lse);
  p.oo = a.o; p.d_o = a.d_o; p.delta = static_cast<float*>(a.workspace);
  p.dq = a.dq; p.dk = a.dk; p.dv = a.dv; p.d_bias = a.d_bias; p.dbias_dtype = a.dbias_dtype;
  MF_REQUIRE(a.L <= 8192, MF_ERR_UNSUPPORTED, "CUDA-core backward keeps dBias rows in shared memory: L=%d > 8192", a.L);
  MF_DISPATCH_FLOAT(a.dtype, T, MF_DISPATCH_DPW(p.DP, W, {
    const int DP = W * 32;
    const int64_t rows = (int64_t)a.B * a.N * a.L * a.H;
    evo_delta_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(
        static_cast<const T*>(a.o), static_cast<const T*>(a.d_o), p.delta, rows, a.N, a.L, a.H, a.D);
    MF_LAUNCHED("evo_delta_kernel");
    {
      size_t smem = sizeof(float) * (2 * kTile * (DP + 1) + 2 * kWarps * DP + (size_t)kWarps * a.L);
      MF_REQUIRE(smem <= 220 * 1024, MF_ERR_UNSUPPORTED, "L=%d too long for the CUDA-core backward", a.L);
      auto kern = evo_bwd_dq_simt_kernel<T, W>;
      int r = set_smem(kern, smem); if (r) return r;
      dim3 grid((a.L + kWarps - 1) / kWarps, a.H, a.B);
      kern<<<grid, kWarps * 32, smem, st>>>(p);
      MF_LAUNCHED("evo_bwd_dq_simt_kernel");
    }
    {
      size_t smem = sizeof(float) * (2 * kTile * (DP + 1) + 2 * kWarps * DP);
      auto kern = evo_bwd_dkv_simt_kernel<T, W>;
      int r = set_smem(kern, smem); if (r) return r;
      dim3 grid((a.L + kWarps - 1) / kWarps, a.H, a.B * a.N);
      kern<<<grid, kWarps * 32, smem, st>>>(p);
      MF_LAUNCHED("evo_bwd_dkv_simt_kernel");
    }
  }));
  return MF_OK;
}

// ---- backward without any allocation ------------------------------------------------------------------
// Scratch for the variant below: the per-query delta = rowsum(dO * O) values, B*N*H*L floats.  The array is part
// of the library image, so every GPU that loads the library holds these 4 MiB until the process exits.
constexpr size_t kNoAllocDeltaFloats = size_t(1) << 20;
static __device__ __align__(256) float g_noalloc_delta[kNoAllocDeltaFloats];

size_t evo_bwd_noalloc_max_rows() { return kNoAllocDeltaFloats; }

int evo_bwd_simt_noalloc(const mf_evo_bwd_args& a, cudaStream_t st) {
  const size_t need = (size_t)a.B * a.N * a.H * a.L;
  MF_REQUIRE(need <= kNoAllocDeltaFloats, MF_ERR_UNSUPPORTED,
             "mf_evo_bwd_noalloc: B*N*H*L = %zu query rows exceed the built-in scratch of %zu rows; use mf_evo_bwd with a workspace",
             need, kNoAllocDeltaFloats);
  // In host code `g_noalloc_delta` is only a handle of the device array, not its address: the address is asked
  // for once per device (with that device current) and remembered.
  static float* dev_ptr[64] = {};
  int dev = 0;
  MF_CUDA(cudaGetDevice(&dev));
  MF_REQUIRE(dev >= 0 && dev < 64, MF_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  float* scratch = __atomic_load_n(&dev_ptr[dev], __ATOMIC_ACQUIRE);
  if (!scratch) {
    MF_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), g_noalloc_delta));
    MF_REQUIRE(scratch != nullptr, MF_ERR_CUDA, "cudaGetSymbolAddress returned a null scratch address");
    __atomic_store_n(&dev_ptr[dev], scratch, __ATOMIC_RELEASE);
  }
  mf_evo_bwd_args b = a;
  b.workspace = scratch;
  b.workspace_bytes = kNoAllocDeltaFloats * sizeof(float);
  return evo_bwd_simt(b, st);     // delta is fully rewritten for the B*N*H*L rows in use: nothing to clear
}

}  // namespace mf
