// Shared helpers of the megafold_b200 CUDA library: error reporting, dtype
// conversion, launch accounting.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "../../include/megafold_b200.h"

namespace mf {

// ---- host-side error state ----------------------------------------------------------------
char* last_error_buf();                 // thread-local, 512 bytes
void set_last_path(const char* p);
extern std::atomic<uint64_t> g_launches;

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define MF_REQUIRE(cond, code, ...) \
  do { if (!(cond)) return ::mf::fail((code), __VA_ARGS__); } while (0)

#define MF_CUDA(expr)                                                                        \
  do {                                                                                       \
    cudaError_t e__ = (expr);                                                                \
    if (e__ != cudaSuccess)                                                                  \
      return ::mf::fail(MF_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                        __FILE__, __LINE__);                                                 \
  } while (0)

// Checks the launch that was just issued and counts it.
inline int after_launch(const char* name) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(MF_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e));
  return MF_OK;
}
#define MF_LAUNCHED(name) \
  do { int r__ = ::mf::after_launch(name); if (r__ != MF_OK) return r__; } while (0)

inline size_t dtype_size(int dt) {
  switch (dt) {
    case MF_F32: return 4;
    case MF_BF16: case MF_F16: return 2;
    case MF_U8: return 1;
    default: return 0;
  }
}
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---- device-side conversion ---------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

// load element `idx` of an array whose dtype is only known at run time
__device__ __forceinline__ float load_rt(const void* p, int64_t idx, int dt) {
  switch (dt) {
    case MF_F32: return static_cast<const float*>(p)[idx];
    case MF_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
    case MF_F16: return __half2float(static_cast<const __half*>(p)[idx]);
    default: return static_cast<float>(static_cast<const uint8_t*>(p)[idx]);
  }
}
__device__ __forceinline__ void store_rt(void* p, int64_t idx, int dt, float v) {
  switch (dt) {
    case MF_F32: static_cast<float*>(p)[idx] = v; break;
    case MF_BF16: static_cast<__nv_bfloat16*>(p)[idx] = __float2bfloat16_rn(v); break;
    case MF_F16: static_cast<__half*>(p)[idx] = __float2half_rn(v); break;
    default: break;
  }
}

// Additive logit term of key j of row (b,n): keep-mask 0 -> -FLT_MAX (acts as a replacement of the
// logit because |logit| << ulp(FLT_MAX)), keep-mask 1 -> 0, floating mask -> its value.
__device__ __forceinline__ float mask_term(const void* mask, int64_t idx, int dt) {
  if (dt == MF_U8) return static_cast<const uint8_t*>(mask)[idx] ? 0.f : -FLT_MAX;
  return load_rt(mask, idx, dt);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- dispatch on the storage dtype ----------------------------------------------------------
#define MF_DISPATCH_FLOAT(dt, T, ...)                                       \
  switch (dt) {                                                             \
    case MF_F32: { using T = float; __VA_ARGS__; } break;                   \
    case MF_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break;          \
    case MF_F16: { using T = __half; __VA_ARGS__; } break;                  \
    default: return ::mf::fail(MF_ERR_BAD_ARG, "unknown dtype %d", (int)(dt)); \
  }

// ---- internal entry points of the kernel families ---------------------------------------------
int evo_fwd_simt(const mf_evo_fwd_args& a, cudaStream_t st);
int evo_bwd_simt(const mf_evo_bwd_args& a, cudaStream_t st);
size_t evo_bwd_simt_workspace(const mf_evo_bwd_args& a);
int evo_bwd_simt_noalloc(const mf_evo_bwd_args& a, cudaStream_t st);
size_t evo_bwd_noalloc_max_rows();

bool evo_tc_supported(int B, int N, int L, int H, int D, int dtype, const int64_t* qs, const int64_t* ks,
                      const int64_t* vs, const void* q, const void* k, const void* v);
int tc_async_status();
int bounded_wait_selftest(cudaStream_t st);
int evo_fwd_tc(const mf_evo_fwd_args& a, cudaStream_t st);
bool evo_fwd_ws_supported(const mf_evo_fwd_args& a);
int evo_fwd_ws(const mf_evo_fwd_args& a, cudaStream_t st);
bool evo_bwd_ws_shape_ok(int L, int D);
int evo_bwd_ws(const mf_evo_bwd_args& a, cudaStream_t st);
size_t evo_bwd_ws_workspace(const mf_evo_bwd_args& a);

int lnl_fwd_simt(const mf_lnl_fwd_args& a, cudaStream_t st);
bool lnl_fwd_tc_supported(const mf_lnl_fwd_args& a);
int lnl_fwd_tc(const mf_lnl_fwd_args& a, cudaStream_t st);
int lnl_bwd(const mf_lnl_bwd_args& a, cudaStream_t st);   // picks tensor-core GEMMs when lnl_bwd_runs_on_tc
bool lnl_bwd_runs_on_tc(const mf_lnl_bwd_args& a);
bool transition_bwd_runs_on_tc(const mf_transition_bwd_args& a);
bool transition_bwd_fused_ok(const mf_transition_bwd_args& a);
int transition_bwd_fused(const mf_transition_bwd_args& a, void* g, void* dh, float* dyln, cudaStream_t st);
int unpermute_dw1(const float* src, float* dst, int dim, int inner, cudaStream_t st);
size_t lnl_bwd_workspace(const mf_lnl_bwd_args& a);

int transition_fwd_simt(const mf_transition_fwd_args& a, cudaStream_t st);
bool transition_fwd_tc_supported(const mf_transition_fwd_args& a);
int transition_fwd_tc(const mf_transition_fwd_args& a, cudaStream_t st);
int transition_bwd(const mf_transition_bwd_args& a, cudaStream_t st);
size_t transition_fwd_simt_workspace(const mf_transition_fwd_args& a);
size_t transition_bwd_workspace(const mf_transition_bwd_args& a);

int swiglu_fwd(const void* x, void* y, int64_t M, int inner, int dtype, cudaStream_t st);
int swiglu_bwd(const void* x, const void* dy, void* dx, int64_t M, int inner, int dtype, cudaStream_t st);

}  // namespace mf
