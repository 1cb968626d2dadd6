// C ABI of the library: argument validation and dispatch to the kernel families.
#include "common.cuh"

#include <nvtx3/nvToolsExt.h>

namespace mf {

char* last_error_buf() {
  static thread_local char buf[512] = "no error";
  return buf;
}
static thread_local const char* t_last_path = "none";
void set_last_path(const char* p) { t_last_path = p; }
std::atomic<uint64_t> g_launches{0};

namespace {

// One NVTX range per entry point (the reference marks its fused operators the same way for its timeline traces); without
// a profiler attached the calls return at once.
struct Range {
  explicit Range(const char* name) { nvtxRangePushA(name); }
  ~Range() { nvtxRangePop(); }
  Range(const Range&) = delete;
  Range& operator=(const Range&) = delete;
};

bool float_dtype(int dt) { return dt == MF_F32 || dt == MF_BF16 || dt == MF_F16; }

int check_device() {
  static thread_local int checked_dev = -1;
  int dev = 0;
  MF_CUDA(cudaGetDevice(&dev));
  if (dev == checked_dev) return MF_OK;
  int major = 0;
  MF_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  MF_REQUIRE(major == 10, MF_ERR_ARCH, "device %d has compute capability %d.x; this library is built for sm_100a only", dev, major);
  checked_dev = dev;
  return MF_OK;
}

template <typename A>
int check_evo_common(const A& a) {
  MF_REQUIRE(a.B > 0 && a.N > 0 && a.L > 0 && a.H > 0 && a.D > 0, MF_ERR_BAD_ARG,
             "sizes must be positive (B=%d N=%d L=%d H=%d D=%d)", a.B, a.N, a.L, a.H, a.D);
  MF_REQUIRE(float_dtype(a.dtype), MF_ERR_BAD_ARG, "q/k/v dtype %d is not a floating type", a.dtype);
  MF_REQUIRE(float_dtype(a.bias_dtype), MF_ERR_BAD_ARG, "pair_bias dtype %d is not a floating type", a.bias_dtype);
  MF_REQUIRE(float_dtype(a.mask_dtype) || a.mask_dtype == MF_U8, MF_ERR_BAD_ARG, "res_mask dtype %d unknown", a.mask_dtype);
  MF_REQUIRE(a.q && a.k && a.v, MF_ERR_BAD_ARG, "q, k and v must not be NULL");
  MF_REQUIRE(a.mask, MF_ERR_BAD_ARG, "res_mask must not be NULL");
  MF_REQUIRE(a.bias, MF_ERR_BAD_ARG, "pair_bias is mandatory and must not be NULL");
  MF_REQUIRE(a.D <= 128, MF_ERR_UNSUPPORTED, "head size %d > 128 is not supported", a.D);
  MF_REQUIRE((int64_t)a.B * a.N <= 65535 && a.H <= 65535, MF_ERR_UNSUPPORTED, "B*N=%lld or H=%d exceeds 65535",
             (long long)a.B * a.N, a.H);
  return MF_OK;
}

}  // namespace
}  // namespace mf

using namespace mf;

extern "C" {

int mf_evo_fwd(const mf_evo_fwd_args* args, void* stream) {
  Range nvtx_range("mf_evo_fwd");
  MF_REQUIRE(args, MF_ERR_BAD_ARG, "args is NULL");
  const mf_evo_fwd_args& a = *args;
  int r = check_evo_common(a); if (r) return r;
  MF_REQUIRE(a.o && a.lse, MF_ERR_BAD_ARG, "o and lse must not be NULL");
  r = check_device(); if (r) return r;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the tensor-core kernels write o with 16-byte stores
  if (!(a.flags & MF_FLAG_FORCE_SIMT) && ((uintptr_t)a.o & 15) == 0 &&
      evo_tc_supported(a.B, a.N, a.L, a.H, a.D, a.dtype, a.q_strides, a.k_strides, a.v_strides, a.q, a.k, a.v)) {
    r = evo_fwd_ws_supported(a) ? evo_fwd_ws(a, st) : evo_fwd_tc(a, st);
    if (r == MF_OK) set_last_path("tcgen05");
    return r;
  }
  r = evo_fwd_simt(a, st);
  if (r == MF_OK) set_last_path("simt");
  return r;
}

static bool evo_bwd_use_tc(const mf_evo_bwd_args& a) {
  // the tensor-core kernels read o / d_o and write dq / dk / dv with 16-byte accesses
  const uintptr_t align = (uintptr_t)a.o | (uintptr_t)a.d_o | (uintptr_t)a.dq | (uintptr_t)a.dk | (uintptr_t)a.dv;
  return !(a.flags & MF_FLAG_FORCE_SIMT) && (align & 15) == 0 && evo_bwd_ws_shape_ok(a.L, a.D) &&
         evo_tc_supported(a.B, a.N, a.L, a.H, a.D, a.dtype, a.q_strides, a.k_strides, a.v_strides, a.q, a.k, a.v);
}

size_t mf_evo_bwd_workspace_bytes(const mf_evo_bwd_args* args) {
  if (!args) return 0;
  return evo_bwd_use_tc(*args) ? evo_bwd_ws_workspace(*args) : evo_bwd_simt_workspace(*args);
}

int mf_evo_bwd(const mf_evo_bwd_args* args, void* stream) {
  Range nvtx_range("mf_evo_bwd");
  MF_REQUIRE(args, MF_ERR_BAD_ARG, "args is NULL");
  const mf_evo_bwd_args& a = *args;
  int r = check_evo_common(a); if (r) return r;
  MF_REQUIRE(a.o && a.d_o && a.lse, MF_ERR_BAD_ARG, "o, d_o and lse must not be NULL");
  MF_REQUIRE(a.dq && a.dk && a.dv && a.d_bias, MF_ERR_BAD_ARG, "dq, dk, dv and d_bias must not be NULL");
  MF_REQUIRE(a.dbias_dtype == MF_F32 || a.dbias_dtype == a.dtype, MF_ERR_BAD_ARG,
             "d_bias dtype must be fp32 or the q/k/v dtype");
  const size_t need = mf_evo_bwd_workspace_bytes(args);
  MF_REQUIRE(a.workspace && a.workspace_bytes >= need, MF_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need,
             a.workspace ? a.workspace_bytes : (size_t)0);
  MF_REQUIRE(((uintptr_t)a.workspace & 255) == 0, MF_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
  r = check_device(); if (r) return r;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (evo_bwd_use_tc(a)) {
    r = evo_bwd_ws(a, st);
    if (r == MF_OK) set_last_path("tcgen05");
    return r;
  }
  r = evo_bwd_simt(a, st);
  if (r == MF_OK && a.dbias_ready_event) MF_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(a.dbias_ready_event), st));
  if (r == MF_OK) set_last_path("simt");
  return r;
}

int mf_evo_bwd_noalloc(const mf_evo_bwd_args* args, void* stream) {
  Range nvtx_range("mf_evo_bwd_noalloc");
  MF_REQUIRE(args, MF_ERR_BAD_ARG, "args is NULL");
  const mf_evo_bwd_args& a = *args;
  int r = check_evo_common(a); if (r) return r;
  MF_REQUIRE(a.o && a.d_o && a.lse, MF_ERR_BAD_ARG, "o, d_o and lse must not be NULL");
  MF_REQUIRE(a.dq && a.dk && a.dv && a.d_bias, MF_ERR_BAD_ARG, "dq, dk, dv and d_bias must not be NULL");
  MF_REQUIRE(a.dbias_dtype == MF_F32 || a.dbias_dtype == a.dtype, MF_ERR_BAD_ARG,
             "d_bias dtype must be fp32 or the q/k/v dtype");
  r = check_device(); if (r) return r;
  r = evo_bwd_simt_noalloc(a, static_cast<cudaStream_t>(stream));
  if (r == MF_OK && a.dbias_ready_event)
    MF_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(a.dbias_ready_event), static_cast<cudaStream_t>(stream)));
  if (r == MF_OK) set_last_path("simt");
  return r;
}

size_t mf_evo_bwd_noalloc_max_rows(void) { return evo_bwd_noalloc_max_rows(); }

int mf_lnl_fwd(const mf_lnl_fwd_args* args, void* stream) {
  Range nvtx_range("mf_lnl_fwd");
  MF_REQUIRE(args, MF_ERR_BAD_ARG, "args is NULL");
  const mf_lnl_fwd_args& a = *args;
  MF_REQUIRE(a.M >= 0 && a.K > 0 && a.N > 0, MF_ERR_BAD_ARG, "bad sizes M=%lld K=%d N=%d", (long long)a.M, a.K, a.N);
  MF_REQUIRE(float_dtype(a.dtype), MF_ERR_BAD_ARG, "dtype %d is not a floating type", a.dtype);
  MF_REQUIRE(a.x && a.ln_w && a.w && a.y && a.mean && a.rstd, MF_ERR_BAD_ARG, "x, ln_w, w, y, mean, rstd must not be NULL");
  if (a.M == 0) return MF_OK;
  int r = check_device(); if (r) return r;
  if (!(a.flags & MF_FLAG_FORCE_SIMT) && lnl_fwd_tc_supported(a)) {
    r = lnl_fwd_tc(a, static_cast<cudaStream_t>(stream));
    if (r == MF_OK) set_last_path("tcgen05");
    return r;
  }
  r = lnl_fwd_simt(a, static_cast<cudaStream_t>(stream));
  if (r == MF_OK) set_last_path("simt");
  return r;
}

size_t mf_lnl_bwd_workspace_bytes(const mf_lnl_bwd_args* args) {
  if (!args) return 0;
  return lnl_bwd_workspace(*args);
}

int mf_lnl_bwd(const mf_lnl_bwd_args* args, void* stream) {
  Range nvtx_range("mf_lnl_bwd");
  MF_REQUIRE(args, MF_ERR_BAD_ARG, "args is NULL");
  const mf_lnl_bwd_args& a = *args;
  MF_REQUIRE(a.M > 0 && a.K > 0 && a.N > 0, MF_ERR_BAD_ARG, "bad sizes M=%lld K=%d N=%d", (long long)a.M, a.K, a.N);
  MF_REQUIRE(float_dtype(a.dtype), MF_ERR_BAD_ARG, "dtype %d is not a floating type", a.dtype);
  MF_REQUIRE(a.x && a.ln_w && a.w && a.dy && a.mean && a.rstd && a.dx && a.dw && a.d_ln_w, MF_ERR_BAD_ARG,
             "x, ln_w, w, dy, mean, rstd, dx, dw, d_ln_w must not be NULL");
  const size_t need = mf_lnl_bwd_workspace_bytes(args);
  MF_REQUIRE(a.workspace && a.workspace_bytes >= need, MF_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need,
             a.workspace ? a.workspace_bytes : (size_t)0);
  MF_REQUIRE(((uintptr_t)a.workspace & 255) == 0, MF_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
  int r = check_device(); if (r) return r;
  r = lnl_bwd(a, static_cast<cudaStream_t>(stream));
  if (r == MF_OK) set_last_path(lnl_bwd_runs_on_tc(a) ? "tcgen05" : "simt");
  return r;
}

int mf_swiglu_fwd(const void* x, void* y, int64_t M, int32_t inner, int32_t dtype, void* stream) {
  Range nvtx_range("mf_swiglu_fwd");
  MF_REQUIRE(x && y && M >= 0 && inner > 0, MF_ERR_BAD_ARG, "bad swiglu arguments");
  MF_REQUIRE(float_dtype(dtype), MF_ERR_BAD_ARG, "dtype %d is not a floating type", dtype);
  int r = check_device(); if (r) return r;
  return swiglu_fwd(x, y, M, inner, dtype, static_cast<cudaStream_t>(stream));
}

int mf_swiglu_bwd(const void* x, const void* dy, void* dx, int64_t M, int32_t inner, int32_t dtype, void* stream) {
  Range nvtx_range("mf_swiglu_bwd");
  MF_REQUIRE(x && dy && dx && M >= 0 && inner > 0, MF_ERR_BAD_ARG, "bad swiglu arguments");
  MF_REQUIRE(float_dtype(dtype), MF_ERR_BAD_ARG, "dtype %d is not a floating type", dtype);
  int r = check_device(); if (r) return r;
  return swiglu_bwd(x, dy, dx, M, inner, dtype, static_cast<cudaStream_t>(stream));
}

static bool transition_fwd_use_tc(const mf_transition_fwd_args& a) {
  return !(a.flags & MF_FLAG_FORCE_SIMT) && transition_fwd_tc_supported(a);
}

size_t mf_transition_fwd_workspace_bytes(const mf_transition_fwd_args* args) {
  if (!args) return 0;
  if (transition_fwd_use_tc(*args)) return 0;      // the fused kernel keeps the hidden activation on chip
  return transition_fwd_simt_workspace(*args);
}

int mf_transition_fwd(const mf_transition_fwd_args* args, void* stream) {
  Range nvtx_range("mf_transition_fwd");
  MF_REQUIRE(args, MF_ERR_BAD_ARG, "args is NULL");
  const mf_transition_fwd_args& a = *args;
  MF_REQUIRE(a.M > 0 && a.dim > 0 && a.inner > 0, MF_ERR_BAD_ARG, "bad sizes");
  MF_REQUIRE(float_dtype(a.dtype), MF_ERR_BAD_ARG, "dtype %d is not a floating type", a.dtype);
  MF_REQUIRE(a.x && a.w1 && a.w2 && a.y, MF_ERR_BAD_ARG, "x, w1, w2, y must not be NULL");
  MF_REQUIRE(!a.ln_w || (a.mean && a.rstd), MF_ERR_BAD_ARG, "mean and rstd are needed with LayerNorm");
  const size_t need = mf_transition_fwd_workspace_bytes(args);
  MF_REQUIRE(need == 0 || (a.workspace && a.workspace_bytes >= need), MF_ERR_WORKSPACE,
             "workspace of %zu bytes needed, %zu given", need, a.workspace ? a.workspace_bytes : (size_t)0);
  int r = check_device(); if (r) return r;
  if (transition_fwd_use_tc(a)) {
    r = transition_fwd_tc(a, static_cast<cudaStream_t>(stream));
    if (r == MF_OK) set_last_path("tcgen05");
    return r;
  }
  r = transition_fwd_simt(a, static_cast<cudaStream_t>(stream));
  if (r == MF_OK) set_last_path("simt");
  return r;
}

size_t mf_transition_bwd_workspace_bytes(const mf_transition_bwd_args* args) {
  if (!args) return 0;
  return transition_bwd_workspace(*args);
}

int mf_transition_bwd(const mf_transition_bwd_args* args, void* stream) {
  Range nvtx_range("mf_transition_bwd");
  MF_REQUIRE(args, MF_ERR_BAD_ARG, "args is NULL");
  const mf_transition_bwd_args& a = *args;
  MF_REQUIRE(a.M > 0 && a.dim > 0 && a.inner > 0, MF_ERR_BAD_ARG, "bad sizes");
  MF_REQUIRE(float_dtype(a.dtype), MF_ERR_BAD_ARG, "dtype %d is not a floating type", a.dtype);
  MF_REQUIRE(a.x && a.w1 && a.w2 && a.dy && a.dx && a.dw1 && a.dw2, MF_ERR_BAD_ARG,
             "x, w1, w2, dy, dx, dw1, dw2 must not be NULL");
  MF_REQUIRE(!a.ln_w || (a.mean && a.rstd && a.d_ln_w), MF_ERR_BAD_ARG, "mean, rstd, d_ln_w are needed with LayerNorm");
  const size_t need = mf_transition_bwd_workspace_bytes(args);
  MF_REQUIRE(a.workspace && a.workspace_bytes >= need, MF_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need,
             a.workspace ? a.workspace_bytes : (size_t)0);
  MF_REQUIRE(((uintptr_t)a.workspace & 255) == 0, MF_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
  int r = check_device(); if (r) return r;
  r = transition_bwd(a, static_cast<cudaStream_t>(stream));
  if (r == MF_OK) set_last_path(transition_bwd_runs_on_tc(a) ? "tcgen05" : "simt");
  return r;
}

const char* mf_last_error_string(void) { return last_error_buf(); }
int mf_version(void) { return MF_ABI_VERSION; }
uint64_t mf_kernel_launch_count(void) { return g_launches.load(); }
const char* mf_last_path(void) { return t_last_path; }
int mf_async_status(void) { return tc_async_status(); }

int mf_selftest_bounded_wait(void* stream) {
  int r = check_device(); if (r) return r;
  return bounded_wait_selftest(static_cast<cudaStream_t>(stream));
}

}  // extern "C"
