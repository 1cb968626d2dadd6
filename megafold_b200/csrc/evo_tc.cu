// Host-side support shared by the tensor-core attention kernels: status word, device queries and the
// test that decides whether a call can take the tensor-core path.
#include <stdlib.h>

#include "evo_tc_common.cuh"

namespace mf {
namespace tcx {

StatusWord* status_slot() {
  static std::mutex mu;
  static StatusWord words[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  StatusWord& w = words[dev];
  if (!w.host) {
    if (cudaHostAlloc(&w.host, sizeof(int), cudaHostAllocMapped) != cudaSuccess) { w.host = nullptr; return nullptr; }
    *w.host = 0;
    if (cudaHostGetDevicePointer(&w.dev, w.host, 0) != cudaSuccess) return nullptr;
  }
  return &w;
}

#ifdef MF_TRACE
long long* g_trace = nullptr;
#endif

int sm_count() {
  static int n[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev] > 0 ? n[dev] : 148;
}

}  // namespace tcx

int tc_async_status() {
  tcx::StatusWord* w = tcx::status_slot();
  return (w && w->host) ? *reinterpret_cast<volatile int*>(w->host) : 0;
}

bool evo_tc_supported(int B, int N, int L, int H, int D, int dtype, const int64_t* qs, const int64_t* ks,
                      const int64_t* vs, const void* q, const void* k, const void* v) {
  if (dtype != MF_BF16 && dtype != MF_F16) return false;
  if (D % 8 != 0 || D > 64 || L > 4096) return false;
  return tcx::qkv_strides_ok(q, qs, B, N, L, H) && tcx::qkv_strides_ok(k, ks, B, N, L, H) &&
         tcx::qkv_strides_ok(v, vs, B, N, L, H);
}

bool evo_bwd_tc_available() { return true; }

bool debug_old_evo(int which) {
  static const bool f = [] { const char* e = getenv("MF_DEBUG_OLD_EVO_FWD"); return e && e[0] == '1'; }();
  static const bool b = [] { const char* e = getenv("MF_DEBUG_OLD_EVO_BWD"); return e && e[0] == '1'; }();
  return which == 0 ? f : b;
}

}  // namespace mf

#ifdef MF_TRACE
// debug builds only: device buffer of 8 * kTraceLen 64-bit words that the attention kernels' phase trace is written to
extern "C" __attribute__((visibility("default"))) void mf_debug_set_trace(long long* p) { mf::tcx::g_trace = p; }
#endif
