// Host-side support shared by the tensor-core attention kernels: status word, device queries and the
// test that decides whether a call can take the tensor-core path.
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

namespace {
// One CTA waits, with a short cap, on an mbarrier that nobody completes, then takes the same exit path as the
// attention kernels: raise the CTA's flag, report through the status word, return normally.
__global__ void bounded_wait_selftest_kernel(int* status, int cap) {
  __shared__ uint64_t bar;
  __shared__ int abort_s;
  if (threadIdx.x == 0) { abort_s = 0; tc::mbar_init(&bar, 1); tc::mbar_fence_init(); }
  __syncthreads();
  bool done = false;
  for (int i = 0; i < cap && !done; ++i) done = tc::mbar_try_wait(&bar, 0);
  if (!done) abort_s = 1;
  __syncthreads();
  if (threadIdx.x == 0 && abort_s) *reinterpret_cast<volatile int*>(status) = 1;
}
}  // namespace

int bounded_wait_selftest(cudaStream_t st) {
  int* status = tcx::status_word();
  MF_REQUIRE(status, MF_ERR_CUDA, "could not allocate the device status word");
  bounded_wait_selftest_kernel<<<1, 128, 0, st>>>(status, 2048);
  MF_LAUNCHED("bounded_wait_selftest_kernel");
  return MF_OK;
}

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

}  // namespace mf

#ifdef MF_TRACE
// debug builds only: device buffer of 8 * kTraceLen 64-bit words that the attention kernels' phase trace is written to
extern "C" __attribute__((visibility("default"))) void mf_debug_set_trace(long long* p) { mf::tcx::g_trace = p; }
#endif
