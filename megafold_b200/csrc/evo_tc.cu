// tcgen05 / TMEM / TMA attention kernels (placeholder while the CUDA-core path is brought up).
#include "common.cuh"
namespace mf {
bool evo_tc_supported(int, int, int, int, int, int, const int64_t*, const int64_t*, const int64_t*, const void*,
                      const void*, const void*) { return false; }
int evo_fwd_tc(const mf_evo_fwd_args&, cudaStream_t) { return fail(MF_ERR_UNSUPPORTED, "no tensor-core path"); }
int evo_bwd_tc(const mf_evo_bwd_args&, cudaStream_t) { return fail(MF_ERR_UNSUPPORTED, "no tensor-core path"); }
size_t evo_bwd_tc_workspace(const mf_evo_bwd_args&) { return 0; }
}  // namespace mf
