// General 16-bit GEMM on the tensor cores (tcgen05 + TMEM + TMA), used by the backward passes of LayernormLinear
// and Transition:   C[M, N] (+)= op(A) op(B)   with fp32 accumulation.
//
// Operands are row-major matrices described by how they are laid out relative to the reduction index r:
//   A "K-major":  stored [M, R]  (r contiguous)        A "MN-major": stored [R, M]  (m contiguous, i.e. A^T is given)
//   B "K-major":  stored [N, R]                        B "MN-major": stored [R, N]
// so that y = x W^T, dW = x^T dy, dg = dy W2 and friends all map onto it without a transposed copy.
//
// Persistent CTAs walk work items (128 x 128 output tile, slice of the reduction).  A 4-stage TMA ring feeds
// 64-deep slabs of A and B (128B-swizzled boxes), one thread issues 4 tcgen05.mma (M = N = 128, K = 16) per slab
// into one of two TMEM accumulators, and four epilogue warps move finished tiles (each its own 32 rows) TMEM ->
// registers -> swizzled staging -> TMA store (16-bit or fp32) or TMA add-reduction (fp32, when the reduction is split over CTAs; the
// output must then be zero on entry).  All waits are bounded.
#include "evo_tc_common.cuh"
#include "gemm_tc.cuh"

namespace mf {
namespace {
using namespace tcx;

constexpr int kBM = 128, kBN = 128, kBK = 64;
constexpr int kStages = 4;
constexpr int kThreads = 256;
constexpr int kStageBytes = 2 * 128 * 128;       // A slab 16 KB + B slab 16 KB

struct GemmP {
  int m_tiles, n_tiles, k_splits, slabs_total, slabs_per_split;
  int n_cols; int64_t n_rows;
  int a_mn, b_mn, out_kind;     // out_kind: 0 = 16-bit store, 1 = fp32 store, 2 = fp32 add-reduction
  uint32_t ab_fmt;
  int* status;
};

struct Bars { uint64_t full[kStages], empty[kStages], acc_full[2], acc_empty[2]; };

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* m, const void* src, int c0, int c1) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap ma, const __grid_constant__ CUtensorMap mb,
               const __grid_constant__ CUtensorMap mc, const GemmP p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sStage = smem;                                  // [kStages][A 16 KB | B 16 KB]
  uint8_t* sOut = smem + kStages * kStageBytes;            // staging: 64 KB (fp32) / 32 KB (16 bit)
  __shared__ Bars bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    abort_s = 0;
    for (int i = 0; i < kStages; ++i) { mbar_init(&bar.full[i], 1); mbar_init(&bar.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bar.acc_full[i], 1); mbar_init(&bar.acc_empty[i], 4); }
    mbar_fence_init();
    prefetch_tmap(&ma); prefetch_tmap(&mb); prefetch_tmap(&mc);
  }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  volatile int* abort_flag = &abort_s;
  const uint32_t tm0 = tmem_base_s;
  const int n_items = p.m_tiles * p.n_tiles * p.k_splits;
  auto decode = [&](int item, int& mt, int& nt, int& s0, int& s1) {
    const int ks = item % p.k_splits, rest = item / p.k_splits;
    nt = rest % p.n_tiles; mt = rest / p.n_tiles;
    s0 = ks * p.slabs_per_split;
    s1 = s0 + p.slabs_per_split; if (s1 > p.slabs_total) s1 = p.slabs_total;
  };

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------------------------------ TMA producer
    uint32_t cnt = 0;
    for (int item = blockIdx.x; item < n_items && !*abort_flag; item += gridDim.x) {
      int mt, nt, s0, s1; decode(item, mt, nt, s0, s1);
      for (int s = s0; s < s1; ++s, ++cnt) {
        const int st = cnt % kStages;
        if (cnt >= kStages) wait_or_flag(&bar.empty[st], ((cnt / kStages) - 1) & 1, abort_flag);
        if (*abort_flag) break;
        uint8_t* a = sStage + st * kStageBytes; uint8_t* b = a + 16384;
        mbar_expect_tx(&bar.full[st], kStageBytes);
        if (p.a_mn) {   // stored [R, M]: two [64 r][64 m] boxes
          tma_load_2d(a, &ma, &bar.full[st], mt * kBM, s * kBK);
          tma_load_2d(a + 8192, &ma, &bar.full[st], mt * kBM + 64, s * kBK);
        } else {        // stored [M, R]: one [128 m][64 r] box
          tma_load_2d(a, &ma, &bar.full[st], s * kBK, mt * kBM);
        }
        if (p.b_mn) {
          tma_load_2d(b, &mb, &bar.full[st], nt * kBN, s * kBK);
          tma_load_2d(b + 8192, &mb, &bar.full[st], nt * kBN + 64, s * kBK);
        } else {
          tma_load_2d(b, &mb, &bar.full[st], s * kBK, nt * kBN);
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------------------------ MMA issuer
    const uint32_t idesc = idesc_f16(128, kBN, p.ab_fmt, p.a_mn, p.b_mn);
    uint32_t cnt = 0, acc_cnt = 0;
    for (int item = blockIdx.x; item < n_items && !*abort_flag; item += gridDim.x, ++acc_cnt) {
      int mt, nt, s0, s1; decode(item, mt, nt, s0, s1);
      const int ab = acc_cnt & 1;
      if (acc_cnt >= 2) wait_or_flag(&bar.acc_empty[ab], ((acc_cnt >> 1) - 1) & 1, abort_flag);
      for (int s = s0; s < s1; ++s, ++cnt) {
        const int st = cnt % kStages;
        wait_or_flag(&bar.full[st], (cnt / kStages) & 1, abort_flag);
        tc_fence_after();
        if (*abort_flag) break;
        const uint32_t a0 = smem_u32(sStage + st * kStageBytes), b0 = a0 + 16384;
        // descriptor low words stepped by (bytes >> 4) per k-step: 16 rows of 128 B for MN-major, 32 B for K-major
        const uint32_t a_lo = p.a_mn ? desc_lo(a0, 8192) : desc_lo(a0, 16), a_step = p.a_mn ? 128u : 2u;
        const uint32_t b_lo = p.b_mn ? desc_lo(b0, 8192) : desc_lo(b0, 16), b_step = p.b_mn ? 128u : 2u;
#pragma unroll
        for (int ks = 0; ks < kBK / 16; ++ks)
          mma_ss_lh(tm0 + ab * kBN, a_lo + ks * a_step, desc_hi(1024, kSw128), b_lo + ks * b_step, desc_hi(1024, kSw128), idesc, s > s0 || ks > 0);
        tc_commit(&bar.empty[st]);
      }
      tc_commit(&bar.acc_full[ab]);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------------------------ epilogue (128 threads)
    const int ew = warp - 4;
    const int row = ew * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(ew * 32) << 16;
    uint32_t acc_cnt = 0;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++acc_cnt) {
      int mt, nt, s0, s1; decode(item, mt, nt, s0, s1);
      const int ab = acc_cnt & 1;
      wait_or_flag(&bar.acc_full[ab], (acc_cnt >> 1) & 1, abort_flag);
      tc_fence_after();
      // every epilogue warp stages and stores its own 32-row slab: no barrier between them
      if (lane == 0) bulk_wait_group_read<0>();             // my slab has been read by my previous store
      if (__any_sync(0xffffffffu, *abort_flag)) break;
#pragma unroll
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t v[32];
        tmem_ld32(tm0 + ab * kBN + cb * 32 + lane_addr, v);
        tmem_ld_wait();
        if (p.out_kind == 0) {
          // 16-bit: columns cb*32.. -> atom cb/2, chunks (cb%2)*4 .. +3
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 o;
            o.x = Pack2<T>::pack(__uint_as_float(v[ch * 8]), __uint_as_float(v[ch * 8 + 1]));
            o.y = Pack2<T>::pack(__uint_as_float(v[ch * 8 + 2]), __uint_as_float(v[ch * 8 + 3]));
            o.z = Pack2<T>::pack(__uint_as_float(v[ch * 8 + 4]), __uint_as_float(v[ch * 8 + 5]));
            o.w = Pack2<T>::pack(__uint_as_float(v[ch * 8 + 6]), __uint_as_float(v[ch * 8 + 7]));
            *reinterpret_cast<uint4*>(sOut + (cb >> 1) * 16384 + swz_offset(row, (cb & 1) * 4 + ch, 128)) = o;
          }
        } else {
          // fp32: columns cb*32.. form one 128-byte row of atom cb
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(sOut + cb * 16384 + swz_offset(row, ch, 128)) = make_uint4(v[ch * 4], v[ch * 4 + 1], v[ch * 4 + 2], v[ch * 4 + 3]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.acc_empty[ab]);
      fence_async_smem();
      __syncwarp();
      if (lane == 0 && (int64_t)mt * kBM + ew * 32 < p.n_rows) {     // never start a store past the last row
        const int r0 = mt * kBM + ew * 32;
        const uint8_t* slab = sOut + ew * (32 * 128);
        if (p.out_kind == 0) {
          tma_store_2d(&mc, slab, nt * kBN, r0);
          if (nt * kBN + 64 < p.n_cols) tma_store_2d(&mc, slab + 16384, nt * kBN + 64, r0);
        } else {
#pragma unroll
          for (int cb = 0; cb < 4; ++cb) {
            if (nt * kBN + cb * 32 >= p.n_cols) break;       // never start a store past the last column
            if (p.out_kind == 2) tma_reduce_add_2d(&mc, slab + cb * 16384, nt * kBN + cb * 32, r0);
            else tma_store_2d(&mc, slab + cb * 16384, nt * kBN + cb * 32, r0);
          }
        }
        bulk_commit_group();
      }
    }
    if (lane == 0) bulk_wait_group<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_s) *reinterpret_cast<volatile int*>(p.status) = 1;
  if (warp == 0) tmem_dealloc(tmem_base_s, 256);
}

}  // namespace

bool gemm_tc_ok(const GemmTcArgs& g) {
  if (g.dtype != MF_BF16 && g.dtype != MF_F16) return false;
  if (g.M < 1 || g.N < 1 || g.R < 1 || g.M > INT32_MAX || g.R > INT32_MAX) return false;
  const int64_t a_pitch = g.a_mn ? g.M : g.R, b_pitch = g.b_mn ? g.N : g.R;
  if (a_pitch % 8 || b_pitch % 8) return false;
  if (g.out_kind == 0 ? (g.N % 8 != 0) : (g.N % 4 != 0)) return false;
  const uintptr_t al = reinterpret_cast<uintptr_t>(g.a) | reinterpret_cast<uintptr_t>(g.b) | reinterpret_cast<uintptr_t>(g.c);
  return (al & 15) == 0;
}

int gemm_tc(const GemmTcArgs& g, cudaStream_t st) {
  MF_REQUIRE(gemm_tc_ok(g), MF_ERR_UNSUPPORTED, "gemm_tc: shape or alignment not supported");
  CUtensorMap ma, mb, mc;
  int r;
  {
    const int64_t dims[2] = {g.a_mn ? g.M : g.R, g.a_mn ? g.R : g.M}, str[2] = {1, dims[0]};
    const int box[2] = {64, g.a_mn ? 64 : 128};
    if ((r = make_tiled_map(&ma, g.a, g.dtype, 2, dims, str, box, 128))) return r;
  }
  {
    const int64_t dims[2] = {g.b_mn ? g.N : g.R, g.b_mn ? g.R : g.N}, str[2] = {1, dims[0]};
    const int box[2] = {64, g.b_mn ? 64 : 128};
    if ((r = make_tiled_map(&mb, g.b, g.dtype, 2, dims, str, box, 128))) return r;
  }
  {
    const int64_t dims[2] = {g.N, g.M}, str[2] = {1, g.N};
    const int box[2] = {g.out_kind == 0 ? 64 : 32, 32};      // one epilogue warp's slab
    if ((r = make_tiled_map(&mc, g.c, g.out_kind == 0 ? g.dtype : MF_F32, 2, dims, str, box, 128))) return r;
  }
  GemmP p{};
  p.m_tiles = (int)((g.M + kBM - 1) / kBM);
  p.n_tiles = (int)((g.N + kBN - 1) / kBN);
  p.slabs_total = (int)((g.R + kBK - 1) / kBK);
  const int sms = sm_count();
  int splits = 1;
  if (g.out_kind == 2) {
    // split the reduction so that every SM has work, but keep slices of at least 8 slabs
    const int tiles = p.m_tiles * p.n_tiles;
    splits = (2 * sms + tiles - 1) / tiles;
    const int cap = p.slabs_total / 8 > 0 ? p.slabs_total / 8 : 1;
    if (splits > cap) splits = cap;
    if (splits < 1) splits = 1;
  }
  p.slabs_per_split = (p.slabs_total + splits - 1) / splits;
  p.k_splits = (p.slabs_total + p.slabs_per_split - 1) / p.slabs_per_split;
  p.n_cols = (int)g.N; p.n_rows = g.M;
  p.a_mn = g.a_mn; p.b_mn = g.b_mn; p.out_kind = g.out_kind;
  p.ab_fmt = g.dtype == MF_BF16 ? 1u : 0u;
  p.status = status_word();
  MF_REQUIRE(p.status, MF_ERR_CUDA, "could not allocate the device status word");
  MF_REQUIRE(tc_async_status() == 0, MF_ERR_CUDA, "an earlier tensor-core kernel gave up on a bounded wait; results are invalid");
  if (g.out_kind == 2 && !g.accumulate) MF_CUDA(cudaMemsetAsync(g.c, 0, sizeof(float) * (size_t)g.M * g.N, st));
  const size_t smem = 1024 + kStages * (size_t)kStageBytes + 65536;
  const int n_items = p.m_tiles * p.n_tiles * p.k_splits;
  int grid = sms < n_items ? sms : n_items;
  if (g.dtype == MF_BF16) {
    auto kern = gemm_tc_kernel<__nv_bfloat16>;
    MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, st>>>(ma, mb, mc, p);
  } else {
    auto kern = gemm_tc_kernel<__half>;
    MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, st>>>(ma, mb, mc, p);
  }
  MF_LAUNCHED("gemm_tc_kernel");
  return MF_OK;
}

}  // namespace mf
