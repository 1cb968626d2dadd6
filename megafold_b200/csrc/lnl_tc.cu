// LayernormLinear forward on the tensor cores:  Y[M,N] = LayerNorm_K(X[M,K]) W[K,N] (+ b),  K in {64, 128}.
//
// The operator is bound by HBM traffic (K = 128 gives 64-140 FLOP per byte), so the kernel is organised around
// touching X and Y exactly once with full-line accesses; the tensor pipe has slack.
//
// Persistent CTA per SM, 128-row tiles of X, four warpgroups with fixed roles:
//   warps 8-11  normalise.  The raw rows of X arrive by TMA in the layout the MMA wants (ring of three tiles); a
//               thread owns one row: two-pass mean / variance in fp32, gain and shift, 16-bit result written back
//               over the raw row; mean and rstd go to global memory for the backward pass.  These warps run
//               ahead of the MMAs as far as the ring allows.
//   warps 0-7   epilogue.  Thread (row, column half) reads 64 accumulator columns from TMEM, adds the linear bias,
//               packs to 16 bit and writes a swizzled staging slab ([32 rows][64 columns] per warp) that the warp's
//               lane 0 hands to a TMA store (full 128-byte lines, clipped at the edges of Y); no barrier between
//               the epilogue warps.
//   warp 12     tcgen05.mma issuer: per 128-column tile of W, K/16 MMAs (M = 128, N = 128) into one of two TMEM
//               accumulators, so the epilogue of one tile overlaps the MMAs of the next.
//   warp 13     TMA producer of X tiles and W tiles ([K rows][64 columns] boxes, MN-major B operand; W is
//               re-streamed from L2 for every row tile).
// Every wait is bounded; on expiry the CTA raises a flag, drains and reports through mf_async_status().
#include <type_traits>

#include "evo_tc_common.cuh"

namespace mf {
namespace {
using namespace tcx;

constexpr int kRows = 128;          // rows of X per tile = TMEM lanes
constexpr int kNT = 128;            // output columns per MMA group
constexpr int kWorkers = 256;
constexpr int kNormWarps = 4;         // warps 8-11 normalise rows; warp 12 issues MMAs, warp 13 TMA loads
constexpr int kThreads = 512;          // four warpgroups: two of epilogue warps, one of normalising warps, one of issuers
constexpr int kWStages = 2;
constexpr int kAStages = 3;         // X tiles in flight (TMA prefetch two tiles ahead)

struct LnlP {
  int64_t M; int K, N, n_mt, n_nt;
  float eps;
  uint32_t ab_fmt;
  const void *x, *gamma, *beta, *bias;
  float *mean, *rstd;
  int* status;
};

struct Bars {
  uint64_t x_full[kAStages], a_full[kAStages], a_empty[kAStages], w_full[kWStages], w_empty[kWStages], acc_full[2], acc_empty[2];
};

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

template <int K, typename T>
__global__ void __launch_bounds__(kThreads, 1)
lnl_fwd_tc_kernel(const __grid_constant__ CUtensorMap mx, const __grid_constant__ CUtensorMap mw,
                  const __grid_constant__ CUtensorMap my, const LnlP p) {
  constexpr int EPL = K / 32;                 // elements of a row per lane
  constexpr int ATOMS = K / 64;               // 64-element swizzle atoms along K
  constexpr int A_BYTES = kRows * K * 2;
  constexpr int W_BYTES = K * kNT * 2;        // one 128-column tile of W: two [K][64] boxes
  constexpr int Y_BYTES = kRows * kNT * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;                         // [kAStages][ATOMS][128 rows][128 B]: raw X from TMA, normalised in place
  uint8_t* sW = sA + kAStages * A_BYTES;             // [kWStages][2][K rows][128 B]
  uint8_t* sY = sW + kWStages * W_BYTES;      // [2][2][128 rows][128 B]

  __shared__ Bars bar;
  __shared__ float gam_s[K], bet_s[K];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    abort_s = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar.acc_full[i], 1); mbar_init(&bar.acc_empty[i], 8);
    }
    for (int i = 0; i < kWStages; ++i) { mbar_init(&bar.w_full[i], 1); mbar_init(&bar.w_empty[i], 1); }
    for (int i = 0; i < kAStages; ++i) { mbar_init(&bar.x_full[i], 1); mbar_init(&bar.a_full[i], 4); mbar_init(&bar.a_empty[i], 1); }
    mbar_fence_init();
    prefetch_tmap(&mw); prefetch_tmap(&my); prefetch_tmap(&mx);
  }
  for (int k = tid; k < K; k += kThreads) {
    gam_s[k] = to_f(static_cast<const T*>(p.gamma)[k]);
    bet_s[k] = p.beta ? to_f(static_cast<const T*>(p.beta)[k]) : 0.f;
  }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  volatile int* abort_flag = &abort_s;
  const uint32_t tm0 = tmem_base_s;
  // Register re-partition (the CTA is launched with 128 per thread): the issuer warpgroup keeps 40, the epilogue
  // warpgroups get 152 and the normalising warpgroup 168; 256 * 152 + 128 * 168 + 128 * 40 = 512 * 128 exactly.
  static_assert(256 * 152 + 128 * 168 + 128 * 40 <= kThreads * 128, "setmaxnreg budget");
  // (each setmaxnreg sits inside its role's branch: the compiler allocates registers per region)
  const int my_tiles = p.n_mt > (int)blockIdx.x ? (p.n_mt - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

  if (warp < 8 + kNormWarps) {
    // ------------------------------------------------------------------------------------ epilogue warps 0-7,
    // normalising warps 8-11
    const int row_l = (warp & 3) * 32 + lane;        // my row of the tile (= my TMEM lane in the epilogue)
    const int half = warp >> 2;                      // epilogue: my 64-column half of the 128-column tile
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t acc_cnt = 0;                            // accumulator tiles consumed (buffer = acc_cnt & 1)

    // LayerNorm in place: the raw rows of X arrive by TMA in the layout the MMA wants (K-major, 128B swizzle); the
    // threads of warps 0-3 own one row each, read it from shared memory (conflict free thanks to the swizzle),
    // compute mean / variance in two passes in fp32 and write the normalised 16-bit row back over the raw one.
    auto normalise = [&](int t_local) {
      const int buf = t_local % kAStages;
      const int64_t row = ((int64_t)blockIdx.x + (int64_t)t_local * gridDim.x) * kRows + row_l;
      wait_or_flag(&bar.x_full[buf], (t_local / kAStages) & 1, abort_flag);
      uint8_t* a = sA + buf * A_BYTES;
      uint4 raw[K / 8];
#pragma unroll
      for (int c = 0; c < K / 8; ++c)
        raw[c] = *reinterpret_cast<const uint4*>(a + (c >> 3) * (kRows * 128) + swz_offset(row_l, c & 7, 128));
      float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < K / 8; ++c) {
        const float2 f0 = Pack2<T>::unpack(raw[c].x), f1 = Pack2<T>::unpack(raw[c].y), f2 = Pack2<T>::unpack(raw[c].z), f3 = Pack2<T>::unpack(raw[c].w);
        s4[0] += f0.x + f0.y; s4[1] += f1.x + f1.y; s4[2] += f2.x + f2.y; s4[3] += f3.x + f3.y;
      }
      const float mu = ((s4[0] + s4[1]) + (s4[2] + s4[3])) * (1.f / K);
      float q4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < K / 8; ++c) {
        const uint32_t u[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = Pack2<T>::unpack(u[e]);
          const float d0 = f.x - mu, d1 = f.y - mu;
          q4[e] = fmaf(d0, d0, q4[e]); q4[e] = fmaf(d1, d1, q4[e]);
        }
      }
      const float rs = rsqrtf(((q4[0] + q4[1]) + (q4[2] + q4[3])) * (1.f / K) + p.eps);
      const bool ok = row < p.M;
      if (ok) { p.mean[row] = mu; p.rstd[row] = rs; }
#pragma unroll
      for (int c = 0; c < K / 8; ++c) {
        const uint32_t u[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = Pack2<T>::unpack(u[e]);
          const int k = c * 8 + e * 2;
          const float y0 = fmaf((f.x - mu) * rs, gam_s[k], bet_s[k]), y1 = fmaf((f.y - mu) * rs, gam_s[k + 1], bet_s[k + 1]);
          o[e] = ok ? Pack2<T>::pack(y0, y1) : 0u;      // rows beyond M arrive as zeros from TMA and stay zero
        }
        *reinterpret_cast<uint4*>(a + (c >> 3) * (kRows * 128) + swz_offset(row_l, c & 7, 128)) = make_uint4(o[0], o[1], o[2], o[3]);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.a_full[buf]);
    };

    if (warp >= 8) {
      // the normalising warps run ahead of the MMAs as far as the ring of X tiles allows
      asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
      for (int t = 0; t < my_tiles && !*abort_flag; ++t) normalise(t);
    } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
    bool dead = false;
    for (int t = 0; t < my_tiles && !dead; ++t) {
      const int64_t row0 = ((int64_t)blockIdx.x + (int64_t)t * gridDim.x) * kRows;
      for (int nt = 0; nt < p.n_nt; ++nt, ++acc_cnt) {
        const int ab = acc_cnt & 1;
        const int n0 = nt * kNT + half * 64;
        // the linear bias of my 64 columns, requested before the wait for the accumulator so that its latency is hidden
        // (loaded inside the conversion loop, each of the eight loads exposed its full latency: 1300 of the 2400 cycles
        // an epilogue warp spent per tile)
        const T* bias = static_cast<const T*>(p.bias);
        const bool bias_vec = bias && (n0 + 64 <= p.N) && ((reinterpret_cast<uintptr_t>(bias) & 15) == 0);
        uint4 braw[8];
        if (bias_vec) {
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) braw[ch] = __ldg(reinterpret_cast<const uint4*>(bias + n0 + ch * 8));
        }
        wait_or_flag(&bar.acc_full[ab], (acc_cnt >> 1) & 1, abort_flag);
        tc_fence_after();
        uint32_t acc[64];
        tmem_ld32(tm0 + ab * kNT + half * 64 + lane_addr, *reinterpret_cast<uint32_t (*)[32]>(acc));
        tmem_ld32(tm0 + ab * kNT + half * 64 + 32 + lane_addr, *reinterpret_cast<uint32_t (*)[32]>(acc + 32));
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar.acc_empty[ab]);
        // Every warp stages and stores its own [32 rows][64 columns] slab, so the epilogue warps never wait for each
        // other.  Slab `ab` was handed to a TMA store by this warp two tiles ago: make sure it has been read.
        uint8_t* ys = sY + ab * Y_BYTES + half * (kRows * 128);
        if (lane == 0) bulk_wait_group_read<1>();
        if (__any_sync(0xffffffffu, *abort_flag)) { dead = true; break; }
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          float b8[8];
          if (bias_vec) {
            const uint4 u = braw[ch];
            const float2 f0 = Pack2<T>::unpack(u.x), f1 = Pack2<T>::unpack(u.y), f2 = Pack2<T>::unpack(u.z), f3 = Pack2<T>::unpack(u.w);
            b8[0] = f0.x; b8[1] = f0.y; b8[2] = f1.x; b8[3] = f1.y; b8[4] = f2.x; b8[5] = f2.y; b8[6] = f3.x; b8[7] = f3.y;
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int n = n0 + ch * 8 + e;
              b8[e] = (bias && n < p.N) ? to_f(bias[n]) : 0.f;
            }
          }
          uint4 v;
          v.x = Pack2<T>::pack(__uint_as_float(acc[ch * 8]) + b8[0], __uint_as_float(acc[ch * 8 + 1]) + b8[1]);
          v.y = Pack2<T>::pack(__uint_as_float(acc[ch * 8 + 2]) + b8[2], __uint_as_float(acc[ch * 8 + 3]) + b8[3]);
          v.z = Pack2<T>::pack(__uint_as_float(acc[ch * 8 + 4]) + b8[4], __uint_as_float(acc[ch * 8 + 5]) + b8[5]);
          v.w = Pack2<T>::pack(__uint_as_float(acc[ch * 8 + 6]) + b8[6], __uint_as_float(acc[ch * 8 + 7]) + b8[7]);
          *reinterpret_cast<uint4*>(ys + swz_offset(row_l, ch, 128)) = v;
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          // [64 columns][32 rows] box; TMA clips rows >= M and columns >= N (a slab wholly beyond N is skipped)
          if (n0 < p.N && row0 + (warp & 3) * 32 < p.M) tma_store_2d(&my, ys + (warp & 3) * (32 * 128), n0, (int)row0 + (warp & 3) * 32);
          bulk_commit_group();
        }
      }
    }
    if (lane == 0) bulk_wait_group<0>();
    }
  } else {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  if (warp == 8 + kNormWarps && lane == 0) {
    // ------------------------------------------------------------------------------------ MMA issuer
    const uint32_t idesc = idesc_f16(128, kNT, p.ab_fmt, 0, 1);     // A K-major, B MN-major
    uint32_t acc_cnt = 0, w_cnt = 0;
    for (int t = 0; t < my_tiles && !*abort_flag; ++t) {
      const int buf = t % kAStages;
      wait_or_flag(&bar.a_full[buf], (t / kAStages) & 1, abort_flag);
      const uint32_t a_lo = desc_lo(smem_u32(sA + buf * A_BYTES), 16);
      for (int nt = 0; nt < p.n_nt; ++nt, ++acc_cnt, ++w_cnt) {
        const int ab = acc_cnt & 1, ws = w_cnt % kWStages;
        wait_or_flag(&bar.w_full[ws], (w_cnt / kWStages) & 1, abort_flag);
        if (acc_cnt >= 2) wait_or_flag(&bar.acc_empty[ab], ((acc_cnt >> 1) - 1) & 1, abort_flag);
        tc_fence_after();
        if (*abort_flag) break;
        const uint32_t w_lo = desc_lo(smem_u32(sW + ws * W_BYTES), K * 128);
#pragma unroll
        for (int ks = 0; ks < K / 16; ++ks)
          mma_ss_lh(tm0 + ab * kNT, a_lo + (ks >> 2) * (kRows * 128 / 16) + (ks & 3) * 2, desc_hi(1024, kSw128),
                    w_lo + ks * (2048 / 16), desc_hi(1024, kSw128), idesc, ks > 0);
        tc_commit(&bar.acc_full[ab]);
        tc_commit(&bar.w_empty[ws]);
      }
      tc_commit(&bar.a_empty[buf]);
    }
  } else if (warp == 9 + kNormWarps && lane == 0) {
    // ------------------------------------------------------------------------------------ TMA producer of X and W tiles
    uint32_t w_cnt = 0;
    auto load_x = [&](int t_local) {
      const int buf = t_local % kAStages;
      if (t_local >= kAStages) wait_or_flag(&bar.a_empty[buf], ((t_local / kAStages) - 1) & 1, abort_flag);
      const int row0 = (int)(((int64_t)blockIdx.x + (int64_t)t_local * gridDim.x) * kRows);
      mbar_expect_tx(&bar.x_full[buf], A_BYTES);
#pragma unroll
      for (int at = 0; at < ATOMS; ++at)
        tma_load_2d(sA + buf * A_BYTES + at * (kRows * 128), &mx, &bar.x_full[buf], at * 64, row0);
    };
    for (int t = 0; t < my_tiles && t < kAStages - 1; ++t) load_x(t);
    for (int t = 0; t < my_tiles && !*abort_flag; ++t) {
      if (t + kAStages - 1 < my_tiles) load_x(t + kAStages - 1);
      for (int nt = 0; nt < p.n_nt; ++nt, ++w_cnt) {
        const int ws = w_cnt % kWStages;
        if (w_cnt >= kWStages) wait_or_flag(&bar.w_empty[ws], ((w_cnt / kWStages) - 1) & 1, abort_flag);
        if (*abort_flag) break;
        mbar_expect_tx(&bar.w_full[ws], W_BYTES);
        tma_load_2d(sW + ws * W_BYTES, &mw, &bar.w_full[ws], nt * kNT, 0);
        tma_load_2d(sW + ws * W_BYTES + K * 128, &mw, &bar.w_full[ws], nt * kNT + 64, 0);
      }
    }
  }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_s) *reinterpret_cast<volatile int*>(p.status) = 1;
  if (warp == 0) tmem_dealloc(tmem_base_s, 256);
}

template <int K, typename T>
int launch_lnl(const mf_lnl_fwd_args& a, cudaStream_t st) {
  CUtensorMap mx, mw, my;
  int r;
  {
    const int64_t dims[2] = {K, a.M}, str[2] = {1, K};
    const int box[2] = {64, kRows};
    if ((r = make_tiled_map(&mx, a.x, a.dtype, 2, dims, str, box, 128))) return r;
  }
  {
    const int64_t dims[2] = {a.N, K}, str[2] = {1, a.N};
    const int box[2] = {64, K};
    if ((r = make_tiled_map(&mw, a.w, a.dtype, 2, dims, str, box, 128))) return r;
  }
  {
    const int64_t dims[2] = {a.N, a.M}, str[2] = {1, a.N};
    const int box[2] = {64, 32};                 // one epilogue warp's slab
    if ((r = make_tiled_map(&my, a.y, a.dtype, 2, dims, str, box, 128))) return r;
  }
  LnlP p{};
  p.M = a.M; p.K = K; p.N = a.N;
  p.n_mt = (int)((a.M + kRows - 1) / kRows);
  p.n_nt = (a.N + kNT - 1) / kNT;
  p.eps = a.eps;
  p.ab_fmt = a.dtype == MF_BF16 ? 1u : 0u;
  p.x = a.x; p.gamma = a.ln_w; p.beta = a.ln_b; p.bias = a.b;
  p.mean = a.mean; p.rstd = a.rstd;
  p.status = status_word();
  MF_REQUIRE(p.status, MF_ERR_CUDA, "could not allocate the device status word");
  MF_REQUIRE(tc_async_status() == 0, MF_ERR_CUDA, "an earlier tensor-core kernel gave up on a bounded wait; results are invalid");
  const size_t smem = 1024 + kAStages * (size_t)kRows * K * 2 + kWStages * (size_t)K * kNT * 2 + 2 * (size_t)kRows * kNT * 2;
  auto kern = lnl_fwd_tc_kernel<K, T>;
  MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int grid = sm_count();
  if (grid > p.n_mt) grid = p.n_mt;
  kern<<<grid, kThreads, smem, st>>>(mx, mw, my, p);
  MF_LAUNCHED("lnl_fwd_tc_kernel");
  return MF_OK;
}

}  // namespace

bool lnl_fwd_tc_supported(const mf_lnl_fwd_args& a) {
  if (a.dtype != MF_BF16 && a.dtype != MF_F16) return false;
  if (a.K != 64 && a.K != 128) return false;
  if (a.N % 8 != 0 || a.M < 1 || a.M > (int64_t)INT32_MAX) return false;
  const uintptr_t al = reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.w) | reinterpret_cast<uintptr_t>(a.y);
  return (al & 15) == 0;
}

int lnl_fwd_tc(const mf_lnl_fwd_args& a, cudaStream_t st) {
  if (a.dtype == MF_BF16) return a.K == 128 ? launch_lnl<128, __nv_bfloat16>(a, st) : launch_lnl<64, __nv_bfloat16>(a, st);
  return a.K == 128 ? launch_lnl<128, __half>(a, st) : launch_lnl<64, __half>(a, st);
}

}  // namespace mf
