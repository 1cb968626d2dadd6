// Fused Transition forward on the tensor cores:
//     Y[M, dim] = ( silu(H[:, inner:]) * H[:, :inner] ) W2^T,   H = LayerNorm(X) W1,   dim in {64, 128}.
// The hidden activation H [M, 2*inner] and the gated product never leave the SM.
//
// Persistent CTA per SM, 128-row tiles of X.  Per tile the hidden dimension is walked in chunks of 64:
//   TMA warp     X tile (raw rows, K-major, 128B swizzle) two tiles ahead; per chunk the two W1 column blocks
//                (value half and gate half, [dim rows][64 columns], MN-major B operands) and the W2 block
//                ([dim rows][64 hidden], K-major B operand).
//   row threads  (warps 8-11, a warpgroup of their own) LayerNorm of the next tile in place in shared memory, as in
//                the LayernormLinear kernel, ahead of the MMAs by as much as the ring of X tiles allows.
//   MMA threads  (warp 12 and warp 14, one GEMM each) GEMM1 of chunk c: H_a, H_g = A W1 blocks (2 x dim/16 MMAs, N = 64) into one of two TMEM buffers;
//                GEMM2 of chunk c-1: Y += G W2-block^T (4 MMAs, N = dim) once the workers have written G.
//   workers      (warps 0-7) thread (row, half): 32 columns of H_a and H_g from TMEM, g = silu(gate) * value with
//                one MUFU op per element (silu(x) = x/2 * (1 + tanh(x/2))), packed 16-bit G tile to shared memory
//                (K-major A operand of GEMM2); after the last chunk the Y tile goes TMEM -> registers -> swizzled
//                staging -> TMA store.
// GEMM1 of the next chunk overlaps the gating of the current one (two H buffers, two G tiles, two weight stages).
// Every wait is bounded; on expiry the CTA raises a flag, drains and reports through mf_async_status().
#include <type_traits>

#include "evo_tc_common.cuh"

namespace mf {
namespace {
using namespace tcx;

constexpr int kRows = 128;
constexpr int kHC = 64;             // hidden columns per chunk
constexpr int kWorkers = 256;
constexpr int kThreads = 512;          // warpgroups: 0-1 SwiGLU / output workers, 2 normalising warps, 3 issuers (warp 12 MMA, warp 13 TMA)
constexpr int kAStages = 2;
constexpr int kWStages = 2;

struct TrP {
  int64_t M; int dim, inner, n_mt, n_ch;
  float eps;
  uint32_t ab_fmt;
  int has_ln;
  const void *x, *gamma, *beta;
  float *mean, *rstd;
  int* status;
};

struct Bars {
  uint64_t x_full[kAStages], a_full[kAStages], a_empty[kAStages];
  uint64_t w1_full[kWStages], w1_empty[kWStages], w2_full[kWStages], w2_empty[kWStages];
  uint64_t h_full[2], h_empty[2], g_full[2], g_empty[2], y_full, y_empty;
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
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int K, typename T>
__global__ void __launch_bounds__(kThreads, 1)
transition_fwd_tc_kernel(const __grid_constant__ CUtensorMap mx, const __grid_constant__ CUtensorMap mw1,
                         const __grid_constant__ CUtensorMap mw2, const __grid_constant__ CUtensorMap my, const TrP p) {
  constexpr int ATOMS = K / 64;
  constexpr int A_BYTES = kRows * K * 2;
  constexpr int W1B = K * 128;                 // one [K rows][64 columns] block of W1
  constexpr int W2B = K * 128;                 // one [dim = K rows][64 hidden] block of W2
  constexpr int W_BYTES = 2 * W1B + W2B;
  constexpr int G_BYTES = kRows * 128;         // [128 rows][64 hidden] 16-bit
  constexpr int Y_BYTES = kRows * K * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sW = sA + kAStages * A_BYTES;
  uint8_t* sG = sW + kWStages * W_BYTES;
  uint8_t* sY = sG + 2 * G_BYTES;

  __shared__ Bars bar;
  __shared__ float gam_s[K], bet_s[K];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    abort_s = 0;
    for (int i = 0; i < kAStages; ++i) { mbar_init(&bar.x_full[i], 1); mbar_init(&bar.a_full[i], 4); mbar_init(&bar.a_empty[i], 1); }
    for (int i = 0; i < kWStages; ++i) {
      mbar_init(&bar.w1_full[i], 1); mbar_init(&bar.w1_empty[i], 1);
      mbar_init(&bar.w2_full[i], 1); mbar_init(&bar.w2_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar.h_full[i], 1); mbar_init(&bar.h_empty[i], 8);
      mbar_init(&bar.g_full[i], 8); mbar_init(&bar.g_empty[i], 1);
    }
    mbar_init(&bar.y_full, 1); mbar_init(&bar.y_empty, 8);
    mbar_fence_init();
    prefetch_tmap(&mx); prefetch_tmap(&mw1); prefetch_tmap(&mw2); prefetch_tmap(&my);
  }
  for (int k = tid; k < K; k += kThreads) {
    gam_s[k] = p.has_ln ? to_f(static_cast<const T*>(p.gamma)[k]) : 1.f;
    bet_s[k] = (p.has_ln && p.beta) ? to_f(static_cast<const T*>(p.beta)[k]) : 0.f;
  }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  volatile int* abort_flag = &abort_s;
  const uint32_t tm0 = tmem_base_s;
  const uint32_t tH = tm0, tY = tm0 + 256;        // H: two buffers of (value 64 | gate 64); Y: K columns
  const int my_tiles = p.n_mt > (int)blockIdx.x ? (p.n_mt - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int nch = p.n_ch;

  // Register re-partition (launched with 128 per thread): issuers keep 40, workers get 152, the normalising
  // warpgroup 168; 256 * 152 + 128 * 168 + 128 * 40 = 512 * 128.  Each setmaxnreg sits inside its role's branch.
  static_assert(256 * 152 + 128 * 168 + 128 * 40 <= kThreads * 128, "setmaxnreg budget");
  if (warp < 12) {
    // ------------------------------------------------------------------------------------ workers (warps 0-7),
    // normalising warps (8-11)
    const int row_l = (warp & 3) * 32 + lane;
    const int half = warp >> 2;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t ch_cnt = 0;                            // chunks consumed (H / G buffer = ch_cnt & 1)

    auto normalise = [&](int t_local) {
      const int buf = t_local % kAStages;
      const int64_t row = ((int64_t)blockIdx.x + (int64_t)t_local * gridDim.x) * kRows + row_l;
      wait_or_flag(&bar.x_full[buf], (t_local / kAStages) & 1, abort_flag);
      if (p.has_ln) {
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
            o[e] = ok ? Pack2<T>::pack(y0, y1) : 0u;
          }
          *reinterpret_cast<uint4*>(a + (c >> 3) * (kRows * 128) + swz_offset(row_l, c & 7, 128)) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        fence_async_smem();
      }
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
      const int row0 = (int)(((int64_t)blockIdx.x + (int64_t)t * gridDim.x) * kRows);
      for (int c = 0; c < nch; ++c, ++ch_cnt) {
        const int hb = ch_cnt & 1;
        wait_or_flag(&bar.h_full[hb], (ch_cnt >> 1) & 1, abort_flag);
        tc_fence_after();
        uint32_t ha[32], hg[32];
        tmem_ld32(tH + hb * 128 + half * 32 + lane_addr, ha);
        tmem_ld32(tH + hb * 128 + 64 + half * 32 + lane_addr, hg);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar.h_empty[hb]);
        uint32_t gp[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float a0 = __uint_as_float(ha[2 * e]), a1 = __uint_as_float(ha[2 * e + 1]);
          const float b0 = 0.5f * __uint_as_float(hg[2 * e]), b1 = 0.5f * __uint_as_float(hg[2 * e + 1]);
          // silu(b) * a = b/2 * (1 + tanh(b/2)) * a
          const float g0 = fmaf(b0, tanh_approx(b0), b0) * a0, g1 = fmaf(b1, tanh_approx(b1), b1) * a1;
          gp[e] = Pack2<T>::pack(g0, g1);
        }
        if (ch_cnt >= 2) wait_or_flag(&bar.g_empty[hb], ((ch_cnt >> 1) - 1) & 1, abort_flag);
        uint8_t* g = sG + hb * G_BYTES;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
          *reinterpret_cast<uint4*>(g + swz_offset(row_l, half * 4 + ch, 128)) = make_uint4(gp[ch * 4], gp[ch * 4 + 1], gp[ch * 4 + 2], gp[ch * 4 + 3]);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar.g_full[hb]);
      }
      // ---- Y tile: TMEM -> registers -> staging -> TMA store
      wait_or_flag(&bar.y_full, t & 1, abort_flag);
      tc_fence_after();
      uint32_t acc[K / 2];
#pragma unroll
      for (int cb = 0; cb < K / 64; ++cb)
        tmem_ld32(tY + half * (K / 2) + cb * 32 + lane_addr, *reinterpret_cast<uint32_t (*)[32]>(acc + cb * 32));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.y_empty);
      if (tid == 0) bulk_wait_group_read<0>();
      if (named_sync_or(2, kWorkers, *abort_flag)) { dead = true; break; }
      // thread (row, half) holds columns [half*K/2, +K/2): K = 128 -> atom `half`, all 8 chunks; K = 64 -> atom 0, chunks half*4..
#pragma unroll
      for (int ch = 0; ch < K / 16; ++ch) {
        uint4 v;
        v.x = Pack2<T>::pack(__uint_as_float(acc[ch * 8]), __uint_as_float(acc[ch * 8 + 1]));
        v.y = Pack2<T>::pack(__uint_as_float(acc[ch * 8 + 2]), __uint_as_float(acc[ch * 8 + 3]));
        v.z = Pack2<T>::pack(__uint_as_float(acc[ch * 8 + 4]), __uint_as_float(acc[ch * 8 + 5]));
        v.w = Pack2<T>::pack(__uint_as_float(acc[ch * 8 + 6]), __uint_as_float(acc[ch * 8 + 7]));
        const int col_chunk = half * (K / 16) + ch;           // 16-byte chunk index inside the K-column row
        *reinterpret_cast<uint4*>(sY + (col_chunk >> 3) * (kRows * 128) + swz_offset(row_l, col_chunk & 7, 128)) = v;
      }
      fence_async_smem();
      named_sync(2, kWorkers);
      if (tid == 0) {
#pragma unroll
        for (int at = 0; at < ATOMS; ++at) tma_store_2d(&my, sY + at * (kRows * 128), at * 64, row0);
        bulk_commit_group();
      }
    }
    if (tid == 0) bulk_wait_group<0>();
    }
  } else {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  if (warp == 12 && lane == 0) {
    // ------------------------------------------------------------------------------------ MMA issuer
    const uint32_t id1 = idesc_f16(128, kHC, p.ab_fmt, 0, 1);     // GEMM1: A K-major, B (W1 block) MN-major, N = 64
    uint32_t ch_cnt = 0;
    for (int t = 0; t < my_tiles && !*abort_flag; ++t) {
      const int buf = t % kAStages;
      wait_or_flag(&bar.a_full[buf], (t / kAStages) & 1, abort_flag);
      const uint32_t a_lo = desc_lo(smem_u32(sA + buf * A_BYTES), 16);
      for (int c = 0; c < nch && !*abort_flag; ++c, ++ch_cnt) {
        const int hb = ch_cnt & 1, ws = ch_cnt % kWStages;
        wait_or_flag(&bar.w1_full[ws], (ch_cnt / kWStages) & 1, abort_flag);
        if (ch_cnt >= 2) wait_or_flag(&bar.h_empty[hb], ((ch_cnt >> 1) - 1) & 1, abort_flag);
        tc_fence_after();
        if (*abort_flag) break;
        const uint32_t w1v_lo = desc_lo(smem_u32(sW + ws * W_BYTES), 16), w1g_lo = desc_lo(smem_u32(sW + ws * W_BYTES + W1B), 16);
#pragma unroll
        for (int ks = 0; ks < K / 16; ++ks)      // value half
          mma_ss_lh(tH + hb * 128, a_lo + (ks >> 2) * (kRows * 128 / 16) + (ks & 3) * 2, desc_hi(1024, kSw128),
                    w1v_lo + ks * (2048 / 16), desc_hi(1024, kSw128), id1, ks > 0);
#pragma unroll
        for (int ks = 0; ks < K / 16; ++ks)      // gate half
          mma_ss_lh(tH + hb * 128 + 64, a_lo + (ks >> 2) * (kRows * 128 / 16) + (ks & 3) * 2, desc_hi(1024, kSw128),
                    w1g_lo + ks * (2048 / 16), desc_hi(1024, kSw128), id1, ks > 0);
        tc_commit(&bar.h_full[hb]);
        tc_commit(&bar.w1_empty[ws]);
      }
      if (*abort_flag) break;
      tc_commit(&bar.a_empty[buf]);
    }
  } else if (warp == 14 && lane == 0) {
    // ------------------------------------------------------------------------------------ second MMA issuer: GEMM2.
    // One thread issuing both GEMMs spends a chunk's time on its own waits, descriptors and commits (about 3200 cycles
    // per chunk measured, against 1250 of worker time); two threads run those two instruction streams side by side.
    const uint32_t id2 = idesc_f16(128, K, p.ab_fmt, 0, 0);       // A (G) K-major, B (W2 block) K-major, N = dim
    auto gemm2 = [&](uint32_t cc, bool first_of_tile, int t) {    // Y (+)= G(cc) W2-block(cc)^T
      const int gb = cc & 1, ws = cc % kWStages;
      wait_or_flag(&bar.w2_full[ws], (cc / kWStages) & 1, abort_flag);
      wait_or_flag(&bar.g_full[gb], (cc >> 1) & 1, abort_flag);
      if (first_of_tile && t > 0) wait_or_flag(&bar.y_empty, (t - 1) & 1, abort_flag);
      tc_fence_after();
      if (*abort_flag) return;
      const uint32_t g_lo = desc_lo(smem_u32(sG + gb * G_BYTES), 16), w2_lo = desc_lo(smem_u32(sW + ws * W_BYTES + 2 * W1B), 16);
#pragma unroll
      for (int ks = 0; ks < kHC / 16; ++ks)
        mma_ss_lh(tY, g_lo + ks * 2, desc_hi(1024, kSw128), w2_lo + ks * 2, desc_hi(1024, kSw128), id2, !first_of_tile || ks > 0);
      tc_commit(&bar.g_empty[gb]);
      tc_commit(&bar.w2_empty[ws]);
    };
    uint32_t ch_cnt = 0;
    for (int t = 0; t < my_tiles && !*abort_flag; ++t) {
      for (int c = 0; c < nch && !*abort_flag; ++c, ++ch_cnt) gemm2(ch_cnt, c == 0, t);
      if (*abort_flag) break;
      tc_commit(&bar.y_full);
    }
  } else if (warp == 13 && lane == 0) {
    // ------------------------------------------------------------------------------------ TMA producer
    uint32_t ch_cnt = 0;
    auto load_x = [&](int t_local) {
      const int buf = t_local % kAStages;
      if (t_local >= kAStages) wait_or_flag(&bar.a_empty[buf], ((t_local / kAStages) - 1) & 1, abort_flag);
      const int row0 = (int)(((int64_t)blockIdx.x + (int64_t)t_local * gridDim.x) * kRows);
      mbar_expect_tx(&bar.x_full[buf], A_BYTES);
#pragma unroll
      for (int at = 0; at < ATOMS; ++at)
        tma_load_2d(sA + buf * A_BYTES + at * (kRows * 128), &mx, &bar.x_full[buf], at * 64, row0);
    };
    if (my_tiles > 0) load_x(0);
    for (int t = 0; t < my_tiles && !*abort_flag; ++t) {
      if (t + 1 < my_tiles) load_x(t + 1);
      for (int c = 0; c < nch; ++c, ++ch_cnt) {
        const int ws = ch_cnt % kWStages;
        uint8_t* w = sW + ws * W_BYTES;
        // the W1 blocks of a stage are free once GEMM1 of its previous chunk is done, the W2 block only after GEMM2
        if (ch_cnt >= kWStages) wait_or_flag(&bar.w1_empty[ws], ((ch_cnt / kWStages) - 1) & 1, abort_flag);
        if (*abort_flag) break;
        mbar_expect_tx(&bar.w1_full[ws], 2 * W1B);
        tma_load_2d(w, &mw1, &bar.w1_full[ws], c * kHC, 0);                    // value columns of W1
        tma_load_2d(w + W1B, &mw1, &bar.w1_full[ws], p.inner + c * kHC, 0);   // gate columns of W1
        if (ch_cnt >= kWStages) wait_or_flag(&bar.w2_empty[ws], ((ch_cnt / kWStages) - 1) & 1, abort_flag);
        if (*abort_flag) break;
        mbar_expect_tx(&bar.w2_full[ws], W2B);
        tma_load_2d(w + 2 * W1B, &mw2, &bar.w2_full[ws], c * kHC, 0);          // W2[:, chunk]
      }
    }
  }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_s) *reinterpret_cast<volatile int*>(p.status) = 1;
  if (warp == 0) tmem_dealloc(tmem_base_s, 512);
}

template <int K, typename T>
int launch_tr(const mf_transition_fwd_args& a, cudaStream_t st) {
  CUtensorMap mx, mw1, mw2, my;
  int r;
  {
    const int64_t dims[2] = {K, a.M}, str[2] = {1, K};
    const int box[2] = {64, kRows};
    if ((r = make_tiled_map(&mx, a.x, a.dtype, 2, dims, str, box, 128))) return r;
    if ((r = make_tiled_map(&my, a.y, a.dtype, 2, dims, str, box, 128))) return r;
  }
  {
    const int64_t dims[2] = {2 * (int64_t)a.inner, K}, str[2] = {1, 2 * (int64_t)a.inner};
    const int box[2] = {64, K};
    if ((r = make_tiled_map(&mw1, a.w1, a.dtype, 2, dims, str, box, 128))) return r;
  }
  {
    const int64_t dims[2] = {a.inner, K}, str[2] = {1, a.inner};
    const int box[2] = {64, K};
    if ((r = make_tiled_map(&mw2, a.w2, a.dtype, 2, dims, str, box, 128))) return r;
  }
  TrP p{};
  p.M = a.M; p.dim = K; p.inner = a.inner;
  p.n_mt = (int)((a.M + kRows - 1) / kRows);
  p.n_ch = a.inner / kHC;
  p.eps = a.eps;
  p.ab_fmt = a.dtype == MF_BF16 ? 1u : 0u;
  p.has_ln = a.ln_w != nullptr;
  p.x = a.x; p.gamma = a.ln_w; p.beta = a.ln_b;
  p.mean = a.mean; p.rstd = a.rstd;
  p.status = status_word();
  MF_REQUIRE(p.status, MF_ERR_CUDA, "could not allocate the device status word");
  MF_REQUIRE(tc_async_status() == 0, MF_ERR_CUDA, "an earlier tensor-core kernel gave up on a bounded wait; results are invalid");
  const size_t smem = 1024 + kAStages * (size_t)kRows * K * 2 + kWStages * (size_t)(3 * K * 128) + 2 * (size_t)kRows * 128 +
                      (size_t)kRows * K * 2;
  auto kern = transition_fwd_tc_kernel<K, T>;
  MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int grid = sm_count();
  if (grid > p.n_mt) grid = p.n_mt;
  kern<<<grid, kThreads, smem, st>>>(mx, mw1, mw2, my, p);
  MF_LAUNCHED("transition_fwd_tc_kernel");
  return MF_OK;
}

}  // namespace

bool transition_fwd_tc_supported(const mf_transition_fwd_args& a) {
  if (a.dtype != MF_BF16 && a.dtype != MF_F16) return false;
  if (a.dim != 64 && a.dim != 128) return false;
  if (a.inner % 64 != 0 || a.inner < 64 || a.M < 1 || a.M > (int64_t)INT32_MAX) return false;
  const uintptr_t al = reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.w1) | reinterpret_cast<uintptr_t>(a.w2) |
                       reinterpret_cast<uintptr_t>(a.y);
  return (al & 15) == 0;
}

int transition_fwd_tc(const mf_transition_fwd_args& a, cudaStream_t st) {
  if (a.dtype == MF_BF16) return a.dim == 128 ? launch_tr<128, __nv_bfloat16>(a, st) : launch_tr<64, __nv_bfloat16>(a, st);
  return a.dim == 128 ? launch_tr<128, __half>(a, st) : launch_tr<64, __half>(a, st);
}

}  // namespace mf
