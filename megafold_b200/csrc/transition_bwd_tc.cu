// Fused core of the Transition backward on the tensor cores (dim = 128, 16-bit types):
//
//     h = LayerNorm(x) W1          (recomputed, never stored)            g  = silu(h_gate) * h_value   -> HBM (for dW2)
//     dg = dy W2                                                          dh = SwiGLU'(h, dg)           -> HBM (for dW1)
//     dyln = dh W1^T               (accumulated on chip over the hidden dimension)                      -> HBM, fp32
//
// so that the [M, 2*inner] pre-activation and the [M, inner] gradient of the gated product never touch HBM, and
// g / dh are written exactly once.  The weight gradients (dW2 = dy^T g, dW1 = LN(x)^T dh) and the LayerNorm backward
// of dyln are separate, streaming kernels.
//
// Persistent CTA per SM, 128-row tiles, the hidden dimension walked in chunks of 32 (value) + 32 (gate) columns:
//   warp 13      TMA loads: X tile (two stages), dY tile, per chunk the W1 value / gate blocks and the W2 block
//                ([128 rows][32 columns], 64-byte swizzle; three stages).
//   warp 14      TMA stores of the dh and g tiles of every chunk.
//   warps 8-11   LayerNorm of the X tile in place (thread per row), one tile ahead.
//   warp 12      MMAs of H(c) = A W1blocks (8 x N=64, the two blocks as the two swizzle atoms of one MN-major B operand)
//                and DG(c) = dY W2block (8 x N=32) into one of two TMEM buffers.
//   warp 15      MMAs of dyln += dh(c) [W1 value block; W1 gate block]^T (4 x N=128; the same shared-memory blocks read
//                K-major) once the workers have written dh(c).
//   warps 0-7    workers, thread (row, half): 16 value, 16 gate, 16 dg columns from TMEM; g, dh in registers with one
//                MUFU op per element; 16-bit tiles to shared memory: dh as the K-major A operand of the dyln GEMM
//                (column order inside a chunk: [value 0-15 | gate 0-15 | value 16-31 | gate 16-31]) and both as
//                sources of the TMA stores.  After the last chunk: dyln TMEM ->
//                registers -> global (fp32).
// dh is stored chunk by chunk in that column order ([M][inner/32][64]); dW1 computed from it has its columns in the same
// order and is put back by a small kernel.
// Every wait is bounded; on expiry the CTA raises a flag, drains and reports through mf_async_status().
#include "evo_tc_common.cuh"

namespace mf {
namespace {
using namespace tcx;

constexpr int kRows = 128;
constexpr int K = 128;               // dim
constexpr int kHC = 32;              // hidden (value) columns per chunk
constexpr int kWorkers = 256;
constexpr int kThreads = 512;        // warpgroups: 0-1 workers, 2 normalising warps, 3 issuers (warp 12 MMA, warp 13 TMA)
constexpr int A_BYTES = kRows * K * 2;          // 32 KB: X / LN(X) tile or dY tile, two 64-column atoms
constexpr int WB = K * 64;                       // 8 KB: one [128 rows][32 columns] weight block
constexpr int W_BYTES = 3 * WB;                  // W1 value | W1 gate | W2
constexpr int DH_BYTES = kRows * 128;            // [128 rows][64 columns] 16 bit
constexpr int G_BYTES = kRows * 64;              // [128 rows][32 columns] 16 bit
constexpr int kWS = 3;                           // weight stages: a stage is released only by the dyln GEMM of its chunk,
                                                 // one chunk after its H / DG GEMMs, so two stages would stall the TMA refill

struct TbP {
  int64_t M; int inner, n_mt, n_ch;
  uint32_t ab_fmt;
  const void *x, *gamma, *beta;
  const float *mean, *rstd;
  float* dyln;
  int* status;
};

struct Bars {
  uint64_t x_full[2], a_full[2], a_empty[2], dy_full, dy_empty;
  uint64_t w_full[kWS], w_empty[kWS];
  uint64_t hd_full[2], hd_empty[2], dh_full[2], dh_empty[2], st_done[2], acc_full, acc_empty;
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

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
transition_bwd_tc_kernel(const __grid_constant__ CUtensorMap mx, const __grid_constant__ CUtensorMap mdy,
                         const __grid_constant__ CUtensorMap mw1, const __grid_constant__ CUtensorMap mw2,
                         const __grid_constant__ CUtensorMap mdh, const __grid_constant__ CUtensorMap mg, const TbP p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;                          // [2] X tiles, normalised in place
  uint8_t* sDY = sA + 2 * A_BYTES;             // dY tile
  uint8_t* sW = sDY + A_BYTES;                 // [kWS] weight stages
  uint8_t* sDH = sW + kWS * W_BYTES;           // [2] dh tiles
  uint8_t* sG = sDH + 2 * DH_BYTES;            // [2] g tiles

  __shared__ Bars bar;
  __shared__ float gam_s[K], bet_s[K];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    abort_s = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar.x_full[i], 1); mbar_init(&bar.a_full[i], 4); mbar_init(&bar.a_empty[i], 1);
      mbar_init(&bar.hd_full[i], 1); mbar_init(&bar.hd_empty[i], 8);
      mbar_init(&bar.dh_full[i], 8); mbar_init(&bar.dh_empty[i], 1); mbar_init(&bar.st_done[i], 1);
    }
    for (int i = 0; i < kWS; ++i) { mbar_init(&bar.w_full[i], 1); mbar_init(&bar.w_empty[i], 1); }
    mbar_init(&bar.dy_full, 1); mbar_init(&bar.dy_empty, 1);
    mbar_init(&bar.acc_full, 1); mbar_init(&bar.acc_empty, 8);
    mbar_fence_init();
    prefetch_tmap(&mx); prefetch_tmap(&mdy); prefetch_tmap(&mw1); prefetch_tmap(&mw2); prefetch_tmap(&mdh); prefetch_tmap(&mg);
  }
  for (int k = tid; k < K; k += kThreads) {
    gam_s[k] = to_f(static_cast<const T*>(p.gamma)[k]);
    bet_s[k] = p.beta ? to_f(static_cast<const T*>(p.beta)[k]) : 0.f;
  }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  volatile int* abort_flag = &abort_s;
  const uint32_t tm0 = tmem_base_s;
  // TMEM columns: two buffers of (H value 32 | H gate 32 | DG 32) at 0 and 128; dyln accumulator (128) at 256
  const uint32_t tHD = tm0, tACC = tm0 + 256;
  const int my_tiles = p.n_mt > (int)blockIdx.x ? (p.n_mt - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int nch = p.n_ch;
  // Register re-partition (launched with 128 per thread): issuers keep 40, workers get 152, the normalising
  // warpgroup 168; 256 * 152 + 128 * 168 + 128 * 40 = 512 * 128.  Each setmaxnreg sits inside its role's branch.
  static_assert(256 * 152 + 128 * 168 + 128 * 40 <= kThreads * 128, "setmaxnreg budget");

  if (warp < 12) {
    const int row_l = (warp & 3) * 32 + lane;
    if (warp >= 8) {
      // -------------------------------------------------------------------------------- normalising warps
      asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
      for (int t = 0; t < my_tiles && !*abort_flag; ++t) {
        const int buf = t & 1;
        const int64_t row = ((int64_t)blockIdx.x + (int64_t)t * gridDim.x) * kRows + row_l;
        wait_or_flag(&bar.x_full[buf], (t >> 1) & 1, abort_flag);
        uint8_t* a = sA + buf * A_BYTES;
        uint4 raw[K / 8];
#pragma unroll
        for (int c = 0; c < K / 8; ++c)
          raw[c] = *reinterpret_cast<const uint4*>(a + (c >> 3) * (kRows * 128) + swz_offset(row_l, c & 7, 128));
        const bool ok = row < p.M;
        const float mu = ok ? p.mean[row] : 0.f, rs = ok ? p.rstd[row] : 0.f;     // saved by the forward pass
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
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar.a_full[buf]);
      }
    } else {
      // -------------------------------------------------------------------------------- workers
      asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
      const int half = warp >> 2;
      const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
      uint32_t ch_cnt = 0;
      bool dead = false;
      for (int t = 0; t < my_tiles && !dead; ++t) {
        const int row0 = (int)(((int64_t)blockIdx.x + (int64_t)t * gridDim.x) * kRows);
        for (int c = 0; c < nch; ++c, ++ch_cnt) {
          const int hb = ch_cnt & 1;
          wait_or_flag(&bar.hd_full[hb], (ch_cnt >> 1) & 1, abort_flag);
          tc_fence_after();
          uint32_t hv[16], hg[16], dg[16];
          tmem_ld16(tHD + hb * 128 + half * 16 + lane_addr, hv);
          tmem_ld16(tHD + hb * 128 + 32 + half * 16 + lane_addr, hg);
          tmem_ld16(tHD + hb * 128 + 64 + half * 16 + lane_addr, dg);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar.hd_empty[hb]);
          uint32_t gp[8], dv[8], db[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float go[2], dvo[2], dbo[2];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const float v = __uint_as_float(hv[2 * e + q]), b = __uint_as_float(hg[2 * e + q]), d = __uint_as_float(dg[2 * e + q]);
              const float sg = fmaf(0.5f, tanh_approx(0.5f * b), 0.5f);      // sigmoid(b)
              const float sl = b * sg;                                        // silu(b)
              go[q] = sl * v;
              dvo[q] = d * sl;
              dbo[q] = d * v * fmaf(sl, 1.f - sg, sg);                        // d/db silu(b) = sg + sl * (1 - sg)
            }
            gp[e] = Pack2<T>::pack(go[0], go[1]); dv[e] = Pack2<T>::pack(dvo[0], dvo[1]); db[e] = Pack2<T>::pack(dbo[0], dbo[1]);
          }
          // tile buffer hb: the dyln MMAs of two chunks ago have read it, and so has the TMA store of that chunk (which
          // the store warp issues and reports)
          if (ch_cnt >= 2) {
            wait_or_flag(&bar.dh_empty[hb], ((ch_cnt >> 1) - 1) & 1, abort_flag);
            wait_or_flag(&bar.st_done[hb], ((ch_cnt >> 1) - 1) & 1, abort_flag);
          }
          if (__any_sync(0xffffffffu, *abort_flag)) { dead = true; break; }
          uint8_t* dh = sDH + hb * DH_BYTES;
          uint8_t* g = sG + hb * G_BYTES;
          // dh row (128 B): [value 0-15 | gate 0-15 | value 16-31 | gate 16-31]; my 16 + 16 columns are chunks half*4 .. +3
          *reinterpret_cast<uint4*>(dh + swz_offset(row_l, half * 4 + 0, 128)) = make_uint4(dv[0], dv[1], dv[2], dv[3]);
          *reinterpret_cast<uint4*>(dh + swz_offset(row_l, half * 4 + 1, 128)) = make_uint4(dv[4], dv[5], dv[6], dv[7]);
          *reinterpret_cast<uint4*>(dh + swz_offset(row_l, half * 4 + 2, 128)) = make_uint4(db[0], db[1], db[2], db[3]);
          *reinterpret_cast<uint4*>(dh + swz_offset(row_l, half * 4 + 3, 128)) = make_uint4(db[4], db[5], db[6], db[7]);
          // g row (64 B): columns in natural order, mine are chunks half*2, half*2 + 1
          *reinterpret_cast<uint4*>(g + swz_offset(row_l, half * 2 + 0, 64)) = make_uint4(gp[0], gp[1], gp[2], gp[3]);
          *reinterpret_cast<uint4*>(g + swz_offset(row_l, half * 2 + 1, 64)) = make_uint4(gp[4], gp[5], gp[6], gp[7]);
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar.dh_full[hb]);
        }
        if (dead) break;
        // ---- dyln of this tile: TMEM -> registers -> global (fp32), thread (row, half) = 64 columns
        wait_or_flag(&bar.acc_full, t & 1, abort_flag);
        tc_fence_after();
        uint32_t acc[64];
        tmem_ld32(tACC + half * 64 + lane_addr, *reinterpret_cast<uint32_t (*)[32]>(acc));
        tmem_ld32(tACC + half * 64 + 32 + lane_addr, *reinterpret_cast<uint32_t (*)[32]>(acc + 32));
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar.acc_empty);
        const int64_t row = (int64_t)row0 + row_l;
        if (row < p.M && !*abort_flag) {
          float4* dst = reinterpret_cast<float4*>(p.dyln + row * K + half * 64);
#pragma unroll
          for (int i = 0; i < 16; ++i)
            dst[i] = make_float4(__uint_as_float(acc[4 * i]), __uint_as_float(acc[4 * i + 1]), __uint_as_float(acc[4 * i + 2]), __uint_as_float(acc[4 * i + 3]));
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 12 && lane == 0) {
      // -------------------------------------------------------------------------------- MMA issuer
      const uint32_t id_h = idesc_f16(128, 64, p.ab_fmt, 0, 1);     // A K-major, B = W1 value|gate blocks MN-major, N = 64
      const uint32_t id_g = idesc_f16(128, 32, p.ab_fmt, 0, 1);     // A = dY K-major, B = W2 block MN-major, N = 32
      uint32_t ch_cnt = 0;
      for (int t = 0; t < my_tiles && !*abort_flag; ++t) {
        const int buf = t & 1;
        wait_or_flag(&bar.a_full[buf], (t >> 1) & 1, abort_flag);
        wait_or_flag(&bar.dy_full, t & 1, abort_flag);
        const uint32_t a_lo = desc_lo(smem_u32(sA + buf * A_BYTES), 16), y_lo = desc_lo(smem_u32(sDY), 16);
        for (int c = 0; c < nch && !*abort_flag; ++c, ++ch_cnt) {
          const int hb = ch_cnt & 1, ws = ch_cnt % kWS;
          wait_or_flag(&bar.w_full[ws], (ch_cnt / kWS) & 1, abort_flag);
          if (ch_cnt >= 2) wait_or_flag(&bar.hd_empty[hb], ((ch_cnt >> 1) - 1) & 1, abort_flag);
          tc_fence_after();
          if (*abort_flag) break;
          const uint32_t w = smem_u32(sW + ws * W_BYTES);
          const uint32_t wh_lo = desc_lo(w, WB), wg_lo = desc_lo(w + 2 * WB, 16);
#pragma unroll
          for (int ks = 0; ks < K / 16; ++ks)      // H value | gate: the two blocks are the two atoms along N (LBO = WB)
            mma_ss_lh(tHD + hb * 128, a_lo + (((ks >> 2) * (kRows * 128) + (ks & 3) * 32) >> 4), desc_hi(1024, kSw128),
                      wh_lo + ((ks * 1024) >> 4), desc_hi(512, kSw64), id_h, ks > 0);
#pragma unroll
          for (int ks = 0; ks < K / 16; ++ks)      // DG
            mma_ss_lh(tHD + hb * 128 + 64, y_lo + (((ks >> 2) * (kRows * 128) + (ks & 3) * 32) >> 4), desc_hi(1024, kSw128),
                      wg_lo + ((ks * 1024) >> 4), desc_hi(512, kSw64), id_g, ks > 0);
          tc_commit(&bar.hd_full[hb]);
        }
        if (*abort_flag) break;
        tc_commit(&bar.a_empty[buf]);      // the H / DG MMAs of this tile are all issued: X and dY tiles are free when they complete
        tc_commit(&bar.dy_empty);
      }
    } else if (warp == 15 && lane == 0) {
      // -------------------------------------------------------------------------------- second MMA issuer: the dyln GEMMs
      // (a single issuing thread spends more time on its own waits, descriptors and commits than the MMAs take)
      const uint32_t id_a = idesc_f16(128, 128, p.ab_fmt, 0, 0);    // A = dh K-major, B = W1 blocks K-major, N = dim
      auto acc_gemm = [&](uint32_t cc, bool first_of_tile, int t) {  // dyln (+)= dh(cc) [W1v; W1g](cc)^T
        const int hb = cc & 1;
        wait_or_flag(&bar.dh_full[hb], (cc >> 1) & 1, abort_flag);
        if (first_of_tile && t > 0) wait_or_flag(&bar.acc_empty, (t - 1) & 1, abort_flag);
        tc_fence_after();
        if (*abort_flag) return;
        const uint32_t dh_lo = desc_lo(smem_u32(sDH + hb * DH_BYTES), 16), w_lo = desc_lo(smem_u32(sW + (cc % kWS) * W_BYTES), 16);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          // k-step ks covers dh columns ks*16 .. +15: value (ks even) or gate (ks odd) columns (ks / 2) * 16 .. of the chunk
          mma_ss_lh(tACC, dh_lo + ((ks * 32) >> 4), desc_hi(1024, kSw128), w_lo + (((ks & 1) * WB + (ks >> 1) * 32) >> 4), desc_hi(512, kSw64),
                    id_a, !first_of_tile || ks > 0);
        }
        tc_commit(&bar.dh_empty[hb]);
        tc_commit(&bar.w_empty[cc % kWS]);
      };
      uint32_t ch_cnt = 0;
      for (int t = 0; t < my_tiles && !*abort_flag; ++t) {
        for (int c = 0; c < nch && !*abort_flag; ++c, ++ch_cnt) acc_gemm(ch_cnt, c == 0, t);
        if (*abort_flag) break;
        tc_commit(&bar.acc_full);
      }
    } else if (warp == 14 && lane == 0) {
      // -------------------------------------------------------------------------------- TMA stores of the dh / g tiles
      uint32_t ch_cnt = 0;
      for (int t = 0; t < my_tiles && !*abort_flag; ++t) {
        const int row0 = (int)(((int64_t)blockIdx.x + (int64_t)t * gridDim.x) * kRows);
        for (int c = 0; c < nch && !*abort_flag; ++c, ++ch_cnt) {
          const int hb = ch_cnt & 1;
          wait_or_flag(&bar.dh_full[hb], (ch_cnt >> 1) & 1, abort_flag);      // written and fenced by all eight worker warps
          if (*abort_flag) break;
          tma_store_2d(&mdh, sDH + hb * DH_BYTES, c * 64, row0);               // rows >= M are clipped
          tma_store_2d(&mg, sG + hb * G_BYTES, c * kHC, row0);
          bulk_commit_group();
          bulk_wait_group_read<0>();
          mbar_arrive(&bar.st_done[hb]);
        }
      }
      bulk_wait_group<0>();
    } else if (warp == 13 && lane == 0) {
      // -------------------------------------------------------------------------------- TMA producer
      uint32_t ch_cnt = 0;
      auto load_x = [&](int tl) {
        const int buf = tl & 1;
        if (tl >= 2) wait_or_flag(&bar.a_empty[buf], ((tl >> 1) - 1) & 1, abort_flag);
        const int row0 = (int)(((int64_t)blockIdx.x + (int64_t)tl * gridDim.x) * kRows);
        mbar_expect_tx(&bar.x_full[buf], A_BYTES);
        tma_load_2d(sA + buf * A_BYTES, &mx, &bar.x_full[buf], 0, row0);
        tma_load_2d(sA + buf * A_BYTES + kRows * 128, &mx, &bar.x_full[buf], 64, row0);
      };
      if (my_tiles > 0) load_x(0);
      for (int t = 0; t < my_tiles && !*abort_flag; ++t) {
        const int row0 = (int)(((int64_t)blockIdx.x + (int64_t)t * gridDim.x) * kRows);
        if (t > 0) wait_or_flag(&bar.dy_empty, (t - 1) & 1, abort_flag);
        if (*abort_flag) break;
        mbar_expect_tx(&bar.dy_full, A_BYTES);
        tma_load_2d(sDY, &mdy, &bar.dy_full, 0, row0);
        tma_load_2d(sDY + kRows * 128, &mdy, &bar.dy_full, 64, row0);
        if (t + 1 < my_tiles) load_x(t + 1);
        for (int c = 0; c < nch; ++c, ++ch_cnt) {
          const int ws = ch_cnt % kWS;
          uint8_t* w = sW + ws * W_BYTES;
          if (ch_cnt >= kWS) wait_or_flag(&bar.w_empty[ws], ((ch_cnt / kWS) - 1) & 1, abort_flag);
          if (*abort_flag) break;
          mbar_expect_tx(&bar.w_full[ws], W_BYTES);
          tma_load_2d(w, &mw1, &bar.w_full[ws], c * kHC, 0);                    // value columns of W1
          tma_load_2d(w + WB, &mw1, &bar.w_full[ws], p.inner + c * kHC, 0);     // gate columns of W1
          tma_load_2d(w + 2 * WB, &mw2, &bar.w_full[ws], c * kHC, 0);           // W2[:, chunk]
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_s) *reinterpret_cast<volatile int*>(p.status) = 1;
  if (warp == 0) tmem_dealloc(tmem_base_s, 512);
}

// dw1[k][n] from the chunk-ordered columns: position c*64 + [v0-15 | g0-15 | v16-31 | g16-31]
__global__ void unpermute_dw1_kernel(const float* __restrict__ src, float* __restrict__ dst, int inner) {
  const int k = blockIdx.x, two_i = 2 * inner;
  for (int pcol = threadIdx.x; pcol < two_i; pcol += blockDim.x) {
    const int c = pcol >> 6, w = pcol & 63;
    const int seg = w >> 4, off = w & 15;            // seg: 0 value lo, 1 gate lo, 2 value hi, 3 gate hi
    const int n = c * kHC + (seg >> 1) * 16 + off + ((seg & 1) ? inner : 0);
    dst[(int64_t)k * two_i + n] = src[(int64_t)k * two_i + pcol];
  }
}

}  // namespace

bool transition_bwd_fused_ok(const mf_transition_bwd_args& a) {
  if (a.dtype != MF_BF16 && a.dtype != MF_F16) return false;
  if (a.dim != 128 || a.inner % 32 != 0 || a.inner < 32 || !a.ln_w) return false;
  if (a.M < 1 || a.M > (int64_t)INT32_MAX) return false;
  const uintptr_t al = reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.dy) | reinterpret_cast<uintptr_t>(a.w1) |
                       reinterpret_cast<uintptr_t>(a.w2);
  return (al & 15) == 0;
}

// g [M, inner], dh [M, inner/32, 64] (chunk-ordered columns), dyln [M, 128] fp32
int transition_bwd_fused(const mf_transition_bwd_args& a, void* g, void* dh, float* dyln, cudaStream_t st) {
  CUtensorMap mx, mdy, mw1, mw2, mdh, mg;
  int r;
  {
    const int64_t dims[2] = {K, a.M}, str[2] = {1, K};
    const int box[2] = {64, kRows};
    if ((r = make_tiled_map(&mx, a.x, a.dtype, 2, dims, str, box, 128))) return r;
    if ((r = make_tiled_map(&mdy, a.dy, a.dtype, 2, dims, str, box, 128))) return r;
  }
  {
    const int64_t dims[2] = {2 * (int64_t)a.inner, K}, str[2] = {1, 2 * (int64_t)a.inner};
    const int box[2] = {kHC, K};
    if ((r = make_tiled_map(&mw1, a.w1, a.dtype, 2, dims, str, box, 64))) return r;
  }
  {
    const int64_t dims[2] = {a.inner, K}, str[2] = {1, a.inner};
    const int box[2] = {kHC, K};
    if ((r = make_tiled_map(&mw2, a.w2, a.dtype, 2, dims, str, box, 64))) return r;
  }
  {
    const int64_t dims[2] = {2 * (int64_t)a.inner, a.M}, str[2] = {1, 2 * (int64_t)a.inner};
    const int box[2] = {64, kRows};
    if ((r = make_tiled_map(&mdh, dh, a.dtype, 2, dims, str, box, 128))) return r;
  }
  {
    const int64_t dims[2] = {a.inner, a.M}, str[2] = {1, a.inner};
    const int box[2] = {kHC, kRows};
    if ((r = make_tiled_map(&mg, g, a.dtype, 2, dims, str, box, 64))) return r;
  }
  TbP p{};
  p.M = a.M; p.inner = a.inner;
  p.n_mt = (int)((a.M + kRows - 1) / kRows);
  p.n_ch = a.inner / kHC;
  p.ab_fmt = a.dtype == MF_BF16 ? 1u : 0u;
  p.x = a.x; p.gamma = a.ln_w; p.beta = a.ln_b; p.mean = a.mean; p.rstd = a.rstd;
  p.dyln = dyln;
  p.status = status_word();
  MF_REQUIRE(p.status, MF_ERR_CUDA, "could not allocate the device status word");
  MF_REQUIRE(tc_async_status() == 0, MF_ERR_CUDA, "an earlier tensor-core kernel gave up on a bounded wait; results are invalid");
  const size_t smem = 1024 + 3 * (size_t)A_BYTES + kWS * (size_t)W_BYTES + 2 * (size_t)DH_BYTES + 2 * (size_t)G_BYTES;
  int grid = sm_count();
  if (grid > p.n_mt) grid = p.n_mt;
  if (a.dtype == MF_BF16) {
    auto kern = transition_bwd_tc_kernel<__nv_bfloat16>;
    MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, st>>>(mx, mdy, mw1, mw2, mdh, mg, p);
  } else {
    auto kern = transition_bwd_tc_kernel<__half>;
    MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, st>>>(mx, mdy, mw1, mw2, mdh, mg, p);
  }
  MF_LAUNCHED("transition_bwd_tc_kernel");
  return MF_OK;
}

int unpermute_dw1(const float* src, float* dst, int dim, int inner, cudaStream_t st) {
  unpermute_dw1_kernel<<<dim, 256, 0, st>>>(src, dst, inner);
  MF_LAUNCHED("unpermute_dw1_kernel");
  return MF_OK;
}

}  // namespace mf
