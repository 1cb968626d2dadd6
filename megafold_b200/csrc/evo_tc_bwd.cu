// Pair-biased masked attention backward on the tensor cores (tcgen05 + TMEM + TMA): dQ, dK, dV and dBias.
//
// One CTA (256 threads, one per SM, persistent) owns a whole (b, n, h) at a time and walks its
// 128-key tiles j and, inside, its 128-query tiles i.  Everything is computed TRANSPOSED, keys on the
// TMEM lanes:
//
//   S^T  = K_j Q_i^T,   dP^T = V_j dO_i^T                       (tcgen05.mma, both into TMEM)
//   thread (w, r): key row r, query half w -> 64 columns of S^T and dP^T into registers, then
//   P^T  = exp2(S^T c1 + bias log2e + mask_j - lse2_i),   dS^T = P^T (dP^T - delta_i)
//   written as 16-bit tiles to shared memory ([128 keys][2 x 64 queries], 128-byte rows, 128B swizzle)
//   dV_j += P^T dO_i      A = P^T tile (K-major),  B = dO_i tile (MN-major)
//   dK_j += dS^T Q_i      A = dS^T tile (K-major), B = Q_i tile  (MN-major)
//   dQ_i += dS K_j        A = the same dS^T tile read MN-major (M = queries), B = K_j tile (MN-major)
//
// dK_j / dV_j accumulate in TMEM over the query tiles, dQ_i (one accumulator per query tile, all kept in
// TMEM for the whole item) over the key tiles; nothing is reduced across CTAs, so dQ/dK/dV are
// bit-reproducible.  The scores for the next block are issued as soon as the current ones have been read
// into registers.  dBias is the sum of dS over the N rows that share the bias: every row adds its dS to
// an fp32 buffer with coalesced red.global.add (lanes = consecutive keys), the same scheme as the
// reference's atomic adds; its summation order is not fixed.
//
// delta_i = rowsum(dO_i * O_i) comes from a small pre-kernel.  All waits are bounded (see tc.cuh).
#include <type_traits>

#include "evo_tc_common.cuh"

namespace mf {
namespace {
using namespace tcx;

constexpr int kT = 128;            // tile edge (keys and queries)
constexpr int kComputeWarps = 16;  // 4 per scheduler, to hide the latencies of the per-element work
constexpr int kThreads = (kComputeWarps + 4) * 32;   // + one warpgroup: accumulate-MMA issuer, TMA producer, score-MMA issuer, idle
constexpr int kTileP = 2 * 128 * 128;   // bytes of a [128 x 128] 16-bit tile (two 64-wide atoms)

template <int DP> struct Cfg {
  static constexpr int ROWB = DP * 2;
  static constexpr int TILEB = 128 * ROWB;
  static constexpr Swizzle SW = DP == 32 ? kSw64 : kSw128;
  static constexpr int SBO = 8 * ROWB;
  static constexpr int MAX_QT = (512 - 256 - 2 * DP) / DP;   // dQ accumulators that fit next to S^T, dP^T, dK, dV
};

struct BwdP {
  int B, N, L, H, D;
  int n_t, n_items, lpad;
  int ksplit;            // work items per (b, n, h): the key tiles are split into this many ranges
  float* dq_acc;         // fp32 [B,N,L,H,D] accumulator of dQ when ksplit > 1 or dq_stream
  int dq_stream;         // more query tiles than dQ accumulators fit in TMEM: dQ leaves the SM block by block
  float c1, scale, inv_L;
  uint32_t ab_fmt;
  const void* bias; int64_t bs[4];
  const void* biasT_;                    // transposed, row-padded copy of the bias (same dtype)
  const void* mask; int64_t ms[3]; int mask_dtype;
  const float* lse; const float* delta;
  void *dq, *dk, *dv; float* dbias;      // dbias: fp32 [B, H, L, L], zeroed by the host side
  int* status;
  long long* timeline;   // debug builds only
};

// Phase timestamps of thread 0 of CTA 0; compiled in only with -DMF_TIMELINE.
#ifdef MF_TIMELINE
long long* g_timeline_bwd = nullptr;
#ifdef MF_TL_MMA
#define MF_TL_WHO (kComputeWarps * 32)
#else
#define MF_TL_WHO 0
#endif
#define MF_TL(tag) do { if (p.timeline && blockIdx.x == 0 && tid == MF_TL_WHO && tl_n < 250) { p.timeline[2 * tl_n] = (tag); p.timeline[2 * tl_n + 1] = clock64(); ++tl_n; } } while (0)
#else
#define MF_TL(tag) do { } while (0)
#endif

struct Bars {
  uint64_t kv_full[2], kv_empty[2], qd_full[3], qd_empty[3], sd_ready, acc_done;
  uint64_t loaded, written, item_sync;     // one arrival per warp
  int special[2];
};

// delta[b,n,h,i] = sum_d dO * O; one thread per (b,n,i,h) row, 16-byte loads (D is a multiple of 8)
template <typename T>
__global__ void evo_delta_tc_kernel(const T* __restrict__ o, const T* __restrict__ d_o, float* __restrict__ delta,
                                    int64_t rows, int L, int H, int D) {
  const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  const uint4* po = reinterpret_cast<const uint4*>(o + row * D);
  const uint4* pg = reinterpret_cast<const uint4*>(d_o + row * D);
  float s = 0.f;
  for (int c = 0; c < D / 8; ++c) {
    const uint4 a = __ldg(po + c), g = __ldg(pg + c);
    const uint32_t av[4] = {a.x, a.y, a.z, a.w}, gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = Pack2<T>::unpack(av[e]), y = Pack2<T>::unpack(gv[e]);
      s = fmaf(x.x, y.x, s); s = fmaf(x.y, y.y, s);
    }
  }
  const int h = (int)(row % H); const int64_t t = row / H; const int i = (int)(t % L); const int64_t bn = t / L;
  delta[(bn * H + h) * L + i] = s;
}

// dst[row][0..L) = src[row][0..L) with the source rows `pitch` floats apart
template <typename T>
__global__ void cast_rows_pitched_kernel(const float* __restrict__ src, T* __restrict__ dst, int64_t rows, int L, int pitch) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * L) return;
  const int64_t row = i / L; const int c = (int)(i - row * L);
  dst[i] = from_f<T>(src[row * pitch + c]);
}

// biasT[b][h][j][i] = bias[b][h][i][j], rows padded to `lpad` entries so that every 64-query run is aligned
// and in bounds.  The backward kernel works with keys on the TMEM lanes, so a thread needs the bias of ONE key
// for a run of queries; with this copy that run is contiguous.
template <typename TB>
__global__ void transpose_bias_kernel(const TB* __restrict__ bias, TB* __restrict__ biasT, int H, int L, int lpad,
                                      int64_t sb, int64_t sh, int64_t si, int64_t sj) {
  __shared__ TB tile[32][33];
  const int bh = blockIdx.z, b = bh / H, h = bh % H;
  const int i0 = blockIdx.y * 32, j0 = blockIdx.x * 32;
  for (int k = threadIdx.y; k < 32; k += blockDim.y) {
    const int i = i0 + k, j = j0 + threadIdx.x;
    if (i < L && j < L) tile[k][threadIdx.x] = bias[b * sb + h * sh + (int64_t)i * si + (int64_t)j * sj];
  }
  __syncthreads();
  for (int k = threadIdx.y; k < 32; k += blockDim.y) {
    const int j = j0 + k, i = i0 + threadIdx.x;
    if (i < L && j < L) biasT[((int64_t)bh * L + j) * lpad + i] = tile[threadIdx.x][k];
  }
}

// 32 consecutive bias values held in registers (packed for 16-bit types)
template <typename TB> struct BiasRun {
  uint4 v[4];
  __device__ __forceinline__ void load(const TB* p) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __ldg(q + i);
  }
  __device__ __forceinline__ float get(int c) const {
    const uint4& x = v[c >> 3];
    const uint32_t u = ((c >> 1) & 3) == 0 ? x.x : ((c >> 1) & 3) == 1 ? x.y : ((c >> 1) & 3) == 2 ? x.z : x.w;
    const float2 f = Pack2<TB>::unpack(u);
    return (c & 1) ? f.y : f.x;
  }
};
template <> struct BiasRun<float> {
  float4 v[8];
  __device__ __forceinline__ void load(const float* p) {
    const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __ldg(q + i);
  }
  __device__ __forceinline__ float get(int c) const {
    const float4& x = v[c >> 2];
    return (c & 3) == 0 ? x.x : (c & 3) == 1 ? x.y : (c & 3) == 2 ? x.z : x.w;
  }
};

// dBias staging: fp32 [16 queries][32 keys] per warp, pushed to global memory with a TMA add-reduction
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, const void* src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

template <int DP, typename T, typename TB, bool DQS>      // DQS: dQ streamed block by block (more query tiles than TMEM holds)
__global__ void __launch_bounds__(kThreads, 1)
evo_bwd_tc_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                  const __grid_constant__ CUtensorMap mv, const __grid_constant__ CUtensorMap mg,
                  const __grid_constant__ CUtensorMap mdb, const BwdP p) {
  using C = Cfg<DP>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sP = smem;                         // P^T tile
  uint8_t* sDS = sP + kTileP;                 // dS^T tile
  uint8_t* sKV = sDS + kTileP;                // [2 stages][K, V]
  uint8_t* sQD = sKV + 4 * C::TILEB;          // [3 stages][Q, dO]
  float* lse2 = reinterpret_cast<float*>(sQD + 6 * C::TILEB);
  float* dlt = lse2 + 2 * p.lpad;            // lse2, dlt: two buffers each (current item / next item)

  __shared__ Bars bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int w = warp >> 2;                          // query quarter (32 columns) handled by this thread
  const int r = (warp & 3) * 32 + lane;             // TMEM lane = key row inside the tile
  float* stage = dlt + 2 * p.lpad + warp * 1024;        // per warp: 2 buffers x [16 queries][32 keys] fp32
  if (tid == 0) {
    abort_s = 0;
    mbar_init(&bar.kv_full[0], 1); mbar_init(&bar.kv_full[1], 1);
    mbar_init(&bar.qd_full[0], 1); mbar_init(&bar.qd_full[1], 1); mbar_init(&bar.qd_full[2], 1);
    mbar_init(&bar.sd_ready, 1);
    mbar_init(&bar.acc_done, 1);
    mbar_init(&bar.kv_empty[0], 1); mbar_init(&bar.kv_empty[1], 1);
    mbar_init(&bar.qd_empty[0], 1); mbar_init(&bar.qd_empty[1], 1); mbar_init(&bar.qd_empty[2], 1);
    mbar_init(&bar.loaded, kComputeWarps); mbar_init(&bar.written, kComputeWarps); mbar_init(&bar.item_sync, kComputeWarps);
    bar.special[0] = 0; bar.special[1] = 0;
    mbar_fence_init();
    prefetch_tmap(&mq); prefetch_tmap(&mk); prefetch_tmap(&mv); prefetch_tmap(&mg);
  }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  volatile int* abort_flag = &abort_s;
  const uint32_t tm0 = tmem_base_s;
  const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
  // dK/dV accumulators are double-buffered over the key tiles when the dQ accumulators leave room for it: their
  // write-out is then deferred by one block and no longer stalls the pipeline at the end of a key tile
  const bool dbuf = DQS || p.n_t <= (512 - 256 - 4 * DP) / DP;
  // dQ: one accumulator per query tile, complete at the end of the item; or (dq_stream) two accumulators used in turn
  // by successive blocks, each block's product added to the fp32 accumulator in global memory by the compute warps
  const uint32_t tST = tm0, tDP = tm0 + 128, tKV = tm0 + 256, tDQ = tm0 + 256 + (dbuf ? 4 : 2) * DP;
  auto tDK_of = [&](uint32_t kc) { return tKV + (dbuf ? (kc & 1) * 2 * DP : 0); };
  auto tDV_of = [&](uint32_t kc) { return tDK_of(kc) + DP; };
  const uint32_t id_s = idesc_f16(128, 128, p.ab_fmt, 0, 0);
  const uint32_t id_kv = idesc_f16(128, DP, p.ab_fmt, 0, 1);    // A K-major, B MN-major
  const uint32_t id_q = idesc_f16(128, DP, p.ab_fmt, 1, 1);     // A MN-major, B MN-major
  const int nt = p.n_t, blocks_per_item = nt * nt;

  uint32_t g = 0;                 // blocks processed by this CTA: sd_ready / acc_done parity g & 1;
                                  // Q/dO tile of block g lives in stage g % 3 (qd_full parity (g / 3) & 1)
  uint32_t kv_cnt = 0;            // (item, j) pairs so far: K/V stage kv_cnt & 1, kv_full parity (kv_cnt >> 1) & 1
  bool dead = false;
  int tl_n = 0; (void)tl_n;
  uint32_t rnd = 0;               // dBias staging rounds of this warp (buffer = rnd & 1)
  uint32_t isync = 0;             // CTA rendezvous counter (one per item)
  int item_no = 0;                // items this CTA has started (statistics buffer = item_no & 1)
  int pend_j = -1; uint32_t pend_kc = 0; int pend_b = 0, pend_n = 0, pend_h = 0;   // deferred dK/dV write-out
  auto qd_stage = [&](uint32_t gg) { return sQD + (gg % 3) * 2 * C::TILEB; };
  auto load_qd = [&](uint32_t gg, int it2, int h, int n, int b) {
    uint64_t* fb = &bar.qd_full[gg % 3];
    mbar_expect_tx(fb, 2 * C::TILEB);
    tma_load_5d(qd_stage(gg), &mq, fb, 0, h, it2 * kT, n, b);
    tma_load_5d(qd_stage(gg) + C::TILEB, &mg, fb, 0, h, it2 * kT, n, b);
  };
  auto load_kv = [&](uint32_t kc, int jt2, int h, int n, int b) {
    uint64_t* fb = &bar.kv_full[kc & 1];
    mbar_expect_tx(fb, 2 * C::TILEB);
    tma_load_5d(sKV + (kc & 1) * 2 * C::TILEB, &mk, fb, 0, h, jt2 * kT, n, b);
    tma_load_5d(sKV + (kc & 1) * 2 * C::TILEB + C::TILEB, &mv, fb, 0, h, jt2 * kT, n, b);
  };
  auto issue_scores = [&](uint32_t gg, uint32_t kc) {     // S^T = K Q^T and dP^T = V dO^T of block gg
    const uint32_t ka = smem_u32(sKV + (kc & 1) * 2 * C::TILEB), qa = smem_u32(qd_stage(gg));
    const uint32_t k_lo = desc_lo(ka, 16), v_lo = desc_lo(ka + C::TILEB, 16), q_lo = desc_lo(qa, 16), g_lo = desc_lo(qa + C::TILEB, 16);
    constexpr uint32_t hi = desc_hi(C::SBO, C::SW);
#pragma unroll
    for (int ks = 0; ks < DP / 16; ++ks) mma_ss_lh(tST, k_lo + ks * 2, hi, q_lo + ks * 2, hi, id_s, ks > 0);
#pragma unroll
    for (int ks = 0; ks < DP / 16; ++ks) mma_ss_lh(tDP, v_lo + ks * 2, hi, g_lo + ks * 2, hi, id_s, ks > 0);
    tc_commit(&bar.sd_ready);
  };

  // dK (scaled) and dV rows of key `j` from accumulator buffer `kc`: quarter 0 writes dK, quarter 1 writes dV
  auto store_kv = [&](uint32_t kc, int j, int b, int n, int h) {
    tc_fence_after();
    if (w < 2) {
      uint32_t o32[DP];
#pragma unroll
      for (int cb = 0; cb < DP / 32; ++cb)
        tmem_ld32((w == 0 ? tDK_of(kc) : tDV_of(kc)) + lane_addr + cb * 32, *reinterpret_cast<uint32_t (*)[32]>(o32 + cb * 32));
      tmem_ld_wait();
      if (j < p.L && !*abort_flag) {
        const float sc = w == 0 ? p.scale : 1.f;
        T* orow = static_cast<T*>(w == 0 ? p.dk : p.dv) + ((((int64_t)b * p.N + n) * p.L + j) * p.H + h) * p.D;
#pragma unroll
        for (int d8 = 0; d8 < DP / 8; ++d8) {
          if (d8 * 8 < p.D) {
            uint4 v;
            v.x = Pack2<T>::pack(__uint_as_float(o32[d8 * 8]) * sc, __uint_as_float(o32[d8 * 8 + 1]) * sc);
            v.y = Pack2<T>::pack(__uint_as_float(o32[d8 * 8 + 2]) * sc, __uint_as_float(o32[d8 * 8 + 3]) * sc);
            v.z = Pack2<T>::pack(__uint_as_float(o32[d8 * 8 + 4]) * sc, __uint_as_float(o32[d8 * 8 + 5]) * sc);
            v.w = Pack2<T>::pack(__uint_as_float(o32[d8 * 8 + 6]) * sc, __uint_as_float(o32[d8 * 8 + 7]) * sc);
            *reinterpret_cast<uint4*>(orow + d8 * 8) = v;
          }
        }
      }
    }
    tc_fence_before();
  };

  // dq_stream: the dQ product of block gg (query tile it2) sits in accumulator gg & 1; the four warps of query
  // quarter gg & 3 add it, scaled, to the fp32 dQ rows in global memory
  auto stream_dq = [&](uint32_t gg, int it2, int b, int n, int h) {
    if (w != (int)(gg & 3)) return;
    tc_fence_after();
    uint32_t o32[DP];
#pragma unroll
    for (int cb = 0; cb < DP / 32; ++cb)
      tmem_ld32(tDQ + (gg & 1) * DP + lane_addr + cb * 32, *reinterpret_cast<uint32_t (*)[32]>(o32 + cb * 32));
    tmem_ld_wait();
    tc_fence_before();
    const int i = it2 * kT + r;
    if (i < p.L && !*abort_flag) {
      float* arow = p.dq_acc + ((((int64_t)b * p.N + n) * p.L + i) * p.H + h) * p.D;
#pragma unroll
      for (int d4 = 0; d4 < DP / 4; ++d4)
        if (d4 * 4 < p.D)
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(arow + d4 * 4),
                       "f"(__uint_as_float(o32[d4 * 4]) * p.scale), "f"(__uint_as_float(o32[d4 * 4 + 1]) * p.scale),
                       "f"(__uint_as_float(o32[d4 * 4 + 2]) * p.scale), "f"(__uint_as_float(o32[d4 * 4 + 3]) * p.scale) : "memory");
    }
  };

  if (warp < kComputeWarps) {
  // Register re-partition: the CTA is launched with 96 registers per thread (640 threads); the issuer warpgroup
  // drops to 32 and the compute warpgroups rise to 112.  The raise can only draw on what the drop releases inside
  // this CTA, so 512 * 112 + 128 * 32 must not exceed 640 * 96 (it is equal) - otherwise the raise never returns.
  static_assert(kComputeWarps * 32 * 112 + 128 * 32 <= kThreads * 96, "setmaxnreg budget");
  asm volatile("setmaxnreg.inc.sync.aligned.u32 112;");
  for (int item = blockIdx.x; item < p.n_items && !dead; item += gridDim.x) {
    // work item = (b, n, h, range of key tiles); with one range per (b, n, h) the dQ rows are complete at the end of
    // the item, otherwise they are partial sums that go to an fp32 accumulator
    const int bnh = item / p.ksplit, sp = item - bnh * p.ksplit;
    const int jt0 = sp * nt / p.ksplit, jt1 = (sp + 1) * nt / p.ksplit;
    const int h = bnh % p.H, bn = bnh / p.H, n = bn % p.N, b = bn / p.N;
    // ---- per-item statistics (lse in base 2, delta; queries beyond L get lse = +inf so that P = 0) live in two
    // buffers: the current item's were stored while the previous item was running.  One CTA-wide rendezvous per item
    // (bounded mbarrier wait, one arrival per warp): everybody has left the previous item, so the other buffer may be
    // refilled, and everybody's earlier stores to this buffer are visible.
    auto load_stats = [&](int item2, int buf, int stamp) {
      if (item2 >= p.n_items) return;
      const int64_t row2 = (int64_t)(item2 / p.ksplit) * p.L;   // ((b*N+n)*H + h) * L
      for (int i = tid; i < p.lpad; i += kComputeWarps * 32) {
        float l2 = INFINITY, dl = 0.f;
        if (i < p.L) {
          const float lv = p.lse[row2 + i];
          if (lv <= -3e38f) bar.special[buf] = stamp;  // a fully masked row: the item (identified by its stamp) takes the careful path
          l2 = lv * kLog2e; dl = p.delta[row2 + i];
        }
        lse2[buf * p.lpad + i] = l2; dlt[buf * p.lpad + i] = dl;
      }
    };
    auto cta_sync = [&]() {
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.item_sync);
      wait_or_flag(&bar.item_sync, isync & 1, abort_flag);
      ++isync;
    };
    const int sbuf = item_no & 1;
    if (item_no == 0) { load_stats(item, 0, 1); }
    cta_sync();
    if (__any_sync(0xffffffffu, *abort_flag)) { dead = true; break; }
    const bool special = *reinterpret_cast<volatile int*>(&bar.special[sbuf]) == item_no + 1;
    load_stats(item + (int)gridDim.x, sbuf ^ 1, item_no + 2);
    const float* lse2c = lse2 + sbuf * p.lpad;
    const float* dltc = dlt + sbuf * p.lpad;
    ++item_no;
    float mask2_next = -INFINITY;
    {
      const int j0r = jt0 * kT + r;
      if (j0r < p.L) {
        const int64_t mi = b * p.ms[0] + n * p.ms[1] + (int64_t)j0r * p.ms[2];
        mask2_next = p.mask_dtype == MF_U8 ? (static_cast<const uint8_t*>(p.mask)[mi] ? 0.f : -FLT_MAX)
                                           : load_rt(p.mask, mi, p.mask_dtype) * kLog2e;
      }
    }

    for (int jt = jt0; jt < jt1 && !dead; ++jt) {
      const int j = jt * kT + r;
      const bool j_ok = j < p.L;
      const float mask2 = mask2_next;          // fetched one key tile ahead
      if (jt + 1 < jt1) {
        const int jn = (jt + 1) * kT + r;
        mask2_next = -INFINITY;
        if (jn < p.L) {
          const int64_t mi = b * p.ms[0] + n * p.ms[1] + (int64_t)jn * p.ms[2];
          mask2_next = p.mask_dtype == MF_U8 ? (static_cast<const uint8_t*>(p.mask)[mi] ? 0.f : -FLT_MAX)
                                             : load_rt(p.mask, mi, p.mask_dtype) * kLog2e;
        }
      }
      const bool masked_key = mask2 <= -FLT_MAX;
      for (int it = 0; it < nt; ++it, ++g) {
        const int i0 = it * kT + w * 32;
        const bool new_j = (it == nt - 1);
        MF_TL(20);
        // ---- bias for my key and my 64 queries: one contiguous run of the transposed copy biasT[b][h][j][i]
        BiasRun<TB> bv;
        bv.load(static_cast<const TB*>(p.biasT_) + (((int64_t)b * p.H + h) * p.L + (j_ok ? j : 0)) * p.lpad + i0);
        MF_TL(21);
        // ---- S^T, dP^T of this block -> registers
        wait_or_flag(&bar.sd_ready, g & 1, abort_flag);
        tc_fence_after();
        MF_TL(22);
        uint32_t sr[32], dr[32];
        {
          uint32_t (*s2)[32] = reinterpret_cast<uint32_t (*)[32]>(sr);
          uint32_t (*d2)[32] = reinterpret_cast<uint32_t (*)[32]>(dr);
          tmem_ld32(tST + lane_addr + w * 32, s2[0]);
          tmem_ld32(tDP + lane_addr + w * 32, d2[0]);
          tmem_ld_wait();
        }
        MF_TL(23);
        tc_fence_before();
        if (__any_sync(0xffffffffu, *abort_flag)) { dead = true; break; }
        if (lane == 0) mbar_arrive(&bar.loaded);
        MF_TL(24);
        MF_TL(25);
        // ---- P^T and dS^T for my 64 queries
        uint32_t pp[16], dd[16];
        auto compute = [&](auto careful) {
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 l4 = *reinterpret_cast<const float4*>(lse2c + i0 + c4 * 4);
          const float4 d4 = *reinterpret_cast<const float4*>(dltc + i0 + c4 * 4);
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, de[4] = {d4.x, d4.y, d4.z, d4.w};
          float pv[4], dv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = c4 * 4 + e;
            const float x = fmaf(__uint_as_float(sr[c]), p.c1, fmaf(bv.get(c), kLog2e, mask2)) - ls[e];
            float pr = ex2f(x);
            if (decltype(careful)::value && ls[e] <= -3e38f) pr = j_ok ? p.inv_L : 0.f;   // fully masked row: uniform
            float ds = pr * (__uint_as_float(dr[c]) - de[e]);
            if (decltype(careful)::value && masked_key) ds = 0.f;                         // no gradient through a masked logit
            pv[e] = pr; dv[e] = ds;
            stage[(rnd & 1) * 512 + ((c4 & 3) * 4 + e) * 32 + lane] = ds;
          }
          if ((c4 & 3) == 3) {
            // 16 queries x 32 keys of dS are staged: add them to dBias[b, h, i, j] (TMA clips rows/columns >= L)
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
#ifndef MF_NO_REDUCE
              tma_reduce_add_4d(&mdb, stage + (rnd & 1) * 512, jt * kT + (warp & 3) * 32, i0 + (c4 >> 2) * 16, h, b);
#endif
              bulk_commit();
              bulk_wait_read<1>();      // the buffer written two rounds ago has been read: it may be refilled
            }
            __syncwarp();
            ++rnd;
          }
          pp[c4 * 2] = Pack2<T>::pack(pv[0], pv[1]); pp[c4 * 2 + 1] = Pack2<T>::pack(pv[2], pv[3]);
          dd[c4 * 2] = Pack2<T>::pack(dv[0], dv[1]); dd[c4 * 2 + 1] = Pack2<T>::pack(dv[2], dv[3]);
        }
        };
        if (special) compute(std::true_type{}); else compute(std::false_type{});
        MF_TL(26);
        // the MMAs of the previous block have finished reading the P^T / dS^T tiles?
        if (g > 0) wait_or_flag(&bar.acc_done, (g - 1) & 1, abort_flag);
        if constexpr (DQS) { if (!(jt == jt0 && it == 0)) stream_dq(g - 1, it == 0 ? nt - 1 : it - 1, b, n, h); }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const uint32_t off = (w >> 1) * 16384 + swz_offset(r, (w & 1) * 4 + ch, 128);
          *reinterpret_cast<uint4*>(sP + off) = make_uint4(pp[ch * 4], pp[ch * 4 + 1], pp[ch * 4 + 2], pp[ch * 4 + 3]);
          *reinterpret_cast<uint4*>(sDS + off) = make_uint4(dd[ch * 4], dd[ch * 4 + 1], dd[ch * 4 + 2], dd[ch * 4 + 3]);
        }
        fence_async_smem();
        tc_fence_before();
        MF_TL(27);
        if (__any_sync(0xffffffffu, *abort_flag)) { dead = true; break; }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar.written);
        MF_TL(28);
        // ---- dK_j, dV_j write-out.  Double-buffered: the key tile that finished one block ago (its MMAs were
        // awaited before this block's tiles were written).  Otherwise: right now, after waiting for this block's MMAs.
        if (dbuf) {
          if (pend_j >= 0) { store_kv(pend_kc, pend_j, pend_b, pend_n, pend_h); pend_j = -1; }
          if (new_j) { pend_j = j; pend_kc = kv_cnt; pend_b = b; pend_n = n; pend_h = h; }
        } else if (new_j) {
          wait_or_flag(&bar.acc_done, g & 1, abort_flag);
          store_kv(kv_cnt, j, b, n, h);
        }
      }
      if (!dead) ++kv_cnt;
    }
    if (dead) break;
    // ---- dQ of every query tile, once the last block's MMAs are complete; and the last key tile's dK/dV
    wait_or_flag(&bar.acc_done, (g - 1) & 1, abort_flag);
    if (pend_j >= 0) { store_kv(pend_kc, pend_j, pend_b, pend_n, pend_h); pend_j = -1; }
    tc_fence_after();
    if constexpr (DQS) stream_dq(g - 1, nt - 1, b, n, h);     // the last block of the item
    for (int it = w; it < nt && !DQS; it += 4) {
      const int i = it * kT + r;
      uint32_t o32[DP];
#pragma unroll
      for (int cb = 0; cb < DP / 32; ++cb) tmem_ld32(tDQ + it * DP + lane_addr + cb * 32, *reinterpret_cast<uint32_t (*)[32]>(o32 + cb * 32));
      tmem_ld_wait();
      if (i < p.L && !*abort_flag && p.ksplit > 1) {
        float* arow = p.dq_acc + ((((int64_t)b * p.N + n) * p.L + i) * p.H + h) * p.D;
#pragma unroll
        for (int d4 = 0; d4 < DP / 4; ++d4)
          if (d4 * 4 < p.D)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(arow + d4 * 4),
                         "f"(__uint_as_float(o32[d4 * 4]) * p.scale), "f"(__uint_as_float(o32[d4 * 4 + 1]) * p.scale),
                         "f"(__uint_as_float(o32[d4 * 4 + 2]) * p.scale), "f"(__uint_as_float(o32[d4 * 4 + 3]) * p.scale) : "memory");
      } else if (i < p.L && !*abort_flag) {
        T* orow = static_cast<T*>(p.dq) + ((((int64_t)b * p.N + n) * p.L + i) * p.H + h) * p.D;
#pragma unroll
        for (int d8 = 0; d8 < DP / 8; ++d8) {
          if (d8 * 8 < p.D) {
            uint4 v;
            v.x = Pack2<T>::pack(__uint_as_float(o32[d8 * 8]) * p.scale, __uint_as_float(o32[d8 * 8 + 1]) * p.scale);
            v.y = Pack2<T>::pack(__uint_as_float(o32[d8 * 8 + 2]) * p.scale, __uint_as_float(o32[d8 * 8 + 3]) * p.scale);
            v.z = Pack2<T>::pack(__uint_as_float(o32[d8 * 8 + 4]) * p.scale, __uint_as_float(o32[d8 * 8 + 5]) * p.scale);
            v.w = Pack2<T>::pack(__uint_as_float(o32[d8 * 8 + 6]) * p.scale, __uint_as_float(o32[d8 * 8 + 7]) * p.scale);
            *reinterpret_cast<uint4*>(orow + d8 * 8) = v;
          }
        }
      }
    }
    tc_fence_before();
  }

  if (lane == 0) bulk_wait<0>();      // my dBias reductions have left shared memory and reached global memory
  } else {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 32;");
  if (warp == kComputeWarps && lane == 0) {
    // ---------------------------------------------------------------- accumulate-MMA issuer: the three
    // accumulations of each block, as soon as its P^T / dS^T tiles have been written
    uint32_t g = 0, kv = 0;
    for (int item = blockIdx.x; item < p.n_items && !*abort_flag; item += gridDim.x) {
      const int sp = item % p.ksplit, jt0 = sp * nt / p.ksplit, jt1 = (sp + 1) * nt / p.ksplit;
      for (int jt = jt0; jt < jt1 && !*abort_flag; ++jt) {
        for (int it = 0; it < nt; ++it, ++g) {
          MF_TL(43);
          wait_or_flag(&bar.written, g & 1, abort_flag);
          MF_TL(44);
          tc_fence_after();
          if (*abort_flag) break;
          const uint32_t kvb = smem_u32(sKV + (kv & 1) * 2 * C::TILEB);
          const uint32_t qdb = smem_u32(qd_stage(g));
          // descriptor low words (address field in units of 16 bytes); the high words are constants
          const uint32_t p_lo = desc_lo(smem_u32(sP), 16), ds_lo = desc_lo(smem_u32(sDS), 16), dst_lo = desc_lo(smem_u32(sDS), 16384);
          const uint32_t q_lo = desc_lo(qdb, 16), do_lo = desc_lo(qdb + C::TILEB, 16), k_lo = desc_lo(kvb, 16);
          constexpr uint32_t hi_t = desc_hi(1024, kSw128), hi_o = desc_hi(C::SBO, C::SW);
          constexpr uint32_t kstep = 16 * C::ROWB / 16;      // 16 rows of an MN-major operand tile
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)      // dV_j += P^T dO_i
            mma_ss_lh(tDV_of(kv), p_lo + (ks >> 2) * (16384 / 16) + (ks & 3) * 2, hi_t, do_lo + ks * kstep, hi_o, id_kv, it > 0 || ks > 0);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)      // dK_j += dS^T Q_i
            mma_ss_lh(tDK_of(kv), ds_lo + (ks >> 2) * (16384 / 16) + (ks & 3) * 2, hi_t, q_lo + ks * kstep, hi_o, id_kv, it > 0 || ks > 0);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)      // dQ_i += dS K_j   (A = dS^T tile read MN-major: M = queries)
            mma_ss_lh(tDQ + (DQS ? (g & 1) : it) * DP, dst_lo + ks * (2048 / 16), hi_t, k_lo + ks * kstep, hi_o, id_q,
                      DQS ? ks > 0 : (jt > jt0 || ks > 0));
          MF_TL(45);
          tc_commit(&bar.acc_done);
          // the stages are also read by this block's score MMAs, which completed before its tiles were written
          tc_commit(&bar.qd_empty[g % 3]);
          if (it == nt - 1) { tc_commit(&bar.kv_empty[kv & 1]); ++kv; }
        }
      }
    }
  } else if (warp == kComputeWarps + 2 && lane == 0) {
    // ---------------------------------------------------------------- score-MMA issuer, one block ahead of
    // the compute warps: S^T, dP^T of block g+1 as soon as every warp holds block g's in registers
    uint32_t g = 0, kv = 0;
    wait_or_flag(&bar.kv_full[0], 0, abort_flag);
    wait_or_flag(&bar.qd_full[0], 0, abort_flag);
    tc_fence_after();
    if (!*abort_flag) issue_scores(0, 0);
    for (int item = blockIdx.x; item < p.n_items && !*abort_flag; item += gridDim.x) {
      const bool last_item = item + (int)gridDim.x >= p.n_items;
      const int sp = item % p.ksplit, jt0 = sp * nt / p.ksplit, jt1 = (sp + 1) * nt / p.ksplit;
      for (int jt = jt0; jt < jt1 && !*abort_flag; ++jt) {
        for (int it = 0; it < nt; ++it, ++g) {
          const bool new_j = (it == nt - 1);
          if (last_item && (jt == jt1 - 1) && new_j) break;
          wait_or_flag(&bar.loaded, g & 1, abort_flag);
          const uint32_t kc = new_j ? kv + 1 : kv;
          if (new_j) wait_or_flag(&bar.kv_full[kc & 1], (kc >> 1) & 1, abort_flag);
          wait_or_flag(&bar.qd_full[(g + 1) % 3], ((g + 1) / 3) & 1, abort_flag);
          tc_fence_after();
          if (*abort_flag) break;
          issue_scores(g + 1, kc);
          if (new_j) ++kv;
        }
      }
    }
  } else if (warp == kComputeWarps + 1 && lane == 0) {
    // ---------------------------------------------------------------- TMA producer, in order of need
    uint32_t g = 0, kv = 0;
    for (int item = blockIdx.x; item < p.n_items && !*abort_flag; item += gridDim.x) {
      const int bnh = item / p.ksplit, sp = item - bnh * p.ksplit;
      const int jt0 = sp * nt / p.ksplit, jt1 = (sp + 1) * nt / p.ksplit;
      const int h = bnh % p.H, bn = bnh / p.H, n = bn % p.N, b = bn / p.N;
      for (int jt = jt0; jt < jt1 && !*abort_flag; ++jt) {
        if (kv >= 2) wait_or_flag(&bar.kv_empty[kv & 1], ((kv >> 1) - 1) & 1, abort_flag);
        if (*abort_flag) break;
        load_kv(kv, jt, h, n, b);
        ++kv;
        for (int it = 0; it < nt; ++it, ++g) {
          if (g >= 3) wait_or_flag(&bar.qd_empty[g % 3], ((g / 3) - 1) & 1, abort_flag);
          if (*abort_flag) break;
          load_qd(g, it, h, n, b);
        }
      }
    }
  }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_s) *reinterpret_cast<volatile int*>(p.status) = 1;
  if (warp == 0) tmem_dealloc(tmem_base_s, 512);
}

// With few (b, n, h) triples (single-representation attention: N = 1) the key tiles of each are spread over several
// CTAs so that the whole GPU works; the partial dQ rows then meet in an fp32 accumulator.  B200: 148 SMs.
int bwd_ksplit(int64_t bnh, int nt) {
  const int64_t sms = 148;
  if (bnh >= sms || nt < 2) return 1;
  int64_t k = sms / bnh;                 // as many ranges as keep every CTA at one work item
  if (k > nt) k = nt;
  return k < 1 ? 1 : (int)k;
}

template <typename T>
__global__ void cast_scaled_rows_kernel(const float* __restrict__ src, T* __restrict__ dst, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = from_f<T>(src[i]);
}

template <int DP, typename T, typename TB>
int launch_bwd(const mf_evo_bwd_args& a, cudaStream_t st) {
  using C = Cfg<DP>;
  CUtensorMap mq, mk, mv, mg, mdb;
  int r;
  const int64_t cs[5] = {(int64_t)a.N * a.L * a.H * a.D, (int64_t)a.L * a.H * a.D, (int64_t)a.H * a.D, a.D, 1};
  if ((r = make_qkv_map(&mq, a.q, a.dtype, a.B, a.N, a.L, a.H, a.D, a.q_strides, DP, kT))) return r;
  if ((r = make_qkv_map(&mk, a.k, a.dtype, a.B, a.N, a.L, a.H, a.D, a.k_strides, DP, kT))) return r;
  if ((r = make_qkv_map(&mv, a.v, a.dtype, a.B, a.N, a.L, a.H, a.D, a.v_strides, DP, kT))) return r;
  if ((r = make_qkv_map(&mg, a.d_o, a.dtype, a.B, a.N, a.L, a.H, a.D, cs, DP, kT))) return r;
  BwdP p{};
  p.B = a.B; p.N = a.N; p.L = a.L; p.H = a.H; p.D = a.D;
  p.n_t = (a.L + kT - 1) / kT;
  p.ksplit = bwd_ksplit((int64_t)a.B * a.N * a.H, (a.L + kT - 1) / kT);
  p.n_items = a.B * a.N * a.H * p.ksplit;
  p.lpad = p.n_t * kT;
  p.scale = 1.0f / sqrtf((float)a.D);
  p.c1 = kLog2e * p.scale;
  p.inv_L = 1.0f / a.L;
  p.ab_fmt = a.dtype == MF_BF16 ? 1u : 0u;
  p.bias = a.bias; for (int i = 0; i < 4; ++i) p.bs[i] = a.bias_strides[i];
  p.mask = a.mask; for (int i = 0; i < 3; ++i) p.ms[i] = a.mask_strides[i];
  p.mask_dtype = a.mask_dtype;
  p.lse = a.lse;
  p.dq = a.dq; p.dk = a.dk; p.dv = a.dv;
#ifdef MF_TIMELINE
  p.timeline = g_timeline_bwd;
#endif
  p.status = status_word();
  MF_REQUIRE(p.status, MF_ERR_CUDA, "could not allocate the device status word");
  MF_REQUIRE(tc_async_status() == 0, MF_ERR_CUDA, "an earlier tensor-core kernel gave up on a bounded wait; results are invalid");
  // workspace: delta [B,N,H,L] fp32 | fp32 dBias accumulator (unless d_bias itself can serve) | transposed bias
  float* delta = static_cast<float*>(a.workspace);
  const size_t delta_bytes = align_up(sizeof(float) * (size_t)a.B * a.N * a.H * a.L, 256);
  const int lp4 = (a.L + 3) / 4 * 4;                 // TMA needs 16-byte row pitch
  const bool direct = a.dbias_dtype == MF_F32 && lp4 == a.L;
  const int64_t nb = (int64_t)a.B * a.H * a.L * lp4;
  const size_t acc_bytes = direct ? 0 : align_up(sizeof(float) * (size_t)nb, 256);
  float* dbias = direct ? static_cast<float*>(a.d_bias) : reinterpret_cast<float*>(static_cast<char*>(a.workspace) + delta_bytes);
  p.delta = delta; p.dbias = dbias;
  {
    const int64_t dims[4] = {a.L, a.L, a.H, a.B};
    const int64_t str[4] = {1, lp4, (int64_t)a.L * lp4, (int64_t)a.H * a.L * lp4};
    const int box[4] = {32, 16, 1, 1};
    if ((r = make_tiled_map(&mdb, dbias, MF_F32, 4, dims, str, box, 0))) return r;
  }
  const int64_t n_dq = (int64_t)a.B * a.N * a.L * a.H * a.D;
  p.dq_stream = (a.L + kT - 1) / kT > Cfg<DP>::MAX_QT;
  const bool dq_fp32 = p.ksplit > 1 || p.dq_stream;
  const size_t dq_bytes = dq_fp32 ? align_up(sizeof(float) * (size_t)n_dq, 256) : 0;
  p.dq_acc = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + delta_bytes + acc_bytes);
  if (dq_fp32) MF_CUDA(cudaMemsetAsync(p.dq_acc, 0, sizeof(float) * (size_t)n_dq, st));
  TB* biasT = reinterpret_cast<TB*>(static_cast<char*>(a.workspace) + delta_bytes + acc_bytes + dq_bytes);
  p.biasT_ = biasT;
  {
    MF_CUDA(cudaMemsetAsync(biasT, 0, sizeof(TB) * (size_t)a.B * a.H * a.L * p.lpad, st));
    dim3 grid((a.L + 31) / 32, (a.L + 31) / 32, a.B * a.H), block(32, 8);
    transpose_bias_kernel<TB><<<grid, block, 0, st>>>(static_cast<const TB*>(a.bias), biasT, a.H, a.L, p.lpad, a.bias_strides[0],
                                                       a.bias_strides[1], a.bias_strides[2], a.bias_strides[3]);
    MF_LAUNCHED("transpose_bias_kernel");
  }
  const int64_t rows = (int64_t)a.B * a.N * a.L * a.H;
  evo_delta_tc_kernel<T><<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(static_cast<const T*>(a.o), static_cast<const T*>(a.d_o),
                                                                      delta, rows, a.L, a.H, a.D);
  MF_LAUNCHED("evo_delta_tc_kernel");
  MF_CUDA(cudaMemsetAsync(dbias, 0, sizeof(float) * nb, st));
  const size_t smem = 1024 + 2 * kTileP + 10 * (size_t)C::TILEB + 4 * sizeof(float) * p.lpad + 16 * 4096;
  int grid = sm_count();
  if (grid > p.n_items) grid = p.n_items;
  if (p.dq_stream) {
    auto kern = evo_bwd_tc_kernel<DP, T, TB, true>;
    MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, st>>>(mq, mk, mv, mg, mdb, p);
  } else {
    auto kern = evo_bwd_tc_kernel<DP, T, TB, false>;
    MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, st>>>(mq, mk, mv, mg, mdb, p);
  }
  MF_LAUNCHED("evo_bwd_tc_kernel");
  if (dq_fp32) {
    cast_scaled_rows_kernel<T><<<(unsigned)((n_dq + 255) / 256), 256, 0, st>>>(p.dq_acc, static_cast<T*>(a.dq), n_dq);
    MF_LAUNCHED("cast_scaled_rows_kernel");
  }
  if (!direct) {
    const int64_t rows_b = (int64_t)a.B * a.H * a.L, n_out = rows_b * a.L;
    if (a.dbias_dtype == MF_F32)
      cast_rows_pitched_kernel<float><<<(unsigned)((n_out + 255) / 256), 256, 0, st>>>(dbias, static_cast<float*>(a.d_bias), rows_b, a.L, lp4);
    else
      cast_rows_pitched_kernel<T><<<(unsigned)((n_out + 255) / 256), 256, 0, st>>>(dbias, static_cast<T*>(a.d_bias), rows_b, a.L, lp4);
    MF_LAUNCHED("cast_rows_pitched_kernel");
  }
  return MF_OK;
}

}  // namespace

#ifdef MF_TIMELINE
extern "C" __attribute__((visibility("default"))) void mf_debug_set_timeline_bwd(long long* p) { g_timeline_bwd = p; }
#endif

bool evo_bwd_tc_shape_ok(int L, int D) {
  const int nt = (L + kT - 1) / kT;
  // head sizes above 32 would need more shared memory than an SM has with this tiling: CUDA-core path
  // up to MAX_QT query tiles keep their dQ accumulators in TMEM; longer rows stream dQ through global memory, up to
  // the length whose row statistics still fit the shared memory (L <= 1024)
  return D <= 32 && nt <= 8;
}

size_t evo_bwd_tc_workspace(const mf_evo_bwd_args& a) {
  size_t b = align_up(sizeof(float) * (size_t)a.B * a.N * a.H * a.L, 256);
  const size_t lp4 = (size_t)(a.L + 3) / 4 * 4;
  if (!(a.dbias_dtype == MF_F32 && lp4 == (size_t)a.L)) b += align_up(sizeof(float) * (size_t)a.B * a.H * a.L * lp4, 256);
  const size_t lpad = (size_t)((a.L + kT - 1) / kT) * kT;
  if (bwd_ksplit((int64_t)a.B * a.N * a.H, (a.L + kT - 1) / kT) > 1 || (a.L + kT - 1) / kT > Cfg<32>::MAX_QT)
    b += align_up(sizeof(float) * (size_t)a.B * a.N * a.L * a.H * a.D, 256);         // fp32 dQ accumulator
  b += align_up(dtype_size(a.bias_dtype) * (size_t)a.B * a.H * a.L * lpad, 256);     // transposed bias copy
  return b;
}

#define MF_DISPATCH_BIAS(dt, TB, ...)                                         \
  switch (dt) {                                                               \
    case MF_F32: { using TB = float; __VA_ARGS__; } break;                    \
    case MF_BF16: { using TB = __nv_bfloat16; __VA_ARGS__; } break;           \
    case MF_F16: { using TB = __half; __VA_ARGS__; } break;                   \
    default: return fail(MF_ERR_BAD_ARG, "unknown bias dtype %d", (int)(dt)); \
  }

int evo_bwd_tc(const mf_evo_bwd_args& a, cudaStream_t st) {
  int r = MF_OK;
  if (a.dtype == MF_BF16) {
    MF_DISPATCH_BIAS(a.bias_dtype, TB, {
      r = a.D <= 32 ? launch_bwd<32, __nv_bfloat16, TB>(a, st) : launch_bwd<64, __nv_bfloat16, TB>(a, st);
    });
  } else {
    MF_DISPATCH_BIAS(a.bias_dtype, TB, {
      r = a.D <= 32 ? launch_bwd<32, __half, TB>(a, st) : launch_bwd<64, __half, TB>(a, st);
    });
  }
  return r;
}

}  // namespace mf
