// Pair-biased masked attention backward on the tensor cores (tcgen05 + TMEM + TMA), head sizes up to 64 (as one or two
// halves of 32 columns, template parameter NH).
//
// Two kernels share the transposed-score scheme (keys on the TMEM lanes):
//
//   S''^T = K_j Q_i^T + sqrt(D) * bias^T + terms        dP''^T = V_j dO_i^T - delta_i      (tcgen05.mma into TMEM; the bias
//   P^T   = 2^(c1 * S''^T)                              dS^T   = P^T dP''^T                 term is itself a product with
//   alpha * I, and the key mask, the log-sum-exp and delta enter through one more K = 16 product: evo_tc_common.cuh)
//
// evo_bwd_ws_kernel (dQ, dK, dV).  A persistent CTA owns a (b, n, h) - or a range of its key tiles - and walks the
// key tiles j and, inside, the query tiles i in HALF blocks of [128 keys x 64 queries].  Two teams of eight compute
// warps take alternate half blocks, each with its own score buffers in TMEM, so that the tensor pipe works on one
// team's products while the other team exponentiates.  A thread (key row, 32 query columns) writes packed 16-bit
// P^T and dS^T back over the scores it has just read: they are the TMEM A operands of  dV_j += P^T dO_i  and
// dK_j += dS^T Q_i.  dS^T also goes to a shared-memory tile, read MN-major as the A operand of  dQ_i += dS K_j.
// dK_j / dV_j accumulate in TMEM over the query tiles and dQ_i over the key tiles (or, for long rows and split
// items, leave block by block through fp32 adds in global memory).
//
// evo_dbias_ws_kernel (dBias = sum of dS over the N rows that share the bias).  A CTA keeps ONE (b, h, i tile,
// j tile) and walks a range of rows n: scores and dP for row n+1 are produced while the 16 compute warps turn row n
// into dS and add it to register accumulators; nothing is reduced through memory until the range is done.  Ranges
// are summed in a fixed order afterwards, so dBias is bit-reproducible.  With one row per bias (N = 1) the kernel is not
// run: dS is the answer and evo_bwd_ws_kernel stores it.
//
// delta_i = rowsum(dO_i * O_i) and the term tiles come from a small pre-kernel.  The bias tile of a half block is the A
// operand [128 keys x 16 queries] of the products that add it: the caller's bias ([queries][keys]) is exactly that in
// MN-major form and is loaded in place when TMA can address it; otherwise a transposed 16-bit copy is made first.  All waits are bounded
// (tc.cuh); on expiry the CTA runs dry without touching global memory and the host sees mf_async_status() != 0.
#include <type_traits>

#include "evo_tc_common.cuh"

namespace mf {
namespace {
using namespace tcx;

constexpr int kT = 128;             // tile edge (keys and queries)
constexpr int kHalf = 64;           // queries per half block
constexpr int kComputeWarps = 16;
constexpr int kThreads = (kComputeWarps + 4) * 32;
constexpr int kTileB = 128 * 64;    // [128 x 32] 16-bit operand tile, 64-byte rows, 64B swizzle
constexpr int kAtomB = 128 * 128;   // [128 x 64] 16-bit tile, 128-byte rows, 128B swizzle (bias^T atoms, dS^T atoms)
constexpr int kDP = 32;             // padded head size
// Head sizes up to 64 are handled as NH = 1 or 2 halves of 32 columns: every operand is loaded as NH tiles of [128 x 32]
// (the same layout whatever the head size), the score products run over 2 * NH slices of 16, and each half has its own
// 32 columns in the dK, dV and dQ accumulators.  With two halves the stages are twice as large, so there are fewer:
template <int NH> struct Geo {
  static constexpr int kStageB = 2 * NH * kTileB + 4096;            // main kernel: a (K, V, XK) or (Q, dO, XQ) stage
  static constexpr int kDbStageB = 4 * NH * kTileB + 2 * 4096;      // dBias kernel: one row's Q, dO, K, V tiles and its two term tiles
  static constexpr int NQ = NH == 1 ? 3 : 2;       // (Q, dO, XQ) stages
  static constexpr int NKV = NH == 1 ? 2 : 1;      // (K, V, XK) stages
  static constexpr int NB = NH == 1 ? 3 : 2;       // bias^T atoms
  static constexpr int NS = NH == 1 ? 3 : 2;       // dBias kernel: operand stages
  static constexpr size_t kMainSmem = 1024 + 4 * (size_t)kAtomB + NB * (size_t)kAtomB + (NQ + NKV) * (size_t)kStageB + 2048 + kXTileB;
  static constexpr size_t kDbSmem = 1024 + 2 * (size_t)kAtomB + NS * (size_t)kDbStageB + 2048 + kXTileB;
};
static_assert(Geo<2>::kMainSmem + 1024 <= 227 * 1024 && Geo<1>::kMainSmem + 1024 <= 227 * 1024, "shared memory of the main kernel");
static_assert(Geo<2>::kDbSmem + 1024 <= 227 * 1024 && Geo<1>::kDbSmem + 1024 <= 227 * 1024, "shared memory of the dBias kernel");
// registers per thread: at launch (640 threads) / compute warps / helper warps after setmaxnreg.  The raise of the
// compute warps can only draw on what the helper warps release inside the CTA - otherwise it never returns.
constexpr int kLaunchRegs = 96, kComputeRegs = 104, kHelperRegs = 64;
static_assert(kComputeWarps * 32 * kComputeRegs + 128 * kHelperRegs <= kThreads * kLaunchRegs, "setmaxnreg budget");

struct BwdWsP {
  int B, N, L, H, D;
  int n_t, n_items, lpad;
  int ksplit;            // work items per (b, n, h): the key tiles are split into this many ranges
  int dq_stream;         // dQ leaves the SM block by block (more query tiles than TMEM holds)
  int dbuf;              // dK/dV accumulators double-buffered over the key tiles
  float* dq_acc;         // fp32 [B,N,L,H,D] accumulator of dQ when ksplit > 1 or dq_stream
  float c1, scale, inv_L;
  uint32_t fmt, bfmt;
  int n_alpha; float alpha[2];
  int bias_b_mul;
  int bias_mn;           // the bias atoms hold the caller's bias as it is ([queries][keys]) and are read MN-major
  const uint8_t* xq; const uint8_t* xk;     // rank-one term tiles (evo_extras_ws_kernel)
  const int* flags;                         // per (b, n, h): every key of the row is masked
  void* dbias_direct;                       // N == 1 and a 16-bit d_pair_bias: dS is the answer, written by this kernel
  void *dq, *dk, *dv;
  int* status;
};

struct Bars {
  uint64_t kv_full[2], kv_empty[2], qd_full[3], qd_empty[3], bt_full[3], bt_empty[3];
  uint64_t sd_ready[2], written[2], buf_free[2];
  uint64_t ds_written[2], dq_done[2];        // per block parity: dS^T tile complete in shared memory / its dQ product complete
  uint64_t kv_done;                          // the dK / dV accumulation of a key tile is complete
  uint64_t item_done[2];                     // the compute warps have read the item's on-chip dQ accumulators
  uint64_t kv_drained, dq_drained[2];
};

// 1-D bulk copy global -> shared, completion counted in bytes on `bar` (addresses and size multiples of 16 bytes)
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// One thread per (b, n, i < lpad, h): delta = sum_d dO * O (16-byte loads; D is a multiple of 8), the XQ row of query i
// and, for h == 0, the XK row of key i.  Consecutive threads take the heads of one token, then the next token: a warp
// reads one contiguous piece of o and dO.  (Measured against a thread per token walking all heads, and against
// consecutive threads taking consecutive tokens of one head: 22.8 us against 27.3 and 28.5 at the benchmark size.)
// flags[bnh] is raised when the row (b, n) has every key masked (lse = -FLT_MAX).
template <typename T>
__global__ void evo_extras_ws_kernel(const T* __restrict__ o, const T* __restrict__ d_o, const float* __restrict__ lse,
                                     const void* __restrict__ mask, int64_t ms_b, int64_t ms_n, int64_t ms_l, int mask_dtype,
                                     uint8_t* __restrict__ xq, uint8_t* __restrict__ xk, int* __restrict__ flags,
                                     int64_t n_threads, int N, int L, int lpad, int H, int D) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_threads) return;
  const int hg = (int)(idx % H); const int64_t t = idx / H; const int i = (int)(t % lpad); const int64_t bn = t / lpad;
  constexpr int hpt = 1;
  const float sqrt_d = sqrtf((float)D);
  const __nv_bfloat16 one = __float2bfloat16_rn(1.f), zero = __float2bfloat16_rn(0.f);
  const int nt = lpad / 128, tile = i >> 7, r = i & 127;
  for (int h = hg * hpt; h < (hg + 1) * hpt; ++h) {
    const int64_t bnh = bn * H + h;
    float nl = kMinusBig, nd = 0.f;
    if (i < L) {
      const int64_t row = (bn * L + i) * H + h;
      const uint4* po = reinterpret_cast<const uint4*>(o + row * D);
      const uint4* pg = reinterpret_cast<const uint4*>(d_o + row * D);
      float dl = 0.f;
      for (int c = 0; c < D / 8; ++c) {
        const uint4 a = __ldg(po + c), g = __ldg(pg + c);
        const uint32_t av[4] = {a.x, a.y, a.z, a.w}, gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x = Pack2<T>::unpack(av[e]), y = Pack2<T>::unpack(gv[e]);
          dl = fmaf(x.x, y.x, dl); dl = fmaf(x.y, y.y, dl);
        }
      }
      nd = -dl;
      const float lv = lse[bnh * L + i];
      if (lv <= -3e38f) flags[bnh] = 1; else nl = -lv * sqrt_d;
    }
    __nv_bfloat16 a[3], b[3];
    split3(nl, a); split3(nd, b);
    uint8_t* base = xq + ((int64_t)bnh * nt + tile) * kXTileB;
    *reinterpret_cast<uint4*>(base + swz_offset(r, 0, 32)) = make_uint4(pack_bf(one, one), pack_bf(one, a[0]), pack_bf(a[1], a[2]), pack_bf(b[0], b[1]));
    *reinterpret_cast<uint4*>(base + swz_offset(r, 1, 32)) = make_uint4(pack_bf(b[2], zero), 0u, 0u, 0u);
  }
  if (hg == 0) {
    float mv = kMinusBig;
    if (i < L) {
      const int n = (int)(bn % N); const int64_t b = bn / N;
      const int64_t mi = b * ms_b + n * ms_n + (int64_t)i * ms_l;
      mv = mask_dtype == MF_U8 ? (static_cast<const uint8_t*>(mask)[mi] ? 0.f : kMinusBig) : fmaxf(load_rt(mask, mi, mask_dtype) * sqrt_d, kMinusBig);
    }
    __nv_bfloat16 m[3];
    split3(mv, m);
    uint8_t* base = xk + ((int64_t)bn * nt + tile) * kXTileB;
    *reinterpret_cast<uint4*>(base + swz_offset(r, 0, 32)) = make_uint4(pack_bf(m[0], m[1]), pack_bf(m[2], one), pack_bf(one, one), 0u);
    *reinterpret_cast<uint4*>(base + swz_offset(r, 1, 32)) = make_uint4(0u, 0u, 0u, 0u);
  }
}

// biasT[b][h][j][i] = bias[b][h][i][j] in the 16-bit type TO, rows padded to `lpad` entries (the padding is zeroed by
// the caller).  The kernels work with keys on the TMEM lanes, so the tile they need has the queries contiguous.
template <typename TB, typename TO>
__global__ void transpose_bias_ws_kernel(const TB* __restrict__ bias, TO* __restrict__ biasT, int H, int L, int lpad,
                                         int64_t sb, int64_t sh, int64_t si, int64_t sj) {
  // 64 x 64 tiles; a thread moves two neighbouring entries at a time, on the way in (two keys of one query) and on the
  // way out (two queries of one key), so that a warp reads and writes 128 or more contiguous bytes
  __shared__ float tile[64][65];
  const int bh = blockIdx.z, b = bh / H, h = bh % H;
  const int i0 = blockIdx.y * 64, j0 = blockIdx.x * 64;
  const TB* src = bias + b * sb + h * sh;
  const bool pair_in = sj == 1 && sizeof(TB) == 2 && (si & 1) == 0 && (((sb | sh) & 1) == 0) && (reinterpret_cast<uintptr_t>(bias) & 3) == 0;
  for (int k = threadIdx.y; k < 64; k += blockDim.y) {
    const int i = i0 + k, j = j0 + 2 * threadIdx.x;
    if (i >= L) continue;
    bool done = false;
    if constexpr (sizeof(TB) == 2) {
      if (pair_in && j + 1 < L) {
        const uint32_t v = *reinterpret_cast<const uint32_t*>(src + (int64_t)i * si + j);
        TB lo, hi;
        *reinterpret_cast<unsigned short*>(&lo) = (unsigned short)(v & 0xffffu);
        *reinterpret_cast<unsigned short*>(&hi) = (unsigned short)(v >> 16);
        tile[k][2 * threadIdx.x] = to_f(lo); tile[k][2 * threadIdx.x + 1] = to_f(hi);
        done = true;
      }
    }
    if (!done) {
      if (j < L) tile[k][2 * threadIdx.x] = to_f(src[(int64_t)i * si + (int64_t)j * sj]);
      if (j + 1 < L) tile[k][2 * threadIdx.x + 1] = to_f(src[(int64_t)i * si + (int64_t)(j + 1) * sj]);
    }
  }
  __syncthreads();
  for (int k = threadIdx.y; k < 64; k += blockDim.y) {
    const int j = j0 + k, i = i0 + 2 * threadIdx.x;
    if (j >= L || i >= L) continue;
    TO* dst = biasT + ((int64_t)bh * L + j) * lpad + i;         // lpad is a multiple of 128 and i is even: 4-byte aligned
    const TO a = from_f<TO>(tile[2 * threadIdx.x][k]);
    const TO c = i + 1 < L ? from_f<TO>(tile[2 * threadIdx.x + 1][k]) : from_f<TO>(0.f);
    uint32_t v = (uint32_t)*reinterpret_cast<const unsigned short*>(&a) | ((uint32_t)*reinterpret_cast<const unsigned short*>(&c) << 16);
    *reinterpret_cast<uint32_t*>(dst) = v;
  }
}

// P^T and dS^T of one thread for 16 query columns.  sr: scores S''^T with the bias, mask and log-sum-exp terms already
// inside (see the rank-one terms above), dr: dP^T - delta.  Results packed two queries per word.  `careful`: the row (b, n)
// has every key masked - P is uniform over the keys of the row and no gradient passes through the (masked) logits.
template <typename T>
__device__ __forceinline__ void p_and_ds(const uint32_t (&sr)[16], const uint32_t (&dr)[16], float c1, bool careful,
                                         float p_uniform, uint32_t* __restrict__ pp, uint32_t* __restrict__ dd) {
  const float2 c1c1 = make_float2(c1, c1);
  if (careful) {
    const uint32_t pu = Pack2<T>::pack(p_uniform, p_uniform);
#pragma unroll
    for (int c = 0; c < 8; ++c) { pp[c] = pu; dd[c] = 0u; }
    return;
  }
#pragma unroll
  for (int c2 = 0; c2 < 8; ++c2) {
    const float2 xx = mul2(make_float2(__uint_as_float(sr[c2 * 2]), __uint_as_float(sr[c2 * 2 + 1])), c1c1);
    const float2 pr = make_float2(ex2f(xx.x), ex2f(xx.y));
    const float2 ds = mul2(pr, make_float2(__uint_as_float(dr[c2 * 2]), __uint_as_float(dr[c2 * 2 + 1])));
    pp[c2] = Pack2<T>::pack(pr.x, pr.y);
    dd[c2] = Pack2<T>::pack(ds.x, ds.y);
  }
}

template <typename T, typename TB, bool DQS, int NH>      // DQS: dQ streamed block by block through global memory
__global__ void __launch_bounds__(kThreads, 1)
evo_bwd_ws_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                  const __grid_constant__ CUtensorMap mv, const __grid_constant__ CUtensorMap mg,
                  const __grid_constant__ CUtensorMap mbt, const BwdWsP p MF_TRACE_PARAM) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr int kStageB = Geo<NH>::kStageB, NQ = Geo<NH>::NQ, NKV = Geo<NH>::NKV, NB = Geo<NH>::NB;
  uint8_t* sDS = smem;                          // [2 blocks][2 atoms]: dS^T tiles for the dQ product
  uint8_t* sBT = sDS + 4 * kAtomB;              // bias^T atoms, ring of NB
  uint8_t* sKV = sBT + NB * kAtomB;             // [NKV stages][K halves, V halves, XK]
  uint8_t* sQD = sKV + NKV * kStageB;           // [NQ stages][Q halves, dO halves, XQ]
  uint8_t* sI = sQD + NQ * kStageB;             // alpha * I, two terms
  uint8_t* sXC = sI + 2048;                     // constant tile of the -delta term

  __shared__ Bars bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    abort_s = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar.kv_full[i], 1); mbar_init(&bar.kv_empty[i], 1);
      mbar_init(&bar.sd_ready[i], 1); mbar_init(&bar.written[i], kComputeWarps / 2);
      mbar_init(&bar.buf_free[i], 1);
      mbar_init(&bar.ds_written[i], kComputeWarps); mbar_init(&bar.dq_done[i], 1);
      mbar_init(&bar.item_done[i], kComputeWarps);
      mbar_init(&bar.dq_drained[i], 4 * NH);
    }
    for (int i = 0; i < 3; ++i) {
      mbar_init(&bar.qd_full[i], 1); mbar_init(&bar.qd_empty[i], 1); mbar_init(&bar.bt_full[i], 1); mbar_init(&bar.bt_empty[i], 1);
    }
    mbar_init(&bar.kv_done, 1);
    mbar_init(&bar.kv_drained, 8 * NH);
    mbar_fence_init();
    prefetch_tmap(&mq); prefetch_tmap(&mk); prefetch_tmap(&mv); prefetch_tmap(&mg); prefetch_tmap(&mbt);
  }
  write_alpha_identity<TB>(sI, p.alpha[0], tid, kThreads);
  write_alpha_identity<TB>(sI + 1024, p.alpha[1], tid, kThreads);
  write_xc_tile(sXC, tid, kThreads);
  fence_async_smem();
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  volatile int* abort_flag = &abort_s;
  const uint32_t tm0 = tmem_base_s;
  const int nt = p.n_t;
  const bool dbuf = p.dbuf != 0;
  // TMEM: team t's scores S''^T at t*128 + [0,64), dP^T at t*128 + [64,128) (P^T / dS^T are packed over them);
  // dK | dV accumulators (one or two sets); dQ accumulators (one per query tile, or two used in turn when streaming)
  // (each accumulator has 32 columns per head half: dK = [0, 32 NH), dV = [32 NH, 64 NH) of a set)
  const uint32_t tKV = tm0 + 256, tDQ = tm0 + 256 + (dbuf ? 128 : 64) * NH;
  const uint32_t kv_set = dbuf ? 64 * NH : 0;    // column distance between the two dK|dV accumulator sets
  // work item = (b, n, h, range of key tiles)
  auto item_range = [&](int item, int& jt0, int& jt1) {
    const int sp = item % p.ksplit;
    jt0 = sp * nt / p.ksplit; jt1 = (sp + 1) * nt / p.ksplit;
  };

  if (warp < kComputeWarps) {
    // ============================================================================ compute warps
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kComputeRegs));
    const int team = warp >> 3;                       // takes the half blocks with (half == team)
    const int ch = (warp >> 2) & 1;                   // which 32 of the half block's 64 query columns
    const int w = warp >> 2;                          // 0..3: role in the write-out of accumulators
    const int r = (warp & 3) * 32 + lane;             // TMEM lane = key row inside the tile
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tST = tm0 + team * 128 + ch * 32 + lane_addr, tDP = tST + 64;
    MF_TRACE_DECL(tr, team, blockIdx.x == 0 && (warp == 0 || warp == 8) && lane == 0);

    // dK (scaled) and dV rows of key `j` from accumulator set `kc`: the warps with w < 2 NH take one (dK or dV, head
    // half) each
    const int kv_which = NH == 1 ? w : (w >> 1), kv_hh = NH == 1 ? 0 : (w & 1);
    auto store_kv = [&](uint32_t kc, int j, int b, int n, int h) {
      tc_fence_after();
      uint32_t o32[32];
      tmem_ld32(tKV + (kc & 1) * kv_set + kv_which * 32 * NH + kv_hh * 32 + lane_addr, o32);
      tmem_ld_wait();
      tc_fence_before();
      if (j < p.L && !*abort_flag) {
        const float sc = kv_which == 0 ? p.scale : 1.f;
        T* orow = static_cast<T*>(kv_which == 0 ? p.dk : p.dv) + ((((int64_t)b * p.N + n) * p.L + j) * p.H + h) * p.D + kv_hh * 32;
#pragma unroll
        for (int d8 = 0; d8 < 4; ++d8) {
          if (kv_hh * 32 + d8 * 8 < p.D) {
            uint4 v;
            v.x = Pack2<T>::pack(__uint_as_float(o32[d8 * 8]) * sc, __uint_as_float(o32[d8 * 8 + 1]) * sc);
            v.y = Pack2<T>::pack(__uint_as_float(o32[d8 * 8 + 2]) * sc, __uint_as_float(o32[d8 * 8 + 3]) * sc);
            v.z = Pack2<T>::pack(__uint_as_float(o32[d8 * 8 + 4]) * sc, __uint_as_float(o32[d8 * 8 + 5]) * sc);
            v.w = Pack2<T>::pack(__uint_as_float(o32[d8 * 8 + 6]) * sc, __uint_as_float(o32[d8 * 8 + 7]) * sc);
            *reinterpret_cast<uint4*>(orow + d8 * 8) = v;
          }
        }
      }
    };
    // rows of a dQ accumulator (TMEM lane = query) added, scaled, to the fp32 dQ rows in global memory
    auto add_dq = [&](uint32_t tacc, int it2, int hh, int b, int n, int h) {
      tc_fence_after();
      uint32_t o32[32];
      tmem_ld32(tacc + hh * 32 + lane_addr, o32);
      tmem_ld_wait();
      tc_fence_before();
      const int i = it2 * kT + r;
      if (i < p.L && !*abort_flag) {
        float* arow = p.dq_acc + ((((int64_t)b * p.N + n) * p.L + i) * p.H + h) * p.D + hh * 32;
#pragma unroll
        for (int d4 = 0; d4 < 8; ++d4)
          if (hh * 32 + d4 * 4 < p.D)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(arow + d4 * 4),
                         "f"(__uint_as_float(o32[d4 * 4]) * p.scale), "f"(__uint_as_float(o32[d4 * 4 + 1]) * p.scale),
                         "f"(__uint_as_float(o32[d4 * 4 + 2]) * p.scale), "f"(__uint_as_float(o32[d4 * 4 + 3]) * p.scale) : "memory");
      }
    };

    // streamed dQ: which warps drain the accumulator of block g2, and which head half each takes
    const int dq_hh = NH == 1 ? 0 : (w & 1);
    auto dq_mine = [&](uint32_t g2) { return NH == 1 ? w == (int)(g2 & 3) : (w >> 1) == (int)(g2 & 1); };
    uint32_t g = 0;                 // full blocks seen by this CTA (both teams count every block)
    uint32_t kv_cnt = 0;            // (item, j) pairs so far
    int item_no = 0;
    int pend_j = -1; uint32_t pend_kc = 0; int pend_b = 0, pend_n = 0, pend_h = 0;   // deferred dK/dV write-out
    int dqp_it = -1; uint32_t dqp_g = 0; int dqp_b = 0, dqp_n = 0, dqp_h = 0;        // deferred streamed dQ
    int special_next = blockIdx.x < p.n_items ? p.flags[blockIdx.x / p.ksplit] : 0;
    for (int item = blockIdx.x; item < p.n_items; item += gridDim.x, ++item_no) {
      const int bnh = item / p.ksplit;
      int jt0, jt1; item_range(item, jt0, jt1);
      const int h = bnh % p.H, bn = bnh / p.H, n = bn % p.N, b = bn / p.N;
      const int sbuf = item_no & 1;
      const bool special = special_next != 0;      // every key of the row is masked: the item takes the careful path
      if (item + (int)gridDim.x < p.n_items) special_next = p.flags[(item + (int)gridDim.x) / p.ksplit];
      for (int jt = jt0; jt < jt1; ++jt, ++kv_cnt) {
        const int j = jt * kT + r;
        const float p_uniform = j < p.L ? p.inv_L : 0.f;       // careful path: P of a fully masked row
        for (int it = 0; it < nt; ++it, ++g) {
          // ---- S''^T, dP^T of my half block -> registers
          tr(1);
          wait_or_flag(&bar.sd_ready[team], g & 1, abort_flag);
          tc_fence_after();
          tr(2);
          uint32_t pp[16], dd[16];
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {        // 16 query columns at a time keeps the live registers down
            uint32_t sr[16], dr[16];
            tmem_ld16(tST + hf * 16, sr);
            tmem_ld16(tDP + hf * 16, dr);
            tmem_ld_wait();
            if (hf == 0) tr(3);
            p_and_ds<T>(sr, dr, p.c1, special, p_uniform, pp + hf * 8, dd + hf * 8);
          }
          tr(4);
          // ---- packed P^T / dS^T over the scores just read (A operands of the dV / dK products)
          tmem_st16(tST, pp);
          tmem_st16(tDP, dd);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar.written[team]);
          // ---- a bias that only this row uses (N = 1): d_pair_bias[b, h, i, j] = dS[i, j], no sum over rows; lanes hold
          // consecutive keys j, so every store instruction writes 64 contiguous bytes
          if (p.dbias_direct && j < p.L) {
            const int i0 = it * kT + team * kHalf + ch * 32;
            T* dst = static_cast<T*>(p.dbias_direct) + (((int64_t)b * p.H + h) * p.L + i0) * p.L + j;
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              if (i0 + 2 * c < p.L) *reinterpret_cast<unsigned short*>(dst) = (unsigned short)(dd[c] & 0xffffu);
              if (i0 + 2 * c + 1 < p.L) *reinterpret_cast<unsigned short*>(dst + p.L) = (unsigned short)(dd[c] >> 16);
              dst += 2 * (int64_t)p.L;
            }
          }
          // ---- dS^T also to the shared-memory tile of this block (A operand of the dQ product), once the dQ
          // product that read this buffer two blocks ago is complete
          if (g >= 2) wait_or_flag(&bar.dq_done[g & 1], ((g >> 1) - 1) & 1, abort_flag);
          tr(5);
          {
            uint8_t* atom = sDS + (g & 1) * 2 * kAtomB + team * kAtomB;
#pragma unroll
            for (int c = 0; c < 4; ++c)
              *reinterpret_cast<uint4*>(atom + swz_offset(r, ch * 4 + c, 128)) = make_uint4(dd[c * 4], dd[c * 4 + 1], dd[c * 4 + 2], dd[c * 4 + 3]);
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar.ds_written[g & 1]);
          tr(6);
          // ---- streamed dQ: the product of the previous block sits in accumulator (g - 1) & 1; the four warps with
          // w == (g - 1) & 3 add it to global memory and hand the accumulator back
          if constexpr (DQS) {
            if (dqp_it >= 0 && dq_mine(dqp_g)) {
              wait_or_flag(&bar.dq_done[dqp_g & 1], (dqp_g >> 1) & 1, abort_flag);
              add_dq(tDQ + (dqp_g & 1) * 32 * NH, dqp_it, dq_hh, dqp_b, dqp_n, dqp_h);
              __syncwarp();
              if (lane == 0) mbar_arrive(&bar.dq_drained[dqp_g & 1]);
            }
            dqp_it = it; dqp_g = g; dqp_b = b; dqp_n = n; dqp_h = h;
          }
          // ---- dK_j, dV_j of the key tile that finished one block ago (warps 0-7)
          if (pend_j >= 0 && w < 2 * NH) {
            wait_or_flag(&bar.kv_done, pend_kc & 1, abort_flag);
            store_kv(pend_kc, pend_j, pend_b, pend_n, pend_h);
            if (!dbuf) { __syncwarp(); if (lane == 0) mbar_arrive(&bar.kv_drained); }
          }
          pend_j = -1;
          if (it == nt - 1) { pend_j = j; pend_kc = kv_cnt; pend_b = b; pend_n = n; pend_h = h; }
        }
      }
      // ---- end of the item: the last key tile's dK/dV, the last streamed dQ, or every query tile's dQ
      tr(7);
      if (pend_j >= 0 && w < 2 * NH) {
        wait_or_flag(&bar.kv_done, pend_kc & 1, abort_flag);
        store_kv(pend_kc, pend_j, pend_b, pend_n, pend_h);
        if (!dbuf) { __syncwarp(); if (lane == 0) mbar_arrive(&bar.kv_drained); }
      }
      pend_j = -1;
      const uint32_t gl = g - 1;
      wait_or_flag(&bar.dq_done[gl & 1], (gl >> 1) & 1, abort_flag);
      if constexpr (DQS) {
        if (dqp_it >= 0 && dq_mine(dqp_g)) {
          add_dq(tDQ + (dqp_g & 1) * 32 * NH, dqp_it, dq_hh, dqp_b, dqp_n, dqp_h);
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar.dq_drained[dqp_g & 1]);
        }
        dqp_it = -1;
      } else {
        for (int u = w; u < nt * NH; u += 4) {          // one (query tile, head half) accumulator per turn
          const int it = u / NH, hh = u - it * NH;
          if (p.ksplit > 1) {
            add_dq(tDQ + it * 32 * NH, it, hh, b, n, h);
          } else {
            tc_fence_after();
            uint32_t o32[32];
            tmem_ld32(tDQ + it * 32 * NH + hh * 32 + lane_addr, o32);
            tmem_ld_wait();
            tc_fence_before();
            const int i = it * kT + r;
            if (i < p.L && !*abort_flag) {
              T* orow = static_cast<T*>(p.dq) + ((((int64_t)b * p.N + n) * p.L + i) * p.H + h) * p.D + hh * 32;
#pragma unroll
              for (int d8 = 0; d8 < 4; ++d8) {
                if (hh * 32 + d8 * 8 < p.D) {
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
        }
      }
      // this item's on-chip dQ accumulators have been read out by this warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.item_done[sbuf]);
      tr(8);
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kHelperRegs));
    // The helper roles are run by whole warps (one elected lane issues: see mma_ss_el); every exit decision is a warp vote.
    auto dead = [&] { return __any_sync(0xffffffffu, *abort_flag) != 0; };
    constexpr uint32_t hi64 = desc_hi(512, kSw64), hi128 = desc_hi(1024, kSw128);
    constexpr uint32_t kTile16 = kTileB / 16, kAtom16 = kAtomB / 16;      // descriptor address units
    constexpr uint32_t hi32 = desc_hi(256, kSw32), kStage16 = kStageB / 16, kX16 = kXTileB / 16;
    // inside a stage: the NH halves of the first operand (K or Q), the NH halves of the second (V or dO), the term tile
    constexpr uint32_t kOp2 = NH * kTile16, kTerm16 = 2 * NH * kTile16;
    const uint32_t kv_base = desc_lo(smem_u32(sKV), 16), qd_base = desc_lo(smem_u32(sQD), 16);
    if (warp == kComputeWarps) {
      // ========================================================================== dV / dK issuer: per half block
      //   dV_j += P^T dO_i,  dK_j += dS^T Q_i   (A = packed P^T / dS^T in TMEM, B = the dO / Q rows of the half, MN-major;
      //   one group of four products per head half, into that half's 32 accumulator columns)
      const uint32_t id_kv = idesc_f16(128, 32, p.fmt, 0, 1);
      MF_TRACE_DECL(tr, 2, blockIdx.x == 0 && lane == 0);
      uint32_t g = 0, kv = 0, qslot = 0;
      for (int item = blockIdx.x; item < p.n_items && !dead(); item += gridDim.x) {
        int jt0, jt1; item_range(item, jt0, jt1);
        for (int jt = jt0; jt < jt1 && !dead(); ++jt, ++kv) {
          if (!dbuf && kv > 0) wait_or_flag(&bar.kv_drained, (kv - 1) & 1, abort_flag);
          const uint32_t tdk = tKV + (kv & 1) * kv_set, tdv = tdk + 32 * NH;
          for (int it = 0; it < nt && !dead(); ++it, ++g) {
            const uint32_t q_lo = qd_base + qslot * kStage16, do_lo = q_lo + kOp2;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              tr(20);
              wait_or_flag(&bar.written[half], g & 1, abort_flag);
              tc_fence_after();
              tr(21);
              const uint32_t tPt = tm0 + half * 128, tDSt = tPt + 64;
              const bool first = it == 0 && half == 0;
#pragma unroll
              for (int hh = 0; hh < NH; ++hh) {
                const uint32_t b_do = do_lo + hh * kTile16 + half * 256, b_q = q_lo + hh * kTile16 + half * 256;
                mma_ts_el(tdv + hh * 32, tPt, b_do, hi64, id_kv, !first);
                mma_ts_el(tdv + hh * 32, tPt + 8, b_do + 64, hi64, id_kv, true);
                mma_ts_el(tdv + hh * 32, tPt + 32, b_do + 128, hi64, id_kv, true);
                mma_ts_el(tdv + hh * 32, tPt + 40, b_do + 192, hi64, id_kv, true);
                mma_ts_el(tdk + hh * 32, tDSt, b_q, hi64, id_kv, !first);
                mma_ts_el(tdk + hh * 32, tDSt + 8, b_q + 64, hi64, id_kv, true);
                mma_ts_el(tdk + hh * 32, tDSt + 32, b_q + 128, hi64, id_kv, true);
                mma_ts_el(tdk + hh * 32, tDSt + 40, b_q + 192, hi64, id_kv, true);
              }
              tc_commit_el(&bar.buf_free[half]);
              tr(22);
            }
            tc_commit_el(&bar.qd_empty[qslot]);
            if (it == nt - 1) tc_commit_el(&bar.kv_done);
            if (++qslot == NQ) qslot = 0;
          }
        }
      }
    } else if (warp == kComputeWarps + 3) {
      // ========================================================================== dQ issuer: per block
      //   dQ_i += dS K_j   (A = the dS^T tile in shared memory read MN-major: M = queries; B = K_j, MN-major)
      const uint32_t id_q = idesc_f16(128, 32, p.fmt, 1, 1);
      const uint32_t ds_base = desc_lo(smem_u32(sDS), kAtomB);
      uint32_t g = 0, kv = 0;
      int item_no = 0;
      for (int item = blockIdx.x; item < p.n_items && !dead(); item += gridDim.x, ++item_no) {
        int jt0, jt1; item_range(item, jt0, jt1);
        // the on-chip dQ accumulators of the previous item must have been read out before they start afresh
        if (!DQS && item_no > 0) wait_or_flag(&bar.item_done[(item_no - 1) & 1], ((item_no - 1) >> 1) & 1, abort_flag);
        for (int jt = jt0; jt < jt1 && !dead(); ++jt, ++kv) {
          const uint32_t k_lo = kv_base + (kv % NKV) * kStage16;
          for (int it = 0; it < nt && !dead(); ++it, ++g) {
            wait_or_flag(&bar.ds_written[g & 1], (g >> 1) & 1, abort_flag);
            if constexpr (DQS) { if (g >= 2) wait_or_flag(&bar.dq_drained[g & 1], ((g >> 1) - 1) & 1, abort_flag); }
            tc_fence_after();
            const uint32_t a_lo = ds_base + (g & 1) * 2 * kAtom16;
            const uint32_t tacc = tDQ + (DQS ? (g & 1) : it) * 32 * NH;
#pragma unroll
            for (int hh = 0; hh < NH; ++hh) {          // one group of eight products per head half
              const uint32_t kh = k_lo + hh * kTile16;
              mma_ss_el(tacc + hh * 32, a_lo, hi128, kh, hi64, id_q, DQS ? false : jt > jt0);
#pragma unroll
              for (int ks = 1; ks < 8; ++ks) mma_ss_el(tacc + hh * 32, a_lo + ks * (2048 / 16), hi128, kh + ks * 64, hi64, id_q, true);
            }
            tc_commit_el(&bar.dq_done[g & 1]);
            if (it == nt - 1) tc_commit_el(&bar.kv_empty[kv % NKV]);
          }
        }
      }
    } else if (warp == kComputeWarps + 2) {
      // ========================================================================== score issuer: per half block
      //   S''^T = K_j Q_i^T + alpha * bias^T,  dP^T = V_j dO_i^T
      const uint32_t id_s = idesc_f16(128, kHalf, p.fmt, 0, 0);
      // The bias atom of a half block is the A operand [128 keys x 64 queries] of four K = 16 products.  Either it holds
      // rows of a transposed copy of the bias (keys as rows, K-major A), or - when TMA can address the caller's bias - the
      // bias as it is: two [64 queries x 64 keys] pieces read MN-major (keys contiguous), and no copy is made.
      const uint32_t id_b = idesc_f16(128, 16, p.bfmt, p.bias_mn ? 1u : 0u, 0);
      const uint32_t id_x = idesc_f16(128, kHalf, 1u, 0, 0);        // the rank-one term tiles are bf16 whatever q/k/v are
      const uint32_t xc_lo = desc_lo(smem_u32(sXC), 16);
      const uint32_t bt_base = desc_lo(smem_u32(sBT), p.bias_mn ? 8192 : 16);
      const uint32_t bstep = p.bias_mn ? 2048 / 16 : 2;            // 16 queries further: 16 rows of 128 bytes, or 32 bytes
      const uint32_t i_lo0 = desc_lo(smem_u32(sI), 16), i_lo1 = i_lo0 + 1024 / 16;
      const bool two_terms = p.n_alpha > 1;
      MF_TRACE_DECL(tr, 3, blockIdx.x == 0 && lane == 0);
      uint32_t g = 0, kv = 0, bslot = 0, buse = 0, qslot = 0, quse = 0;
      for (int item = blockIdx.x; item < p.n_items && !dead(); item += gridDim.x) {
        int jt0, jt1; item_range(item, jt0, jt1);
        for (int jt = jt0; jt < jt1 && !dead(); ++jt, ++kv) {
          wait_or_flag(&bar.kv_full[kv % NKV], (kv / NKV) & 1, abort_flag);
          const uint32_t k_lo = kv_base + (kv % NKV) * kStage16, v_lo = k_lo + kOp2, xk_lo = k_lo + kTerm16;
          for (int it = 0; it < nt && !dead(); ++it, ++g) {
            wait_or_flag(&bar.qd_full[qslot], quse & 1, abort_flag);
            const uint32_t q_blk = qd_base + qslot * kStage16;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              tr(30);
              wait_or_flag(&bar.bt_full[bslot], buse & 1, abort_flag);
              if (g >= 1) wait_or_flag(&bar.buf_free[half], (g - 1) & 1, abort_flag);
              tc_fence_after();
              tr(31);
              const uint32_t tS = tm0 + half * 128, tD = tS + 64;
              const uint32_t q_lo = q_blk + half * 256, g_lo = q_lo + kOp2, xq_lo = q_blk + kTerm16 + half * (kX16 / 2);
#pragma unroll
              for (int hh = 0; hh < NH; ++hh) {
                mma_ss_el(tS, k_lo + hh * kTile16, hi64, q_lo + hh * kTile16, hi64, id_s, hh > 0);
                mma_ss_el(tS, k_lo + hh * kTile16 + 2, hi64, q_lo + hh * kTile16 + 2, hi64, id_s, true);
              }
              mma_ss_el(tS, xk_lo, hi32, xq_lo, hi32, id_x, true);               // + mask_j - lse_i
              const uint32_t a_lo = bt_base + bslot * kAtom16;
#pragma unroll
              for (int c = 0; c < 4; ++c) mma_ss_el(tS + c * 16, a_lo + c * bstep, hi128, i_lo0, hi64, id_b, true);
              if (two_terms) {
#pragma unroll
                for (int c = 0; c < 4; ++c) mma_ss_el(tS + c * 16, a_lo + c * bstep, hi128, i_lo1, hi64, id_b, true);
              }
#pragma unroll
              for (int hh = 0; hh < NH; ++hh) {
                mma_ss_el(tD, v_lo + hh * kTile16, hi64, g_lo + hh * kTile16, hi64, id_s, hh > 0);
                mma_ss_el(tD, v_lo + hh * kTile16 + 2, hi64, g_lo + hh * kTile16 + 2, hi64, id_s, true);
              }
              mma_ss_el(tD, xc_lo, hi32, xq_lo, hi32, id_x, true);               // - delta_i
              tc_commit_el(&bar.sd_ready[half]);
              tc_commit_el(&bar.bt_empty[bslot]);
              if (++bslot == NB) { bslot = 0; ++buse; }
              tr(32);
            }
            if (++qslot == NQ) { qslot = 0; ++quse; }
          }
        }
      }
    } else if (warp == kComputeWarps + 1) {
      // ========================================================================== TMA producer, in order of need
      uint32_t g = 0, kv = 0, bslot = 0, buse = 0, nbt = 0, qslot = 0, quse = 0;
      int item_no = 0;
      for (int item = blockIdx.x; item < p.n_items && !dead(); item += gridDim.x, ++item_no) {
        const int bnh = item / p.ksplit;
        int jt0, jt1; item_range(item, jt0, jt1);
        const int h = bnh % p.H, bn = bnh / p.H, n = bn % p.N, b = bn / p.N;
        for (int jt = jt0; jt < jt1 && !dead(); ++jt, ++kv) {
          if (kv >= (uint32_t)NKV) wait_or_flag(&bar.kv_empty[kv % NKV], ((kv / NKV) - 1) & 1, abort_flag);
          if (dead()) break;
          if (elect_one()) {
            uint64_t* fb = &bar.kv_full[kv % NKV];
            uint8_t* st = sKV + (kv % NKV) * kStageB;
            mbar_expect_tx(fb, kStageB);
#pragma unroll
            for (int hh = 0; hh < NH; ++hh) {
              tma_load_5d(st + hh * kTileB, &mk, fb, hh * kDP, h, jt * kT, n, b);
              tma_load_5d(st + (NH + hh) * kTileB, &mv, fb, hh * kDP, h, jt * kT, n, b);
            }
            bulk_load_1d(st + 2 * NH * kTileB, p.xk + ((int64_t)bn * nt + jt) * kXTileB, kXTileB, fb);
          }
          for (int it = 0; it < nt; ++it, ++g) {
            if (quse >= 1) wait_or_flag(&bar.qd_empty[qslot], (quse - 1) & 1, abort_flag);
            if (dead()) break;
            if (elect_one()) {
              uint64_t* fb = &bar.qd_full[qslot];
              uint8_t* st = sQD + qslot * kStageB;
              mbar_expect_tx(fb, kStageB);
#pragma unroll
              for (int hh = 0; hh < NH; ++hh) {
                tma_load_5d(st + hh * kTileB, &mq, fb, hh * kDP, h, it * kT, n, b);
                tma_load_5d(st + (NH + hh) * kTileB, &mg, fb, hh * kDP, h, it * kT, n, b);
              }
              bulk_load_1d(st + 2 * NH * kTileB, p.xq + ((int64_t)bnh * nt + it) * kXTileB, kXTileB, fb);
            }
            if (++qslot == NQ) { qslot = 0; ++quse; }
            for (int half = 0; half < 2; ++half) {
              if (buse >= 1) wait_or_flag(&bar.bt_empty[bslot], (buse - 1) & 1, abort_flag);
              if (dead()) break;
              if (elect_one()) {
                mbar_expect_tx(&bar.bt_full[bslot], kAtomB);
                if (p.bias_mn) {       // [64 queries x 64 keys] pieces of the bias itself: keys 0-63 | 64-127 of the tile
                  tma_load_4d(sBT + bslot * kAtomB, &mbt, &bar.bt_full[bslot], jt * kT, it * kT + half * kHalf, h, b * p.bias_b_mul);
                  tma_load_4d(sBT + bslot * kAtomB + 8192, &mbt, &bar.bt_full[bslot], jt * kT + 64, it * kT + half * kHalf, h, b * p.bias_b_mul);
                } else {
                  tma_load_4d(sBT + bslot * kAtomB, &mbt, &bar.bt_full[bslot], it * kT + half * kHalf, jt * kT, h, b * p.bias_b_mul);
                }
              }
              ++nbt;
              if (++bslot == NB) { bslot = 0; ++buse; }
            }
          }
        }
      }
      if (dead() && lane == 0) {
        // the copies already requested must land before the CTA's shared memory is given back (bounded)
        for (uint32_t back = 0; back < (uint32_t)NKV && back < kv; ++back) { const uint32_t c = kv - 1 - back; mbar_wait(&bar.kv_full[c % NKV], (c / NKV) & 1); }
        for (uint32_t back = 0; back < (uint32_t)NQ && back < g; ++back) { const uint32_t c = g - 1 - back; mbar_wait(&bar.qd_full[c % NQ], (c / NQ) & 1); }
        for (uint32_t back = 0; back < (uint32_t)NB && back < nbt; ++back) { const uint32_t c = nbt - 1 - back; mbar_wait(&bar.bt_full[c % NB], (c / NB) & 1); }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_s) *reinterpret_cast<volatile int*>(p.status) = 1;
  if (warp == 0) tmem_dealloc(tmem_base_s, 512);
}

// ------------------------------------------------------------------------------------------------ dBias
struct DbP {
  int B, N, L, H, D;
  int n_t, lpad, nsplit, n_units;
  float c1;
  uint32_t fmt, bfmt;
  int n_alpha; float alpha[2];
  int bias_b_mul;
  int bias_mn;            // as in BwdWsP
  const uint8_t* xq; const uint8_t* xk;      // rank-one term tiles (evo_extras_ws_kernel)
  float* part;            // fp32 [nsplit][B][H][L][L] partial sums
  void* out16;            // with a single row range and a 16-bit d_bias: the result itself, [B][H][L][L] in the q/k/v type
  int* status;
};

struct DbBars {
  uint64_t op_full[3], op_empty[3];          // Q, dO, K, V, XQ, XK of one row n
  uint64_t bt_full, bt_free;                 // the unit's two bias^T atoms
  uint64_t sd_ready[2], loaded[2];
};

template <typename T, typename TB, int NH>
__global__ void __launch_bounds__(kThreads, 1)
evo_dbias_ws_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                    const __grid_constant__ CUtensorMap mv, const __grid_constant__ CUtensorMap mg,
                    const __grid_constant__ CUtensorMap mbt, const DbP p MF_TRACE_PARAM) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sBT = smem;                          // two bias^T atoms (queries 0-63 | 64-127 of the tile)
  constexpr int kDbStageB = Geo<NH>::kDbStageB, NS = Geo<NH>::NS;
  uint8_t* sOP = sBT + 2 * kAtomB;              // [NS stages][Q halves, dO halves, K halves, V halves, XQ, XK]
  uint8_t* sI = sOP + NS * kDbStageB;
  uint8_t* sXC = sI + 2048;                     // constant tile of the -delta term

  __shared__ DbBars bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    abort_s = 0;
    for (int i = 0; i < 3; ++i) {
      mbar_init(&bar.op_full[i], 1); mbar_init(&bar.op_empty[i], 2);      // two issuers commit
    }
    mbar_init(&bar.bt_full, 1); mbar_init(&bar.bt_free, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&bar.sd_ready[i], 2); mbar_init(&bar.loaded[i], kComputeWarps); }
    mbar_fence_init();
    prefetch_tmap(&mq); prefetch_tmap(&mk); prefetch_tmap(&mv); prefetch_tmap(&mg); prefetch_tmap(&mbt);
  }
  write_alpha_identity<TB>(sI, p.alpha[0], tid, kThreads);
  write_alpha_identity<TB>(sI + 1024, p.alpha[1], tid, kThreads);
  write_xc_tile(sXC, tid, kThreads);
  fence_async_smem();
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  volatile int* abort_flag = &abort_s;
  const uint32_t tm0 = tmem_base_s;
  const int nt = p.n_t;
  // unit = ((b * H + h) * nt + jt) * nt + it, split `sp` of the rows
  struct Unit { int b, h, jt, it, n0, n1; };
  auto unit_of = [&](int u) {
    Unit x;
    const int sp = u % p.nsplit; int c = u / p.nsplit;
    x.it = c % nt; c /= nt; x.jt = c % nt; c /= nt; x.h = c % p.H; x.b = c / p.H;
    x.n0 = (int)((int64_t)sp * p.N / p.nsplit); x.n1 = (int)((int64_t)(sp + 1) * p.N / p.nsplit);
    return x;
  };

  if (warp < kComputeWarps) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kComputeRegs));
    const int w = warp >> 2;                          // query quarter (32 columns) handled by this thread
    const int r = (warp & 3) * 32 + lane;             // TMEM lane = key row inside the tile
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t g = 0;                                   // rows processed by this CTA (TMEM buffer g & 1)
    const float2 c1c1 = make_float2(p.c1, p.c1);
    MF_TRACE_DECL(tr, 0, blockIdx.x == 0 && tid == 0);
    for (int u = blockIdx.x; u < p.n_units; u += gridDim.x) {
      const Unit x = unit_of(u);
      const int j = x.jt * kT + r;
      float2 acc[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) acc[c] = make_float2(0.f, 0.f);
      for (int n = x.n0; n < x.n1; ++n, ++g) {
        const uint32_t tST = tm0 + (g & 1) * 256 + w * 32 + lane_addr, tDP = tST + 128;
        tr(1);
        wait_or_flag(&bar.sd_ready[g & 1], (g >> 1) & 1, abort_flag);
        tc_fence_after();
        tr(2);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {          // 16 query columns at a time keeps the live registers down
          uint32_t sr[16], dr[16];
          tmem_ld16(tST + hf * 16, sr);
          tmem_ld16(tDP + hf * 16, dr);
          tmem_ld_wait();
          if (hf == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar.loaded[g & 1]);
            tr(3);
          }
          // mask, lse and delta are already inside the accumulators: P = 2^(c1 S''), dS = P dP''
#pragma unroll
          for (int c2 = 0; c2 < 8; ++c2) {
            const float2 xx = mul2(make_float2(__uint_as_float(sr[c2 * 2]), __uint_as_float(sr[c2 * 2 + 1])), c1c1);
            const float2 pr = make_float2(ex2f(xx.x), ex2f(xx.y));
            acc[hf * 8 + c2] = fma2(pr, make_float2(__uint_as_float(dr[c2 * 2]), __uint_as_float(dr[c2 * 2 + 1])), acc[hf * 8 + c2]);
          }
        }
        tr(4);
      }
      // the unit's partial sum: part[sp][b][h][i][j], lanes = consecutive keys
      if (j < p.L && !*abort_flag) {
        const int sp = u % p.nsplit;
        const int64_t at = ((((int64_t)sp * p.B + x.b) * p.H + x.h) * p.L) * (int64_t)p.L + j;
        const int i0 = x.it * kT + w * 32;
        if (p.out16) {
          T* dst = static_cast<T*>(p.out16) + at;
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            if (i0 + 2 * c < p.L) dst[(int64_t)(i0 + 2 * c) * p.L] = from_f<T>(acc[c].x);
            if (i0 + 2 * c + 1 < p.L) dst[(int64_t)(i0 + 2 * c + 1) * p.L] = from_f<T>(acc[c].y);
          }
        } else {
          float* dst = p.part + at;
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            if (i0 + 2 * c < p.L) dst[(int64_t)(i0 + 2 * c) * p.L] = acc[c].x;
            if (i0 + 2 * c + 1 < p.L) dst[(int64_t)(i0 + 2 * c + 1) * p.L] = acc[c].y;
          }
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kHelperRegs));
    // The helper roles are run by whole warps (one elected lane issues: see mma_ss_el); every exit decision is a warp vote.
    auto dead = [&] { return __any_sync(0xffffffffu, *abort_flag) != 0; };
    constexpr uint32_t hi64 = desc_hi(512, kSw64), hi128 = desc_hi(1024, kSw128);
    constexpr uint32_t kTile16 = kTileB / 16, kAtom16 = kAtomB / 16;
    constexpr uint32_t hi32 = desc_hi(256, kSw32), kStage16 = kDbStageB / 16;
    const uint32_t op_base = desc_lo(smem_u32(sOP), 16);
    const uint32_t id_s = idesc_f16(128, 128, p.fmt, 0, 0);
    const uint32_t id_x = idesc_f16(128, 128, 1u, 0, 0);          // the rank-one term tiles are bf16 whatever q/k/v are
    if (warp == kComputeWarps) {
      // ========================================================================== score issuer: S''^T = K Q^T + alpha * bias^T
      const uint32_t id_b = idesc_f16(128, 16, p.bfmt, p.bias_mn ? 1u : 0u, 0);      // see the main kernel's score issuer
      const uint32_t bt_lo = desc_lo(smem_u32(sBT), p.bias_mn ? 8192 : 16);
      const uint32_t bstep = p.bias_mn ? 2048 / 16 : 2;
      const uint32_t i_lo0 = desc_lo(smem_u32(sI), 16), i_lo1 = i_lo0 + 1024 / 16;
      const bool two_terms = p.n_alpha > 1;
      MF_TRACE_DECL(tr, 2, blockIdx.x == 0 && lane == 0);
      uint32_t g = 0, un = 0, stage = 0, suse = 0;
      for (int u = blockIdx.x; u < p.n_units && !dead(); u += gridDim.x, ++un) {
        const Unit x = unit_of(u);
        wait_or_flag(&bar.bt_full, un & 1, abort_flag);
        for (int n = x.n0; n < x.n1 && !dead(); ++n, ++g) {
          tr(20);
          wait_or_flag(&bar.op_full[stage], suse & 1, abort_flag);
          if (g >= 2) wait_or_flag(&bar.loaded[g & 1], ((g >> 1) - 1) & 1, abort_flag);
          tc_fence_after();
          tr(21);
          const uint32_t q_lo = op_base + stage * kStage16, k_lo = q_lo + 2 * NH * kTile16;
          const uint32_t xq_lo = q_lo + 4 * NH * kTile16, xk_lo = xq_lo + kXTileB / 16;
          const uint32_t tST = tm0 + (g & 1) * 256;
#pragma unroll
          for (int hh = 0; hh < NH; ++hh) {
            mma_ss_el(tST, k_lo + hh * kTile16, hi64, q_lo + hh * kTile16, hi64, id_s, hh > 0);
            mma_ss_el(tST, k_lo + hh * kTile16 + 2, hi64, q_lo + hh * kTile16 + 2, hi64, id_s, true);
          }
          mma_ss_el(tST, xk_lo, hi32, xq_lo, hi32, id_x, true);                 // + mask_j - lse_i
#pragma unroll
          for (int c = 0; c < 8; ++c) mma_ss_el(tST + c * 16, bt_lo + (c >> 2) * kAtom16 + (c & 3) * bstep, hi128, i_lo0, hi64, id_b, true);
          if (two_terms) {
#pragma unroll
            for (int c = 0; c < 8; ++c) mma_ss_el(tST + c * 16, bt_lo + (c >> 2) * kAtom16 + (c & 3) * bstep, hi128, i_lo1, hi64, id_b, true);
          }
          tc_commit_el(&bar.sd_ready[g & 1]);
          tc_commit_el(&bar.op_empty[stage]);
          if (++stage == NS) { stage = 0; ++suse; }
          tr(22);
        }
        tc_commit_el(&bar.bt_free);       // every product that reads this unit's bias atoms is complete
      }
    } else if (warp == kComputeWarps + 2) {
      // ========================================================================== dP issuer: dP^T = V dO^T
      uint32_t g = 0, stage = 0, suse = 0;
      for (int u = blockIdx.x; u < p.n_units && !dead(); u += gridDim.x) {
        const Unit x = unit_of(u);
        for (int n = x.n0; n < x.n1 && !dead(); ++n, ++g) {
          wait_or_flag(&bar.op_full[stage], suse & 1, abort_flag);
          if (g >= 2) wait_or_flag(&bar.loaded[g & 1], ((g >> 1) - 1) & 1, abort_flag);
          tc_fence_after();
          const uint32_t g_lo = op_base + stage * kStage16 + NH * kTile16, v_lo = g_lo + 2 * NH * kTile16;
          const uint32_t xq_lo = op_base + stage * kStage16 + 4 * NH * kTile16;
          const uint32_t tDP = tm0 + (g & 1) * 256 + 128;
#pragma unroll
          for (int hh = 0; hh < NH; ++hh) {
            mma_ss_el(tDP, v_lo + hh * kTile16, hi64, g_lo + hh * kTile16, hi64, id_s, hh > 0);
            mma_ss_el(tDP, v_lo + hh * kTile16 + 2, hi64, g_lo + hh * kTile16 + 2, hi64, id_s, true);
          }
          mma_ss_el(tDP, desc_lo(smem_u32(sXC), 16), hi32, xq_lo, hi32, id_x, true);      // - delta_i
          tc_commit_el(&bar.sd_ready[g & 1]);
          tc_commit_el(&bar.op_empty[stage]);
          if (++stage == NS) { stage = 0; ++suse; }
        }
      }
    } else if (warp == kComputeWarps + 1) {
      // ========================================================================== TMA producer
      uint32_t g = 0, un = 0, stage = 0, suse = 0;
      for (int u = blockIdx.x; u < p.n_units && !dead(); u += gridDim.x, ++un) {
        const Unit x = unit_of(u);
        if (un >= 1) wait_or_flag(&bar.bt_free, (un - 1) & 1, abort_flag);
        if (dead()) break;
        if (elect_one()) {
          mbar_expect_tx(&bar.bt_full, 2 * kAtomB);
          if (p.bias_mn) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)       // (query half, key half) pieces of [64 x 64]
              tma_load_4d(sBT + (q4 >> 1) * kAtomB + (q4 & 1) * 8192, &mbt, &bar.bt_full, x.jt * kT + (q4 & 1) * 64,
                          x.it * kT + (q4 >> 1) * kHalf, x.h, x.b * p.bias_b_mul);
          } else {
            tma_load_4d(sBT, &mbt, &bar.bt_full, x.it * kT, x.jt * kT, x.h, x.b * p.bias_b_mul);
            tma_load_4d(sBT + kAtomB, &mbt, &bar.bt_full, x.it * kT + kHalf, x.jt * kT, x.h, x.b * p.bias_b_mul);
          }
        }
        for (int n = x.n0; n < x.n1; ++n, ++g) {
          if (suse >= 1) wait_or_flag(&bar.op_empty[stage], (suse - 1) & 1, abort_flag);
          if (dead()) break;
          if (elect_one()) {
            uint64_t* fb = &bar.op_full[stage];
            uint8_t* st = sOP + stage * kDbStageB;
            mbar_expect_tx(fb, kDbStageB);
#pragma unroll
            for (int hh = 0; hh < NH; ++hh) {
              tma_load_5d(st + hh * kTileB, &mq, fb, hh * kDP, x.h, x.it * kT, n, x.b);
              tma_load_5d(st + (NH + hh) * kTileB, &mg, fb, hh * kDP, x.h, x.it * kT, n, x.b);
              tma_load_5d(st + (2 * NH + hh) * kTileB, &mk, fb, hh * kDP, x.h, x.jt * kT, n, x.b);
              tma_load_5d(st + (3 * NH + hh) * kTileB, &mv, fb, hh * kDP, x.h, x.jt * kT, n, x.b);
            }
            const int64_t bn = (int64_t)x.b * p.N + n;
            bulk_load_1d(st + 4 * NH * kTileB, p.xq + ((bn * p.H + x.h) * nt + x.it) * kXTileB, kXTileB, fb);
            bulk_load_1d(st + 4 * NH * kTileB + kXTileB, p.xk + (bn * nt + x.jt) * kXTileB, kXTileB, fb);
          }
          if (++stage == NS) { stage = 0; ++suse; }
        }
      }
      if (dead() && lane == 0) {
        for (uint32_t back = 0; back < (uint32_t)NS && back < g; ++back) { const uint32_t c = g - 1 - back; mbar_wait(&bar.op_full[c % NS], (c / NS) & 1); }
        if (un > 0) mbar_wait(&bar.bt_full, (un - 1) & 1);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_s) *reinterpret_cast<volatile int*>(p.status) = 1;
  if (warp == 0) tmem_dealloc(tmem_base_s, 512);
}

// d_bias[b][h][i][j] = sum over the row ranges, in order, cast to the output type
template <typename TO>
__global__ void dbias_finish_kernel(const float* __restrict__ part, TO* __restrict__ out, int64_t n, int nsplit) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  if (i + 4 <= n && (n & 3) == 0) {            // four entries per thread; every range starts on a 16-byte boundary
    float4 s = *reinterpret_cast<const float4*>(part + i);
    for (int k = 1; k < nsplit; ++k) {
      const float4 t = *reinterpret_cast<const float4*>(part + (int64_t)k * n + i);
      s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
    }
    out[i] = from_f<TO>(s.x); out[i + 1] = from_f<TO>(s.y); out[i + 2] = from_f<TO>(s.z); out[i + 3] = from_f<TO>(s.w);
    return;
  }
  for (int64_t e = i; e < n && e < i + 4; ++e) {
    float s = part[e];
    for (int k = 1; k < nsplit; ++k) s += part[(int64_t)k * n + e];
    out[e] = from_f<TO>(s);
  }
}

template <typename T>
__global__ void cast_rows_ws_kernel(const float* __restrict__ src, T* __restrict__ dst, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = from_f<T>(src[i]);
}

// With few (b, n, h) triples (single-representation attention: N = 1) the key tiles of each are spread over several
// CTAs so that the whole GPU works; the partial dQ rows then meet in an fp32 accumulator.
int bwd_ksplit(int64_t bnh, int nt, int sms) {
  if (bnh >= sms || nt < 2) return 1;
  int64_t k = sms / bnh;                 // as many ranges as keep every CTA at one work item
  if (k > nt) k = nt;
  return k < 1 ? 1 : (int)k;
}

// Can TMA address the caller's bias ([.., queries, keys], 16-bit, keys contiguous, 16-byte multiples elsewhere)?  Then its
// tiles are loaded as they are and read MN-major; otherwise a transposed 16-bit copy is made first.
bool bias_tma_ok(const mf_evo_bwd_args& a) {
  if (a.bias_dtype != MF_BF16 && a.bias_dtype != MF_F16) return false;
  const int64_t* s = a.bias_strides;
  if (s[3] != 1 || (reinterpret_cast<uintptr_t>(a.bias) & 15) != 0) return false;
  if ((s[2] * 2) % 16 != 0 || s[2] <= 0) return false;
  if (a.H > 1 && ((s[1] * 2) % 16 != 0 || s[1] <= 0)) return false;
  if (a.B > 1 && s[0] != 0 && ((s[0] * 2) % 16 != 0 || s[0] < 0)) return false;
  return true;
}

struct BwdPlan {
  int nt, lpad, ksplit, dq_stream, dbuf, nsplit;
  bool dq_fp32, part_direct, bias_direct;
  size_t off_flags, off_xq, off_xk, off_part, off_dq, off_biasT, total;
};

BwdPlan plan_bwd(const mf_evo_bwd_args& a) {
  BwdPlan pl{};
  const int sms = sm_count();
  pl.nt = (a.L + kT - 1) / kT;
  pl.lpad = pl.nt * kT;
  pl.ksplit = bwd_ksplit((int64_t)a.B * a.N * a.H, pl.nt, sms);
  // dQ accumulators of all query tiles next to one set (up to six tiles) or two sets (up to four) of dK/dV accumulators;
  // longer rows stream dQ
  if (a.D <= kDP) {
    pl.dq_stream = pl.nt > 6;
    pl.dbuf = pl.dq_stream || pl.nt <= 4;
  } else {
    // two head halves: one set of dK|dV accumulators (128 columns) leaves room for two dQ accumulators of 64 columns
    pl.dq_stream = pl.nt > 2;
    pl.dbuf = 0;
  }
  pl.dq_fp32 = pl.ksplit > 1 || pl.dq_stream;
  const int64_t combos = (int64_t)a.B * a.H * pl.nt * pl.nt;
  int64_t ns = sms / combos;
  if (ns < 1) ns = 1;
  if (ns > a.N) ns = a.N;
  pl.nsplit = (int)ns;
  pl.part_direct = pl.nsplit == 1;      // a single range writes d_bias itself, in its own type
  size_t off = 0;
  pl.off_flags = off; off += align_up(sizeof(int) * (size_t)a.B * a.N * a.H, 256);
  pl.off_xq = off; off += (size_t)a.B * a.N * a.H * pl.nt * kXTileB;
  pl.off_xk = off; off += (size_t)a.B * a.N * pl.nt * kXTileB;
  pl.off_part = off; if (!pl.part_direct) off += align_up(sizeof(float) * (size_t)pl.nsplit * a.B * a.H * a.L * a.L, 256);
  pl.off_dq = off; if (pl.dq_fp32) off += align_up(sizeof(float) * (size_t)a.B * a.N * a.L * a.H * a.D, 256);
  pl.bias_direct = bias_tma_ok(a);
  pl.off_biasT = off; if (!pl.bias_direct) off += align_up(2 * (size_t)a.B * a.H * a.L * pl.lpad, 256);
  pl.total = off;
  return pl;
}

template <typename T, typename TB, int NH>
int launch_bwd_ws(const mf_evo_bwd_args& a, cudaStream_t st) {
  const BwdPlan pl = plan_bwd(a);
  CUtensorMap mq, mk, mv, mg, mbt;
  int r;
  const int64_t cs[5] = {(int64_t)a.N * a.L * a.H * a.D, (int64_t)a.L * a.H * a.D, (int64_t)a.H * a.D, a.D, 1};
  if ((r = make_qkv_map(&mq, a.q, a.dtype, a.B, a.N, a.L, a.H, a.D, a.q_strides, kDP, kT))) return r;
  if ((r = make_qkv_map(&mk, a.k, a.dtype, a.B, a.N, a.L, a.H, a.D, a.k_strides, kDP, kT))) return r;
  if ((r = make_qkv_map(&mv, a.v, a.dtype, a.B, a.N, a.L, a.H, a.D, a.v_strides, kDP, kT))) return r;
  if ((r = make_qkv_map(&mg, a.d_o, a.dtype, a.B, a.N, a.L, a.H, a.D, cs, kDP, kT))) return r;
  int* status = status_word();
  MF_REQUIRE(status, MF_ERR_CUDA, "could not allocate the device status word");
  MF_REQUIRE(tc_async_status() == 0, MF_ERR_CUDA, "an earlier tensor-core kernel gave up on a bounded wait; results are invalid");
  char* ws = static_cast<char*>(a.workspace);
  int* flags = reinterpret_cast<int*>(ws + pl.off_flags);
  uint8_t* xq = reinterpret_cast<uint8_t*>(ws + pl.off_xq);
  uint8_t* xk = reinterpret_cast<uint8_t*>(ws + pl.off_xk);
  float* part = !pl.part_direct ? reinterpret_cast<float*>(ws + pl.off_part) : (a.dbias_dtype == MF_F32 ? static_cast<float*>(a.d_bias) : nullptr);
  float* dq_acc = reinterpret_cast<float*>(ws + pl.off_dq);
  // the transposed bias copy is kept in a 16-bit type: the bias dtype when that is one, else the q/k/v dtype
  using TT = typename std::conditional<sizeof(TB) == 2, TB, T>::type;
  const int bt_dtype = sizeof(TB) == 2 ? a.bias_dtype : a.dtype;
  TT* biasT = reinterpret_cast<TT*>(ws + pl.off_biasT);
  const int lpad = pl.lpad;
  const int bias_b_mul = pl.bias_direct ? (a.bias_strides[0] == 0 ? 0 : 1) : 1;
  if (pl.bias_direct) {
    const int64_t dims[4] = {a.L, a.L, a.H, bias_b_mul ? a.B : 1};
    const int64_t str[4] = {1, a.bias_strides[2], a.bias_strides[1], a.bias_strides[0]};
    const int box[4] = {64, 64, 1, 1};
    if ((r = make_tiled_map(&mbt, a.bias, a.bias_dtype, 4, dims, str, box, 128))) return r;
  } else {
    if (lpad != a.L) MF_CUDA(cudaMemsetAsync(biasT, 0, 2 * (size_t)a.B * a.H * a.L * lpad, st));      // the row padding
    dim3 grid((a.L + 63) / 64, (a.L + 63) / 64, a.B * a.H), block(32, 8);
    transpose_bias_ws_kernel<TB, TT><<<grid, block, 0, st>>>(static_cast<const TB*>(a.bias), biasT, a.H, a.L, lpad, a.bias_strides[0],
                                                             a.bias_strides[1], a.bias_strides[2], a.bias_strides[3]);
    MF_LAUNCHED("transpose_bias_ws_kernel");
    const int64_t dims[4] = {lpad, a.L, a.H, a.B};
    const int64_t str[4] = {1, lpad, (int64_t)a.L * lpad, (int64_t)a.H * a.L * lpad};
    const int box[4] = {kHalf, 128, 1, 1};
    if ((r = make_tiled_map(&mbt, biasT, bt_dtype, 4, dims, str, box, 128))) return r;
  }
  MF_CUDA(cudaMemsetAsync(flags, 0, sizeof(int) * (size_t)a.B * a.N * a.H, st));
  {
    const int64_t n_threads = (int64_t)a.B * a.N * lpad * a.H;
    evo_extras_ws_kernel<T><<<(unsigned)((n_threads + 255) / 256), 256, 0, st>>>(static_cast<const T*>(a.o), static_cast<const T*>(a.d_o), a.lse,
                                                                             a.mask, a.mask_strides[0], a.mask_strides[1], a.mask_strides[2], a.mask_dtype,
                                                                             xq, xk, flags, n_threads, a.N, a.L, lpad, a.H, a.D);
  }
  MF_LAUNCHED("evo_extras_ws_kernel");
  const int64_t n_dq = (int64_t)a.B * a.N * a.L * a.H * a.D;
  if (pl.dq_fp32) MF_CUDA(cudaMemsetAsync(dq_acc, 0, sizeof(float) * (size_t)n_dq, st));

  float alpha[2];
  const int n_alpha = split_alpha(a.D, bt_dtype, alpha);
  // With one row per bias (N = 1, single-representation attention) and d_pair_bias in the q/k/v type, dS is the answer:
  // the dQ/dK/dV kernel writes it and the d_pair_bias kernel is not needed.
  const bool dbias_direct = a.N == 1 && a.dbias_dtype == a.dtype;
  // ---- dBias first: a caller that all-reduces it over row shards can start while dQ / dK / dV are computed
  if (!dbias_direct) {
    DbP p{};
    p.B = a.B; p.N = a.N; p.L = a.L; p.H = a.H; p.D = a.D;
    p.n_t = pl.nt; p.lpad = lpad; p.nsplit = pl.nsplit;
    p.n_units = a.B * a.H * pl.nt * pl.nt * pl.nsplit;
    p.c1 = kLog2e / sqrtf((float)a.D);
    p.fmt = a.dtype == MF_BF16 ? 1u : 0u; p.bfmt = bt_dtype == MF_BF16 ? 1u : 0u;
    p.n_alpha = n_alpha; p.alpha[0] = alpha[0]; p.alpha[1] = alpha[1];
    p.bias_b_mul = bias_b_mul; p.bias_mn = pl.bias_direct ? 1 : 0;
    p.xq = xq; p.xk = xk;
    p.part = part;
    p.out16 = pl.part_direct && a.dbias_dtype != MF_F32 ? a.d_bias : nullptr;
    p.status = status;
    const size_t smem = Geo<NH>::kDbSmem;
    int grid = sm_count();
    if (grid > p.n_units) grid = p.n_units;
    auto kern = evo_dbias_ws_kernel<T, TT, NH>;
    MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, st>>>(mq, mk, mv, mg, mbt, p MF_TRACE_ARG);
    MF_LAUNCHED("evo_dbias_ws_kernel");
    if (!pl.part_direct) {
      const int64_t n_out = (int64_t)a.B * a.H * a.L * a.L;
      if (a.dbias_dtype == MF_F32)
        dbias_finish_kernel<float><<<(unsigned)((n_out + 1023) / 1024), 256, 0, st>>>(part, static_cast<float*>(a.d_bias), n_out, pl.nsplit);
      else
        dbias_finish_kernel<T><<<(unsigned)((n_out + 1023) / 1024), 256, 0, st>>>(part, static_cast<T*>(a.d_bias), n_out, pl.nsplit);
      MF_LAUNCHED("dbias_finish_kernel");
    }
  }
  if (a.dbias_ready_event && !dbias_direct) MF_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(a.dbias_ready_event), st));
  // ---- dQ, dK, dV
  {
    BwdWsP p{};
    p.B = a.B; p.N = a.N; p.L = a.L; p.H = a.H; p.D = a.D;
    p.n_t = pl.nt; p.lpad = lpad; p.ksplit = pl.ksplit; p.dq_stream = pl.dq_stream; p.dbuf = pl.dbuf;
    p.n_items = a.B * a.N * a.H * pl.ksplit;
    p.dq_acc = dq_acc;
    p.scale = 1.0f / sqrtf((float)a.D); p.c1 = kLog2e * p.scale; p.inv_L = 1.0f / a.L;
    p.fmt = a.dtype == MF_BF16 ? 1u : 0u; p.bfmt = bt_dtype == MF_BF16 ? 1u : 0u;
    p.n_alpha = n_alpha; p.alpha[0] = alpha[0]; p.alpha[1] = alpha[1];
    p.bias_b_mul = bias_b_mul; p.bias_mn = pl.bias_direct ? 1 : 0;
    p.xq = xq; p.xk = xk; p.flags = flags;
    p.dbias_direct = dbias_direct ? a.d_bias : nullptr;
    p.dq = a.dq; p.dk = a.dk; p.dv = a.dv;
    p.status = status;
    const size_t smem = Geo<NH>::kMainSmem;
    int grid = sm_count();
    if (grid > p.n_items) grid = p.n_items;
    if (pl.dq_stream) {
      auto kern = evo_bwd_ws_kernel<T, TT, true, NH>;
      MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      kern<<<grid, kThreads, smem, st>>>(mq, mk, mv, mg, mbt, p MF_TRACE_ARG);
    } else {
      auto kern = evo_bwd_ws_kernel<T, TT, false, NH>;
      MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      kern<<<grid, kThreads, smem, st>>>(mq, mk, mv, mg, mbt, p MF_TRACE_ARG);
    }
    MF_LAUNCHED("evo_bwd_ws_kernel");
    if (a.dbias_ready_event && dbias_direct) MF_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(a.dbias_ready_event), st));
  }
  if (pl.dq_fp32) {
    cast_rows_ws_kernel<T><<<(unsigned)((n_dq + 255) / 256), 256, 0, st>>>(dq_acc, static_cast<T*>(a.dq), n_dq);
    MF_LAUNCHED("cast_rows_ws_kernel");
  }
  return MF_OK;
}

}  // namespace

bool evo_bwd_ws_shape_ok(int L, int D) {
  // head sizes up to 64 (two halves of 32 columns); rows of more than six query tiles (two with a head size above 32)
  // stream dQ through an fp32 accumulator in global memory, which has been validated up to 2048 tokens
  return D <= 64 && L <= 2048;
}

size_t evo_bwd_ws_workspace(const mf_evo_bwd_args& a) { return plan_bwd(a).total; }

#define MF_DISPATCH_BIAS(dt, TB, ...)                                         \
  switch (dt) {                                                               \
    case MF_F32: { using TB = float; __VA_ARGS__; } break;                    \
    case MF_BF16: { using TB = __nv_bfloat16; __VA_ARGS__; } break;           \
    case MF_F16: { using TB = __half; __VA_ARGS__; } break;                   \
    default: return fail(MF_ERR_BAD_ARG, "unknown bias dtype %d", (int)(dt)); \
  }

int evo_bwd_ws(const mf_evo_bwd_args& a, cudaStream_t st) {
  int r = MF_OK;
  if (a.dtype == MF_BF16) {
    MF_DISPATCH_BIAS(a.bias_dtype, TB, { r = a.D <= kDP ? launch_bwd_ws<__nv_bfloat16, TB, 1>(a, st) : launch_bwd_ws<__nv_bfloat16, TB, 2>(a, st); });
  } else {
    MF_DISPATCH_BIAS(a.bias_dtype, TB, { r = a.D <= kDP ? launch_bwd_ws<__half, TB, 1>(a, st) : launch_bwd_ws<__half, TB, 2>(a, st); });
  }
  return r;
}

}  // namespace mf
