// Pair-biased masked attention forward, warp-specialised (tcgen05 + TMEM + TMA), head sizes up to 32.
//
// A persistent CTA (one per SM, 512 threads) runs TWO independent streams.  A stream walks a contiguous range of
// work items (b, n, h, 128-query tile) and, per item, the key tiles of 128.  Roles:
//
//   warps 0-3 / 4-7   softmax warpgroup of stream 0 / 1: one query row (= one TMEM lane) per thread
//   warp 8 / 9        issuer of the score MMAs of stream 0 / 1 (one thread)
//   warp 10 / 11      issuer of the P V MMAs of stream 0 / 1 (one thread)
//   warp 12 / 13      TMA producer of stream 0 / 1 (one thread); warps 14, 15 idle
// (a single thread issues an MMA every ~60 cycles at best, so the two kinds of products get a thread each)
//
// Per key tile the issuer builds   S = Q K^T + sqrt(D) * bias   entirely on the tensor core: two MMAs for Q K^T and
// eight [128 x 16] x [16 x 16] MMAs that add the bias tile (A operand, straight from the TMA-loaded tile) times
// alpha * I (B operand), plus one K = 16 step that adds the key-mask term (a [128 x 16] tile per key tile, written by
// the producer warp, times a constant tile) - see evo_tc_common.cuh.  The softmax thread reads its 128 logits, takes
// the maximum with three-input max (the positive scale commutes with it), and writes
// packed 16-bit P = 2^(x - m) back to TMEM while adding up the row sum (packed adds that hide under the
// exponentials).  P V accumulates into O in TMEM over the key tiles; O and the sum are only multiplied by
// 2^(m_old - m_new) when the running maximum has grown by more than 8 (rare after the first tile; P then stays
// below 2^8, far inside the 16-bit range).  Only O and the log-sum-exp reach global memory.
//
// Every wait is bounded; on expiry the CTA raises a flag, all roles run dry without touching global memory, TMEM is
// freed and the host sees mf_async_status() != 0.
#include "evo_tc_common.cuh"

namespace mf {
namespace {
using namespace tcx;

constexpr int kT = 128;                      // tile edge (queries and keys)
constexpr int kThreads = 512;             // registers are allocated to warps in groups of four
constexpr int kTileB = 128 * 64;             // [128 x 32] 16-bit tile, 64-byte rows, 64B swizzle
constexpr int kAtomB = 128 * 128;            // bias atom: [128 rows x 64 columns] 16-bit, 128-byte rows, 128B swizzle
constexpr int kStreamBytes = 6 * kTileB + 3 * kAtomB + 2 * kXTileB;     // Q x2, K x2, V x2, three bias atoms, mask-term tile x2
constexpr float kRescaleStep = 8.f;          // O is rescaled only when the running maximum grows by more than this (base-2 logits)

struct FwdWsP {
  int B, N, L, H, D;
  int n_qt, n_kt, n_items, lpad, items_per_stream, bias_b_mul;
  float c1;               // D^-1/2 * log2(e)
  uint32_t fmt, bfmt;     // tcgen05 operand formats of q/k/v and of the bias (1 = bf16, 0 = f16)
  int n_alpha; float alpha[2];
  const void* mask; int64_t ms[3]; int mask_dtype;
  void* o; float* lse; int* status;
};

struct StreamBars {
  uint64_t q_full[2], q_empty[2], k_full[2], k_empty[2], v_full[2], v_empty[2], b_full[3], b_empty[3];
  uint64_t xk_full[2];       // the key tile's mask-term tile has been written (by the producer warp)
  uint64_t s_ready, s_free, p_ready, pv_done;
};

// position of a stream's work item
struct ItemPos { int qt, h, n, b, bn; };
__device__ __forceinline__ ItemPos item_pos(int it, const FwdWsP& p) {
  ItemPos x;
  x.qt = it % p.n_qt;
  const int r = it / p.n_qt;
  x.h = r % p.H; x.bn = r / p.H; x.n = x.bn % p.N; x.b = x.bn / p.N;
  return x;
}

constexpr int kLaunchRegs = 128, kSoftmaxRegs = 208, kHelperRegs = 48;      // registers per thread: at launch / after setmaxnreg
static_assert(kLaunchRegs * kThreads <= 65536, "register file");
static_assert(256 * kSoftmaxRegs + (kThreads - 256) * kHelperRegs <= kThreads * kLaunchRegs, "setmaxnreg budget");

template <typename T, typename TB>
__global__ void __maxnreg__(kLaunchRegs)
evo_fwd_ws_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                  const __grid_constant__ CUtensorMap mv, const __grid_constant__ CUtensorMap mb, const FwdWsP p MF_TRACE_PARAM) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sI = smem + 2 * kStreamBytes;              // alpha * I tiles, 1 KB each
  uint8_t* sXO = sI + 2048;                           // constant partner tile of the mask term

  __shared__ StreamBars bars[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    abort_s = 0;
    for (int q = 0; q < 2; ++q) {
      StreamBars& b = bars[q];
      for (int i = 0; i < 2; ++i) {
        mbar_init(&b.q_full[i], 1); mbar_init(&b.q_empty[i], 1); mbar_init(&b.k_full[i], 1); mbar_init(&b.k_empty[i], 1);
        mbar_init(&b.v_full[i], 1); mbar_init(&b.v_empty[i], 1);
        mbar_init(&b.xk_full[i], 1);
      }
      for (int i = 0; i < 3; ++i) { mbar_init(&b.b_full[i], 1); mbar_init(&b.b_empty[i], 1); }
      mbar_init(&b.s_ready, 1); mbar_init(&b.pv_done, 1);
      mbar_init(&b.s_free, 4); mbar_init(&b.p_ready, 4);          // one arrival per softmax warp
    }
    mbar_fence_init();
    prefetch_tmap(&mq); prefetch_tmap(&mk); prefetch_tmap(&mv); prefetch_tmap(&mb);
  }
  // constant MMA operand: alpha * I (bias)
  write_alpha_identity<TB>(sI, p.alpha[0], tid, kThreads);
  write_alpha_identity<TB>(sI + 1024, p.alpha[1], tid, kThreads);
  write_xo_tile(sXO, tid, kThreads);
  fence_async_smem();
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  volatile int* abort_flag = &abort_s;

  const int s = warp < 8 ? (warp >> 2) : (warp & 1);          // stream of this warp (helper warps alternate)
  StreamBars& bar = bars[s];
  uint8_t* sb = smem + s * kStreamBytes;
  uint8_t* sQ = sb;
  uint8_t* sK = sb + 2 * kTileB;
  uint8_t* sV = sb + 4 * kTileB;
  uint8_t* sB = sb + 6 * kTileB;
  uint8_t* sXK = sB + 3 * kAtomB;
  const uint32_t tbase = tmem_base_s + s * 256;               // S [0,128) | P [128,192) | O [192,224)

  const int stream = blockIdx.x * 2 + s;
  const int item_begin = stream * p.items_per_stream;
  int item_end = item_begin + p.items_per_stream;
  if (item_end > p.n_items) item_end = p.n_items;
  const int n_my = item_end > item_begin ? item_end - item_begin : 0;
  const int n_kt = p.n_kt;

  if (warp < 8) {
    // =========================================================================== softmax warpgroup
    // Register re-partition: the CTA is launched with kLaunchRegs registers per thread; the helper warps drop to
    // kHelperRegs and the softmax warpgroups rise to kSoftmaxRegs.  The raise can only draw on what the drop releases
    // inside this CTA (otherwise it never returns): the launcher checks the launch figure.
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tbase + lane_addr, tP = tS + 128, tO = tS + 192;
    const float2 c1c1 = make_float2(p.c1, p.c1);
    uint32_t g = 0;
    MF_TRACE_DECL(tr, 0, blockIdx.x == 0 && tid == 0);
    for (int il = 0; il < n_my; ++il) {
      const ItemPos ip = item_pos(item_begin + il, p);
      const int i = ip.qt * kT + r;
      float m_used = 0.f;
      float2 lsum0 = make_float2(0.f, 0.f), lsum1 = lsum0;        // row sum of P relative to m_used (four partial sums)
      for (int t = 0; t < n_kt; ++t, ++g) {
        // ---------------------------------------------------------------- S(g) -> registers
        tr(1);
        wait_or_flag(&bar.s_ready, g & 1, abort_flag);
        tc_fence_after();
        tr(2);
        uint32_t sr[kT];
        {
          uint32_t (*s4)[32] = reinterpret_cast<uint32_t (*)[32]>(sr);
          tmem_ld32(tS, s4[0]); tmem_ld32(tS + 32, s4[1]); tmem_ld32(tS + 64, s4[2]); tmem_ld32(tS + 96, s4[3]);
          tmem_ld_wait();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar.s_free);          // the issuer may overwrite S with the next tile's scores
        tr(3);
        // ---------------------------------------------------------------- pass 1: the maximum.  Bias and key mask are
        // already inside S (tensor core), and the scale c1 > 0 commutes with the maximum: nothing but three-input maxima
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c4 = 0; c4 < kT / 4; ++c4) {
          mx[c4 & 1 ? 2 : 0] = max3f(mx[c4 & 1 ? 2 : 0], __uint_as_float(sr[c4 * 4]), __uint_as_float(sr[c4 * 4 + 1]));
          mx[c4 & 1 ? 3 : 1] = max3f(mx[c4 & 1 ? 3 : 1], __uint_as_float(sr[c4 * 4 + 2]), __uint_as_float(sr[c4 * 4 + 3]));
        }
        const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));      // in units of the unscaled scores
        tr(4);
        if (t == 0) {
          m_used = m_blk;
        } else {
          const bool grow = (m_blk - m_used) * p.c1 > kRescaleStep;
          if (__any_sync(0xffffffffu, grow)) {
            // rare: bring O and the row sum of this warp's rows to the new maximum
            wait_or_flag(&bar.pv_done, (g - 1) & 1, abort_flag);
            tc_fence_after();
            const float f = grow ? ex2f((m_used - m_blk) * p.c1) : 1.f;
            if (grow) m_used = m_blk;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              uint32_t o16[16];
              tmem_ld16(tO + hf * 16, o16);
              tmem_ld_wait();
#pragma unroll
              for (int d = 0; d < 16; ++d) o16[d] = __float_as_uint(__uint_as_float(o16[d]) * f);
              tmem_st16(tO + hf * 16, o16);
            }
            tmem_st_wait();
            lsum0.x *= f; lsum0.y *= f; lsum1.x *= f; lsum1.y *= f;
          }
        }
        // ---------------------------------------------------------------- pass 2: P = 2^(x - m) as packed 16-bit
        if (g > 0) wait_or_flag(&bar.pv_done, (g - 1) & 1, abort_flag);      // the previous product has read P
        tr(5);
        // x = c1 * (s - m): the difference first, so that logits equal to the maximum give exactly 0 whatever their size
        // (a fully masked row sits at about -1e30, where a fused c1 * s - c1 * m would leave a huge rounding residue)
        const float2 mm = make_float2(m_used, m_used);
#pragma unroll
        for (int qr = 0; qr < 4; ++qr) {
          uint32_t pk[16];
#pragma unroll
          for (int jj = 0; jj < 16; jj += 2) {
            const float2 xa = mul2(sub2(make_float2(__uint_as_float(sr[qr * 32 + 2 * jj]), __uint_as_float(sr[qr * 32 + 2 * jj + 1])), mm), c1c1);
            const float2 xb = mul2(sub2(make_float2(__uint_as_float(sr[qr * 32 + 2 * jj + 2]), __uint_as_float(sr[qr * 32 + 2 * jj + 3])), mm), c1c1);
            const float2 ea = make_float2(ex2f(xa.x), ex2f(xa.y)), eb = make_float2(ex2f(xb.x), ex2f(xb.y));
            lsum0 = add2(lsum0, ea); lsum1 = add2(lsum1, eb);
            pk[jj] = Pack2<T>::pack(ea.x, ea.y); pk[jj + 1] = Pack2<T>::pack(eb.x, eb.y);
          }
          tmem_st16(tP + qr * 16, pk);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar.p_ready);
        tr(6);
      }
      // ------------------------------------------------------------------ item done: O / l and the log-sum-exp
      wait_or_flag(&bar.pv_done, (g - 1) & 1, abort_flag);
      tc_fence_after();
      tr(7);
      uint32_t o32[32];
      tmem_ld32(tO, o32);
      const float l = (lsum0.x + lsum0.y) + (lsum1.x + lsum1.y);
      tmem_ld_wait();
      tc_fence_before();
      tr(8);
      if (i < p.L && !*abort_flag) {
        const float inv = 1.f / l;
        T* orow = static_cast<T*>(p.o) + ((((int64_t)ip.b * p.N + ip.n) * p.L + i) * p.H + ip.h) * p.D;
#pragma unroll
        for (int d8 = 0; d8 < 4; ++d8) {
          if (d8 * 8 < p.D) {
            uint4 v;
            v.x = Pack2<T>::pack(__uint_as_float(o32[d8 * 8]) * inv, __uint_as_float(o32[d8 * 8 + 1]) * inv);
            v.y = Pack2<T>::pack(__uint_as_float(o32[d8 * 8 + 2]) * inv, __uint_as_float(o32[d8 * 8 + 3]) * inv);
            v.z = Pack2<T>::pack(__uint_as_float(o32[d8 * 8 + 4]) * inv, __uint_as_float(o32[d8 * 8 + 5]) * inv);
            v.w = Pack2<T>::pack(__uint_as_float(o32[d8 * 8 + 6]) * inv, __uint_as_float(o32[d8 * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + d8 * 8) = v;
          }
        }
        // a row whose keys are all masked has every logit at the mask term (about -1e30): uniform attention over its L
        // keys; its log-sum-exp is stored as -FLT_MAX, the value the backward kernels recognise
        p.lse[(((int64_t)ip.b * p.N + ip.n) * p.H + ip.h) * p.L + i] = m_used <= -1e28f ? -FLT_MAX : (m_used * p.c1 + lg2f(l)) * kLn2;
      }
      tr(9);
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kHelperRegs));
    // The helper roles are run by whole warps (one elected lane issues: see mma_ss_el); every exit decision is a warp vote.
    auto dead = [&] { return __any_sync(0xffffffffu, *abort_flag) != 0; };
    if (warp < 10) {
      // ========================================================================= score-MMA issuer of stream s
      const uint32_t id_s = idesc_f16(128, 128, p.fmt, 0, 0);
      const uint32_t id_b = idesc_f16(128, 16, p.bfmt, 0, 0);
      const uint32_t id_x = idesc_f16(128, 128, 1u, 0, 0);         // the mask-term tiles are bf16 whatever q/k/v are
      constexpr uint32_t hi64 = desc_hi(512, kSw64), hi128 = desc_hi(1024, kSw128), hi32 = desc_hi(256, kSw32);
      const uint32_t xo_lo = desc_lo(smem_u32(sXO), 16), xk_base = desc_lo(smem_u32(sXK), 16);
      const uint32_t tS = tbase;
      const uint32_t q_base = desc_lo(smem_u32(sQ), 16), k_base = desc_lo(smem_u32(sK), 16), b_base = desc_lo(smem_u32(sB), 16);
      const uint32_t i_lo0 = desc_lo(smem_u32(sI), 16), i_lo1 = i_lo0 + 1024 / 16;
      const bool two_terms = p.n_alpha > 1;
      uint32_t bslot = 0, buse = 0;               // bias atoms consumed: ring slot and use count of the next one
      MF_TRACE_DECL(tr, 1, blockIdx.x == 0 && warp == 8 && lane == 0);
      const uint32_t g_total = (uint32_t)n_my * n_kt;
      int il = 0, t = 0;
      for (uint32_t g = 0; g < g_total; ++g) {       // S(g) = Q K^T + alpha * bias
        tr(10);
        if (t == 0) wait_or_flag(&bar.q_full[il & 1], (il >> 1) & 1, abort_flag);
        wait_or_flag(&bar.k_full[g & 1], (g >> 1) & 1, abort_flag);
        wait_or_flag(&bar.xk_full[g & 1], (g >> 1) & 1, abort_flag);
        const uint32_t slot0 = bslot, use0 = buse;
        uint32_t slot1 = slot0 + 1, use1 = use0;
        if (slot1 == 3) { slot1 = 0; ++use1; }
        wait_or_flag(&bar.b_full[slot0], use0 & 1, abort_flag);
        wait_or_flag(&bar.b_full[slot1], use1 & 1, abort_flag);
        bslot = slot1 + 1; buse = use1;
        if (bslot == 3) { bslot = 0; ++buse; }
        tr(11);
        if (g > 0) wait_or_flag(&bar.s_free, (g - 1) & 1, abort_flag);
        tc_fence_after();
        tr(12);
        if (!dead()) {
          const uint32_t q_lo = q_base + (il & 1) * (kTileB / 16), k_lo = k_base + (g & 1) * (kTileB / 16);
          mma_ss_el(tS, q_lo, hi64, k_lo, hi64, id_s, false);
          mma_ss_el(tS, q_lo + 2, hi64, k_lo + 2, hi64, id_s, true);
          mma_ss_el(tS, xo_lo, hi32, xk_base + (g & 1) * (kXTileB / 16), hi32, id_x, true);        // + key mask
          const uint32_t a0 = b_base + slot0 * (kAtomB / 16), a1 = b_base + slot1 * (kAtomB / 16);
#pragma unroll
          for (int c = 0; c < 4; ++c) mma_ss_el(tS + c * 16, a0 + c * 2, hi128, i_lo0, hi64, id_b, true);      // 16 key columns each
#pragma unroll
          for (int c = 0; c < 4; ++c) mma_ss_el(tS + 64 + c * 16, a1 + c * 2, hi128, i_lo0, hi64, id_b, true);
          if (two_terms) {
#pragma unroll
            for (int c = 0; c < 4; ++c) mma_ss_el(tS + c * 16, a0 + c * 2, hi128, i_lo1, hi64, id_b, true);
#pragma unroll
            for (int c = 0; c < 4; ++c) mma_ss_el(tS + 64 + c * 16, a1 + c * 2, hi128, i_lo1, hi64, id_b, true);
          }
          tc_commit_el(&bar.s_ready);
          tc_commit_el(&bar.k_empty[g & 1]);
          tc_commit_el(&bar.b_empty[slot0]);
          tc_commit_el(&bar.b_empty[slot1]);
          if (t == n_kt - 1) tc_commit_el(&bar.q_empty[il & 1]);
        }
        tr(13);
        if (++t == n_kt) { t = 0; ++il; }
      }
    } else if (warp < 12) {
      // ========================================================================= P V issuer of stream s
      const uint32_t id_o = idesc_f16(128, 32, p.fmt, 0, 1);           // B (V) MN-major
      constexpr uint32_t hi64 = desc_hi(512, kSw64);
      const uint32_t tP = tbase + 128, tO = tbase + 192;
      const uint32_t v_base = desc_lo(smem_u32(sV), 16);
      MF_TRACE_DECL(tr, 2, blockIdx.x == 0 && warp == 10 && lane == 0);
      const uint32_t g_total = (uint32_t)n_my * n_kt;
      int t = 0;
      for (uint32_t g = 0; g < g_total; ++g) {       // O (+)= P V
        tr(15);
        wait_or_flag(&bar.v_full[g & 1], (g >> 1) & 1, abort_flag);
        wait_or_flag(&bar.p_ready, g & 1, abort_flag);
        tc_fence_after();
        tr(16);
        if (!dead()) {
          const uint32_t v_lo = v_base + (g & 1) * (kTileB / 16);
          mma_ts_el(tO, tP, v_lo, hi64, id_o, t > 0);
#pragma unroll
          for (int ks = 1; ks < 8; ++ks) mma_ts_el(tO, tP + ks * 8, v_lo + ks * 64, hi64, id_o, true);
          tc_commit_el(&bar.pv_done);
          tc_commit_el(&bar.v_empty[g & 1]);
        }
        tr(17);
        if (++t == n_kt) t = 0;
      }
    } else if (warp < 14) {
      // ========================================================================= TMA producer of stream s
      uint32_t g = 0, bslot = 0, buse = 0;
      uint32_t nq = 0, nk = 0, nv = 0, nb = 0;      // loads issued, for the drain on abort
      auto load_q = [&](int il) {        // the Q tile of item il (requested one key tile before the item starts)
        const ItemPos iq = item_pos(item_begin + il, p);
        if (il >= 2) wait_or_flag(&bar.q_empty[il & 1], ((il >> 1) - 1) & 1, abort_flag);
        if (dead()) return;
        if (elect_one()) {
          mbar_expect_tx(&bar.q_full[il & 1], kTileB);
          tma_load_5d(sQ + (il & 1) * kTileB, &mq, &bar.q_full[il & 1], 0, iq.h, iq.qt * kT, iq.n, iq.b);
        }
        ++nq;
      };
      // Mask term of key j of row (b, n), in units of the unscaled scores (x sqrt(D)): 0 / -1e30 for a keep-mask, the value
      // for an additive mask; keys beyond L get -2e30 so that even a fully masked row (all its keys at -1e30) excludes them.
      // The mask values of a tile are fetched one tile ahead as raw bits (four independent loads) and converted when the
      // tile is written, so that their latency is never waited for.
      const float sqrt_d = sqrtf((float)p.D);
      uint32_t raw[4] = {0u, 0u, 0u, 0u};
      auto fetch = [&](const ItemPos& x, int j0) {
        int64_t mi[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          int j = j0 + k * 32 + lane;
          if (j >= p.L) j = p.L - 1;
          mi[k] = x.b * p.ms[0] + x.n * p.ms[1] + (int64_t)j * p.ms[2];
        }
        if (p.mask_dtype == MF_U8) {
#pragma unroll
          for (int k = 0; k < 4; ++k) raw[k] = static_cast<const uint8_t*>(p.mask)[mi[k]];
        } else if (p.mask_dtype == MF_F32) {
#pragma unroll
          for (int k = 0; k < 4; ++k) raw[k] = static_cast<const uint32_t*>(p.mask)[mi[k]];
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) raw[k] = static_cast<const uint16_t*>(p.mask)[mi[k]];
        }
      };
      auto term = [&](uint32_t bits, int j) {
        float v;
        if (p.mask_dtype == MF_U8) v = bits ? 0.f : kMinusBig;
        else {
          const float x = p.mask_dtype == MF_F32 ? __uint_as_float(bits)
                          : p.mask_dtype == MF_BF16 ? __uint_as_float(bits << 16) : __half2float(__ushort_as_half((unsigned short)bits));
          v = fmaxf(x * sqrt_d, kMinusBig);
        }
        return j < p.L ? v : 2.f * kMinusBig;
      };
      if (n_my > 0) fetch(item_pos(item_begin, p), 0);
      if (n_my > 0) load_q(0);
      // A bulk-tensor copy keeps the thread that issues it busy for a few hundred cycles whatever its size; several lanes of
      // one warp issuing in the same instruction cost little more than one.  So the K tile and the two bias atoms of a key
      // tile are requested by lanes 0, 1 and 2 together (the waits before them are taken by the whole warp).
      const CUtensorMap* map3 = lane == 0 ? &mk : &mb;
      for (int il = 0; il < n_my && !dead(); ++il) {
        const ItemPos ip = item_pos(item_begin + il, p);
        for (int t = 0; t < n_kt; ++t, ++g) {
          if (t == n_kt - 1 && il + 1 < n_my) load_q(il + 1);
          if (g >= 2) wait_or_flag(&bar.k_empty[g & 1], ((g >> 1) - 1) & 1, abort_flag);
          if (dead()) break;
          {
            // the key tile's mask-term tile XK (rows = keys; columns 0..2 = split3 of the term), written by the whole warp
            uint8_t* xt = sXK + (g & 1) * kXTileB;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              __nv_bfloat16 m3[3];
              const int r = k * 32 + lane;
              split3(term(raw[k], t * kT + r), m3);
              *reinterpret_cast<uint4*>(xt + swz_offset(r, 0, 32)) = make_uint4(pack_bf(m3[0], m3[1]), pack_bf(m3[2], __float2bfloat16_rn(0.f)), 0u, 0u);
              *reinterpret_cast<uint4*>(xt + swz_offset(r, 1, 32)) = make_uint4(0u, 0u, 0u, 0u);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar.xk_full[g & 1]);
            // next tile's mask values: same item, or the first tile of the next item
            if (t + 1 < n_kt) fetch(ip, (t + 1) * kT);
            else if (il + 1 < n_my) fetch(item_pos(item_begin + il + 1, p), 0);
          }
          const uint32_t slot0 = bslot, use0 = buse;
          uint32_t slot1 = slot0 + 1, use1 = use0;
          if (slot1 == 3) { slot1 = 0; ++use1; }
          if (use0 >= 1) wait_or_flag(&bar.b_empty[slot0], (use0 - 1) & 1, abort_flag);
          if (use1 >= 1) wait_or_flag(&bar.b_empty[slot1], (use1 - 1) & 1, abort_flag);
          if (dead()) break;
          if (lane == 0) {
            mbar_expect_tx(&bar.k_full[g & 1], kTileB);
            tma_load_5d(sK + (g & 1) * kTileB, map3, &bar.k_full[g & 1], 0, ip.h, t * kT, ip.n, ip.b);
          } else if (lane <= 2) {
            const uint32_t slot = lane == 1 ? slot0 : slot1;
            mbar_expect_tx(&bar.b_full[slot], kAtomB);
            tma_load_5d(sB + slot * kAtomB, map3, &bar.b_full[slot], t * kT + (lane - 1) * 64, ip.qt * kT, ip.h, ip.b * p.bias_b_mul, 0);
          }
          __syncwarp();
          ++nk; nb += 2;
          bslot = slot1 + 1; buse = use1;
          if (bslot == 3) { bslot = 0; ++buse; }
          if (g >= 2) wait_or_flag(&bar.v_empty[g & 1], ((g >> 1) - 1) & 1, abort_flag);
          if (dead()) break;
          if (elect_one()) {
            mbar_expect_tx(&bar.v_full[g & 1], kTileB);
            tma_load_5d(sV + (g & 1) * kTileB, &mv, &bar.v_full[g & 1], 0, ip.h, t * kT, ip.n, ip.b);
          }
          ++nv;
        }
      }
      if (dead() && lane == 0) {
        // the copies already requested must land before the CTA's shared memory is given back (bounded)
        auto drain = [&](uint64_t* ring, uint32_t n, uint32_t depth) {
          for (uint32_t back = 0; back < depth && back < n; ++back) {
            const uint32_t c = n - 1 - back;
            mbar_wait(&ring[c % depth], (c / depth) & 1);
          }
        };
        drain(bar.q_full, nq, 2); drain(bar.k_full, nk, 2); drain(bar.v_full, nv, 2); drain(bar.b_full, nb, 3);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_s) *reinterpret_cast<volatile int*>(p.status) = 1;
  if (warp == 0) tmem_dealloc(tmem_base_s, 512);
}

template <typename T, typename TB>
int launch_fwd_ws(const mf_evo_fwd_args& a, cudaStream_t st) {
  CUtensorMap mq, mk, mv, mb;
  int r;
  if ((r = make_qkv_map(&mq, a.q, a.dtype, a.B, a.N, a.L, a.H, a.D, a.q_strides, 32, kT))) return r;
  if ((r = make_qkv_map(&mk, a.k, a.dtype, a.B, a.N, a.L, a.H, a.D, a.k_strides, 32, kT))) return r;
  if ((r = make_qkv_map(&mv, a.v, a.dtype, a.B, a.N, a.L, a.H, a.D, a.v_strides, 32, kT))) return r;
  FwdWsP p{};
  p.B = a.B; p.N = a.N; p.L = a.L; p.H = a.H; p.D = a.D;
  p.n_qt = (a.L + kT - 1) / kT; p.n_kt = p.n_qt;
  p.n_items = a.B * a.N * a.H * p.n_qt;
  p.lpad = p.n_kt * kT;
  p.c1 = kLog2e / sqrtf((float)a.D);
  p.fmt = a.dtype == MF_BF16 ? 1u : 0u;
  p.bfmt = a.bias_dtype == MF_BF16 ? 1u : 0u;
  p.n_alpha = split_alpha(a.D, a.bias_dtype, p.alpha);
  p.mask = a.mask; for (int i = 0; i < 3; ++i) p.ms[i] = a.mask_strides[i];
  p.mask_dtype = a.mask_dtype;
  p.o = a.o; p.lse = a.lse;
  p.status = status_word();
  MF_REQUIRE(p.status, MF_ERR_CUDA, "could not allocate the device status word");
  MF_REQUIRE(tc_async_status() == 0, MF_ERR_CUDA, "an earlier tensor-core kernel gave up on a bounded wait; results are invalid");
  p.bias_b_mul = a.bias_strides[0] == 0 ? 0 : 1;
  {
    // five dimensions (the last one a dummy) so that one instruction, issued by several lanes, loads K and bias tiles alike
    const int64_t dims[5] = {a.L, a.L, a.H, p.bias_b_mul ? a.B : 1, 1};
    const int64_t str[5] = {1, a.bias_strides[2], a.bias_strides[1], a.bias_strides[0], 0};
    const int box[5] = {64, 128, 1, 1, 1};
    if ((r = make_tiled_map(&mb, a.bias, a.bias_dtype, 5, dims, str, box, 128))) return r;
  }
  int grid = sm_count();
  const int pairs = (p.n_items + 1) / 2;
  if (grid > pairs) grid = pairs;
  p.items_per_stream = (p.n_items + 2 * grid - 1) / (2 * grid);
  const size_t smem = 1024 + 2 * (size_t)kStreamBytes + 2048 + kXTileB;
  auto kern = evo_fwd_ws_kernel<T, TB>;
  cudaFuncAttributes fa;
  MF_CUDA(cudaFuncGetAttributes(&fa, kern));
  MF_REQUIRE(fa.numRegs == kLaunchRegs, MF_ERR_CUDA, "evo_fwd_ws_kernel was built with %d registers per thread, %d expected", fa.numRegs, kLaunchRegs);
  MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<grid, kThreads, smem, st>>>(mq, mk, mv, mb, p MF_TRACE_ARG);
  MF_LAUNCHED("evo_fwd_ws_kernel");
  return MF_OK;
}

}  // namespace

// The warp-specialised kernel covers head sizes up to 32, rows up to 2048 tokens and a 16-bit pair bias whose rows
// TMA can address (unit stride on keys, 16-byte multiples elsewhere); other calls use the general kernel.
bool evo_fwd_ws_supported(const mf_evo_fwd_args& a) {
  if (a.D > 32 || a.L > 2048) return false;
  if (a.bias_dtype != MF_BF16 && a.bias_dtype != MF_F16) return false;
  const int64_t* s = a.bias_strides;
  if (s[3] != 1 || (reinterpret_cast<uintptr_t>(a.bias) & 15) != 0) return false;
  if ((s[2] * 2) % 16 != 0 || s[2] <= 0) return false;
  if (a.H > 1 && ((s[1] * 2) % 16 != 0 || s[1] <= 0)) return false;
  if (a.B > 1 && s[0] != 0 && ((s[0] * 2) % 16 != 0 || s[0] < 0)) return false;
  return true;
}

int evo_fwd_ws(const mf_evo_fwd_args& a, cudaStream_t st) {
  if (a.dtype == MF_BF16)
    return a.bias_dtype == MF_BF16 ? launch_fwd_ws<__nv_bfloat16, __nv_bfloat16>(a, st) : launch_fwd_ws<__nv_bfloat16, __half>(a, st);
  return a.bias_dtype == MF_BF16 ? launch_fwd_ws<__half, __nv_bfloat16>(a, st) : launch_fwd_ws<__half, __half>(a, st);
}

}  // namespace mf
