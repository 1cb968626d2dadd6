// Pair-biased masked attention forward on the tensor cores (tcgen05 + TMEM + TMA): the GENERAL kernel, for the calls
// the warp-specialised kernel (evo_fwd_ws.cu) does not take - head sizes 33..64, an fp32 or unaligned pair bias,
// rows longer than 2048 tokens.
//
// A persistent CTA (one per SM, 256 threads) runs TWO independent streams, one per warpgroup.  A stream walks a
// contiguous range of work items (b, n, h, 128-query tile) and, per item, the key tiles of 128.  Inside a stream every
// thread owns one query row (= one TMEM lane); three "officer" threads of the warpgroup also issue the stream's
// tcgen05.mma instructions (thread 0), its Q/K/V TMA loads (thread 32) and its bias TMA loads (thread 64):
//
//   wait S(t) in TMEM -> tcgen05.ld the whole 128-column row into registers -> group barrier ->
//   S(t+1) = Q K(t+1)^T is issued at once (the S buffer is free again: registers double-buffer it)
//   -> row thread: logits in base 2 (scale, bias from shared memory, key mask), running max, exp2,
//   row sum, packed 16-bit P -> fold O_tile(t-1) from TMEM into the register accumulator ->
//   tcgen05.st P -> group barrier -> O_tile(t) = P V(t) is issued (P as TMEM A operand, V as
//   MN-major B operand) and the TMA rings are topped up.
//
// Operand tiles are [128 rows x DP] (DP = 32: 64-byte rows, 64B swizzle; DP = 64: 128-byte rows) fetched
// from the strided [B, N, L, H, D] tensors by 5-D tensor maps; smaller head sizes are zero-filled by TMA.
// A 16-bit pair bias with TMA-addressable rows is staged as [128 rows x 64 columns] chunks (128-byte rows, 128B
// swizzle, DP = 32 only); otherwise the row thread reads it from global memory.
//
// Every wait is bounded; on expiry the CTA raises a flag that all threads honour at their next group
// barrier, TMEM is freed and the host sees mf_async_status() != 0.
#include "evo_tc_common.cuh"

namespace mf {
namespace {
using namespace tcx;

constexpr int kQT = 128, kKT = 128;
constexpr int kThreads = 256;
constexpr int kVS = 2;        // V ring stages per stream
constexpr int kBC = 3;        // bias chunk ring per stream (2 chunks per key tile: every TMA issue costs the
                              // issuing thread, a lane of a compute warp, some hundreds of cycles)
constexpr int kBCW = 64;      // columns per bias chunk (128-byte rows)
constexpr int kBChunkBytes = 128 * kBCW * 2;

template <int DP> struct Cfg {
  static constexpr int ROWB = DP * 2;
  static constexpr int TILEB = 128 * ROWB;
  static constexpr int KS = DP == 32 ? 3 : 2;     // K ring stages per stream
  static constexpr Swizzle SW = DP == 32 ? kSw64 : kSw128;
  static constexpr int SBO = 8 * ROWB;
  static constexpr int STREAM_BYTES(bool btma) { return TILEB * (1 + KS + kVS) + (btma ? kBC * kBChunkBytes : 0); }
};

struct FwdP {
  int B, N, L, H, D;
  int n_qt, n_kt, n_items, lpad, items_per_stream, bias_b_mul;
  float c1;               // D^-1/2 * log2(e)
  uint32_t ab_fmt;        // 1 = bf16, 0 = f16
  const void* bias; int64_t bs[4]; int bias_fast;
  const void* mask; int64_t ms[3]; int mask_dtype;
  void* o; float* lse; int* status;
};

struct StreamBars {
  uint64_t q_full, k_full[3], v_full[kVS], b_full[kBC], b_empty[kBC], s_ready, pv_done;
};

// 32 consecutive bias values of one row as fp32 from global memory; `p` 16-byte aligned, in bounds.
template <typename TB>
__device__ __forceinline__ void load_bias32_fast(const TB* p, float (&out)[32]) {
  if constexpr (sizeof(TB) == 4) {
    const float4* v = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float4 x = __ldg(v + i);
      out[4 * i] = x.x; out[4 * i + 1] = x.y; out[4 * i + 2] = x.z; out[4 * i + 3] = x.w;
    }
  } else {
    const uint4* v = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 x = __ldg(v + i);
      float2 a = Pack2<TB>::unpack(x.x), b = Pack2<TB>::unpack(x.y), c = Pack2<TB>::unpack(x.z), d = Pack2<TB>::unpack(x.w);
      out[8 * i] = a.x; out[8 * i + 1] = a.y; out[8 * i + 2] = b.x; out[8 * i + 3] = b.y;
      out[8 * i + 4] = c.x; out[8 * i + 5] = c.y; out[8 * i + 6] = d.x; out[8 * i + 7] = d.y;
    }
  }
}
template <typename TB>
__device__ __forceinline__ void load_bias32_slow(const TB* row, int64_t sj, int j0, int L, float (&out)[32]) {
#pragma unroll
  for (int i = 0; i < 32; ++i) out[i] = (j0 + i < L) ? to_f(row[(int64_t)(j0 + i) * sj]) : 0.f;
}

template <int DP, typename T, typename TB, bool BTMA>
__global__ void __launch_bounds__(kThreads, 1)
evo_fwd_tc_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                  const __grid_constant__ CUtensorMap mv, const __grid_constant__ CUtensorMap mb, const FwdP p) {
  using C = Cfg<DP>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr int kStreamBytes = C::STREAM_BYTES(BTMA);

  __shared__ StreamBars bars[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int s = warp >> 2;                    // stream = warpgroup
  const int wg_tid = tid & 127;
  const bool leader = wg_tid == 0;
  if (tid == 0) {
    abort_s = 0;
    for (int q = 0; q < 2; ++q) {
      StreamBars& b = bars[q];
      mbar_init(&b.q_full, 1);
      for (int i = 0; i < 3; ++i) mbar_init(&b.k_full[i], 1);
      for (int i = 0; i < kVS; ++i) mbar_init(&b.v_full[i], 1);
      for (int i = 0; i < kBC; ++i) { mbar_init(&b.b_full[i], 1); mbar_init(&b.b_empty[i], 128); }
      mbar_init(&b.s_ready, 1);
      mbar_init(&b.pv_done, 1);
    }
    mbar_fence_init();
    prefetch_tmap(&mq); prefetch_tmap(&mk); prefetch_tmap(&mv);
    if (BTMA) prefetch_tmap(&mb);
  }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  volatile int* abort_flag = &abort_s;
  StreamBars& bar = bars[s];
  uint8_t* sb = smem + s * kStreamBytes;
  uint8_t* sQ = sb;
  uint8_t* sK = sQ + C::TILEB;
  uint8_t* sV = sK + C::KS * C::TILEB;
  uint8_t* sB = sV + kVS * C::TILEB;
  float* mask2 = reinterpret_cast<float*>(smem + 2 * kStreamBytes) + s * p.lpad;

  const int r = (warp & 3) * 32 + lane;                              // TMEM lane = query row in the tile
  const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
  const uint32_t tS = tmem_base_s + s * 256 + lane_addr, tP = tS + 128, tO = tS + 192;
  const uint32_t tS0 = tmem_base_s + s * 256;                        // lane 0 addresses for the MMA issuer
  const uint32_t id_s = idesc_f16(128, kKT, p.ab_fmt, 0, 0);
  const uint32_t id_o = idesc_f16(128, DP, p.ab_fmt, 0, 1);

  const int stream = blockIdx.x * 2 + s;
  const int item_begin = stream * p.items_per_stream;
  int item_end = item_begin + p.items_per_stream;
  if (item_end > p.n_items) item_end = p.n_items;
  const int n_my = item_end > item_begin ? item_end - item_begin : 0;
  const int g_total = n_my * p.n_kt;
  const int per_bn = p.H * p.n_qt;

  // ---- TMA bookkeeping.  Three "officer" threads per stream share the issue work so that none of it
  // piles up on one warp: thread 0 issues the MMAs, thread 32 the Q/K/V loads, thread 64 the bias loads.
  // A cursor walks (item, key tile) incrementally: no divisions on the hot path.
  struct Cursor {
    int qt, h, n, b, t, item_local;
  };
  auto cursor_init = [&](Cursor& c) {
    const int it = item_begin;
    c.qt = it % p.n_qt; c.h = (it / p.n_qt) % p.H;
    const int bn = it / per_bn;
    c.n = bn % p.N; c.b = bn / p.N; c.t = 0; c.item_local = 0;
  };
  auto cursor_next_item = [&](Cursor& c) {
    c.t = 0; ++c.item_local;
    if (++c.qt == p.n_qt) { c.qt = 0; if (++c.h == p.H) { c.h = 0; if (++c.n == p.N) { c.n = 0; ++c.b; } } }
  };
  auto cursor_next_tile = [&](Cursor& c) { if (++c.t == p.n_kt) cursor_next_item(c); };
  const bool officer_kv = wg_tid == 32, officer_b = wg_tid == 64;
  Cursor ck, cv, cq, cbias;
  cursor_init(ck); cursor_init(cv); cursor_init(cq); cursor_init(cbias);
  int gk = 0, gv = 0, cb_next = 0, cb_quarter = 0;
  uint32_t kslot = 0, vslot = 0, pslot = 0, puse = 0;
  auto issue_q = [&]() {      // Q of the cursor's item, then advance to the next item
    mbar_expect_tx(&bar.q_full, C::TILEB);
    tma_load_5d(sQ, &mq, &bar.q_full, 0, cq.h, cq.qt * kQT, cq.n, cq.b);
    cursor_next_item(cq);
  };
  // K tiles may be requested up to KS ahead of the last S that is known to be complete (s_done tiles)
  auto pump_k = [&](int s_done) {
    while (gk < g_total && gk < s_done + C::KS) {
      mbar_expect_tx(&bar.k_full[kslot], C::TILEB);
      tma_load_5d(sK + kslot * C::TILEB, &mk, &bar.k_full[kslot], 0, ck.h, ck.t * kKT, ck.n, ck.b);
      cursor_next_tile(ck); ++gk;
      if (++kslot == C::KS) kslot = 0;
    }
  };
  auto pump_v = [&](int pv_done_cnt) {
    while (gv < g_total && gv < pv_done_cnt + kVS) {
      mbar_expect_tx(&bar.v_full[vslot], C::TILEB);
      tma_load_5d(sV + vslot * C::TILEB, &mv, &bar.v_full[vslot], 0, cv.h, cv.t * kKT, cv.n, cv.b);
      cursor_next_tile(cv); ++gv;
      if (++vslot == kVS) vslot = 0;
    }
  };
  auto pump_b = [&]() {
    if (!BTMA) return;
    while (cb_next < g_total * (kKT / kBCW)) {
      if (puse > 0 && !mbar_test(&bar.b_empty[pslot], (puse - 1) & 1)) break;
      mbar_expect_tx(&bar.b_full[pslot], kBChunkBytes);
      tma_load_4d(sB + pslot * kBChunkBytes, &mb, &bar.b_full[pslot], cbias.t * kKT + cb_quarter * kBCW, cbias.qt * kQT,
                  cbias.h, cbias.b * p.bias_b_mul);
      ++cb_next;
      if (++cb_quarter == kKT / kBCW) { cb_quarter = 0; cursor_next_tile(cbias); }
      if (++pslot == kBC) { pslot = 0; ++puse; }
    }
  };
  auto issue_s = [&](int g) {     // S(g) = Q K(g)^T
    const uint32_t q_lo = desc_lo(smem_u32(sQ), 16), k_lo = desc_lo(smem_u32(sK + (g % C::KS) * C::TILEB), 16);
#pragma unroll
    for (int ks = 0; ks < DP / 16; ++ks)
      mma_ss_lh(tS0, q_lo + ks * 2, desc_hi(C::SBO, C::SW), k_lo + ks * 2, desc_hi(C::SBO, C::SW), id_s, ks > 0);
    tc_commit(&bar.s_ready);
  };
  auto issue_pv = [&](int g) {    // O_tile(g) = P V(g)
    const uint32_t v_lo = desc_lo(smem_u32(sV + (g % kVS) * C::TILEB), 16);
#pragma unroll
    for (int ks = 0; ks < kKT / 16; ++ks)
      mma_ts_lh(tS0 + 192, tS0 + 128 + ks * 8, v_lo + ks * (16 * C::ROWB / 16), desc_hi(C::SBO, C::SW), id_o, ks > 0);
    tc_commit(&bar.pv_done);
  };

  if (g_total > 0) {
    if (officer_kv) { issue_q(); pump_k(0); pump_v(0); }
    if (officer_b) pump_b();
  }

  const TB* bias = static_cast<const TB*>(p.bias);
  int prev_bn = -1;
  int t = 0, item_local = 0;
  int b = 0, n = 0, h = 0, i = 0;
  bool row_ok = false;
  const TB* brow = bias;
  float m = -INFINITY, l = 0.f, corr_prev = 0.f;
  float acc[DP];
  uint32_t bslot = 0, bphase = 0;          // bias chunk ring position of the consumer

  auto fold = [&]() {   // acc = acc * corr_prev + O_tile
    tc_fence_after();
#pragma unroll
    for (int cb = 0; cb < DP / 32; ++cb) {
      uint32_t o32[32];
      tmem_ld32(tO + cb * 32, o32);
      tmem_ld_wait();
#pragma unroll
      for (int d = 0; d < 32; ++d) acc[cb * 32 + d] = fmaf(acc[cb * 32 + d], corr_prev, __uint_as_float(o32[d]));
    }
  };

  for (int g = 0; g < g_total; ++g) {
    if (t == 0) {
      // ---------------------------------------------------------------- new item
      const int it = item_begin + item_local;
      const int qt = it % p.n_qt, bn = it / per_bn;
      h = (it / p.n_qt) % p.H; n = bn % p.N; b = bn / p.N;
      i = qt * kQT + r;
      row_ok = i < p.L;
      brow = bias + b * p.bs[0] + h * p.bs[1] + (int64_t)(row_ok ? i : p.L - 1) * p.bs[2];
      if (bn != prev_bn) {
        // additive key terms of row (b, n) in the base-2 domain; columns beyond L are -inf
        named_sync(1 + s, 128);
        for (int j = wg_tid; j < p.lpad; j += 128) {
          float v = -INFINITY;
          if (j < p.L) {
            const int64_t mi = b * p.ms[0] + n * p.ms[1] + j * p.ms[2];
            v = p.mask_dtype == MF_U8 ? (static_cast<const uint8_t*>(p.mask)[mi] ? 0.f : -FLT_MAX)
                                      : load_rt(p.mask, mi, p.mask_dtype) * kLog2e;
          }
          mask2[j] = v;
        }
        named_sync(1 + s, 128);
        prev_bn = bn;
      }
      m = -INFINITY; l = 0.f; corr_prev = 0.f;
#pragma unroll
      for (int d = 0; d < DP; ++d) acc[d] = 0.f;
      if (leader) {
        wait_or_flag(&bar.q_full, item_local & 1, abort_flag);
        wait_or_flag(&bar.k_full[g % C::KS], (g / C::KS) & 1, abort_flag);
        tc_fence_after();
        if (!*abort_flag) issue_s(g);
      }
    }
    // ------------------------------------------------------------------ S(g) -> registers
    wait_or_flag(&bar.s_ready, g & 1, abort_flag);
    tc_fence_after();
    uint32_t sr[kKT];
    {
      uint32_t (*s4)[32] = reinterpret_cast<uint32_t (*)[32]>(sr);
      tmem_ld32(tS, s4[0]); tmem_ld32(tS + 32, s4[1]); tmem_ld32(tS + 64, s4[2]); tmem_ld32(tS + 96, s4[3]);
      tmem_ld_wait();
    }
    tc_fence_before();
    if (named_sync_or(1 + s, 128, *abort_flag)) break;
    if (leader) {
      // the S buffer is free: start the next tile's scores right away
      if (t + 1 < p.n_kt) {
        wait_or_flag(&bar.k_full[(g + 1) % C::KS], ((g + 1) / C::KS) & 1, abort_flag);
        tc_fence_after();
        if (!*abort_flag) issue_s(g + 1);
      }
    }
    if (officer_kv) {
      if (t + 1 == p.n_kt && item_local + 1 < n_my) issue_q();   // every S of this item is complete: Q is free
      pump_k(g + 1);
    }
    if (officer_b) pump_b();
    // ------------------------------------------------------------------ pass 1: base-2 logits, row max
    const int j0 = t * kKT;
    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int cb = 0; cb < 4; ++cb) {
      float bv[32];
      if (BTMA) {
        // a chunk holds 64 columns: two passes of this loop read its two halves
        if ((cb & 1) == 0) wait_or_flag(&bar.b_full[bslot], bphase, abort_flag);
        const uint8_t* chunk = sB + bslot * kBChunkBytes;
#pragma unroll
        for (int pc = 0; pc < 4; ++pc) {
          const uint4 x = *reinterpret_cast<const uint4*>(chunk + swz_offset(r, (cb & 1) * 4 + pc, 128));
          float2 a = Pack2<TB>::unpack(x.x), b2 = Pack2<TB>::unpack(x.y), c2 = Pack2<TB>::unpack(x.z), d2 = Pack2<TB>::unpack(x.w);
          bv[8 * pc] = a.x; bv[8 * pc + 1] = a.y; bv[8 * pc + 2] = b2.x; bv[8 * pc + 3] = b2.y;
          bv[8 * pc + 4] = c2.x; bv[8 * pc + 5] = c2.y; bv[8 * pc + 6] = d2.x; bv[8 * pc + 7] = d2.y;
        }
        if (cb & 1) {
          mbar_arrive(&bar.b_empty[bslot]);
          if (++bslot == kBC) { bslot = 0; bphase ^= 1; }
        }
      } else {
        if (p.bias_fast && (j0 + kKT <= p.L)) load_bias32_fast<TB>(brow + j0 + cb * 32, bv);
        else load_bias32_slow<TB>(brow, p.bs[3], j0 + cb * 32, p.L, bv);
      }
#pragma unroll
      for (int q4 = 0; q4 < 8; ++q4) {
        const float4 mk4 = *reinterpret_cast<const float4*>(mask2 + j0 + cb * 32 + q4 * 4);
        const float mk[4] = {mk4.x, mk4.y, mk4.z, mk4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int jj = cb * 32 + q4 * 4 + e;
          const float v = fmaf(__uint_as_float(sr[jj]), p.c1, fmaf(bv[q4 * 4 + e], kLog2e, mk[e]));
          sr[jj] = __float_as_uint(v);
          mx4[e] = fmaxf(mx4[e], v);
        }
      }
    }
    const float m_new = fmaxf(fmaxf(m, fmaxf(mx4[0], mx4[1])), fmaxf(mx4[2], mx4[3]));
    const float corr = ex2f(m - m_new);
    // ------------------------------------------------------------------ fold O_tile(g-1), then P(g)
    if (t > 0) {
      wait_or_flag(&bar.pv_done, (g - 1) & 1, abort_flag);
      fold();
    }
    float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int cb = 0; cb < 2; ++cb) {
      uint32_t pk[32];
#pragma unroll
      for (int jj = 0; jj < 32; ++jj) {
        const float p0 = ex2f(__uint_as_float(sr[cb * 64 + 2 * jj]) - m_new);
        const float p1 = ex2f(__uint_as_float(sr[cb * 64 + 2 * jj + 1]) - m_new);
        rs4[jj & 3] += p0 + p1;
        pk[jj] = Pack2<T>::pack(p0, p1);
      }
      tmem_st32(tP + cb * 32, pk);
    }
    l = fmaf(l, corr, (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
    m = m_new;
    corr_prev = corr;
    tmem_st_wait();
    tc_fence_before();
    if (named_sync_or(1 + s, 128, *abort_flag)) break;
    if (leader) {
      wait_or_flag(&bar.v_full[g % kVS], (g / kVS) & 1, abort_flag);
      tc_fence_after();
      if (!*abort_flag) issue_pv(g);
    }
    if (officer_kv) pump_v(g);          // P V(g-1) and earlier are known complete
    if (officer_b) pump_b();
    if (++t == p.n_kt) {
      // ---------------------------------------------------------------- item done
      wait_or_flag(&bar.pv_done, g & 1, abort_flag);
      fold();
      if (row_ok && !*abort_flag) {
        const float inv = 1.f / l;
        T* orow = static_cast<T*>(p.o) + ((((int64_t)b * p.N + n) * p.L + i) * p.H + h) * p.D;
#pragma unroll
        for (int d8 = 0; d8 < DP / 8; ++d8) {
          if (d8 * 8 < p.D) {
            uint4 v;
            v.x = Pack2<T>::pack(acc[d8 * 8] * inv, acc[d8 * 8 + 1] * inv);
            v.y = Pack2<T>::pack(acc[d8 * 8 + 2] * inv, acc[d8 * 8 + 3] * inv);
            v.z = Pack2<T>::pack(acc[d8 * 8 + 4] * inv, acc[d8 * 8 + 5] * inv);
            v.w = Pack2<T>::pack(acc[d8 * 8 + 6] * inv, acc[d8 * 8 + 7] * inv);
            *reinterpret_cast<uint4*>(orow + d8 * 8) = v;
          }
        }
        // a row whose keys are all masked keeps m = -FLT_MAX: its log-sum-exp is stored as -FLT_MAX, the value the
        // backward kernels recognise
        p.lse[(((int64_t)b * p.N + n) * p.H + h) * p.L + i] = m <= -1e38f ? -FLT_MAX : (m + lg2f(l)) * kLn2;
      }
      t = 0;
      ++item_local;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_s) *reinterpret_cast<volatile int*>(p.status) = 1;
  if (warp == 0) tmem_dealloc(tmem_base_s, 512);
}

template <int DP, typename T, typename TB>
int launch_fwd(const mf_evo_fwd_args& a, cudaStream_t st) {
  using C = Cfg<DP>;
  CUtensorMap mq, mk, mv, mb;
  int r;
  if ((r = make_qkv_map(&mq, a.q, a.dtype, a.B, a.N, a.L, a.H, a.D, a.q_strides, DP, kQT))) return r;
  if ((r = make_qkv_map(&mk, a.k, a.dtype, a.B, a.N, a.L, a.H, a.D, a.k_strides, DP, kKT))) return r;
  if ((r = make_qkv_map(&mv, a.v, a.dtype, a.B, a.N, a.L, a.H, a.D, a.v_strides, DP, kKT))) return r;
  FwdP p{};
  p.B = a.B; p.N = a.N; p.L = a.L; p.H = a.H; p.D = a.D;
  p.n_qt = (a.L + kQT - 1) / kQT; p.n_kt = (a.L + kKT - 1) / kKT;
  p.n_items = a.B * a.N * a.H * p.n_qt;
  p.lpad = p.n_kt * kKT;
  p.c1 = kLog2e / sqrtf((float)a.D);
  p.ab_fmt = a.dtype == MF_BF16 ? 1u : 0u;
  p.bias = a.bias; for (int i = 0; i < 4; ++i) p.bs[i] = a.bias_strides[i];
  const size_t bes = sizeof(TB);
  p.bias_fast = a.bias_strides[3] == 1 && (reinterpret_cast<uintptr_t>(a.bias) & 15) == 0 &&
                (a.bias_strides[0] * bes) % 16 == 0 && (a.bias_strides[1] * bes) % 16 == 0 && (a.bias_strides[2] * bes) % 16 == 0;
  p.mask = a.mask; for (int i = 0; i < 3; ++i) p.ms[i] = a.mask_strides[i];
  p.mask_dtype = a.mask_dtype;
  p.o = a.o; p.lse = a.lse;
  p.status = status_word();
  MF_REQUIRE(p.status, MF_ERR_CUDA, "could not allocate the device status word");
  MF_REQUIRE(tc_async_status() == 0, MF_ERR_CUDA, "an earlier tensor-core kernel gave up on a bounded wait; results are invalid");

  // bias through TMA: 16-bit dtype, unit inner stride, 16-byte aligned rows, and room in shared memory (DP = 32)
  const bool btma = DP == 32 && bes == 2 && p.bias_fast;
  mb = mq;
  if (btma) {
    p.bias_b_mul = a.bias_strides[0] == 0 ? 0 : 1;
    const int64_t dims[4] = {a.L, a.L, a.H, p.bias_b_mul ? a.B : 1};
    const int64_t str[4] = {1, a.bias_strides[2], a.bias_strides[1], a.bias_strides[0]};
    const int box[4] = {kBCW, 128, 1, 1};
    if ((r = make_tiled_map(&mb, a.bias, a.bias_dtype, 4, dims, str, box, kBCW * 2))) return r;
  }
  int grid = sm_count();
  const int pairs = (p.n_items + 1) / 2;
  if (grid > pairs) grid = pairs;
  p.items_per_stream = (p.n_items + 2 * grid - 1) / (2 * grid);
  const size_t smem = 1024 + 2 * (size_t)C::STREAM_BYTES(btma) + 2 * sizeof(float) * p.lpad;
  if (btma) {
    auto kern = evo_fwd_tc_kernel<DP, T, TB, true>;
    MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, st>>>(mq, mk, mv, mb, p);
  } else {
    auto kern = evo_fwd_tc_kernel<DP, T, TB, false>;
    MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, st>>>(mq, mk, mv, mb, p);
  }
  MF_LAUNCHED("evo_fwd_tc_kernel");
  return MF_OK;
}

}  // namespace

#define MF_DISPATCH_BIAS(dt, TB, ...)                                         \
  switch (dt) {                                                               \
    case MF_F32: { using TB = float; __VA_ARGS__; } break;                    \
    case MF_BF16: { using TB = __nv_bfloat16; __VA_ARGS__; } break;           \
    case MF_F16: { using TB = __half; __VA_ARGS__; } break;                   \
    default: return fail(MF_ERR_BAD_ARG, "unknown bias dtype %d", (int)(dt)); \
  }

int evo_fwd_tc(const mf_evo_fwd_args& a, cudaStream_t st) {
  int r = MF_OK;
  if (a.dtype == MF_BF16) {
    MF_DISPATCH_BIAS(a.bias_dtype, TB, {
      r = a.D <= 32 ? launch_fwd<32, __nv_bfloat16, TB>(a, st) : launch_fwd<64, __nv_bfloat16, TB>(a, st);
    });
  } else {
    MF_DISPATCH_BIAS(a.bias_dtype, TB, {
      r = a.D <= 32 ? launch_fwd<32, __half, TB>(a, st) : launch_fwd<64, __half, TB>(a, st);
    });
  }
  return r;
}

}  // namespace mf
