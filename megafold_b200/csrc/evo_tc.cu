// Pair-biased masked attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), sm_100a.
//
// Forward.  A persistent CTA (one per SM) runs TWO independent streams; a stream walks work items
// (b, n, h, 128-query tile) and, for each, the key tiles of 128:
//
//   warp 0 (one lane)  TMA producer: Q tile and K/V tiles of both streams into shared-memory rings
//   warp 1 (one lane)  tcgen05.mma issuer: S = Q K^T into TMEM, later O_tile = P V into TMEM
//   warps 4-7 / 8-11   softmax group of stream 0 / 1, one thread per query row: reads its S row from
//                      TMEM, adds bias and mask, exponentiates in base 2 with a running maximum, writes
//                      bf16 P back to TMEM (the A operand of the second MMA), and keeps the output row
//                      and the running sum in registers (O_tile is read back from TMEM once per key tile,
//                      which is cheap because the head size is small).
//
// While one stream's softmax group is busy, the tensor pipe works for the other stream.  No L x L
// tensor ever reaches global memory: only O and the log-sum-exp per query row are written.
//
// Operand layouts: Q, K, V tiles are [128 rows x DP] with DP = 32 (64-byte rows, 64B swizzle) or 64
// (128-byte rows, 128B swizzle), fetched straight out of the strided [B, N, L, H, D] tensors by 5-D
// tensor maps (box DP x 1 x 128 x 1 x 1); head sizes below DP are zero-filled by TMA.  Q and K are
// K-major operands, V is an MN-major B operand, P is an A operand in TMEM.
//
// Every wait is bounded; on expiry the CTA raises a flag, all roles drain, TMEM is freed and the
// host reports MF_ERR_CUDA from the status word.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "tc.cuh"

namespace mf {
namespace {
using namespace tc;

#ifdef MF_TIMELINE
long long* g_timeline = nullptr;
#endif
constexpr int kQT = 128;            // query rows per tile = TMEM lanes
constexpr int kKT = 128;            // keys per tile
constexpr int kFwdThreads = 384;    // warpgroup 0: producer warp, MMA warp, 2 idle; warpgroups 1, 2: softmax
constexpr float kLog2e = 1.4426950408889634f;

template <int DP> struct Cfg {
  static constexpr int ROWB = DP * 2;              // bytes per shared-memory row
  static constexpr int TILEB = 128 * ROWB;         // bytes per 128-row tile
  static constexpr int ST = DP == 32 ? 4 : 2;      // K/V ring stages per stream
  static constexpr Swizzle SW = DP == 32 ? kSw64 : kSw128;
  static constexpr int SBO = 8 * ROWB;             // 8-row group stride
};

struct FwdP {
  int B, N, L, H, D;
  int n_qt, n_kt, n_items, lpad;
  float c1;               // D^-1/2 * log2(e)
  uint32_t ab_fmt;        // 1 = bf16, 0 = f16
  const void* bias; int64_t bs[4]; int bias_fast;
  const void* mask; int64_t ms[3]; int mask_dtype;
  void* o; float* lse; int* status;
  long long* timeline;   // optional per-phase clock samples of one softmax thread (debug builds only)
};

struct StreamBars {
  uint64_t q_full[2], q_empty[2], kv_full[4], kv_empty[4], s_ready, p_ready, o_ready;
};

__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kWaitCap; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
// Phase timestamps of thread 0 of stream 0 in CTA 0; compiled in only with -DMF_TIMELINE.
#ifdef MF_TIMELINE
#define MF_TL(tag) do { if (p.timeline && blockIdx.x == 0 && s == 0 && wg_tid == 0 && tl_n < 250) { p.timeline[2 * tl_n] = (tag); p.timeline[2 * tl_n + 1] = clock64(); ++tl_n; } } while (0)
#else
#define MF_TL(tag) do { } while (0)
#endif
__device__ __forceinline__ void named_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2f(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T> struct Pack2;
template <> struct Pack2<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
  }
};
template <> struct Pack2<__half> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
};

// 32 consecutive bias values of one row as fp32; `p` is 16-byte aligned and fully in bounds.
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
// guarded scalar variant: columns >= L read as 0 (their mask term is -inf anyway)
template <typename TB>
__device__ __forceinline__ void load_bias32_slow(const TB* row, int64_t sj, int j0, int L, float (&out)[32]) {
#pragma unroll
  for (int i = 0; i < 32; ++i) out[i] = (j0 + i < L) ? to_f(row[(int64_t)(j0 + i) * sj]) : 0.f;
}

// --------------------------------------------------------------------------------------------------
// forward kernel
// --------------------------------------------------------------------------------------------------
template <int DP, typename T, typename TB>
__global__ void __launch_bounds__(kFwdThreads, 1)
evo_fwd_tc_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                  const __grid_constant__ CUtensorMap mv, const FwdP p) {
  using C = Cfg<DP>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  // per stream: Q[2], {K,V}[ST], then the mask rows of both streams
  constexpr int kStreamBytes = 2 * C::TILEB + C::ST * 2 * C::TILEB;
  float* mask2_all = reinterpret_cast<float*>(smem + 2 * kStreamBytes);

  __shared__ StreamBars bars[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    abort_s = 0;
    for (int s = 0; s < 2; ++s) {
      for (int i = 0; i < 2; ++i) { mbar_init(&bars[s].q_full[i], 1); mbar_init(&bars[s].q_empty[i], 1); }
      for (int i = 0; i < 4; ++i) { mbar_init(&bars[s].kv_full[i], 1); mbar_init(&bars[s].kv_empty[i], 1); }
      mbar_init(&bars[s].s_ready, 1);
      mbar_init(&bars[s].p_ready, 128);
      mbar_init(&bars[s].o_ready, 1);
    }
    mbar_fence_init();
    prefetch_tmap(&mq); prefetch_tmap(&mk); prefetch_tmap(&mv);
  }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  volatile int* abort_flag = &abort_s;
  const int stride_items = gridDim.x * 2;
  const int per_bn = p.H * p.n_qt;


  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int item[2], t[2] = {0, 0}, c[2] = {0, 0};
      uint32_t g[2] = {0, 0};
      bool q_issued[2] = {false, false};
      item[0] = blockIdx.x * 2; item[1] = blockIdx.x * 2 + 1;
      uint32_t idle = 0;
      while ((item[0] < p.n_items || item[1] < p.n_items) && !*abort_flag) {
        bool progress = false;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (item[s] >= p.n_items) continue;
          uint8_t* sb = smem + s * kStreamBytes;
          const int it = item[s];
          const int qt = it % p.n_qt, h = (it / p.n_qt) % p.H, bn = it / per_bn, n = bn % p.N, b = bn / p.N;
          if (!q_issued[s]) {
            const int qb = c[s] & 1;
            if (!mbar_test(&bars[s].q_empty[qb], ((c[s] >> 1) & 1) ^ 1)) continue;
            mbar_expect_tx(&bars[s].q_full[qb], C::TILEB);
            tma_load_5d(sb + qb * C::TILEB, &mq, &bars[s].q_full[qb], 0, h, qt * kQT, n, b);
            q_issued[s] = true; progress = true;
          } else {
            const int st = g[s] % C::ST;
            if (!mbar_test(&bars[s].kv_empty[st], ((g[s] / C::ST) & 1) ^ 1)) continue;
            uint8_t* kv = sb + 2 * C::TILEB + st * 2 * C::TILEB;
            mbar_expect_tx(&bars[s].kv_full[st], 2 * C::TILEB);
            tma_load_5d(kv, &mk, &bars[s].kv_full[st], 0, h, t[s] * kKT, n, b);
            tma_load_5d(kv + C::TILEB, &mv, &bars[s].kv_full[st], 0, h, t[s] * kKT, n, b);
            ++g[s]; progress = true;
            if (++t[s] == p.n_kt) { t[s] = 0; ++c[s]; q_issued[s] = false; item[s] += stride_items; }
          }
        }
        if (progress) idle = 0;
        else if (++idle > kWaitCap) { *abort_flag = 1; break; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int item[2], t[2] = {0, 0}, c[2] = {0, 0};
      uint32_t g[2] = {0, 0};
      bool need_s[2] = {true, true};
      item[0] = blockIdx.x * 2; item[1] = blockIdx.x * 2 + 1;
      const uint32_t id_s = idesc_f16(128, kKT, p.ab_fmt, 0, 0);
      const uint32_t id_o = idesc_f16(128, DP, p.ab_fmt, 0, 1);
      uint32_t idle = 0;
      while ((item[0] < p.n_items || item[1] < p.n_items) && !*abort_flag) {
        bool progress = false;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (item[s] >= p.n_items) continue;
          uint8_t* sb = smem + s * kStreamBytes;
          const uint32_t tS = tmem_base + s * 256, tP = tS + 128, tO = tS + 192;
          const int st = g[s] % C::ST;
          const int qb = c[s] & 1;
          uint8_t* kv = sb + 2 * C::TILEB + st * 2 * C::TILEB;
          if (need_s[s]) {
            if (t[s] == 0 && !mbar_test(&bars[s].q_full[qb], (c[s] >> 1) & 1)) continue;
            if (!mbar_test(&bars[s].kv_full[st], (g[s] / C::ST) & 1)) continue;
            tc_fence_after();
            const uint32_t qa = smem_u32(sb + qb * C::TILEB), ka = smem_u32(kv);
#pragma unroll
            for (int ks = 0; ks < DP / 16; ++ks)
              mma_ss(tS, smem_desc(qa + ks * 32, 16, C::SBO, C::SW), smem_desc(ka + ks * 32, 16, C::SBO, C::SW), id_s, ks > 0);
            tc_commit(&bars[s].s_ready);
            need_s[s] = false; progress = true;
          } else {
            if (!mbar_test(&bars[s].p_ready, g[s] & 1)) continue;
            tc_fence_after();
            const uint32_t va = smem_u32(kv + C::TILEB);
#pragma unroll
            for (int ks = 0; ks < kKT / 16; ++ks)
              mma_ts(tO, tP + ks * 8, smem_desc(va + ks * 16 * C::ROWB, 16, C::SBO, C::SW), id_o, ks > 0);
            tc_commit(&bars[s].o_ready);
            tc_commit(&bars[s].kv_empty[st]);
            ++g[s]; need_s[s] = true; progress = true;
            if (++t[s] == p.n_kt) {
              tc_commit(&bars[s].q_empty[qb]);
              t[s] = 0; ++c[s]; item[s] += stride_items;
            }
          }
        }
        if (progress) idle = 0;
        else if (++idle > kWaitCap) { *abort_flag = 1; break; }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax groups
    const int s = (warp - 4) >> 2;                 // stream
    const int wg_tid = tid - 128 - s * 128;        // 0..127
    const int r = (warp & 3) * 32 + lane;          // TMEM lane = query row inside the tile
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + s * 256 + lane_addr, tP = tS + 128, tO = tS + 192;
    float* mask2 = mask2_all + s * p.lpad;
    const TB* bias = static_cast<const TB*>(p.bias);
    uint32_t g = 0;
    bool ok = true;
    int tl_n = 0; (void)tl_n;
    for (int it = blockIdx.x * 2 + s; it < p.n_items && ok; it += stride_items) {
      const int qt = it % p.n_qt, h = (it / p.n_qt) % p.H, bn = it / per_bn, n = bn % p.N, b = bn / p.N;
      const int i = qt * kQT + r;
      const bool row_ok = i < p.L;
      const TB* brow = bias + b * p.bs[0] + h * p.bs[1] + (int64_t)(row_ok ? i : p.L - 1) * p.bs[2];
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
      MF_TL(0);

      float m = -INFINITY, l = 0.f, corr_prev = 0.f;
      float acc[DP];
#pragma unroll
      for (int d = 0; d < DP; ++d) acc[d] = 0.f;

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
      for (int t = 0; t < p.n_kt && ok; ++t, ++g) {
        // S(t) ready; the same commit also covers P(t-1) V(t-1), issued before it
        ok = __all_sync(0xffffffffu, wait_bar(&bars[s].s_ready, g & 1, abort_flag));
        MF_TL(1);
        if (!ok) break;
        tc_fence_after();
        if (t > 0) fold();
        MF_TL(2);
        const int j0 = t * kKT;
        const bool fast = p.bias_fast && (j0 + kKT <= p.L);
        // pass 1: logits in the base-2 domain, written back over S in TMEM; row maximum
        float mx = -INFINITY;
#pragma unroll
        for (int cb = 0; cb < 4; ++cb) {
          uint32_t s32[32];
          tmem_ld32(tS + cb * 32, s32);
          float bv[32];
          if (fast) load_bias32_fast<TB>(brow + j0 + cb * 32, bv);
          else load_bias32_slow<TB>(brow, p.bs[3], j0 + cb * 32, p.L, bv);
          tmem_ld_wait();
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4) {
            const float4 mk4 = *reinterpret_cast<const float4*>(mask2 + j0 + cb * 32 + q4 * 4);
            const float mk[4] = {mk4.x, mk4.y, mk4.z, mk4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int jj = q4 * 4 + e;
              const float v = fmaf(__uint_as_float(s32[jj]), p.c1, fmaf(bv[jj], kLog2e, mk[e]));
              s32[jj] = __float_as_uint(v);
              mx = fmaxf(mx, v);
            }
          }
          tmem_st32(tS + cb * 32, s32);
        }
        tmem_st_wait();
        MF_TL(3);
        const float m_new = fmaxf(m, mx);
        const float corr = ex2f(m - m_new);
        // pass 2: probabilities, row sum, P (packed 16-bit pairs) into TMEM
        float rs = 0.f;
#pragma unroll
        for (int cb = 0; cb < 2; ++cb) {
          uint32_t pk[32];
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) {
            uint32_t s32[32];
            tmem_ld32(tS + cb * 64 + hb * 32, s32);
            tmem_ld_wait();
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) {
              const float p0 = ex2f(__uint_as_float(s32[2 * jj]) - m_new), p1 = ex2f(__uint_as_float(s32[2 * jj + 1]) - m_new);
              rs += p0 + p1;
              pk[hb * 16 + jj] = Pack2<T>::pack(p0, p1);
            }
          }
          tmem_st32(tP + cb * 32, pk);
        }
        l = fmaf(l, corr, rs);
        m = m_new;
        corr_prev = corr;
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&bars[s].p_ready);
        MF_TL(5);
      }
      MF_TL(6);
      if (ok) {
        ok = __all_sync(0xffffffffu, wait_bar(&bars[s].o_ready, (g - 1) & 1, abort_flag));
        if (ok) fold();
      }
      if (!ok) break;
      MF_TL(7);
      if (row_ok) {
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
        p.lse[(((int64_t)b * p.N + n) * p.H + h) * p.L + i] = (m + lg2f(l)) * (1.f / kLog2e);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_s) *reinterpret_cast<volatile int*>(p.status) = 1;
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

// --------------------------------------------------------------------------------------------------
// host side
// --------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess) f = nullptr;
    return reinterpret_cast<EncodeFn>(f);
  }();
  return fn;
}

// 5-D map over a [B, N, L, H, D] operand (element strides s), box = DP x 1 x rows x 1 x 1
int make_map(CUtensorMap* m, const void* ptr, int dtype, int B, int N, int L, int H, int D, const int64_t* s, int DP,
             int rows) {
  EncodeFn enc = encode_fn();
  MF_REQUIRE(enc, MF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const uint64_t es = 2;
  cuuint64_t gdim[5] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)L, (cuuint64_t)N, (cuuint64_t)B};
  int64_t st[4] = {s[3], s[2], s[1], s[0]};
  const int sizes[4] = {H, L, N, B};
  cuuint64_t gstr[4];
  for (int i = 0; i < 4; ++i) gstr[i] = (cuuint64_t)((sizes[i] == 1 || st[i] == 0) ? 16 : st[i] * (int64_t)es);
  cuuint32_t box[5] = {(cuuint32_t)DP, 1, (cuuint32_t)rows, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(m, dtype == MF_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5,
                   const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   DP == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MF_REQUIRE(r == CUDA_SUCCESS, MF_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return MF_OK;
}

bool strides_ok(const void* p, const int64_t* s, int B, int N, int L, int H) {
  if ((reinterpret_cast<uintptr_t>(p) & 15) != 0 || s[4] != 1) return false;
  const int sizes[4] = {B, N, L, H};
  for (int i = 0; i < 4; ++i)
    if (sizes[i] > 1 && (s[i] <= 0 || (s[i] % 8) != 0)) return false;
  return true;
}

// Status word of the calling thread's device: pinned host memory mapped into the device, so that a
// kernel that gave up on a bounded wait can say so and the host can read it without a device sync.
struct StatusWord { int* host = nullptr; int* dev = nullptr; };
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
int* status_word() {
  StatusWord* w = status_slot();
  return w ? w->dev : nullptr;
}

int sm_count() {
  static int n[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev] > 0 ? n[dev] : 148;
}

template <int DP, typename T, typename TB>
int launch_fwd(const mf_evo_fwd_args& a, cudaStream_t st) {
  using C = Cfg<DP>;
  CUtensorMap mq, mk, mv;
  int r;
  if ((r = make_map(&mq, a.q, a.dtype, a.B, a.N, a.L, a.H, a.D, a.q_strides, DP, kQT))) return r;
  if ((r = make_map(&mk, a.k, a.dtype, a.B, a.N, a.L, a.H, a.D, a.k_strides, DP, kKT))) return r;
  if ((r = make_map(&mv, a.v, a.dtype, a.B, a.N, a.L, a.H, a.D, a.v_strides, DP, kKT))) return r;
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
#ifdef MF_TIMELINE
  p.timeline = g_timeline;
#endif
  p.status = status_word();
  MF_REQUIRE(p.status, MF_ERR_CUDA, "could not allocate the device status word");
  MF_REQUIRE(tc_async_status() == 0, MF_ERR_CUDA, "an earlier tensor-core kernel gave up on a bounded wait; results are invalid");
  const size_t smem = 1024 + 2 * (2 * C::TILEB + C::ST * 2 * C::TILEB) + 2 * sizeof(float) * p.lpad;
  auto kern = evo_fwd_tc_kernel<DP, T, TB>;
  MF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int grid = sm_count();
  const int pairs = (p.n_items + 1) / 2;
  if (grid > pairs) grid = pairs;
  kern<<<grid, kFwdThreads, smem, st>>>(mq, mk, mv, p);
  MF_LAUNCHED("evo_fwd_tc_kernel");
  return MF_OK;
}

}  // namespace

bool evo_tc_supported(int B, int N, int L, int H, int D, int dtype, const int64_t* qs, const int64_t* ks,
                      const int64_t* vs, const void* q, const void* k, const void* v) {
  if (dtype != MF_BF16 && dtype != MF_F16) return false;
  if (D % 8 != 0 || D > 64 || L > 4096) return false;
  return strides_ok(q, qs, B, N, L, H) && strides_ok(k, ks, B, N, L, H) && strides_ok(v, vs, B, N, L, H);
}

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

#ifdef MF_TIMELINE
extern "C" __attribute__((visibility("default"))) void mf_debug_set_timeline(long long* p) { g_timeline = p; }
#endif

bool evo_bwd_tc_available() { return false; }

int tc_async_status() {
  StatusWord* w = status_slot();
  return (w && w->host) ? *reinterpret_cast<volatile int*>(w->host) : 0;
}
int evo_bwd_tc(const mf_evo_bwd_args&, cudaStream_t) { return fail(MF_ERR_UNSUPPORTED, "no tensor-core backward yet"); }
size_t evo_bwd_tc_workspace(const mf_evo_bwd_args&) { return 0; }

}  // namespace mf
