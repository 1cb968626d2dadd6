// Pieces shared by the tensor-core attention kernels (forward, backward, bias gradient):
// bounded waits with a CTA-wide abort flag, 16-bit packing, base-2 exponentials, tensor-map
// construction and the host-visible status word.
#pragma once

#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "tc.cuh"

namespace mf {
namespace tcx {
using namespace tc;

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Waits for a phase; on expiry raises the CTA's abort flag and returns (the caller carries on to its
// next group barrier, where everybody sees the flag and leaves the loop).
__device__ __forceinline__ void wait_or_flag(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  // cheap non-blocking probe first: try_wait costs ~270 cycles even when the phase is already complete (measured with
  // clock stamps in the MMA issuer threads), and that is the common case for the threads that issue MMAs and TMA copies
  if (mbar_test(bar, parity)) return;
  if (*abort_flag) return;            // the CTA is already draining: nobody blocks any more
  for (uint32_t i = 0; i < kWaitCap; ++i) {
    if (mbar_try_wait(bar, parity)) return;
    if ((i & 63u) == 63u && *abort_flag) return;
  }
  *abort_flag = 1;
}
__device__ __forceinline__ void named_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// Group barrier that also ORs a flag over the group: every thread gets the same answer, so the whole
// group takes the same exit decision.
__device__ __forceinline__ bool named_sync_or(int id, int threads, int flag) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %3, 0;\n\t"
      "bar.red.or.pred q, %1, %2, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(out)
      : "r"(id), "r"(threads), "r"(flag)
      : "memory");
  return out != 0;
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

// ---- packed fp32 pairs (one issue slot for two lanes of work) and the three-input maximum ------------
__device__ __forceinline__ uint64_t pack_f2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float2 unpack_f2(uint64_t r) {
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(r));
  return d;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(pack_f2(a.x, a.y)), "l"(pack_f2(b.x, b.y)), "l"(pack_f2(c.x, c.y)));
  return unpack_f2(d);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(pack_f2(a.x, a.y)), "l"(pack_f2(b.x, b.y)));
  return unpack_f2(d);
}
__device__ __forceinline__ float2 sub2(float2 a, float2 b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(pack_f2(a.x, a.y)), "l"(pack_f2(b.x, b.y)));
  return unpack_f2(d);
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(pack_f2(a.x, a.y)), "l"(pack_f2(b.x, b.y)));
  return unpack_f2(d);
}
__device__ __forceinline__ float max3f(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// One 32-bit column of this thread's TMEM lane
__device__ __forceinline__ uint32_t tmem_ld1(uint32_t taddr) {
  uint32_t r;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
  return r;
}
__device__ __forceinline__ void tmem_st1(uint32_t taddr, uint32_t v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(v) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
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
template <> struct Pack2<float> {   // only so that code templated on the bias type compiles; never packed
  static __device__ __forceinline__ float2 unpack(uint32_t u) { return make_float2(__uint_as_float(u), 0.f); }
};

// 4-D tiled TMA load
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// ---- the pair bias through the tensor core ----------------------------------------------------------
// logits * sqrt(D) = Q K^T + sqrt(D) * bias.  The second term is a matrix product too: bias tile (A operand, 16 columns
// at a time) times alpha * I_16 (B operand) lands in 16 columns of the score accumulator, so no thread ever touches a
// bias value.  alpha = sqrt(D) is split into one or two terms of the bias dtype (hi + lo), each with its own B tile.
// Layout of one B tile: K-major [16 rows x 32 columns], 64-byte rows, 64B swizzle (1 KB, 1024-byte aligned); only the
// first 16 columns (one MMA K step) are used.
template <typename TB>
__device__ __forceinline__ void write_alpha_identity(uint8_t* tile, float alpha, int tid, int nthreads) {
  for (int e = tid; e < 16 * 32; e += nthreads) {
    const int n = e >> 5, k = e & 31;
    *reinterpret_cast<TB*>(tile + swz_offset(n, k >> 3, 64) + (k & 7) * 2) = from_f<TB>(k == n ? alpha : 0.f);
  }
}

// ---- rank-one terms of the scores through the tensor core --------------------------------------------------
// x[j,i] = c1 * (K Q^T + sqrt(D) bias^T)[j,i] + mask2_j - lse2_i  and  dP[j,i] - delta_i  both contain terms that depend on
// the key or on the query alone.  Read per logit from shared memory they cost two wavefronts of the shared-memory
// pipe per logit-warp - as much as the exponential costs on its pipe.  Instead they ride on one extra K = 16 MMA step:
//
//   XK[j, 0:3] = split3(mask_j * sqrt(D))     XK[j, 3:6] = 1                          (per (b, n), key tile)
//   XQ[i, 0:3] = 1                            XQ[i, 3:6] = split3(-lse_i * sqrt(D))   XQ[i, 6:9] = split3(-delta_i)
//   XC[j, 6:9] = 1                            (constant)
//
//   S''^T += XK XQ^T   (mask + lse terms; c1 * sqrt(D) = log2 e brings them into the base-2 domain)
//   dP^T  += XC XQ^T   (-delta)
//
// split3 writes an fp32 value as the sum of three bf16 numbers (24 significant bits); the products are exact and the
// accumulation is fp32.  Masked keys, keys and queries beyond L and fully masked query rows get -1e30 (finite: no NaN can
// arise from 0 * inf), which the exponential turns into exactly 0.  Tiles are bf16 [128 rows x 16 columns], 32-byte rows,
// 32B swizzle (4 KB), written here in the shared-memory layout so that a plain bulk copy fetches them.
constexpr int kXTileB = 128 * 32;
constexpr float kMinusBig = -1e30f;

__device__ __forceinline__ void split3(float v, __nv_bfloat16 (&o)[3]) {
  o[0] = __float2bfloat16_rn(v);
  const float r1 = v - __bfloat162float(o[0]);
  o[1] = __float2bfloat16_rn(r1);
  o[2] = __float2bfloat16_rn(r1 - __bfloat162float(o[1]));
}
__device__ __forceinline__ uint32_t pack_bf(__nv_bfloat16 a, __nv_bfloat16 b) {
  return (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
}

// XC: ones in columns 6..8 of every row
__device__ __forceinline__ void write_xc_tile(uint8_t* tile, int tid, int nthreads) {
  const uint32_t one = 0x3f80u;      // bf16 1.0
  for (int r = tid; r < 128; r += nthreads) {
    *reinterpret_cast<uint4*>(tile + swz_offset(r, 0, 32)) = make_uint4(0u, 0u, 0u, one | (one << 16));
    *reinterpret_cast<uint4*>(tile + swz_offset(r, 1, 32)) = make_uint4(one, 0u, 0u, 0u);
  }
}

// XO: ones in columns 0..2 of every row (the forward kernel's partner of the mask columns of XK)
__device__ __forceinline__ void write_xo_tile(uint8_t* tile, int tid, int nthreads) {
  const uint32_t one = 0x3f80u;      // bf16 1.0
  for (int r = tid; r < 128; r += nthreads) {
    *reinterpret_cast<uint4*>(tile + swz_offset(r, 0, 32)) = make_uint4(one | (one << 16), one, 0u, 0u);
    *reinterpret_cast<uint4*>(tile + swz_offset(r, 1, 32)) = make_uint4(0u, 0u, 0u, 0u);
  }
}

// ---- phase trace (debug builds only: -DMF_TRACE) -------------------------------------------------------
// One elected thread per role of CTA 0 records (tag, clock64) pairs into a global buffer handed in through
// mf_debug_set_trace(); role `r` owns entries [r * kTraceLen, (r + 1) * kTraceLen).  Compiled out otherwise.
constexpr int kTraceLen = 512;
#ifdef MF_TRACE
extern long long* g_trace;
struct Tracer {
  long long* buf; int n;
  __device__ __forceinline__ Tracer(long long* base, int role, bool on) : buf(on && base ? base + role * kTraceLen : nullptr), n(0) {}
  __device__ __forceinline__ void operator()(int tag) {
    if (buf && n + 2 <= kTraceLen) { buf[n] = tag; buf[n + 1] = clock64(); n += 2; }
  }
};
#define MF_TRACE_DECL(name, role, on) Tracer name(g_trace_dev, (role), (on))
#define MF_TRACE_PARAM , long long* g_trace_dev
#define MF_TRACE_ARG , ::mf::tcx::g_trace
#else
#define MF_TRACE_DECL(name, role, on) auto name = [](int) {}
#define MF_TRACE_PARAM
#define MF_TRACE_ARG
#endif

// ---- host side ------------------------------------------------------------------------------------
// sqrt(D) as a sum of values representable in the 16-bit type `dt`; returns the number of terms (1 when the first
// one is within 2.5e-4 relative, which is below the rounding of the bias values themselves)
inline int split_alpha(int D, int dt, float (&alpha)[2]) {
  const float a = sqrtf((float)D);
  const float hi = dt == MF_BF16 ? __bfloat162float(__float2bfloat16_rn(a)) : __half2float(__float2half_rn(a));
  const float rest = a - hi;
  const float lo = dt == MF_BF16 ? __bfloat162float(__float2bfloat16_rn(rest)) : __half2float(__float2half_rn(rest));
  alpha[0] = hi; alpha[1] = lo;
  return fabsf(rest) > 2.5e-4f * a ? 2 : 1;
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess) f = nullptr;
    return reinterpret_cast<EncodeFn>(f);
  }();
  return fn;
}

inline CUtensorMapDataType tm_dtype(int dt) {
  return dt == MF_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : dt == MF_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                         : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
}
inline CUtensorMapSwizzle tm_swizzle(int row_bytes) {
  return row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
       : row_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
}

// Generic tiled map: `rank` dims, innermost first; strides in ELEMENTS for dims 1..rank-1 (dim 0 is unit
// stride).  Dims of size 1 get a dummy 16-byte stride.  The box's innermost extent times the element size
// must equal the swizzle width (`row_bytes`).
inline int make_tiled_map(CUtensorMap* m, const void* ptr, int dtype, int rank, const int64_t* dims, const int64_t* strides,
                          const int* box, int row_bytes) {
  EncodeFn enc = encode_fn();
  MF_REQUIRE(enc, MF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const int64_t es = (int64_t)dtype_size(dtype);
  cuuint64_t gdim[5], gstr[4];
  cuuint32_t bx[5], estr[5];
  for (int i = 0; i < rank; ++i) { gdim[i] = (cuuint64_t)dims[i]; bx[i] = (cuuint32_t)box[i]; estr[i] = 1; }
  for (int i = 1; i < rank; ++i) gstr[i - 1] = (cuuint64_t)((dims[i] == 1 || strides[i] <= 0) ? 16 : strides[i] * es);
  CUresult r = enc(m, tm_dtype(dtype), (cuuint32_t)rank, const_cast<void*>(ptr), gdim, gstr, bx, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, tm_swizzle(row_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MF_REQUIRE(r == CUDA_SUCCESS, MF_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return MF_OK;
}

// 5-D map over a [B, N, L, H, D] operand (element strides s = {b, n, l, h, d}); box = DP x 1 x rows x 1 x 1
inline int make_qkv_map(CUtensorMap* m, const void* ptr, int dtype, int B, int N, int L, int H, int D, const int64_t* s,
                        int DP, int rows) {
  const int64_t dims[5] = {D, H, L, N, B};
  const int64_t str[5] = {1, s[3], s[2], s[1], s[0]};
  const int box[5] = {DP, 1, rows, 1, 1};
  return make_tiled_map(m, ptr, dtype, 5, dims, str, box, DP * 2);
}

inline bool qkv_strides_ok(const void* p, const int64_t* s, int B, int N, int L, int H) {
  if ((reinterpret_cast<uintptr_t>(p) & 15) != 0 || s[4] != 1) return false;
  const int sizes[4] = {B, N, L, H};
  for (int i = 0; i < 4; ++i)
    if (sizes[i] > 1 && (s[i] <= 0 || (s[i] % 8) != 0)) return false;
  return true;
}

// Status word of the calling thread's device: pinned host memory mapped into the device, so that a
// kernel that gave up on a bounded wait can say so and the host can read it without a device sync.
struct StatusWord { int* host = nullptr; int* dev = nullptr; };
StatusWord* status_slot();
inline int* status_word() {
  StatusWord* w = status_slot();
  return w ? w->dev : nullptr;
}
int sm_count();

}  // namespace tcx
}  // namespace mf
