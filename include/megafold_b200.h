/*
 * megafold_b200 -- C ABI of the B200 (sm_100a) fused Pairformer operators.
 *
 * Every entry point takes plain device pointers, sizes and strides; no C++ or
 * torch types cross this boundary and no exception leaves the library.  All
 * buffers (inputs, outputs, saved statistics, workspaces) are owned by the
 * caller.  Work is enqueued on the CUDA stream passed as `stream` (a
 * cudaStream_t cast to void*; NULL = legacy default stream) and the call
 * returns without synchronising.
 *
 * Return value: MF_OK (0) or a negative mf_status code;
 * mf_last_error_string() gives the reason for the calling thread's last
 * failure.
 *
 * The citations name the interface of the MegaFold reference project that each
 * entry point stands in for (path:line inside that project).
 */
#ifndef MEGAFOLD_B200_H_
#define MEGAFOLD_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MF_ABI_VERSION 2

#if defined(__GNUC__)
#define MF_API __attribute__((visibility("default")))
#else
#define MF_API
#endif

typedef enum mf_status {
  MF_OK = 0,
  MF_ERR_BAD_ARG = -1,       /* null pointer, non-positive size, unknown dtype          */
  MF_ERR_UNSUPPORTED = -2,   /* shape / dtype / stride outside what the kernels cover  */
  MF_ERR_WORKSPACE = -3,     /* workspace missing or smaller than *_workspace_bytes()   */
  MF_ERR_CUDA = -4,          /* a CUDA runtime / driver call or a launch failed        */
  MF_ERR_ARCH = -5,          /* device is not sm_100                                    */
  MF_ERR_ALIGNMENT = -6      /* pointer or stride not aligned as the entry point needs */
} mf_status;

typedef enum mf_dtype {
  MF_F32 = 0,
  MF_BF16 = 1,
  MF_F16 = 2,
  MF_U8 = 3                  /* bool / uint8: only for res_mask (keep-mask)             */
} mf_dtype;

/* flags */
#define MF_FLAG_FORCE_SIMT 1u   /* use the fp32 CUDA-core kernels even where a tensor-core path exists */

/* ------------------------------------------------------------------------------------------
 * Pair-biased, key-masked attention ("Evoformer attention").
 *
 *   O[b,n,i,h,:] = sum_j softmax_j( D^-1/2 q[b,n,i,h,:].k[b,n,j,h,:] + bias[b,0,h,i,j] (+) mask[b,n,j] ) v[b,n,j,h,:]
 *
 * q,k,v: logical shape [B,N,L,H,D] with arbitrary element strides (s_b,s_n,s_l,s_h,s_d).
 * mask : [B,N,1,1,L]; MF_U8 = keep-mask (0 => the logit is replaced by -FLT_MAX, so the key gets
 *        probability exactly 0 unless every key of the row is masked, in which case the row is
 *        uniform); a floating dtype = values added to the logits.
 * bias : [B,1,H,L,L] with element strides (s_b,s_h,s_i,s_j).
 * o    : contiguous [B,N,L,H,D], same dtype as q.
 * lse  : contiguous fp32 [B,N,H,L], natural-log sum-exp of the logits of each query (saved for backward).
 *
 * Replaces EvoformerAttention.forward, megafold/model/FusedEvoAttention/evoattention.py:690-779
 * (kernel _attn_fwd :123-261).
 * ------------------------------------------------------------------------------------------ */
typedef struct mf_evo_fwd_args {
  int32_t B, N, L, H, D;
  int32_t dtype;            /* q,k,v,o */
  int32_t bias_dtype;
  int32_t mask_dtype;
  uint32_t flags;
  const void* q; const void* k; const void* v;
  int64_t q_strides[5], k_strides[5], v_strides[5];
  const void* mask; int64_t mask_strides[3];     /* b, n, l */
  const void* bias; int64_t bias_strides[4];     /* b, h, i, j */
  void* o;
  float* lse;
} mf_evo_fwd_args;

MF_API int mf_evo_fwd(const mf_evo_fwd_args* args, void* stream);

/*
 * Backward of the above.  d_o, o: contiguous [B,N,L,H,D].  dq,dk,dv: contiguous [B,N,L,H,D] in
 * `dtype`.  d_bias: contiguous [B,1,H,L,L] in `dbias_dtype` (MF_F32 or `dtype`), the sum of dS over
 * the N rows; it is fully overwritten (no need to zero it).  d_bias is summed in a fixed order on every
 * path and is bit-reproducible run to run; so are dk and dv.  dq is bit-reproducible except where the
 * tensor-core path spreads one row's key tiles over several CTAs or streams dq through memory (N*B*H below
 * the SM count, or more than six query tiles of 128 - two with a head size above 32): those partial sums meet in
 * fp32 atomic adds whose order varies.
 * workspace: at least mf_evo_bwd_workspace_bytes() bytes, 256-byte aligned.
 *
 * Replaces EvoformerAttention.backward, evoattention.py:783-903 (kernels _attn_bwd_preprocess
 * :273-301, _attn_bwd_dk_dv :515-686, _attn_bwd_dq :326-490).
 */
typedef struct mf_evo_bwd_args {
  int32_t B, N, L, H, D;
  int32_t dtype;
  int32_t bias_dtype;
  int32_t mask_dtype;
  int32_t dbias_dtype;
  uint32_t flags;
  const void* q; const void* k; const void* v;
  int64_t q_strides[5], k_strides[5], v_strides[5];
  const void* mask; int64_t mask_strides[3];
  const void* bias; int64_t bias_strides[4];
  const void* o; const void* d_o; const float* lse;
  void* dq; void* dk; void* dv;
  void* d_bias;
  void* workspace; size_t workspace_bytes;
  /* Optional cudaEvent_t (NULL = none), recorded on `stream` as soon as d_bias is final.  The tensor-core path
   * computes d_bias first, so a caller that shards the rows over GPUs can all-reduce d_bias on another stream
   * while dq / dk / dv are still being computed; on the CUDA-core path the event is recorded at the end. */
  void* dbias_ready_event;
} mf_evo_bwd_args;

MF_API size_t mf_evo_bwd_workspace_bytes(const mf_evo_bwd_args* args);
MF_API int mf_evo_bwd(const mf_evo_bwd_args* args, void* stream);

/*
 * mf_evo_bwd without a workspace and without any allocation.  (No counterpart in the reference; added for
 * hosts that cannot allocate.)
 *
 * Who needs it: a process that handed the whole of the GPU's memory to its own pool at start-up (so that a
 * cudaMalloc would fail), or one that may not run into the device-wide synchronisation that cudaMalloc and
 * cudaFree imply, has no way to provide the scratch buffer mf_evo_bwd asks for.  This variant keeps its
 * scratch (one float per query row, i.e. B*N*H*L floats) in an array that is part of the library image:
 * 4 MiB, held by every GPU that loads the library until the process exits.  It never calls cudaMalloc,
 * cudaFree or any allocating library routine, and it ignores args->workspace / workspace_bytes.
 *
 *  - Limit: B*N*H*L <= mf_evo_bwd_noalloc_max_rows() (1,048,576); larger problems get MF_ERR_UNSUPPORTED and
 *    must use mf_evo_bwd.
 *  - It always runs the fp32 CUDA-core kernels (the tensor-core path needs more scratch), so its results
 *    equal those of mf_evo_bwd called with MF_FLAG_FORCE_SIMT.
 *  - The first call on a device looks up the device address of the built-in array (with that device
 *    current); make that first call before any stream capture is begun.
 *  - All calls share the one array.  Its previous contents do not matter (the kernels overwrite every entry
 *    they read), but two calls whose kernels overlap on the GPU - different streams, or different host
 *    threads - race on it: serialise them.
 */
MF_API int mf_evo_bwd_noalloc(const mf_evo_bwd_args* args, void* stream);
MF_API size_t mf_evo_bwd_noalloc_max_rows(void);

/* ------------------------------------------------------------------------------------------
 * LayernormLinear:  y[M,N] = LayerNorm_K(x[M,K]; ln_w, ln_b, eps) @ w[K,N] (+ b[N])
 *
 * x,y,w,b,ln_w,ln_b share `dtype`; x,y,w contiguous row-major.  ln_b and b may be NULL.
 * mean, rstd: fp32 [M], written by forward and read by backward.
 *
 * Replaces layernorm_linear_forward, megafold/model/FusedLayernormLinear/fused_layernorm_linear.py:351-405
 * (kernels :110-140, :148-218) as called from LayernormLinearFunction.forward :477-486.
 * ------------------------------------------------------------------------------------------ */
typedef struct mf_lnl_fwd_args {
  int64_t M; int32_t K, N;
  int32_t dtype;
  uint32_t flags;
  float eps;
  const void* x; const void* ln_w; const void* ln_b; const void* w; const void* b;
  void* y; float* mean; float* rstd;
} mf_lnl_fwd_args;

MF_API int mf_lnl_fwd(const mf_lnl_fwd_args* args, void* stream);

/*
 * Backward.  dy [M,N], dx [M,K] in `dtype`; dw [K,N], d_ln_w [K], d_ln_b [K] (NULL if no LN bias),
 * db [N] (NULL if no linear bias) are fp32 and fully overwritten.
 * Replaces layernorm_linear_backward, fused_layernorm_linear.py:408-474 (kernels :227-308, :312-348,
 * and the torch reduction :465-467).
 */
typedef struct mf_lnl_bwd_args {
  int64_t M; int32_t K, N;
  int32_t dtype;
  uint32_t flags;
  const void* x; const void* ln_w; const void* ln_b; const void* w; const void* dy;
  const float* mean; const float* rstd;
  void* dx; float* dw; float* db; float* d_ln_w; float* d_ln_b;
  void* workspace; size_t workspace_bytes;
} mf_lnl_bwd_args;

MF_API size_t mf_lnl_bwd_workspace_bytes(const mf_lnl_bwd_args* args);
MF_API int mf_lnl_bwd(const mf_lnl_bwd_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * SwiGLU:  y[M,I] = silu(x[M, I:2I]) * x[M, 0:I]   (gate = right half)
 * Replaces swiglu_forward / swiglu_backward, megafold/model/FusedTransition/fused_transition.py:55-93
 * (kernels :12-26, :30-52).  Backward writes dx[M,2I] to its own buffer (the reference overwrites x).
 * ------------------------------------------------------------------------------------------ */
MF_API int mf_swiglu_fwd(const void* x, void* y, int64_t M, int32_t inner, int32_t dtype, void* stream);
MF_API int mf_swiglu_bwd(const void* x, const void* dy, void* dx, int64_t M, int32_t inner, int32_t dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * Transition:  y[M,dim] = ( SwiGLU( LayerNorm(x) @ w1[dim,2*inner] ) ) @ w2[dim,inner]^T
 *
 * ln_w == NULL means "no LayerNorm" (the include_ln=False variant).  w2 is laid out like
 * nn.Linear.weight.  mean,rstd fp32 [M] are written by forward (unused without LN).
 * The hidden activations are not kept: backward recomputes them from x.
 *
 * Replaces FusedTransition.forward, fused_transition.py:118-151 (LayernormLinear -> FusedSwiGLU ->
 * nn.Linear) and the autograd chain behind it.
 * ------------------------------------------------------------------------------------------ */
typedef struct mf_transition_fwd_args {
  int64_t M; int32_t dim, inner;
  int32_t dtype;
  uint32_t flags;
  float eps;
  const void* x; const void* ln_w; const void* ln_b; const void* w1; const void* w2;
  void* y; float* mean; float* rstd;
  void* workspace; size_t workspace_bytes;
} mf_transition_fwd_args;

MF_API size_t mf_transition_fwd_workspace_bytes(const mf_transition_fwd_args* args);
MF_API int mf_transition_fwd(const mf_transition_fwd_args* args, void* stream);

typedef struct mf_transition_bwd_args {
  int64_t M; int32_t dim, inner;
  int32_t dtype;
  uint32_t flags;
  const void* x; const void* ln_w; const void* ln_b; const void* w1; const void* w2; const void* dy;
  const float* mean; const float* rstd;
  void* dx; float* dw1; float* dw2; float* d_ln_w; float* d_ln_b;   /* fp32, fully overwritten */
  void* workspace; size_t workspace_bytes;
} mf_transition_bwd_args;

/* The scratch size is that of the path these very arguments take (it depends on dtype, sizes and pointer alignment):
 * ask with the structure filled in as it will be passed to mf_transition_bwd. */
MF_API size_t mf_transition_bwd_workspace_bytes(const mf_transition_bwd_args* args);
MF_API int mf_transition_bwd(const mf_transition_bwd_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * Library queries.
 * ------------------------------------------------------------------------------------------ */
MF_API const char* mf_last_error_string(void);   /* thread-local, never NULL */
MF_API int mf_version(void);                     /* MF_ABI_VERSION the library was built with */
/* Number of kernels this library has launched since it was loaded (all threads). */
MF_API uint64_t mf_kernel_launch_count(void);
/* Name of the kernel family the last successful call on this thread used: "tcgen05" or "simt". */
MF_API const char* mf_last_path(void);
/* Non-zero once a kernel on the current device gave up on one of its bounded waits (its outputs are
 * then invalid).  Readable without a device synchronisation; sticky until the process ends. */
MF_API int mf_async_status(void);
/* Self-test of that mechanism (no counterpart in the reference): launches one small kernel whose only wait, on a
 * barrier that nobody completes, runs into its cap after a few milliseconds; the kernel then leaves through the same
 * exit path as the attention kernels, so afterwards mf_async_status() is non-zero and the tensor-core entry points of
 * this process refuse to launch.  Nothing faults and the context stays usable.  Meant for a throw-away process. */
MF_API int mf_selftest_bounded_wait(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MEGAFOLD_B200_H_ */
