/*
 * deltarule_sm100 -- C ABI of the B200 (sm_100a) delta-rule linear-attention kernels.
 *
 * Every entry point replaces one or more pure-JAX functions of LinearNexus
 * (paths below are relative to the LinearNexus source tree).  The caller owns every
 * buffer; all pointers are DEVICE pointers unless a name ends in `_host`; kernels are
 * enqueued on `stream` (a cudaStream_t passed as void*) and the call returns without
 * synchronising.  The library allocates no device memory in any entry point of this
 * header; scratch comes from the caller (`workspace`, sized by dr_workspace_bytes).
 *
 * Tensors are contiguous in one of two layouts selected by DrDesc.layout:
 *   DR_LAYOUT_BHTD : q,k [B,H,T,K]  v,o [B,H,T,V]  beta [B,H,T]  g [B,H,T] or [B,H,T,K]
 *   DR_LAYOUT_BTHD : q,k [B,T,H,K]  v,o [B,T,H,V]  beta [B,T,H]  g [B,T,H] or [B,T,H,K]
 * The recurrent state is always [B,H,K,V] float32 with S[k][v], o = S^T q.
 *
 * Return value: DR_OK (0) or a negative DrStatus; dr_strerror() names it.
 */
#ifndef DELTARULE_SM100_H_
#define DELTARULE_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum DrVariant {
  DR_DELTA = 0, /* DeltaNet: no decay, no in-op l2norm   (modules/linear_attn/delta_net.py) */
  DR_GATED = 1, /* Gated DeltaNet: scalar log-decay g    (modules/linear_attn/gated_deltanet.py) */
  DR_KDA = 2    /* KDA: per-channel log-decay g[...,K]   (modules/linear_attn/kda.py) */
} DrVariant;

typedef enum DrDtype { DR_F32 = 0, DR_BF16 = 1 } DrDtype;

typedef enum DrLayout { DR_LAYOUT_BHTD = 0, DR_LAYOUT_BTHD = 1 } DrLayout;

typedef enum DrStatus {
  DR_OK = 0,
  DR_ERR_NULL = -1,        /* a required pointer is null */
  DR_ERR_SHAPE = -2,       /* B,H,T,K,V or chunk out of the supported range */
  DR_ERR_DTYPE = -3,       /* unknown dtype tag or unsupported combination */
  DR_ERR_ALIGN = -4,       /* a pointer is not 16-byte aligned */
  DR_ERR_WORKSPACE = -5,   /* workspace too small (see dr_workspace_bytes) */
  DR_ERR_VARIANT = -6,     /* unknown variant, or g missing/present against the variant */
  DR_ERR_CHUNK = -7,       /* chunk size not accepted (Gated/KDA: must be a multiple of 16) */
  DR_ERR_CUDA = -8,        /* a CUDA runtime call failed; see dr_last_cuda_error() */
  DR_ERR_UNSUPPORTED = -9, /* valid request that no kernel of this build covers */
  DR_ERR_DEVICE = -10,     /* a kernel reported a problem through the status word */
  DR_ERR_STATIC_LIMIT = -11 /* dr_chunk_bwd_static: scratch need exceeds DR_STATIC_SCRATCH_BYTES */
} DrStatus;

/* Which kernel family serves a chunk-forward call. */
typedef enum DrChunkPath {
  DR_PATH_AUTO = 0,   /* tensor-core kernel when the shape qualifies, else the register-resident token recurrence */
  DR_PATH_FP32 = 1,   /* CUDA-core fp32 chunk kernel (any K,V multiple of 16 up to 256) */
  DR_PATH_TCGEN05 = 2, /* tcgen05/TMEM bf16-operand kernel (K=V=128, chunk 64, bf16 q,k,v) */
  DR_PATH_SPLIT = 3    /* two kernels: chunk-parallel intra-chunk pass + tcgen05 state pass over a caller
                          workspace (dr_workspace_bytes(desc, 0)); every variant, K=V=128, chunk 64, bf16
                          q,k,v.  AUTO picks it for KDA when the workspace is given. */
} DrChunkPath;

/* Values the device status word can take (written by kernels, never trapped). */
#define DR_DEV_OK 0
#define DR_DEV_TIMEOUT 1 /* a bounded wait on an mbarrier ran out */
#define DR_DEV_BOUNDS 2  /* an index check failed: only the debug build (compiled with -DDR_BOUNDS_CHECK) checks */
/* With DR_DEV_TIMEOUT from the tcgen05 kernels, bits 8..15 say where the first wait of the launch gave up: the number
 * of the barrier in the kernel's control block (bits 8..13) and the warp group that waited (bits 14..15).  For reading
 * by the library's maintainers; callers test the low bits only. */
#define DR_DEV_SITE(word) (((word) >> 8) & 0xff)

typedef struct DrDesc {
  int32_t variant;       /* DrVariant */
  int32_t layout;        /* DrLayout */
  int32_t B, H, T, K, V; /* T is the number of tokens (1 for dr_step) */
  int32_t chunk;         /* chunk size C for the chunk entry points, ignored elsewhere */
  int32_t qkv_dtype;     /* DrDtype of q, k, v (and of do / dq, dk, dv in the backward) */
  int32_t g_dtype;       /* DrDtype of g (ignored for DR_DELTA) */
  int32_t out_dtype;     /* DrDtype of o */
  int32_t use_qk_l2norm; /* 1: normalise q,k rows as x/(||x||+1e-6) inside the kernel */
  float scale;           /* multiplies q after normalisation */
  int32_t path;          /* DrChunkPath, chunk entry points only */
  int32_t qk_heads;      /* heads of q and k when fewer than H (grouped value attention: head h of v, o, g, beta,
                            state uses q/k head h / (H / qk_heads)); 0 or H: one q/k head per head.  Replaces the
                            jnp.repeat of q, k before the op (gated_deltanet.py:798-801, kda.py:917-922).
                            Backward entry points: dq, dk have qk_heads heads and hold the sum over each group
                            (the transpose of that repeat). */
  int32_t reserved;      /* must be zero */
} DrDesc;

/* Library / build identification, e.g. "deltarule_sm100 0.1 (sm_100a)". */
const char* dr_version(void);

/* Text for a DrStatus. */
const char* dr_strerror(int status);

/* cudaError_t (as int) of the most recent failing CUDA call made by this library on the
 * calling thread, 0 if none. */
int dr_last_cuda_error(void);

/* Number of kernel launches this library has issued since load (all threads); the
 * benchmark reports the difference across its timed region. */
uint64_t dr_launch_count(void);

/*
 * Device status word.  Kernels never trap and never wait without a limit; a wait that runs out ORs
 * DR_DEV_TIMEOUT into the int32 the caller passed as `status_dev` and the kernel finishes (its results are
 * then meaningless).  Entry points do not synchronise, so they cannot return that outcome themselves:
 * dr_check_status copies the word back on `stream`, WAITS for the stream, and returns DR_ERR_DEVICE if any
 * kernel enqueued before it reported a problem (the word is cleared so that the next check starts clean;
 * dr_last_device_status() then gives the DR_DEV_* bits that were found), DR_OK otherwise.  Call it where the
 * host synchronises anyway (end of a step, before results are consumed).  The reference has no counterpart:
 * its one GPU kernel falls back silently (modules/linear_attn/delta_net.py:150-156).
 */
int dr_check_status(int32_t* status_dev, void* stream);
int dr_last_device_status(void);

/* Name of the kernel family the most recent call on this thread dispatched to
 * ("step", "recurrent", "chunk_fp32", "chunk_tcgen05", "bwd", ...). */
const char* dr_last_path(void);

/* Bytes of caller-provided scratch that dr_chunk_fwd (op=0) or dr_chunk_bwd (op=1)
 * needs for `desc`; 0 when none is needed.  Negative DrStatus (cast) on a bad desc.
 * For op=0 the figure is what the path desc->path resolves to would use; a forward that is
 * given less returns DR_ERR_WORKSPACE (there is no silent downgrade to a slower kernel: ask for
 * DR_PATH_FP32 to run without scratch).
 * op=1 returns DR_ERR_UNSUPPORTED for shapes the backward does not cover: chunk > 64, K > 128,
 * or DR_KDA with K % 16 != 0 (the forward entry points accept those shapes). */
int64_t dr_workspace_bytes(const DrDesc* desc, int op);

/*
 * Chunkwise forward.  Replaces
 *   delta_rule_chunkwise        modules/linear_attn/delta_net.py:216-354
 *   gated_delta_rule_chunkwise  modules/linear_attn/gated_deltanet.py:232-534
 *   kda_chunkwise               modules/linear_attn/kda.py:350-655
 * g: null for DR_DELTA.  beta: float32.  h0: float32 [B,H,K,V] or null (zero state).
 * o: desc->out_dtype.  hT: float32 [B,H,K,V] or null (final state not wanted).
 * status_dev: one int32 in device memory, or null; kernels OR problems into it.
 * A ragged tail (T % chunk != 0) behaves as the reference's zero padding does.
 */
int dr_chunk_fwd(const DrDesc* desc, const void* q, const void* k, const void* v, const void* g,
                 const float* beta, const float* h0, void* o, float* hT, void* workspace,
                 size_t workspace_bytes, int32_t* status_dev, void* stream);

/*
 * Chunkwise forward over a PACKED batch of variable-length sequences (the layout core/padding.py:13-53 of the
 * reference produces with compute_unpadded_indices / unpad: valid tokens of all sequences back to back).
 * q,k [total_T, Hq, K]  v,o [total_T, H, V]  beta [total_T, H]  g [total_T, H] or [total_T, H, K], token-major;
 * cu_seqlens_host: n_seqs + 1 token offsets in HOST memory (cu_seqlens[0] = 0, cu_seqlens[n_seqs] = total_T);
 * h0, hT: float32 [n_seqs, H, K, V] or null.  desc: B and T are ignored (B = 1 and T = each sequence's length are
 * filled in per sequence), layout must be DR_LAYOUT_BTHD.  Every sequence starts from its own initial state and
 * is cut into chunks from its own first token, so no chunk straddles a boundary; the result equals the
 * reference op run on each sequence alone.  One launch sequence per sequence on `stream`, no copies; workspace as
 * for dr_chunk_fwd sized for the longest sequence (dr_workspace_bytes with T = that length, B = 1).
 */
int dr_chunk_fwd_varlen(const DrDesc* desc, const void* q, const void* k, const void* v, const void* g,
                        const float* beta, const int32_t* cu_seqlens_host, int32_t n_seqs, const float* h0, void* o,
                        float* hT, void* workspace, size_t workspace_bytes, int32_t* status_dev, void* stream);

/*
 * Token-by-token forward.  Replaces
 *   delta_rule_recurrent         modules/linear_attn/delta_net.py:126-213
 *   delta_rule_recurrent_pallas  kernels/pallas/delta_rule.py:47-281
 *   gated_delta_rule_recurrent   modules/linear_attn/gated_deltanet.py:136-229
 *   kda_recurrent                modules/linear_attn/kda.py:179-283
 * Same argument meaning as dr_chunk_fwd; needs no workspace.
 */
int dr_recurrent_fwd(const DrDesc* desc, const void* q, const void* k, const void* v,
                     const void* g, const float* beta, const float* h0, void* o, float* hT,
                     int32_t* status_dev, void* stream);

/*
 * Single-token decode step (desc->T must be 1).  Replaces
 *   delta_rule_step        modules/linear_attn/delta_net.py:357-397
 *   gated_delta_rule_step  modules/linear_attn/gated_deltanet.py:539-597
 *   kda_step               modules/linear_attn/kda.py:286-347
 * q,k [B,H,K]  v [B,H,V]  g [B,H] or [B,H,K]  beta [B,H] float32.
 * state_in/state_out: float32 [B,H,K,V]; they may be the same pointer (in-place update of
 * the decode cache, the case the kernel is tuned for).  o [B,H,V] in desc->out_dtype.
 * status_dev as in dr_chunk_fwd; a unit whose state never arrived in shared memory (bounded wait ran out)
 * is NOT written back, so a reported time-out leaves the cache entries it touched as they were.
 */
int dr_step(const DrDesc* desc, const void* q, const void* k, const void* v, const void* g,
            const float* beta, const float* state_in, float* state_out, void* o, int32_t* status_dev,
            void* stream);

/*
 * Training-step pair: ONE forward per step instead of two.  dr_chunk_bwd recomputes the forward to get the
 * state at the start of every chunk; a caller that is about to differentiate can instead run
 * dr_chunk_fwd_saving, which is dr_chunk_fwd (same o, hT) that also leaves those states at the head of the
 * BACKWARD workspace (dr_workspace_bytes(desc, 1) bytes, kept by the caller until the backward), and later
 * dr_chunk_bwd_saved, which is dr_chunk_bwd without the recomputation.  Under jax this is the fwd / bwd pair of a
 * jax.custom_vjp around the three *_chunkwise functions, the workspace being the residual.
 * desc->path is ignored (the forward kernel is chosen by shape as in dr_chunk_bwd); out_dtype as in dr_chunk_fwd.
 * For bf16 DeltaNet / Gated DeltaNet the saving forward also leaves the adjoint's chunk-parallel pre-pass results in
 * the workspace; that kernel runs beside the forward on a non-blocking side stream the library creates once per
 * device, forked from and joined to `stream` with events (stream order as seen by the caller is unchanged).
 */
int dr_chunk_fwd_saving(const DrDesc* desc, const void* q, const void* k, const void* v, const void* g,
                        const float* beta, const float* h0, void* o, float* hT, void* bwd_workspace,
                        size_t bwd_workspace_bytes, int32_t* status_dev, void* stream);
int dr_chunk_bwd_saved(const DrDesc* desc, const void* q, const void* k, const void* v, const void* g,
                       const float* beta, const void* d_o, const float* d_hT, void* dq, void* dk, void* dv,
                       float* dbeta, float* dg, float* dh0, void* bwd_workspace, size_t bwd_workspace_bytes,
                       int32_t* status_dev, void* stream);

/*
 * Backward of the chunkwise/recurrent forward (the reference has no backward function:
 * its gradients are jax.grad through the three *_chunkwise functions cited above).
 * Inputs: the forward inputs, d_o [like o, desc->qkv_dtype] and d_hT (float32 [B,H,K,V] or
 * null).  Outputs: dq,dk [like q], dv [like v] in desc->qkv_dtype; dbeta float32 [like beta];
 * dg float32 [like g] (null for DR_DELTA); dh0 float32 [B,H,K,V] or null.
 */
int dr_chunk_bwd(const DrDesc* desc, const void* q, const void* k, const void* v, const void* g,
                 const float* beta, const float* h0, const void* d_o, const float* d_hT, void* dq,
                 void* dk, void* dv, float* dbeta, float* dg, float* dh0, void* workspace,
                 size_t workspace_bytes, int32_t* status_dev, void* stream);

/*
 * dr_chunk_bwd over a PACKED batch (the tensors of dr_chunk_fwd_varlen; d_o, dq, dk, dv packed like their
 * primal tensors; dbeta [total_T, H], dg like g, both float32; d_hT, dh0 float32 [n_seqs, H, K, V] or null).
 * Each sequence is differentiated on its own, one after another on `stream`, so one workspace sized for the longest
 * sequence (dr_workspace_bytes(desc with B = 1 and T = that length, 1)) serves all of them.
 */
int dr_chunk_bwd_varlen(const DrDesc* desc, const void* q, const void* k, const void* v, const void* g,
                        const float* beta, const int32_t* cu_seqlens_host, int32_t n_seqs, const float* h0,
                        const void* d_o, const float* d_hT, void* dq, void* dk, void* dv, float* dbeta, float* dg,
                        float* dh0, void* workspace, size_t workspace_bytes, int32_t* status_dev, void* stream);

/* Size of the scratch array built into the library for dr_chunk_bwd_static: 32 MiB per GPU. */
#define DR_STATIC_SCRATCH_BYTES (32u << 20)

/*
 * dr_chunk_bwd for callers that have no way to hand over a workspace.  It has no counterpart in
 * the reference.  Same arguments and results as dr_chunk_bwd minus `workspace`/`workspace_bytes`:
 * the scratch is a fixed DR_STATIC_SCRATCH_BYTES array inside the library's device image, so this
 * entry point calls neither cudaMalloc/cudaFree nor any allocating routine.  It is meant for hosts
 * where an allocation at call time is impossible or unwelcome: a runtime that has already claimed
 * the whole device for its own pool (an XLA/JAX custom call gets only the buffers the compiler
 * planned), a plug-in that must not touch the allocator of the framework it lives in, or a serving
 * loop that may not stall on the driver's allocation lock.
 *   - Limit: dr_workspace_bytes(desc, 1) must not exceed DR_STATIC_SCRATCH_BYTES, otherwise
 *     DR_ERR_STATIC_LIMIT is returned and nothing is launched (use dr_chunk_bwd then).
 *     Every GPU that loads the library keeps the 32 MiB array until the process exits.
 *   - The first call on each device resolves the array's device address (cudaGetSymbolAddress, with
 *     that device current); make that first call outside any stream capture.
 *   - All calls on a device share the one array, which still holds the previous call's data when
 *     the next one starts (everything that must start at zero is cleared by the call itself).
 *     Two calls that overlap on the GPU -- different streams, or different host threads -- race on
 *     it: serialise them.
 */
int dr_chunk_bwd_static(const DrDesc* desc, const void* q, const void* k, const void* v, const void* g,
                        const float* beta, const float* h0, const void* d_o, const float* d_hT, void* dq,
                        void* dk, void* dv, float* dbeta, float* dg, float* dh0, int32_t* status_dev,
                        void* stream);

/*
 * The element-wise steps of a block next to the op, one HBM pass each, in the token-major layout the op reads
 * with DR_LAYOUT_BTHD (so the block needs no transposes around it).  dtype tags are DrDtype.
 *
 * dr_short_conv_silu -- depthwise_conv1d_causal (core/conv.py:13-68) followed by jax.nn.silu
 *   (gated_deltanet.py:764-783).  x, y [B,T,C]; weight float32 [W,C] (w[W-1] meets the current step); bias
 *   float32 [C] or null; cache_in [B,W-1,C] (null: zeros); cache_out [B,W-1,C] (null: not wanted) = the last W-1
 *   rows of concat(cache_in, x).  W in 1..8; W == 1 returns x (+ bias) as the reference does, weight unused.
 *   C a multiple of 8.  y must not be x; cache_out may be cache_in only for T <= 4 (decode).
 *   apply_silu 0 leaves the convolution output as is.
 *
 * dr_gate_activations -- mode 0: g = -exp(A_log[h]) softplus(a + bias[h]), beta = beta_scale sigmoid(b) with
 *   a, b [B,T,H] (gated_deltanet.py:804-815; beta_scale 2 for allow_neg_eigval), K = 1.  mode 1 (kda_gate,
 *   kda.py:120-172): a [B,T,H,K] (+ bias [H*K] or null), g = -exp(A_log[h]) (x > threshold ? x : softplus(x)),
 *   beta = beta_scale sigmoid(b), b [B,T,H].  b and beta may both be null.  g, beta float32, token-major.
 *
 * dr_gated_rmsnorm -- y[b,t,h,:] = o / sqrt(mean(o^2) + eps) * weight * sigmoid(gate[b,t,h,:]) (RMSNorm
 *   common.py:42-53 with the gate of gated_deltanet.py:853-865; FusedRMSNormGated kda.py:664-700).  o in
 *   o_layout ([B,H,T,V] as the op writes it, or [B,T,H,V]); gate [B,T,H,V] or null (plain o_norm); weight
 *   float32 [V]; y [B,T,H,V].  V a multiple of 4, at most 512.
 */
int dr_short_conv_silu(const void* x, const float* weight, const float* bias, const void* cache_in, void* y,
                       void* cache_out, int B, int T, int C, int W, int dtype, int apply_silu, void* stream);
int dr_gate_activations(int mode, const void* a, const void* b, const float* A_log, const float* bias, float* g,
                        float* beta, int B, int T, int H, int K, int a_dtype, int b_dtype, float beta_scale,
                        float threshold, void* stream);
int dr_gated_rmsnorm(const void* o, const void* gate, const float* weight, void* y, int B, int H, int T, int V,
                     int o_layout, int o_dtype, int gate_dtype, int y_dtype, float eps, void* stream);

/*
 * Other matrix-state scans of the reference, token by token with the fp32 state in registers (no chunk form yet).
 * io_dtype tags every activation tensor and the output; states, u, A, D, dt_bias are float32.  h0 null = zero state,
 * hT null = not wanted, hT may be h0 (in place: the decode step).  T = 1 is the single-step function.
 * K, V (N, P for the SSD) in 1..256.  Activation pointers need the alignment of their element type only.
 *
 * dr_dplr_recurrent -- dplr_delta_rule_recurrent / dplr_delta_rule_step (modules/linear_attn/rwkv7.py:114-259):
 *   h <- exp(gk) * h + b (a^T h) + k v^T;  o = h^T (q * scale).  q, k, a, b, gk [B,H,T,K] (or [B,T,H,K] with
 *   DR_LAYOUT_BTHD), v, o [.., V]; state [B,H,K,V].
 *
 * dr_rwkv6_recurrent -- rwkv6_recurrent / rwkv6_step (modules/linear_attn/rwkv6.py:115-189, 360-398), which is also
 *   what the reference's RWKV6Block runs in "chunk" mode (rwkv6.py:837-850):
 *   o = (h + (u * k) v^T)^T (sigmoid(r) * scale);  h <- exp(-exp(w)) * h + k v^T.  u float32 [H,K].
 *
 * dr_ssd_scan -- ssd_chunk_scan / ssd_recurrent_step (modules/ssm/mamba2.py:161-425), as the token recurrence the
 *   chunked scan equals: dt' = clamp(softplus(dt + dt_bias[h]), dt_lo, dt_hi);
 *   state <- exp(A[h] dt') state + (dt' x) B^T;  y = state C + D[h] x.
 *   x, y [B,T,H,P]; dt float32 [B,T,H]; Bm, Cm [B,T,G,N] with H % G == 0 (head h reads group h / (H/G));
 *   state [B,H,P,N].
 */
int dr_dplr_recurrent(const void* q, const void* k, const void* v, const void* a, const void* b, const void* gk,
                      const float* h0, void* o, float* hT, int B, int H, int T, int K, int V, float scale,
                      int io_dtype, int layout, int32_t* status_dev, void* stream);
int dr_rwkv6_recurrent(const void* r, const void* k, const void* v, const void* w, const float* u, const float* h0,
                       void* o, float* hT, int B, int H, int T, int K, int V, float scale, int io_dtype, int layout,
                       int32_t* status_dev, void* stream);
int dr_ssd_scan(const void* x, const void* dt, const float* A, const void* Bm, const void* Cm, const float* D,
                const float* dt_bias, const float* h0, void* y, float* hT, int B, int T, int H, int P, int N,
                int groups, float dt_lo, float dt_hi, int io_dtype, int32_t* status_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DELTARULE_SM100_H_ */
