/*
 * flab200 — C ABI of the B200 (sm_100a) chunked linear-attention kernels.
 *
 * The reference project (flash-linear-attention) has no FFI layer: its boundary is the Python
 * functional API in fla/ops/<family>/{chunk,fused_recurrent}.py, whose autograd Functions launch
 * Triton kernels stage by stage.  This header defines one entry point per such stage, so a Python
 * (ctypes) or C++ host can drive the same pipeline.  Each declaration cites the reference launch
 * wrapper it replaces (path inside the reference repository : line).
 *
 * Conventions
 *  - Every entry point returns 0 on success and a negative FLAB_E_* code otherwise;
 *    flab_last_error() returns a thread-local, human readable message for the last failure.
 *  - All pointers are device pointers on the current device. Nothing is allocated, freed or
 *    synchronised by the library (except where an entry point says otherwise); kernels are
 *    enqueued on `stream` (a cudaStream_t passed as void*).
 *  - Token-major tensors are contiguous in either seq-first [B,T,H,D] (head_first = 0) or
 *    head-first [B,H,T,D] (head_first = 1) layout; per-token scalars (g, beta) use D = 1.
 *  - Variable-length batches: B = 1, T = total tokens, `cu_seqlens` (int32[N+1]) gives sequence
 *    starts, `chunk_indices` (int32[NT][2]) = (sequence, chunk-in-sequence) per chunk and
 *    `chunk_offsets` (int32[N+1]) = exclusive prefix sum of per-sequence chunk counts.
 *  - The chunk length is fixed at 64 tokens. Chunk states are laid out [total_chunks, H, K, V].
 *  - Initial/final states and their gradients are fp32 [N,H,K,V].
 */
#ifndef FLAB200_H
#define FLAB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLAB_ABI_VERSION 1
#define FLAB_CHUNK 64

enum { FLAB_BF16 = 0, FLAB_FP16 = 1, FLAB_FP32 = 2 };

enum {
  FLAB_OK = 0,
  FLAB_E_BADARG = -1,      /* NULL / inconsistent argument                    */
  FLAB_E_UNSUPPORTED = -2, /* shape or dtype outside what the kernels handle  */
  FLAB_E_LAUNCH = -3,      /* CUDA reported an error at launch                */
  FLAB_E_TIMEOUT = -4      /* a bounded device-side wait ran out: returned by flab_tc_check() */
};

enum {
  FLAB_F_REVERSE = 1 << 0,       /* cumsum / recurrence run from the last token to the first */
  FLAB_F_BETA_VECTOR = 1 << 1,   /* fused_recurrent_delta_rule: beta is [.., V] not scalar    */
  FLAB_F_INPLACE_STATE = 1 << 2, /* flab_recurrent_fwd / _delta_fwd: the caller passes ht == h0 (state updated in place); without
                                    the flag an aliased pair is rejected with FLAB_E_BADARG                 */
  FLAB_F_DESCENDING = 1 << 3,    /* flab_recurrent_delta_fwd: walk the (sequence, head) state tiles from the last to the
                                    first. A decode loop alternates the direction from step to step, so that a step
                                    starts on the tiles its predecessor wrote last, which are still in L2    */
  FLAB_F_STATE_ONLY = 1 << 4,    /* delta scans: only the final state is wanted (h, v_new / dh, dv2 may be NULL) */
  FLAB_F_TRANSPOSE = 1 << 5      /* flab_state_chain: apply the transposed transitions (backward chain)         */
};

typedef struct flab_args {
  /* geometry */
  int32_t B, T, H, K, V;
  int32_t N;          /* number of sequences (B, or len(cu_seqlens) - 1)        */
  int32_t NT;         /* total number of 64-token chunks over all sequences     */
  int32_t dtype;      /* FLAB_BF16 / FLAB_FP16 / FLAB_FP32: element type of q,k,v,o,... */
  int32_t head_first; /* 0: [B,T,H,D]   1: [B,H,T,D]                            */
  int32_t flags;      /* FLAB_F_*                                               */
  float scale;
  int32_t S;          /* innermost extent for the vector cumsum entry points    */
  /* variable-length tables (NULL for fixed length) */
  const int32_t *cu_seqlens;
  const int32_t *chunk_indices;
  const int32_t *chunk_offsets;
  /* tensor slots; each entry point documents the ones it reads and writes */
  void *q, *k, *v;
  void *g;     /* fp32 log-gates per token/head (chunk entry points: already chunk-cumsummed) */
  void *gk;    /* fp32 log-gates per token/head/key channel                                  */
  void *gv;    /* fused_recurrent only: log-gates per value channel                          */
  void *beta;
  void *w, *u;     /* WY factors                                                    */
  void *aw, *au;   /* [.., 64] inverse factors of the WY transform (au: gated only) */
  void *h;         /* chunk states [NT,H,K,V], element type = dtype                 */
  void *h0, *ht;   /* fp32 [N,H,K,V]                                                */
  void *v_new;
  void *o;
  void *d_o;       /* gradient of o */
  void *dh;        /* chunk state gradients [NT,H,K,V] */
  void *dht, *dh0; /* fp32 [N,H,K,V] */
  void *dq, *dk, *dv, *dv2, *dw, *du, *dg, *dgk, *dgv, *dbeta;
  void *a, *da;    /* GLA intra-chunk score matrix [.., 64] fp32 and its gradient */
  void *x, *y;     /* generic in / out (cumsum entry points)                      */
  void *ws;        /* caller-provided scratch                                     */
  size_t ws_bytes;
} flab_args;

int flab_abi_version(void);
const char *flab_last_error(void);

/* ---- gate cumulative sums ------------------------------------------------------------------
 * x -> y (fp32). Replaces chunk_local_cumsum (fla/ops/utils/cumsum.py:389) and
 * chunk_global_cumsum (fla/ops/utils/cumsum.py:369). x has element type `dtype`;
 * scalar variants treat x as [B,T,H] (head_first: [B,H,T]); vector variants as [..., S].
 * FLAB_F_REVERSE selects suffix sums. */
int flab_chunk_local_cumsum_scalar(const flab_args *a, void *stream);
int flab_chunk_local_cumsum_vector(const flab_args *a, void *stream);
int flab_chunk_global_cumsum_scalar(const flab_args *a, void *stream);
int flab_chunk_global_cumsum_vector(const flab_args *a, void *stream);

/* ---- row-wise L2 normalisation (the step before the chunk ops in the reference's layers) ------
 * Replaces l2norm_fwd / l2norm_bwd (fla/modules/l2norm.py:89, :131): x is [rows, n] contiguous,
 *   y = x / sqrt(sum_n x^2 + eps);  dx = dy r - sum_n(dy x) r / (sum_n x^2 + eps) x,  r = 1 / sqrt(sum_n x^2 + eps).
 * Element types are FLAB_BF16 / FLAB_FP16 / FLAB_FP32; the forward output may be fp32 for 16-bit input or
 * 16-bit for fp32 input (the reference's output_dtype). Arithmetic is fp32. rows == 0 is a no-op. */
int flab_l2norm_fwd(const void *x, void *y, long long rows, int n, int in_dtype, int out_dtype, float eps, void *stream);
int flab_l2norm_bwd(const void *x, const void *dy, void *dx, long long rows, int n, int dtype, float eps, void *stream);

/* ---- RMS norm with weight times a swish gate (the step after the chunk ops in the reference's layers) ----
 * Replaces layer_norm_fwd / layer_norm_bwd of fla/modules/fused_norm_gate.py (:103, :301) for the case the
 * delta-rule layers use: IS_RMS_NORM, weight, no bias, no residual (FusedRMSNormSwishGate, :728).
 *   y = (x rstd w) * (g sigmoid(g)),  rstd = 1 / sqrt(mean_n x^2 + eps)   (rstd [rows] fp32 is written for backward)
 *   backward writes dx, dgate (element type) and one partial row of dw (fp32 [partials, n]) per thread block;
 *   the caller sums the partial rows. flab_rms_norm_swish_gate_partials gives their number for (rows, n, dtype).
 * x, gate, y, dy, dx, dgate: [rows, n] contiguous of element type dtype; weight: fp32 [n]. */
int flab_rms_norm_swish_gate_partials(long long rows, int n, int dtype);
int flab_rms_norm_swish_gate_fwd(const void *x, const void *gate, const float *weight, void *y, float *rstd, long long rows, int n, int dtype,
                                 float eps, void *stream);
int flab_rms_norm_swish_gate_bwd(const void *x, const void *gate, const float *weight, const void *dy, const float *rstd, void *dx, void *dgate,
                                 float *dw_partial, long long rows, int n, int dtype, void *stream);

/* ---- causal depthwise short convolution (q, k, v of the reference's layers pass through it first) ----
 * Replaces the convolution of ShortConvolution.forward / .step (fla/modules/convolution.py:142-216):
 *   y[b,t,d] = act(bias[d] + sum_{w<W} weight[d,w] x[b, t-(W-1)+w, d]),  x = 0 before the sequence, act = SiLU or none.
 * x, y, dy, dx: [B, T, D] contiguous of element type dtype (D a multiple of 4, 16-byte aligned);
 * weight fp32 [D, W] (W = 2, 3 or 4), bias fp32 [D] or NULL. Backward adds into dweight (fp32 [D, W]) and dbias
 * (fp32 [D], with a bias) with atomics: the caller zeroes them. The update entry is the one-token decode step:
 * cache [B, D, W] (element type dtype) is shifted by one in place, x [B, D] appended, y [B, D] written (W <= 8). */
int flab_short_conv_fwd(const void *x, const float *weight, const float *bias, void *y, int B, int T, int D, int W, int silu, int dtype,
                        void *stream);
int flab_short_conv_bwd(const void *x, const float *weight, const float *bias, const void *dy, void *dx, float *dweight, float *dbias, int B, int T,
                        int D, int W, int silu, int dtype, void *stream);
int flab_short_conv_update(const void *x, void *cache, const float *weight, const float *bias, void *y, int B, int D, int W, int silu, int dtype,
                           void *stream);

/* ---- gate / beta prologue of the gated delta rule layer (the elementwise step right before the chunk op) ----
 * Replaces the two lines of GatedDeltaNet.forward that make the op's gate and beta (fla/layers/gated_deltanet.py:236-237)
 *   beta = sigmoid(b_proj(x)),   g = -exp(A_log) * softplus(a_proj(x) + dt_bias)
 * and, in the same pass, the chunk-local cumulative sum of g that opens the chunk op (chunk_local_cumsum,
 * fla/ops/gated_delta_rule/chunk.py:33). `geo` supplies B, T, H, N, NT, head_first, dtype (element type of a_proj, b_proj,
 * beta and their gradients) and the variable-length tables; its tensor slots are ignored. a_proj, b_proj, beta: [B,T,H]
 * (or [B,H,T]); A_log, dt_bias (may be NULL): fp32 [H]; g, g_cumsum (may be NULL), dg: fp32 [B,T,H].
 * Backward: da, db as above; dA_log, ddt_bias (may be NULL) fp32 [H] are ADDED to with atomics: the caller zeroes them. */
int flab_gdn_gate_fwd(const flab_args *geo, const void *a_proj, const void *b_proj, const float *A_log, const float *dt_bias, float *g,
                      float *g_cumsum, void *beta, void *stream);
int flab_gdn_gate_bwd(const flab_args *geo, const void *a_proj, const void *b_proj, const float *A_log, const float *dt_bias, const float *dg,
                      const void *dbeta, void *da, void *db, float *dA_log, float *ddt_bias, void *stream);

/* ---- inter-chunk state recurrence for diagonal decay ---------------------------------------
 * Replaces chunk_fwd_h (fla/ops/common/chunk_h.py:282): reads k, v, the gates g, gk, gv (each may be NULL;
 * gv, fp32 [.., V], decays the value channels of the state as the reference's GSA op needs,
 * fla/ops/gsa/chunk.py:664-675; g cannot be combined with gk or gv), h0 (optional); writes h (state at the
 * start of every chunk) and ht (optional). */
int flab_chunk_fwd_h(const flab_args *a, void *stream);
/* Replaces chunk_bwd_dh (fla/ops/common/chunk_h.py:338): reads q, d_o, g / gk / gv (as above), dht
 * (optional); writes dh and dh0 (optional). */
int flab_chunk_bwd_dh(const flab_args *a, void *stream);

/* ---- intra-chunk output and its gradients ---------------------------------------------------
 * Replaces chunk_fwd_o (fla/ops/common/chunk_o.py:444): reads q, k, v, h, g (optional); writes o. */
int flab_chunk_fwd_o(const flab_args *a, void *stream);
/* Replaces chunk_bwd_dv (fla/ops/common/chunk_o.py:499): reads q, k, g, d_o, dh; writes dv. */
int flab_chunk_bwd_dv(const flab_args *a, void *stream);
/* Replaces chunk_bwd_dv_local (fla/ops/common/chunk_o.py:551): reads q, k, g (optional), d_o;
 * writes dv. */
int flab_chunk_bwd_dv_local(const flab_args *a, void *stream);
/* Replaces chunk_bwd_dqkwg (fla/ops/common/chunk_o.py:602): reads q, k, v, h, dh, d_o, g (optional),
 * and for the delta-rule family w and dv; writes dq, dk, dg (fp32, gradient w.r.t. the cumsummed
 * gate, when g is given) and dw (when w is given). */
int flab_chunk_bwd_dqkwg(const flab_args *a, void *stream);

/* ---- WY / UT transform of the (gated) delta rule --------------------------------------------
 * Replaces fwd_prepare_wy_repr (fla/ops/delta_rule/wy_fast.py:436,
 * fla/ops/gated_delta_rule/wy_fast.py:320): reads k, v, beta, g (gated only); writes aw, au (gated
 * only), w, u. */
int flab_wy_fwd(const flab_args *a, void *stream);
/* Replaces fwd_recompute_w_u (fla/ops/delta_rule/wy_fast.py:532,
 * fla/ops/gated_delta_rule/wy_fast.py:379): reads k, v, beta, aw, au (gated only); writes w, u. */
int flab_wy_recompute(const flab_args *a, void *stream);
/* Replaces bwd_prepare_wy_repr (fla/ops/delta_rule/wy_fast.py:619,
 * fla/ops/gated_delta_rule/wy_fast.py:565): reads k, v, beta, g (gated only), aw, au (gated only),
 * dw, du; writes dk, dv, dbeta (fp32) and dg (fp32, gated only). Optional x: a dk of the element type
 * to accumulate onto (the reference adds the dk of chunk_bwd_dqkwg afterwards, chunk.py:168); the sum
 * is formed in fp32 and rounded once. Optional dgk (gated only; fp32 [B,T,H], used here as "the dg of the
 * preceding stage"): when given, dg is not this stage's share but the finished gradient of the raw gate,
 * dg = reverse chunk-local cumsum of (dgk + this stage's dg), which the reference forms with an add and a
 * cumsum launch (fla/ops/gated_delta_rule/chunk.py:173-176). */
int flab_wy_bwd(const flab_args *a, void *stream);

/* ---- state recurrence of the (gated) delta rule ----------------------------------------------
 * Replaces chunk_gated_delta_rule_fwd_h (fla/ops/common/chunk_delta_h.py:248): reads k, w, u,
 * g (optional), h0 (optional); writes h, v_new, ht (optional). With FLAB_F_STATE_ONLY only ht is
 * written (h and v_new may be NULL): the first pass of a scan split into slabs along T, which needs
 * each slab's transition only. bf16 / fp16, K = 128, V a multiple of 64; FLAB_E_UNSUPPORTED otherwise.
 * In that mode S > 0 gives the number of value columns u really has (S < V, a multiple of 64): the state
 * columns past S see u = 0, which is how the transition matrix is obtained next to the offset. */
int flab_delta_fwd_h(const flab_args *a, void *stream);
/* Replaces chunk_gated_delta_rule_bwd_dhu (fla/ops/common/chunk_delta_h.py:323): reads q, k, w,
 * g (optional), dht (optional), d_o, dv; writes dh, dv2, dh0 (optional). FLAB_F_STATE_ONLY: only
 * dh0 is written (dh and dv2 may be NULL), same domain as above. */
int flab_delta_bwd_dhu(const flab_args *a, void *stream);

/* ---- attention scores of simple GLA ----------------------------------------------------------
 * Replaces the `attn` output of parallel_simple_gla_fwd (fla/ops/simple_gla/parallel.py:474-544, written by the
 * kernel at :95-131): a[b,h,i,j] = scale <q_i, k_j> exp(g_i - g_j) for j <= i, else 0, with g the cumulative
 * log decay over the whole sequence (fp32, NULL = no decay). Reads q, k, g; writes a ([B,H,T,T], element type
 * dtype, every entry). Fixed-length batches only, like the reference. */
int flab_simple_gla_attn(const flab_args *a, void *stream);

/* ---- chain of slab transitions (scans cut along T) -------------------------------------------
 * No single counterpart in the reference (its two-level scan, fla/ops/common/chunk_h_split.py:164-260, is
 * unused and covers diagonal decay only). A slab of tokens maps the state entering it to the state leaving it
 * as S_out = M S_in + b. Given the transitions of the S slabs of every (sequence, head) this walks the chain in
 * one launch, fp32:   for s = 0 .. S-1:  s_in[s] = cur;  cur = op(M[s]) cur + b[s]      (cur starts at s0 or 0)
 * and writes the last cur to s_last. FLAB_F_REVERSE walks s = S-1 .. 0, FLAB_F_TRANSPOSE uses M[s]^T (the two
 * together are the backward chain dS_in = M^T dS_out + c).
 * M: [B,S,H,K,K]; b: [B,S,H,K,ldb] of which the first V columns are read (ldb >= V lets b be a column slice of
 * a wider buffer); s0: [B,H,K,V] or NULL; s_in: [B,S,H,K,V] or NULL; s_last: [B,H,K,V] or NULL. K <= 256. */
int flab_state_chain(const float *M, const float *b, long long ldb, const float *s0, float *s_in, float *s_last, int B, int S, int H, int K,
                     int V, int flags, void *stream);

/* ---- GLA (per-channel gates) -----------------------------------------------------------------
 * Replaces chunk_gla_fwd_intra_gk (fla/ops/gla/chunk.py:840): reads q, k, gk; writes a (fp32). */
int flab_gla_fwd_intra(const flab_args *a, void *stream);
/* Replaces chunk_gla_fwd_o_gk (fla/ops/gla/chunk.py:941): reads q, v, gk, h, a; writes o. */
int flab_gla_fwd_o(const flab_args *a, void *stream);
/* Replaces chunk_gla_bwd_dA (fla/ops/gla/chunk.py:982) and chunk_gla_bwd_dv
 * (fla/ops/gla/chunk.py:1018): reads k, v, gk, a, d_o, dh; writes da (fp32) and dv. */
int flab_gla_bwd_dav(const flab_args *a, void *stream);
/* Replaces chunk_gla_bwd_dqk_intra (fla/ops/gla/chunk.py:1057) and chunk_gla_bwd_dqkg
 * (fla/ops/gla/chunk.py:1102): reads q, k, v, gk, h, dh, d_o, da; writes dq, dk, dgk (fp32,
 * gradient w.r.t. the raw gate). */
int flab_gla_bwd_dqkg(const flab_args *a, void *stream);

/* ---- token-recurrent kernels -----------------------------------------------------------------
 * Replaces fused_recurrent_fwd (fla/ops/common/fused_recurrent.py:322): reads q, k, v, g/gk/gv
 * (each optional, element type `dtype` except g/gk/gv which are fp32), h0; writes o (fp32) and ht. */
int flab_recurrent_fwd(const flab_args *a, void *stream);
/* Replaces the kernel launch inside fused_recurrent_bwd (fla/ops/common/fused_recurrent.py:385):
 * reads q, k, v, gates, h0, d_o, dht; writes dq, dk, dv (fp32) and dh0. Gate gradients are formed by
 * the caller with the global cumsum entry points, as the reference does. */
int flab_recurrent_bwd(const flab_args *a, void *stream);
/* Replaces fused_recurrent_delta_rule_fwd (fla/ops/delta_rule/fused_recurrent.py:293) and
 * fused_recurrent_gated_delta_rule_fwd (fla/ops/gated_delta_rule/fused_recurrent.py:113):
 * reads q, k, v, beta, g (optional, fp32), h0; writes o (element type dtype), ht, and u (optional:
 * the pre-beta corrected values the backward kernel needs). */
int flab_recurrent_delta_fwd(const flab_args *a, void *stream);
/* Replaces fused_recurrent_delta_rule_bwd (fla/ops/delta_rule/fused_recurrent.py:350): reads q, k,
 * v, beta, h0, d_o, dht; writes dq, dk, dv (fp32), dbeta (fp32), dh0. */
int flab_recurrent_delta_bwd(const flab_args *a, void *stream);

/* ---- whole-forward entry points --------------------------------------------------------------
 * Replaces chunk_gated_delta_rule_fwd (fla/ops/gated_delta_rule/chunk.py:20-73): the four stages
 * (gate cumsum, WY factors, state scan, output) enqueued by one call. Reads q, k, v, g (the RAW fp32
 * log gate, not cumsummed), beta, h0 (optional); writes o and ht (optional). Intermediates go to
 * `ws` (256-byte aligned, at least flab_gated_delta_rule_fwd_workspace(a) bytes in ws_bytes). */
size_t flab_gated_delta_rule_fwd_workspace(const flab_args *a);
int flab_gated_delta_rule_fwd(const flab_args *a, void *stream);
/* No counterpart in the reference. Same computation and arguments as flab_gated_delta_rule_fwd
 * (ws / ws_bytes ignored), for callers that must not allocate device memory at all: code running
 * while a stream is being captured into a CUDA graph, inside a pre-sized serving arena, or in a
 * host callback, where cudaMalloc (or torch's allocator growing its pool) is either illegal or
 * would stall the device. The intermediates live in a 16 MiB device array that is part of the
 * library image: every GPU that loads the library holds those 16 MiB until the process exits.
 * Limits and rules:
 *  - problems whose scratch exceeds the 16 MiB (B*T*H > 8192 token-heads at K = V = 128) are
 *    rejected with FLAB_E_UNSUPPORTED and a message, nothing is launched;
 *  - the first call on each device looks up the array's device address (no allocation, but a
 *    runtime query), and the first call of each host thread binds that thread to the device's
 *    context: make the first call per device and per calling thread before any stream capture
 *    begins;
 *  - all calls share the one array and it keeps the previous call's contents; every call fully
 *    overwrites what it reads, so nothing needs clearing, but two calls that overlap on the GPU
 *    (different streams, or two threads) race on it: serialise them. */
int flab_gated_delta_rule_fwd_noalloc(const flab_args *a, void *stream);

/* ---- diagnostics -----------------------------------------------------------------------------
 * None of these has a counterpart in the reference.
 *
 * Every wait inside the tcgen05 / TMA kernels (on an mbarrier) is bounded: a wait that runs out makes its
 * kernel record the id of the wait in a device-side error word and return normally, so the context stays
 * usable but the outputs of that launch are invalid. The ordinary entry points do not synchronise and
 * therefore cannot report this themselves; the three calls below do (each synchronises the device):
 *   flab_tc_error_state()  0, or the id of the first wait that ran out since the last clear;
 *   flab_tc_check()        FLAB_OK, or FLAB_E_TIMEOUT with the id in flab_last_error();
 *   flab_tc_error_clear()  zeroes the error words.
 * A host that wants every launch checked calls flab_tc_check() after synchronising (the ctypes binding does
 * so after every call when FLA_B200_CHECK=1). */
int flab_tc_error_state(void);
int flab_tc_check(void);
int flab_tc_error_clear(void);
/* Runs four small bf16 products through the TMA + tcgen05 + TMEM path (every shared-memory operand form
 * the kernels use) and writes them to `out` (fp32: [64x64] A B^T, [64x128] A H, [128x64] A^T V,
 * [64x64] bf16(A B^T) V) for the caller to compare with a plain matmul. a, b: [64x128], h: [128x128],
 * v: [64x64], row-major bf16. *status = 0 on success, else the index of the bounded wait that ran out. */
int flab_tc_selftest(const void *a, const void *b, const void *h, const void *v, float *out, int *status, void *stream);
/* Exercises the way out of a wait that gives up: one warp waits for `limit_ticks` clock ticks
 * (1 .. 2^28, i.e. well under a second) on a barrier nothing arrives at, then writes the wait id (99) to
 * *status (device int) and to the error word, and returns. Afterwards flab_tc_check() reports
 * FLAB_E_TIMEOUT until flab_tc_error_clear(). */
int flab_tc_wait_selftest(long long limit_ticks, int *status, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* FLAB200_H */
