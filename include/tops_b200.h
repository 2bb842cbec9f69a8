/*
 * tops_b200 — C ABI of the B200 (sm_100a) gated-linear-attention kernels.
 *
 * The reference (`tops`, a pure-Python JAX package) has no native interface:
 * its boundary for this path is the Python signature of each op.  Every entry
 * point below therefore names the reference function it replaces; the Python
 * package `tops_b200` keeps those signatures and calls these symbols through
 * ctypes (and, where JAX is installed, through a `jax.ffi` shim).
 *
 * Conventions
 *  - All tensors are dense row-major.  Activations are `[B, T, H, D]`
 *    (time-major, head-minor), states are `[N, H, K, V]` fp32, chunk states
 *    are `[B, NT, H, K, V]` with NT = ceil(T / chunk).
 *  - Pointers are device pointers owned by the caller.  Nothing is allocated,
 *    freed or synchronised here; all work is enqueued on `stream`.
 *  - `workspace` is caller-provided scratch of at least
 *    `*_workspace_bytes(params)` bytes, 256-byte aligned.
 *  - Return value: 0 on success, a negative `TOPS_E_*` code otherwise
 *    (`tops_b200_strerror` gives the text).  No entry point aborts or traps.
 *  - Optional pointers may be NULL where the comment says so.
 */
#ifndef TOPS_B200_H_
#define TOPS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  TOPS_OK = 0,
  TOPS_E_BAD_SHAPE = -1,   /* a dimension is outside what the kernels accept */
  TOPS_E_BAD_DTYPE = -2,
  TOPS_E_NULL = -3,        /* a required pointer is NULL */
  TOPS_E_WORKSPACE = -4,   /* workspace missing or too small */
  TOPS_E_CUDA = -5,        /* a CUDA runtime / driver call failed */
  TOPS_E_UNSUPPORTED = -6, /* valid request that no kernel covers */
  TOPS_E_ALIGN = -7,       /* a pointer is not 16-byte aligned */
  TOPS_E_STATIC_LIMIT = -8 /* the problem needs more scratch than the built-in static buffer holds */
};

enum { TOPS_F32 = 0, TOPS_BF16 = 1, TOPS_F16 = 2 };

/* Which gate drives the recurrence. */
enum {
  TOPS_GATE_NONE = 0,
  TOPS_GATE_PER_CHANNEL = 1, /* GLA: g is [B,T,H,K]            */
  TOPS_GATE_SCALAR = 2,      /* simple_gla: g is [B,T,H]       */
  TOPS_GATE_GAMMA = 3        /* simple_gla: constant g_gamma[H] */
};

/* Kernel selection.  AUTO picks the tcgen05 path when the shape allows it. */
enum { TOPS_IMPL_AUTO = 0, TOPS_IMPL_GENERIC = 1, TOPS_IMPL_SM100 = 2 };

const char* tops_b200_strerror(int code);
/* Text of the CUDA error behind the most recent TOPS_E_CUDA ("<call>: <cudaGetErrorString> (<code>)"),
 * copied NUL-terminated into `buf`.  No counterpart in the reference. */
int tops_b200_last_cuda_error(char* buf, size_t cap);
/* Number of kernels launched by this library since load (all entry points). */
int64_t tops_b200_launch_count(void);

/* Every wait inside the tcgen05 kernels (on a TMA or tensor-core completion
 * barrier) is bounded; a wait that gives up records a small positive code in a
 * device word and the kernel returns early.  This call copies that word to
 * `*out` (0 = no wait has ever given up).  It synchronises with the device.
 * No counterpart in the reference. */
int tops_b200_device_error(int* out);
/* The word is sticky: it keeps the first code until it is cleared.  A kernel that gives up also
 * writes NaN into the first element of an output it owns (o, ht, dq, a chunk state), so that a
 * caller who never reads the word still sees a poisoned result instead of stale memory.
 * `_reset` clears the word; `_set` overwrites it from the host (host-side fault injection for
 * tests of the error reporting path; no kernel is involved).  Both synchronise with the device. */
int tops_b200_device_error_reset(void);
int tops_b200_device_error_set(int code);
/* Test hook for the bounded waits themselves: the next tcgen05 state-scan launch of this process never
 * issues the tile load of chunk `chunk` (>= 3) of each block, so the wait for that tile runs out after its
 * limit (tens of milliseconds), the kernel records code 1, poisons its outputs and returns on its own; the
 * hook clears itself after that one launch.  Nothing traps or faults.  No counterpart in the reference. */
int tops_b200_test_skip_load(int chunk);

/* Per-kernel device timing (no counterpart behind the reference's op API; its
 * benchmarks wrap timed loops in jax.profiler traces, `benchmarks/utils.py:71-83`).
 * While enabled, every kernel this library launches is bracketed by a CUDA event
 * pair on its stream.  `tops_b200_profile_read` waits for the recorded events,
 * writes one line per kernel label — "<label> <launches> <total_ms>\n" — into
 * `buf` (NUL-terminated, truncated to `cap`), and clears the records. */
int tops_b200_profile_enable(int on);
int tops_b200_profile_read(char* buf, size_t cap);

/* ------------------------------------------------------------------------ *
 * chunk_local_cumsum — replaces `tops/cpu/ops/common/chunk_o.py:18-112`
 * (accelerator: `tops/ops/common/cumsum.py:472-540`).
 * Inclusive (or, reversed, suffix) sum of `g` inside each chunk along T.
 * `D` is K for per-channel gates, 1 for scalar gates.  Output is fp32.
 * Dense batches only: with `cu_seqlens` set this stand-alone call returns
 * TOPS_E_UNSUPPORTED (packed batches restart chunks per sequence inside the
 * fused chunk entry points, which carry the chunk tables in their workspace).
 * ------------------------------------------------------------------------ */
typedef struct {
  int32_t B, T, H, D, chunk;
  int32_t dtype;   /* dtype of g */
  int32_t reverse; /* 0 prefix sums, 1 suffix sums */
  const void* g;
  float* out;
  const int32_t* cu_seqlens; /* must be NULL (see above) */
  int32_t N;                 /* unused */
} tops_cumsum_params;
int tops_b200_chunk_local_cumsum(const tops_cumsum_params* p, void* stream);

/* ------------------------------------------------------------------------ *
 * Problem description shared by the chunked GLA / simple_gla entry points.
 * ------------------------------------------------------------------------ */
typedef struct {
  int32_t B, T, H, K, V, chunk;
  int32_t dtype;      /* dtype of q, k, v, o, do, dv */
  int32_t gate_dtype; /* dtype of g */
  int32_t gate_kind;  /* TOPS_GATE_* */
  int32_t impl;       /* TOPS_IMPL_* */
  float scale;
  const int32_t* cu_seqlens; /* device int32 [N+1] or NULL */
  const int32_t* cu_seqlens_host; /* the same values in host memory (needed when cu_seqlens != NULL) */
  int32_t N;                 /* sequences when packed; else ignored (N = B) */
} tops_chunk_problem;

/* ------------------------------------------------------------------------ *
 * chunk_fwd_h — replaces `tops/cpu/ops/common/chunk_h.py:31-226`
 * (accelerator `tops/ops/common/chunk_h.py:100-272`): chunk-start states of
 * h <- h*exp(g_last) + k~^T v.  `g_cumsum` is the chunk-local cumsum (fp32),
 * `[B,T,H,K]`, `[B,T,H]` or, for TOPS_GATE_GAMMA, the raw `g_gamma[H]`.
 * h is written as `[B,NT,H,K,V]` in `h_dtype` (TOPS_F32 or the input dtype).
 * ------------------------------------------------------------------------ */
typedef struct {
  tops_chunk_problem pb;
  const void *k, *v;
  const float* g_cumsum;
  const float* h0; /* [N,H,K,V] or NULL */
  void* h;         /* [B,NT,H,K,V] or NULL (only ht wanted) */
  int32_t h_dtype;
  float* ht;       /* [N,H,K,V] or NULL */
} tops_fwd_h_params;
int tops_b200_chunk_fwd_h(const tops_fwd_h_params* p, void* stream);

/* ------------------------------------------------------------------------ *
 * chunk_bwd_dh — replaces `tops/cpu/ops/common/chunk_h.py:229-427`
 * (accelerator `tops/ops/common/chunk_h.py:781-884`): reverse scan
 * dh <- dh*exp(g_last) + (q*scale*exp(g))^T do, seeded by dht.
 * ------------------------------------------------------------------------ */
typedef struct {
  tops_chunk_problem pb;
  const void *q, *do_;
  const float* g_cumsum;
  const float* dht; /* [N,H,K,V] or NULL */
  float* dh;        /* [B,NT,H,K,V] fp32 or NULL */
  float* dh0;       /* [N,H,K,V] or NULL */
} tops_bwd_dh_params;
int tops_b200_chunk_bwd_dh(const tops_bwd_dh_params* p, void* stream);

/* ------------------------------------------------------------------------ *
 * chunk_gla_fwd / chunk_simple_gla_fwd — replace
 * `tops/cpu/ops/gla/chunk.py:159-269` (public `chunk_gla` :648-709,
 * `fused_chunk_gla` `tops/cpu/ops/gla/fused_chunk.py:4-44`) and
 * `tops/cpu/ops/simple_gla/chunk.py:53-129` (public :796-889):
 * cumsum, state scan, masked intra-chunk product and output combine.
 * Optional outputs (NULL to skip): g_cumsum fp32 (shape of g), A fp32
 * `[B,T,H,chunk]`, h `[B,NT,H,K,V]` in the input dtype, ht fp32.
 * ------------------------------------------------------------------------ */
typedef struct {
  tops_chunk_problem pb;
  const void *q, *k, *v;
  const void* g;   /* raw log-gates: [B,T,H,K] / [B,T,H] / g_gamma[H] fp32 / NULL */
  const float* h0; /* [N,H,K,V] or NULL */
  void* o;         /* [B,T,H,V] input dtype */
  float* ht;       /* NULL unless the final state is wanted */
  float* g_cumsum_out;
  float* A_out;
  void* h_out;
  /* Optional scratch kept for the backward call of the same problem:
   * B*NT*H*K*V elements of the input dtype.  Its content is private to the
   * kernel family that ran (the tcgen05 kernels store pre-scaled bf16 states);
   * hand it to tops_b200_chunk_gla_bwd as `h_saved` only when
   * tops_b200_chunk_selected_impl reports TOPS_IMPL_SM100 for the problem. */
  void* saved_out;
  /* Optional (tcgen05 path, few (batch, head) pairs): the workspace a `tops_b200_chunk_state_exchange_pack`
   * call (reverse = 0) on this same problem left behind.  It holds the time segments' summaries, so the
   * forward skips its own summary scan and only chains the segments from `h0`.  NULL otherwise. */
  void* segments;
} tops_chunk_fwd_params;
/* Which kernel family TOPS_IMPL_AUTO resolves to for this problem on the current device. */
int tops_b200_chunk_selected_impl(const tops_chunk_problem* pb);
size_t tops_b200_chunk_fwd_workspace_bytes(const tops_chunk_fwd_params* p);
int tops_b200_chunk_gla_fwd(const tops_chunk_fwd_params* p, void* workspace, size_t workspace_bytes,
                            void* stream);

/* ------------------------------------------------------------------------ *
 * chunk_gla_fwd without a caller-provided workspace.  This entry point has no
 * counterpart in the reference.
 *
 * Some hosts of this library cannot give it scratch memory: a runtime that
 * owns the whole device heap and hands a custom call only its operand and
 * result buffers (no scratch allocator, no way to call cudaMalloc on its
 * behalf), or a serving process whose memory pool is carved up at start-up.
 * For them this variant runs exactly the forward pass of
 * tops_b200_chunk_gla_fwd (same params, same kernels, same results) with its
 * scratch (cumulative gates, chunk-start states) in a device array that is
 * part of the library image: TOPS_STATIC_SCRATCH_BYTES on every GPU that
 * loads the library, held until the process exits.  Nothing is allocated or
 * freed, here or in anything it calls.
 *
 *  - Problems whose scratch need (tops_b200_chunk_fwd_workspace_bytes) exceeds
 *    TOPS_STATIC_SCRATCH_BYTES are refused with TOPS_E_STATIC_LIMIT; nothing
 *    is launched.
 *  - The first call on each device looks up the array's device address (with
 *    that device current); the CUDA runtime may load the part of the library
 *    image that holds the array at that moment, which is when the
 *    TOPS_STATIC_SCRATCH_BYTES leave the device's free memory.  Make that
 *    first call outside any stream capture.  From the second call on the
 *    free memory of the device is the same before and after a call.
 *  - All calls on a device share the one array and it keeps whatever the last
 *    call left there.  The forward pass overwrites every element it later
 *    reads, so nothing has to be cleared; but two calls whose kernels overlap
 *    on the GPU (different streams, or different host threads) race on it.
 *    Serialise them.
 * ------------------------------------------------------------------------ */
#define TOPS_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)
int tops_b200_chunk_gla_fwd_static(const tops_chunk_fwd_params* p, void* stream);

/* ------------------------------------------------------------------------ *
 * chunk_gla_bwd / chunk_simple_gla_bwd — replace
 * `tops/cpu/ops/gla/chunk.py:469-640` and
 * `tops/cpu/ops/simple_gla/chunk.py:668-788`: recompute cumsum, states and
 * the intra matrix, reverse-scan dh, then dq, dk, dv, dg (and dh0 when h0 is
 * given).  Output dtypes: `grad_dtype` for dq/dk (TOPS_F32 for GLA as in the
 * reference's CPU path, the input dtype for simple_gla), dv in the input
 * dtype, dg in `dg_dtype` (`[B,T,H,K]` per-channel, `[B,T,H]` scalar; NULL
 * for GAMMA/NONE).  `dg_dtype` is TOPS_F32 (the default, what
 * `tops/cpu/ops/gla/chunk.py:637-638` returns) or, on the tcgen05 path with
 * `grad_dtype == TOPS_BF16`, TOPS_BF16: the reference's accelerator kernel
 * writes dq, dk and dg in the dtypes of q, k and g
 * (`tops/ops/gla/chunk.py:1551-1554`).
 * ------------------------------------------------------------------------ */
typedef struct {
  tops_chunk_problem pb;
  const void *q, *k, *v;
  const void* g;
  const float* h0;
  const void* do_;
  const float* dht; /* NULL: zero */
  void *dq, *dk;
  int32_t grad_dtype;
  void* dv;
  void* dg;
  float* dh0; /* NULL unless h0 given and wanted */
  /* Optional: the `saved_out` scratch written by the forward call on the same
   * inputs (tcgen05 path only).  When given the backward skips recomputing the
   * chunk-start states; NULL recomputes (the reference always recomputes,
   * `tops/cpu/ops/gla/chunk.py:551-561`). */
  const void* h_saved;
  int32_t dg_dtype; /* TOPS_F32 (0) or TOPS_BF16, see above */
  /* The same for the reverse scan: the workspace of a `tops_b200_chunk_state_exchange_pack` call with
   * reverse = 1 (x = q, y = do, the same scale) on this problem.  NULL otherwise. */
  void* rev_segments;
} tops_chunk_bwd_params;
size_t tops_b200_chunk_bwd_workspace_bytes(const tops_chunk_bwd_params* p);
int tops_b200_chunk_gla_bwd(const tops_chunk_bwd_params* p, void* workspace, size_t workspace_bytes,
                            void* stream);

/* ------------------------------------------------------------------------ *
 * fused_recurrent_gla forward — replaces
 * `tops/cpu/ops/gla/fused_recurrent.py:51-162` (public :362-422): token-serial
 * h*=exp(gk); h*=exp(gv); h+=k(x)v; o=scale*q^T h.  `state_in` may equal
 * `state_out` (in-place decode).  o is written in `o_dtype`.
 * ------------------------------------------------------------------------ */
typedef struct {
  int32_t B, T, H, K, V;
  int32_t dtype;      /* q, k, v */
  int32_t gate_dtype; /* gk, gv */
  int32_t o_dtype;
  int32_t reverse;
  float scale;
  const void *q, *k, *v;
  const void* gk; /* [B,T,H,K] or NULL */
  const void* gv; /* [B,T,H,V] or NULL */
  const float* state_in; /* [N,H,K,V] or NULL (zero) */
  float* state_out;      /* [N,H,K,V] or NULL */
  void* o;
  const int32_t* cu_seqlens;
  int32_t N;
} tops_recurrent_fwd_params;
int tops_b200_fused_recurrent_gla_fwd(const tops_recurrent_fwd_params* p, void* stream);

/* ------------------------------------------------------------------------ *
 * fused_recurrent_gla backward — replaces
 * `tops/cpu/ops/gla/fused_recurrent.py:171-353`.  Two passes over time.
 * workspace: see tops_b200_fused_recurrent_gla_bwd_workspace_bytes.
 * ------------------------------------------------------------------------ */
typedef struct {
  int32_t B, T, H, K, V;
  int32_t dtype, gate_dtype;
  int32_t reverse;
  float scale;
  const void *q, *k, *v, *gk, *gv;
  const float* o; /* fp32 forward output; required with gv */
  const void* do_;
  const float* h0;
  const float* dht;
  void *dq, *dk, *dv; /* input dtype */
  void *dgk, *dgv;    /* gate dtype, NULL when the gate is absent */
  float* dh0;         /* NULL unless h0 given */
  const int32_t* cu_seqlens;
  int32_t N;
} tops_recurrent_bwd_params;
size_t tops_b200_fused_recurrent_gla_bwd_workspace_bytes(const tops_recurrent_bwd_params* p);
int tops_b200_fused_recurrent_gla_bwd(const tops_recurrent_bwd_params* p, void* workspace,
                                      size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------ *
 * KDA (gated delta rule) forward — replaces the forward of `chunk_kda`
 * (`tops/ops/kda/chunk.py:193-216`, oracle `tops/cpu/ops/kda/naive.py:121-313`)
 * and `fused_recurrent_kda` (`tops/ops/kda/fused_recurrent.py:19-105`,
 * `tops/cpu/ops/kda/naive.py:10-118`):
 *   S' = S exp(g_t); e = v_t - k_t^T S'; S = S' + beta_t k_t (x) e; o_t = scale q_t^T S.
 * g is the natural-log decay [B,T,H,K]; beta [B,T,H] in the dtype of q.
 * ------------------------------------------------------------------------ */
typedef struct {
  int32_t B, T, H, K, V;
  int32_t dtype;      /* q, k, v, beta, o */
  int32_t gate_dtype; /* g */
  float scale;
  const void *q, *k, *v, *g, *beta;
  const float* h0; /* [B,H,K,V] or NULL */
  void* o;
  float* ht;       /* [B,H,K,V] or NULL */
} tops_kda_fwd_params;
int tops_b200_kda_fwd(const tops_kda_fwd_params* p, void* stream);

/* ------------------------------------------------------------------------ *
 * chunk_kda_fwd — replaces `chunk_kda_fwd` (`tops/ops/kda/chunk.py:25-190`): the
 * chunked WY / UT-transform forward built from the intra-chunk kernel
 * (`tops/ops/kda/chunk_intra.py:91-165`, blocked unit-lower solve `:28-88`), the
 * delta-rule state scan (`tops/ops/common/chunk_delta_h.py:569-736`) and the
 * output kernel (`tops/ops/gla/chunk.py:1279-1440`), here one pass per (batch,
 * head) on the tensor cores.  bf16 q, k, v, g (natural-log gate), beta `[B,T,H]`;
 * K = V = 128, chunk = 64, T % 64 == 0 (`tops_b200_chunk_kda_supported` says
 * whether a problem qualifies; other problems go to `tops_b200_kda_fwd`).
 * Optional outputs (NULL to skip):
 *   Aqk_out, Akk_out  fp32 `[B,T,H,64]`: row i of its chunk at token i —
 *                     tril(scale q k^T exp(G_i - G_j)) and (I + stril(beta k k^T exp(G_i - G_j)))^-1,
 *                     the matrices `chunk_kda_fwd` returns;
 *   saved_h     bf16 `[B,NT,H,K,V]`  chunk-start states times exp(mid) per key channel,
 *   saved_vnew  bf16 `[B,T,H,V]`     the delta-corrected values v' = u - w h,
 *   saved_R     bf16 `[B,T,H,V]`     beta (v - k exp(G) h), the right-hand side of the solve (v' = Akk R),
 *   saved_T     bf16 `[B,T,H,64]`    the inverse above in bf16:
 *               residuals `tops_b200_chunk_kda_bwd` takes back (opaque to callers).
 * ------------------------------------------------------------------------ */
typedef struct {
  int32_t B, T, H, K, V, chunk;
  int32_t dtype, gate_dtype;
  float scale;
  const void *q, *k, *v, *g, *beta;
  const float* h0; /* [B,H,K,V] or NULL */
  void* o;         /* [B,T,H,V] */
  float* ht;       /* [B,H,K,V] or NULL */
  float *Aqk_out, *Akk_out;
  void *saved_h, *saved_vnew, *saved_T, *saved_R;
} tops_chunk_kda_fwd_params;
int tops_b200_chunk_kda_supported(const tops_chunk_kda_fwd_params* p);
int tops_b200_chunk_kda_fwd(const tops_chunk_kda_fwd_params* p, void* stream);

/* ------------------------------------------------------------------------ *
 * chunk_kda_bwd — replaces `chunk_kda_bwd` (`tops/cpu/ops/kda/chunk_bwd.py:525-668`;
 * accelerator kernels `tops/ops/kda/chunk_bwd.py:19-141, 309-351, 457-520`,
 * `tops/ops/kda/chunk_intra.py:283-574`) for the problems `tops_b200_chunk_kda_fwd` takes.
 * Its stages are regrouped into three kernels on the tensor cores: the reverse scan of the state
 * gradient (`chunk_gated_delta_rule_bwd_dhu` together with the dv part of `chunk_kda_bwd_dAv` and of
 * the WY backward), the gradients of the two per-chunk matrices (dAqk of `chunk_kda_bwd_dAv`, the
 * inverse's gradient of `prepare_wy_repr_bwd` `tops/cpu/ops/kda/wy_fast.py:96-224`), and the chunk
 * outputs (`chunk_kda_bwd_wy_dqkg_fused` + `chunk_kda_bwd_intra` + the reverse cumsum of dg).
 * `saved_*` are the residuals the forward wrote.  dq, dk, dg `[B,T,H,K]` and dbeta `[B,T,H]` in
 * `grad_dtype` (TOPS_F32 as the reference's orchestrator returns them, or TOPS_BF16); dv bf16;
 * dg is with respect to the natural-log gate; dh0 fp32 (NULL to skip).
 * State gradient only: with dq = dk = dg = dbeta = NULL the call runs the reverse scan alone and
 * writes dh0 (and dv).  The state gradient entering a span of tokens depends on the one leaving it
 * linearly, dh_in = M^T dh_out + D; a call with dht = NULL gives D, the summary a rank needs when one
 * sequence is sharded over time (no counterpart in the reference, which has no multi-device path).
 * ------------------------------------------------------------------------ */
typedef struct {
  int32_t B, T, H, K, V, chunk;
  int32_t dtype, gate_dtype;
  float scale;
  const void *q, *k, *v, *g, *beta;
  const void* do_;
  const float* dht; /* [B,H,K,V] or NULL */
  const void *saved_h, *saved_vnew, *saved_T, *saved_R;
  void *dq, *dk, *dg, *dbeta; /* all four, or all NULL (state gradient only) */
  int32_t grad_dtype;
  void* dv;
  float* dh0;
} tops_chunk_kda_bwd_params;
size_t tops_b200_chunk_kda_bwd_workspace_bytes(const tops_chunk_kda_bwd_params* p);
int tops_b200_chunk_kda_bwd(const tops_chunk_kda_bwd_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------ *
 * KDA backward — replaces `chunk_kda_bwd` (`tops/cpu/ops/kda/chunk_bwd.py:525-668`)
 * and the explicit recurrent backward (`tops/cpu/ops/kda/fused_recurrent.py:212-418`):
 * dq, dk, dv, dbeta in the input dtype, dg in the gate dtype (with respect to
 * the natural-log gate), dh0 fp32 (NULL to skip).  K, V <= 128.
 * ------------------------------------------------------------------------ */
typedef struct {
  int32_t B, T, H, K, V;
  int32_t dtype, gate_dtype;
  float scale;
  const void *q, *k, *v, *g, *beta;
  const float* h0;
  const void* do_;
  const float* dht; /* NULL: zero */
  void *dq, *dk, *dv, *dg, *dbeta;
  float* dh0;
} tops_kda_bwd_params;
size_t tops_b200_kda_bwd_workspace_bytes(const tops_kda_bwd_params* p);
int tops_b200_kda_bwd(const tops_kda_bwd_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------ *
 * State exchange of a sequence sharded over time across ranks.  No counterpart
 * in the reference, which has no multi-device path; it generalises its
 * `initial_state` / `output_final_state` contract (`tops/cpu/ops/gla/chunk.py:655-656,694-709`,
 * state-split test `tests/ops/gla/test_pallas_chunk_gla.py:223-247`) to R shards: a shard acts on
 * the state entering it as h_out = h_in * exp(P) + S.
 *   pack   the summary S of this rank's shard: the end state from a zero start (reverse = 0:
 *          x = k, y = v) or the state gradient before the shard for a zero gradient after it
 *          (reverse = 1: x = q, y = do; x is scaled by pb.scale).  tcgen05 problems only (bf16,
 *          K = V = 128, chunk 64, per-channel gate `[B,T,H,K]`): TOPS_E_UNSUPPORTED otherwise.
 *          P, the summed log-gates of the shard `[B,H,K]`, is a plain sum the caller makes.
 *          The workspace keeps the summaries of the time segments the scan was cut into: handed to the
 *          forward (`segments`) / backward (`rev_segments`) call of the same shard it saves their own
 *          summary scan, so a shard is scanned twice per direction, as on a single GPU.
 *   apply  after the ranks have all-gathered P `[R,B*H,K]` and S `[R,B*H,K,V]` (fp32): the state
 *          entering shard `rank` (reverse: the gradient leaving it on its right) from `first`
 *          (h0 / dht, NULL = zero) in `out_in`, and the value pushed through all R shards (final
 *          state / dh0) in `out_all` (NULL to skip).  Any K, V with K*V % 4 == 0.
 * ------------------------------------------------------------------------ */
typedef struct {
  tops_chunk_problem pb;
  int32_t reverse;
  const void *x, *g, *y;
  float* state_out; /* [B,H,K,V] */
} tops_state_pack_params;
size_t tops_b200_chunk_state_exchange_pack_workspace_bytes(const tops_state_pack_params* p);
int tops_b200_chunk_state_exchange_pack(const tops_state_pack_params* p, void* workspace, size_t workspace_bytes,
                                        void* stream);
typedef struct {
  int32_t R, rank, reverse;
  int64_t BH;
  int32_t K, V;
  const float* first;
  const float* P;
  const float* S;
  float* out_in;
  float* out_all;
} tops_state_apply_params;
int tops_b200_chunk_state_exchange_apply(const tops_state_apply_params* p, void* stream);

/* ------------------------------------------------------------------------ *
 * Gate activations — the step before the attention kernels.
 *   TOPS_GATE_ACT_KDA              y = -exp(A_log[h]) softplus(g + dt_bias[h,k])
 *   TOPS_GATE_ACT_KDA_LOWER_BOUND  y = lower_bound sigmoid(exp(A_log[h]) (g + dt_bias[h,k]))
 *       replace `kda_gate_fwd` / `fused_kda_gate` / `kda_gate_bwd`
 *       (`tops/cpu/ops/kda/gate.py:60-204`, `tops/ops/kda/gate.py:54-125`);
 *   TOPS_GATE_ACT_LOG_SIGMOID      y = log_sigmoid(g) / normalizer, optionally clipped from below
 *       replaces the gate of the GLA layer (`tops/layers/gla.py:277-279`).
 * g is `[rows, H, K]` (rows = B*T), K % 4 == 0.  The backward writes dg in the dtype of g and, for the
 * KDA kinds, dA_log `[H]` and d dt_bias `[H*K]` (fp32; NULL to skip) through per-row-block partial sums
 * in the workspace, added in a fixed order.
 * ------------------------------------------------------------------------ */
enum { TOPS_GATE_ACT_KDA = 0, TOPS_GATE_ACT_KDA_LOWER_BOUND = 1, TOPS_GATE_ACT_LOG_SIGMOID = 2 };
typedef struct {
  int64_t rows;
  int32_t H, K;
  int32_t kind;
  int32_t dtype, out_dtype;
  const void* g;
  const float* A_log;   /* [H]; KDA kinds */
  const float* dt_bias; /* [H*K] or NULL */
  float lower_bound, normalizer, clamp_min;
  int32_t has_clamp_min;
  void* out;            /* [rows,H,K] in out_dtype */
} tops_gate_act_params;
typedef struct {
  tops_gate_act_params fwd; /* `out` unused */
  const void* dy;           /* [rows,H,K] */
  int32_t dy_dtype;
  void* dg;                 /* [rows,H,K] in fwd.dtype */
  float* dA_log;            /* [H] or NULL */
  float* dbias;             /* [H*K] or NULL */
} tops_gate_act_bwd_params;
int tops_b200_gate_act_fwd(const tops_gate_act_params* p, void* stream);
size_t tops_b200_gate_act_bwd_workspace_bytes(const tops_gate_act_bwd_params* p);
int tops_b200_gate_act_bwd(const tops_gate_act_bwd_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------ *
 * Row normalisations over the last dimension D (D % 4 == 0, D <= 1024), `[rows, D]`.
 *   l2norm          y = x / sqrt(sum(x^2) + eps)      — the q/k normalisation of KDA
 *                   (`tops/cpu/ops/kda/fused_recurrent.py:14-18`, eps 1e-6); `rstd` (fp32 [rows]) optional.
 *   rmsnorm_gated   y = x rsqrt(mean(x^2) + eps) weight silu(gate)   — `FusedRMSNormGated`
 *                   (`tops/modules/fused_norm_gate.py:6-37`); weight fp32 [D] or NULL.
 * Backward: dx (and dgate, dweight fp32 [D] or NULL for the gated norm) from x, gate, dy.
 * ------------------------------------------------------------------------ */
typedef struct {
  int64_t rows;
  int32_t D;
  int32_t dtype;
  float eps;
  const void* x;
  const void* gate;     /* rmsnorm_gated only */
  const float* weight;  /* rmsnorm_gated only, may be NULL */
  void* y;              /* forward output (unused by the backward) */
  float* rstd;          /* l2norm forward, may be NULL */
  const void* dy;       /* backward */
  void* dx;             /* backward */
  void* dgate;          /* rmsnorm_gated backward */
  float* dweight;       /* rmsnorm_gated backward, may be NULL */
} tops_norm_params;
int tops_b200_l2norm_fwd(const tops_norm_params* p, void* stream);
int tops_b200_l2norm_bwd(const tops_norm_params* p, void* stream);
int tops_b200_rmsnorm_gated_fwd(const tops_norm_params* p, void* stream);
size_t tops_b200_rmsnorm_gated_bwd_workspace_bytes(const tops_norm_params* p);
int tops_b200_rmsnorm_gated_bwd(const tops_norm_params* p, void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TOPS_B200_H_ */
