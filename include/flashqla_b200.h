/*
 * flashqla_b200 - C ABI of the B200 (sm_100a) gated-delta-rule kernels.
 *
 * The reference (FlashQLA) has no C ABI: its boundary is the Python module surface
 *   flash_qla/__init__.py:6-38.  Each entry point below is what a binding for one of those
 * Python functions calls; the struct fields carry exactly the tensors / scalars of the
 * Python signature (raw device pointers, element counts, dtype codes).  No entry point
 * allocates device memory, synchronises the device or touches torch: the caller owns
 * every buffer, including the scratch ("workspace") whose size the *_workspace_bytes
 * functions report.  Everything is launched on the stream passed in (a cudaStream_t).
 *
 * Return value: 0 on success, a negative QLA_ERR_* code otherwise;
 * qla_status_string() maps it to text, qla_last_error() gives the detail of the last
 * failure on the calling thread.
 */
#ifndef FLASHQLA_B200_H_
#define FLASHQLA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QLA_ABI_VERSION 2

#if defined(QLA_BUILDING_LIB)
#define QLA_API __attribute__((visibility("default")))
#else
#define QLA_API
#endif

enum {
  QLA_OK = 0,
  QLA_ERR_INVALID_ARG = -1, /* shape / pointer / flag combination rejected               */
  QLA_ERR_UNSUPPORTED = -2, /* valid in the reference but outside K=V=128, chunk 64, ...  */
  QLA_ERR_CUDA = -3,        /* a CUDA runtime / driver call failed                        */
  QLA_ERR_WORKSPACE = -4,   /* workspace missing or too small                             */
  QLA_ERR_DEVICE = -5       /* the device status word reported a fault (bounded wait ...) */
};

enum { QLA_DT_F32 = 0, QLA_DT_BF16 = 1, QLA_DT_F16 = 2 };

enum { /* flags of QlaRecurrentArgs */
  QLA_REC_QK_L2NORM = 1,            /* use_qk_l2norm_in_kernel                      */
  QLA_REC_DISABLE_STATE_UPDATE = 2, /* disable_state_update                         */
  QLA_REC_A_IS_LOG_DECAY = 4,       /* a_is_log_decay: a already holds g            */
  QLA_REC_B_IS_BETA = 8             /* b_is_beta: b already holds beta              */
};

/*
 * Recurrent decode / spec-decode verify / tree verify.
 * Replaces fused_sigmoid_gating_delta_rule_update,
 *   flash_qla/ops/gated_delta_rule/recurrent_fused.py:6287-7534 (dispatcher) and the kernels
 *   :290-487 (ragged), :4003-4256 (decode), :5656-5944 (verify), :5952-6249 (tree verify).
 * Layouts (all contiguous): q,k [NT,Hk,128]; v,o [NT,Hv,128]; a,b [NT,Hv]; A_log,dt_bias [Hv];
 * state [slots,Hv,128(V),128(K)] fp32 or bf16 (state_dtype), updated in place;
 * inter [slots,inter_steps,Hv,128,128].  Index tensors are checked on the device: a slot outside its pool,
 * cu_seqlens boundaries outside [0, total_tokens] or a parent outside the cached steps never touch memory
 * (the sequence is treated as padding / the access is skipped) and raise the status word.
 */
typedef struct QlaRecurrentArgs {
  int32_t num_seqs;        /* N                                                              */
  int32_t total_tokens;    /* NT                                                             */
  int32_t tokens_per_seq;  /* > 0: every sequence has this many tokens; 0: use cu_seqlens    */
  int32_t num_k_heads;     /* Hk                                                             */
  int32_t num_v_heads;     /* Hv, multiple of Hk                                             */
  int32_t qkv_dtype;       /* QLA_DT_BF16 | QLA_DT_F16 (q, k, v and o)                       */
  int32_t a_dtype;         /* dtype of a and b                                               */
  int32_t a_log_dtype;     /* dtype of A_log                                                 */
  int32_t dt_bias_dtype;   /* dtype of dt_bias                                               */
  int32_t inter_dtype;     /* QLA_DT_F32 | QLA_DT_BF16, ignored when inter == NULL           */
  int32_t inter_steps;     /* second extent of inter                                         */
  int32_t parents_stride;  /* row stride (elements) of parents                               */
  int32_t flags;           /* QLA_REC_*                                                      */
  int32_t rows_per_cta;    /* 0 = choose; 16 or 32 rows of V per CTA                         */
  int64_t state_slots;     /* first extent of state                                          */
  int64_t inter_slots;     /* first extent of inter                                          */
  float scale;
  float softplus_beta;
  float softplus_threshold;
  const void* A_log;
  const void* a;
  const void* dt_bias;
  const void* q;
  const void* k;
  const void* v;
  const void* b;
  void* state;                  /* initial_state_source                                      */
  const int32_t* state_indices; /* [N] slot per sequence, < 0 = zero state and no write-back; NULL = identity */
  const int32_t* cu_seqlens;    /* [N+1] or NULL                                             */
  void* inter;                  /* intermediate_states_buffer or NULL                        */
  const int32_t* inter_indices; /* [N] or NULL (identity)                                    */
  const int32_t* parents;       /* retrieve_parent_token [N,parents_steps] or NULL           */
  void* o;
  int32_t* status;              /* device int32 status word or NULL (see qla_chunk_fwd)      */
  int32_t state_dtype;          /* QLA_DT_F32 | QLA_DT_BF16: element type of the state pool  */
  int32_t parents_steps;        /* second extent of parents (0 when parents == NULL)         */
} QlaRecurrentArgs;

QLA_API int qla_recurrent_update(const QlaRecurrentArgs* args, void* stream);

/* Commit of accepted draft tokens after a speculative-decoding verify step.  The reference's verify
 * convention leaves the state pool untouched (disable_state_update) and caches the state after every draft
 * token in intermediate_states_buffer (recurrent_fused.py:5912-5925); writing the accepted one back is left
 * to the serving framework there.  For every sequence n with accepted[n] > 0:
 *   state[state_indices[n]] = fp32(inter[inter_indices[n], accepted[n] - 1])      (all heads, V x K)
 * accepted[n] == 0 keeps the old state.  Slots outside their pools raise the device status word.      */
typedef struct QlaStateCommitArgs {
  int32_t num_seqs;        /* N                                                               */
  int32_t num_v_heads;     /* Hv                                                              */
  int32_t inter_dtype;     /* QLA_DT_F32 | QLA_DT_BF16                                        */
  int32_t inter_steps;     /* second extent of inter                                          */
  int64_t inter_slots;     /* first extent of inter                                           */
  int64_t state_slots;     /* first extent of state                                           */
  const void* inter;       /* [inter_slots, inter_steps, Hv, 128, 128]                        */
  const int32_t* accepted; /* [N] number of accepted tokens, 0 .. inter_steps                 */
  const int32_t* state_indices; /* [N] or NULL (identity)                                     */
  const int32_t* inter_indices; /* [N] or NULL (identity)                                     */
  void* state;             /* [state_slots, Hv, 128, 128] fp32 or bf16, updated in place      */
  int32_t* status;         /* device int32 status word or NULL                                */
  int32_t state_dtype;     /* QLA_DT_F32 | QLA_DT_BF16                                        */
  int32_t reserved;
} QlaStateCommitArgs;

QLA_API int qla_state_commit(const QlaStateCommitArgs* args, void* stream);

enum { /* flags of QlaChunkFwdArgs / QlaChunkBwdArgs */
  QLA_CHUNK_TRANSPOSE_STATE = 1, /* states are [N,Hv,V,K] instead of [N,Hv,K,V]            */
  QLA_CHUNK_STATE_ONLY = 2,      /* skip q / o: only h, v_new and the final state           */
  QLA_CHUNK_QK_L2NORM = 4,       /* use q / |q| and k / |k| (rows, eps 1e-6) without a pass
                                    over q and k: needs qk_rnorm                            */
  QLA_CHUNK_SKIP_PREPARE = 8,    /* g_cumsum, A and w are inputs (from an earlier call)     */
  QLA_CHUNK_INIT_IDENTITY = 16,  /* start every sequence from S = I instead of h0          */
  QLA_CHUNK_ZERO_V = 32,         /* treat v as zero (with INIT_IDENTITY: the K x K transition
                                    matrix of the chunks, used by context parallelism)      */
  QLA_CHUNK_PREPARE_ONLY = 64,   /* compute g_cumsum, A and w only; no scan                  */
  QLA_CHUNK_A_GIVEN = 128,       /* g_cumsum and A are inputs, w is rebuilt from them (the
                                    backward's recomputation of h / v_new)                  */
  QLA_CHUNK_TABLES_READY = 256,  /* the workspace already holds the chunk tables of these
                                    cu_seqlens (an earlier call with the same cu_seqlens,
                                    num_seqs and workspace filled it): no table launch      */
  QLA_CHUNK_GATE_ACT = 512,      /* g holds the raw gate input a: the preparation step uses
                                    g = -exp(A_log[h]) * softplus(a + dt_bias[h]) (softplus
                                    with beta 1, threshold 20, as the recurrent op)          */
  QLA_CHUNK_BETA_LOGIT = 1024,   /* beta holds logits: the preparation step uses sigmoid(beta)
                                    and writes it to beta_out, which the scan reads           */
  QLA_CHUNK_H0_KV_F32 = 2048,    /* h0 is fp32 [N,Hv,K,V] whatever QLA_CHUNK_TRANSPOSE_STATE and
                                    state_dtype say for final_state (the start states of
                                    context-parallel segments)                                */
  QLA_CHUNK_OUT_GATED_RMSNORM = 8192, /* o leaves through the gated RMS norm that follows the op in a GDN
                                    layer: o * rsqrt(mean_v(o^2) + norm_eps) * norm_weight[v] *
                                    silu(norm_gate[t,h,v]); inference epilogue (no h / v_new)    */
  QLA_CHUNK_DUAL_TRANSITION = 4096 /* with QLA_CHUNK_STATE_ONLY: the same launch also runs the
                                    INIT_IDENTITY | ZERO_V pass of every (sequence, head) with
                                    chunk_limit_b, writing its K x K result to row seq_map_b[n]
                                    of final_state_b (fp32): warm-up and transition pass of
                                    context parallelism as one grid                           */
};

/*
 * Chunked prefill forward (chunk 64, K = V = 128).
 * Replaces chunk_gated_delta_rule_fwd, flash_qla/ops/gated_delta_rule/chunk/__init__.py:23-86
 * (chunk_local_cumsum ops/utils/cumsum.py:134, kkt_solve chunk/hopper/kkt_solve.py:302,
 *  fused_gdr_fwd chunk/hopper/fused_fwd.py:532).
 * Layouts: q,k [B,T,Hk,128]; v,o,v_new [B,T,Hv,128]; g,beta,g_cumsum [B,T,Hv];
 * A [B,T,Hv,64]; h [B*NC or total chunks,Hv,128,128] bf16; states fp32 [N,Hv,128,128].
 * With cu_seqlens (device int32 [N+1]) B must be 1 and T is the packed token count.
 * seq_map (device int32 [N], optional) gives for every sequence the row of final_state
 * it writes (< 0: none); NULL = identity.  h0_map (device int32 [N], optional) likewise gives the row of
 * h0 a sequence starts from (< 0: zero state).  With both maps set to the slot indices of a state pool and
 * h0 == final_state == the pool ([slots,Hv,V,K] with QLA_CHUNK_TRANSPOSE_STATE; fp32 or bf16, state_dtype)
 * a batch is prefilled from and into the pool of the recurrent op in place; sequences must not share a slot.
 * Workspace: qla_chunk_fwd_workspace_bytes(args) bytes of device memory, 16-byte aligned;
 * it holds the per-sequence chunk tables when cu_seqlens is given.
 */
typedef struct QlaChunkFwdArgs {
  int32_t batch;       /* B                                                                  */
  int32_t seq_len;     /* T                                                                  */
  int32_t num_seqs;    /* N: B, or the number of cu_seqlens intervals                        */
  int32_t num_k_heads;
  int32_t num_v_heads;
  int32_t qkv_dtype;   /* QLA_DT_BF16 | QLA_DT_F16                                           */
  int32_t gate_dtype;  /* dtype of g                                                         */
  int32_t beta_dtype;  /* dtype of beta                                                      */
  int32_t flags;       /* QLA_CHUNK_*                                                        */
  int32_t max_chunks_per_seq; /* upper bound used to size grids; 0 = derive from T           */
  float scale;
  const void* q;
  const void* k;
  const void* v;
  const void* g;       /* raw per-token log decay                                            */
  const void* beta;
  const void* h0;      /* NULL = zero                                                        */
  const int32_t* cu_seqlens;
  const int32_t* seq_map;
  const int32_t* seq_order;   /* device int32 [N] or NULL: the order in which sequences are handed to the
                                 GPU (a permutation of 0..N-1); longest first shortens the tail of
                                 batches with very different lengths                          */
  const int32_t* chunk_limit; /* device int32 [N,Hv] or NULL: run only the last chunk_limit chunks
                                 of each (sequence, head), starting from a zero state        */
  float* g_cumsum;     /* out; in with QLA_CHUNK_SKIP_PREPARE                                */
  void* A;             /* out; in with QLA_CHUNK_SKIP_PREPARE                                */
  void* w;             /* [B,T,Hv,K] in the q/k/v dtype: -(A diag(beta e^g) K), the state-dependent
                          operand of every chunk; out, in with QLA_CHUNK_SKIP_PREPARE        */
  float* qk_rnorm;     /* [B,T,Hk,2] fp32, only with QLA_CHUNK_QK_L2NORM: 1/|q_t|, 1/|k_t|; written by
                          the preparation step, read by the scan (in with QLA_CHUNK_SKIP_PREPARE) */
  const float* A_log;  /* [Hv] fp32, only with QLA_CHUNK_GATE_ACT                            */
  const float* dt_bias;/* [Hv] fp32, only with QLA_CHUNK_GATE_ACT                            */
  float* beta_out;     /* [B,T,Hv] fp32 out, only with QLA_CHUNK_BETA_LOGIT: sigmoid(beta); pass it as
                          `beta` (fp32) to later QLA_CHUNK_SKIP_PREPARE calls                 */
  void* o;             /* out, NULL with QLA_CHUNK_STATE_ONLY                                */
  void* h;             /* out or NULL                                                        */
  void* v_new;         /* out or NULL                                                        */
  void* final_state;   /* out or NULL                                                        */
  void* workspace;
  size_t workspace_bytes;
  int32_t* status;     /* device int32, must be 0 on entry; kernels write a non-zero code on a fault */
  const int32_t* h0_map; /* device int32 [N] or NULL: row of h0 per sequence, < 0 = zero state        */
  int32_t state_dtype; /* QLA_DT_F32 | QLA_DT_BF16: element type of h0 and final_state               */
  int32_t reserved;
  const int32_t* chunk_limit_b; /* QLA_CHUNK_DUAL_TRANSITION: chunk limits [N,Hv] of the second pass  */
  const int32_t* seq_map_b;     /* QLA_CHUNK_DUAL_TRANSITION: output rows [N] of the second pass      */
  float* final_state_b;         /* QLA_CHUNK_DUAL_TRANSITION: fp32 [rows,Hv,128,128] out              */
  const void* norm_gate;        /* QLA_CHUNK_OUT_GATED_RMSNORM: z [B,T,Hv,128] in the q/k/v dtype     */
  const float* norm_weight;     /* QLA_CHUNK_OUT_GATED_RMSNORM: fp32 [128]                            */
  float norm_eps;
  int32_t reserved2;
  const int32_t* lead;          /* [num_seqs, Hv] or NULL: chunks in FRONT of an interval (tokens of the interval
                                   before it in the same sequence) that are run first from a zero state, their
                                   outputs not stored: the warm-up of a context-parallel segment inside its own
                                   scan (qla_cp_plan writes it); an interval with lead > 0 ignores h0          */
} QlaChunkFwdArgs;

QLA_API size_t qla_chunk_fwd_workspace_bytes(const QlaChunkFwdArgs* args);
QLA_API int qla_chunk_fwd(const QlaChunkFwdArgs* args, void* stream);

/*
 * qla_chunk_fwd for callers that cannot allocate device memory.  No counterpart in the reference (its
 * Python layer allocates freely through torch).  Meant for hosts that reserve the whole GPU at start-up
 * and forbid cudaMalloc afterwards: the chunk tables qla_chunk_fwd would put into a caller-provided
 * workspace live in a fixed device array inside the library (about 32 KiB per GPU, kept until exit).
 * args->workspace / workspace_bytes are ignored.  Calls with cu_seqlens and more than
 * QLA_NOALLOC_MAX_SEQS sequences are rejected with QLA_ERR_INVALID_ARG.  All calls on one GPU share the
 * array: calls that can overlap on the GPU race.  QLA_CHUNK_TABLES_READY has no meaning with a shared
 * array (another call may have rewritten it) and is ignored: every call recomputes the tables.  The first
 * call on each GPU resolves the array's device address and sets the kernels' shared-memory attribute
 * (cudaFuncSetAttribute), so it should be made before any stream capture.  No cudaMalloc / cudaFree inside.
 */
#define QLA_NOALLOC_MAX_SEQS 4096
QLA_API int qla_chunk_fwd_noalloc(const QlaChunkFwdArgs* args, void* stream);

/*
 * Chunked backward: dq, dk, dv, dbeta, dg (w.r.t. the raw gate) and dh0.
 * Replaces chunk_gated_delta_rule_bwd, flash_qla/ops/gated_delta_rule/chunk/__init__.py:89-182
 * (fused_gdr_bwd chunk/hopper/fused_bwd.py:898, the decomposed stages chunk/blackwell/bwd_sm12x.py:768-780,
 * group_reduce_vector ops/utils/group_reduce.py:60, reverse chunk_local_cumsum ops/utils/cumsum.py:134).
 * g_cumsum, A, w, h and v_new are the tensors qla_chunk_fwd produced for the same inputs (h with one entry
 * per chunk: the state entering it; v_new = the "new values" of every token; w = the prepared operand, which
 * QLA_CHUNK_PREPARE_ONLY | QLA_CHUNK_A_GIVEN rebuilds from g_cumsum and A when it was not kept).  dq / dk come out already
 * summed over the v-heads that share a k-head; dg is already mapped back from cumulative to per-token
 * gates.  dh0 is written iff the pointer is non-NULL.
 * Workspace: qla_chunk_bwd_workspace_bytes(args) bytes, 16-byte aligned.
 */
typedef struct QlaChunkBwdArgs {
  int32_t batch;
  int32_t seq_len;
  int32_t num_seqs;
  int32_t num_k_heads;
  int32_t num_v_heads;
  int32_t qkv_dtype;   /* q, k, v, A, h, v_new, do, dq, dk, dv                                  */
  int32_t beta_dtype;
  int32_t flags;       /* QLA_CHUNK_TRANSPOSE_STATE applies to dht and dh0                       */
  float scale;
  const void* q;
  const void* k;
  const void* v;
  const float* g_cumsum;
  const void* beta;
  const void* A;
  const void* h;
  const void* v_new;
  const void* w;            /* [B,T,Hv,128] as in QlaChunkFwdArgs                               */
  const void* d_o;          /* gradient of o                                                     */
  const float* dht;         /* gradient of the final state or NULL                               */
  const int32_t* cu_seqlens;
  void* dq;
  void* dk;
  void* dv;
  float* dbeta;
  float* dg;
  float* dh0;               /* or NULL                                                           */
  void* workspace;
  size_t workspace_bytes;
  int32_t* status;
  /* Context parallelism of the reverse scan (long sequences, few heads; the reference's backward has none: its
   * grid is sequences x heads, chunk/hopper/fused_bwd.py:79).  Main call: with num_segments > 0 the scan runs over
   * the intervals seg_cu (multiples of 64 tokens inside a sequence) starting from seg_dht (fp32 [num_segments,Hv,
   * K,V]: the state gradient entering every segment from the right) and the first segment of every sequence
   * writes dh0 (seg_dh0_map: row of dh0 or < 0).  State-only call (QLA_CHUNK_STATE_ONLY): cu_seqlens are the
   * intervals; only the first chunk_limit[n,h] chunks of an interval are scanned and the gradient leaving them on
   * the left goes to row out_map[n] of dh0; with QLA_CHUNK_DUAL_TRANSITION the same launch also produces the
   * K x K transition matrices of those scans (chunk_limit_b, out_map_b, out_b). */
  int32_t num_segments;
  int32_t reserved;
  const int32_t* seg_cu;
  const float* seg_dht;
  const int32_t* seg_dh0_map;
  const int32_t* chunk_limit;
  const int32_t* out_map;
  const int32_t* chunk_limit_b;
  const int32_t* out_map_b;
  float* out_b;
  const int32_t* seg_lead;   /* with num_segments: [num_segments, Hv] chunks BEHIND a segment that its reverse scan runs
                                first from a zero gradient, nothing of them stored (qla_cp_plan with reverse and lead
                                writes it); a segment with seg_lead > 0 ignores its row of seg_dht; NULL: none        */
} QlaChunkBwdArgs;

QLA_API size_t qla_chunk_bwd_workspace_bytes(const QlaChunkBwdArgs* args);
QLA_API int qla_chunk_bwd(const QlaChunkBwdArgs* args, void* stream);

/*
 * Intra-card context parallelism (long sequences, few heads): helpers around qla_chunk_fwd.
 * Replaces intra_card_cp_preprocess, flash_qla/ops/gated_delta_rule/chunk/cp_context.py:117-176
 * (get_warmup_chunks chunk/hopper/cp_fwd.py:66, correct_initial_states chunk/hopper/cp_fwd.py:253;
 * the segment-end states come from qla_chunk_fwd with QLA_CHUNK_STATE_ONLY and chunk_limit).
 *
 * qla_cp_plan: for every (segment, head) the number of trailing chunks whose accumulated log decay
 * first drops below `threshold` (warm_limit), or - when the segment never decays that far - all its
 * chunks, in which case m_limit holds the same count (0 otherwise) and the K x K transition matrix of
 * the segment is required.  seg_next[s] = index of the segment that continues segment s, < 0 if s ends
 * its sequence (then both limits are 0).
 */
typedef struct QlaCpPlanArgs {
  int32_t num_segments;
  int32_t num_v_heads;
  float threshold;            /* e.g. -10: contributions below exp(-10) are dropped            */
  const float* g_cumsum;      /* [NT, Hv] chunk-local cumulative gates                          */
  const int32_t* cu_seqlens;  /* [num_segments + 1] segment boundaries (multiples of 64 inside a sequence) */
  const int32_t* seg_next;    /* [num_segments]                                                 */
  int32_t* warm_limit;        /* out [num_segments, Hv]                                         */
  int32_t* m_limit;           /* out [num_segments, Hv]                                         */
  /* optional: start states of the segments, written by the same launch.  seg_start_of[s] = index of the
   * original sequence segment s starts (< 0: s continues a sequence).  Row s of cp_h0 becomes the caller's
   * initial state of that sequence (row h0_map[r] of h0, or r; < 0 or h0 == NULL: zero), converted to fp32
   * [K,V]; rows of continuing segments are zeroed (the warm-up pass adds their state).                    */
  float* cp_h0;               /* out fp32 [num_segments, Hv, 128, 128] or NULL                  */
  const int32_t* seg_start_of; /* [num_segments], with cp_h0                                    */
  const void* h0;             /* caller's initial states or NULL                                */
  const int32_t* h0_map;      /* [number of original sequences] or NULL                         */
  int32_t h0_dtype;           /* QLA_DT_F32 | QLA_DT_BF16                                       */
  int32_t h0_transposed;      /* caller's states are [V,K]                                      */
  int32_t reverse;            /* plan for the backward scan: count LEADING chunks of a segment (the
                                 accumulated decay from its start) instead of trailing ones; seg_next
                                 then names the segment's predecessor (< 0: none)                 */
  int32_t num_raw_seqs;       /* with lead: number of original sequences                        */
  /* optional (with cp_h0; with reverse the roles of predecessor and successor swap): warm-up inside the main scan.  lead[s,h] = trailing chunks of the
   * segment before s that the main scan's CTA of s runs first, from a zero state and without storing their
   * output (QlaChunkFwdArgs.lead): the state-only pass then has nothing to do for that sequence and head
   * (warm_limit = 0).  A sequence and head in which some segment never decays below the threshold keeps the
   * state-only pass, the transition matrices and the chain (lead = 0 there).  Only the rows of cp_h0 that start a
   * sequence are initialised in this mode (the others are written by the state-only pass or not read at all).  */
  int32_t* lead;              /* out [num_segments, Hv] or NULL                                 */
  const int32_t* raw_first_seg; /* [num_raw_seqs + 1] first segment of every original sequence; with lead */
} QlaCpPlanArgs;

QLA_API int qla_cp_plan(const QlaCpPlanArgs* args, void* stream);

/*
 * qla_cp_chain: h0[seg + 1] += M[seg] * h0[seg] for every (segment, head) with m_limit != 0, walking
 * the segments of each original sequence in order.  h0 and M are fp32 [num_segments, Hv, 128, 128]
 * ([K, V] and [K, K]); raw_first_seg [num_raw_seqs + 1] gives the first segment of every original
 * sequence.
 */
typedef struct QlaCpChainArgs {
  int32_t num_raw_seqs;
  int32_t num_v_heads;
  float* h0;
  const float* M;
  const int32_t* m_limit;
  const int32_t* raw_first_seg;
  int32_t reverse;            /* backward: h0[seg - 1] += M[seg] * h0[seg], last segment first  */
  int32_t reserved;
} QlaCpChainArgs;

QLA_API int qla_cp_chain(const QlaCpChainArgs* args, void* stream);

/*
 * Tracing (no counterpart in the reference, whose profiling is torch.profiler around whole kernels,
 * flash_qla/utils/profiler.py:8-25): when a device buffer of at least 192 int64 is registered, CTA 0 of
 * every later chunk-scan launch stamps clock64() at its phase boundaries for chunks 4..7, laid out as
 * [role: 0 MMA issuer, 1 chain warpgroup, 2 side warpgroup][chunk][16 events].  If the buffer holds
 * 192 + 3 * CTAs entries, every CTA also records (start ns, end ns, SM id) there.  NULL switches it off.
 */
QLA_API int qla_set_trace_buffer(long long* device_buffer, size_t count);

/*
 * Self-test of the fault path (no counterpart in the reference, whose kernels wait without a bound): launches
 * one warp that waits, with the bounded mbarrier wait every kernel of the library uses, for a barrier nothing
 * completes.  After limit_ns (at most one second) the wait gives up, writes (1 | 255 << 8 | parity << 16 |
 * warp << 20) to *status and the kernel returns; the context stays usable.
 */
QLA_API int qla_selftest_bounded_wait(int32_t* status, uint64_t limit_ns, void* stream);

/*
 * Launch constants of the library's main kernels ("chunk_fwd_kernel", "kkt_solve_kernel", "bwd_scan_kernel",
 * "bwd_chunk_kernel", "recurrent_kernel"): threads per block and dynamic shared-memory bytes, as compiled.
 * The manifest written beside the library (and beside the per-kernel cubins) carries the same figures for
 * launchers that load the cubins without the CUDA runtime, the role of the reference's AOT export
 * (flash_qla/compile_sm12x_gdn.py:580-669).
 */
QLA_API int qla_kernel_launch_info(const char* kernel, int32_t* block_threads, size_t* dynamic_smem_bytes);

QLA_API const char* qla_status_string(int code);
QLA_API const char* qla_last_error(void);
QLA_API int qla_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FLASHQLA_B200_H_ */
