// Parameter blocks shared between the chunk kernels and their host entry points.
#pragma once

#include "ptx_sm100.cuh"

namespace qla {

struct KktParams {
  const void* g;
  const void* beta;
  float* g_cumsum;              // out; in when A_in is given
  void* A;                      // out (unused when A_in is given)
  const void* A_in;             // optional: A from an earlier call -> only w is produced
  void* w;                      // out: -(A diag(beta gamma) K), [NT, Hv, 128]
  float* rnorm;                 // out or NULL: [NT, Hk, 2] = 1/|q_t|, 1/|k_t| (in-kernel q/k L2 norm)
  float norm_eps;               // added to the squared norm
  const float* A_log;           // [Hv] or NULL: g = -exp(A_log[h]) * softplus(raw gate + dt_bias[h])
  const float* dt_bias;         // [Hv], with A_log
  float* beta_out;              // [NT, Hv] or NULL: beta holds logits, sigmoid(beta) is used and written here
  const int32_t* cu_seqlens;    // NULL: equal-length batch of `seq_len` tokens
  const int32_t* pair_offsets;  // [num_seqs + 1] exclusive scan of ceil(len / 128), varlen only
  int* status;
  int num_seqs, seq_len, num_k_heads, num_v_heads;
  int gate_dtype, beta_dtype;
};

struct FwdParams {
  const float* g_cumsum;        // [NT, Hv]
  const void* beta;             // [NT, Hv]
  const void* h0;               // [n_h0, Hv, 128, 128] (state_dtype) or NULL
  const int32_t* h0_map;        // [num_seqs] row of h0 a sequence starts from (< 0: zero state) or NULL (identity)
  const int32_t* cu_seqlens;    // [num_seqs + 1] or NULL (equal-length batch)
  const int32_t* seq_map;       // [num_seqs] row of final_state (< 0: none) or NULL (identity)
  const int32_t* seq_order;     // [num_seqs] launch order (permutation) or NULL
  const float* rnorm;           // [NT, Hk, 2] = 1/|q_t|, 1/|k_t| or NULL (q, k used as they are)
  const int32_t* chunk_offsets; // [num_seqs + 1] first chunk index of each sequence (varlen h output)
  const int32_t* chunk_limit;   // [num_seqs, Hv] optional: only the LAST chunk_limit chunks are processed
  const int32_t* lead;          // [num_seqs, Hv] optional: chunks in front of the interval run first from a zero state, outputs not stored
  void* o;                      // [NT, Hv, 128]
  void* v_new;                  // [NT, Hv, 128] or NULL
  void* h;                      // [total_chunks, Hv, 128, 128] bf16/fp16 or NULL
  const void* norm_gate;        // [NT, Hv, 128] gate z of the output gated RMS norm or NULL (no norm)
  const float* norm_weight;     // [128] with norm_gate
  float norm_eps;
  void* final_state;            // [n_out, Hv, 128, 128] (state_dtype) or NULL
  int* status;
  int num_seqs, seq_len, num_k_heads, num_v_heads;
  int beta_dtype;
  int state_dtype;              // QLA_DT_F32 | QLA_DT_BF16: element type of h0 and final_state
  int transpose_state;          // final_state (and h0, unless h0_kv) stored [V, K] instead of [K, V]
  int h0_kv;                    // h0 is fp32 [K, V] whatever transpose_state / state_dtype say (context-parallel segments)
  int init_identity;            // start from S = I (ignores h0)
  int zero_v;                   // treat V as 0
  int dual;                     // second half of the grid = transition-matrix pass (identity start, zero V) with:
  const int32_t* chunk_limit_b; //   its chunk limits,
  const int32_t* seq_map_b;     //   its output rows,
  void* final_state_b;          //   and its fp32 output
  float scale;
  long long* trace;             // optional phase trace (see qla_set_trace_buffer), NULL in normal use
  long long trace_count;        // capacity of `trace` in entries
};

struct BwdParams {
  const void* q;                // [NT, Hk, 128]
  const void* k;
  const void* v;                // [NT, Hv, 128]
  const void* v_new;            // [NT, Hv, 128] saved by the forward
  const void* d_o;              // [NT, Hv, 128]
  const void* A;                // [NT, Hv, 64]
  const void* w;                // [NT, Hv, 128] -(A diag(beta gamma) K), the forward's prepared operand
  const void* h;                // [chunks, Hv, 128, 128] state entering every chunk, saved by the forward
  const float* g_cumsum;        // [NT, Hv]
  const void* beta;             // [NT, Hv]
  const float* dht;             // [N, Hv, 128, 128] or NULL
  const int32_t* cu_seqlens;
  const int32_t* chunk_offsets;
  void* dh;                     // workspace [chunks, Hv, 128 v, 128 k]: gradient of the state leaving every chunk
  void* du;                     // workspace [chunks, Hv, 128 v, 64 tokens]: gradient of v_new, transposed per chunk
  void* dq;                     // [NT, Hk, 128]
  void* dk;
  void* dv;                     // [NT, Hv, 128]
  float* dbeta;                 // [NT, Hv]
  float* dg;                    // [NT, Hv] w.r.t. the raw per-token gate
  float* dh0;                   // [N, Hv, 128, 128] or NULL
  int* status;
  long long* trace;             // optional phase trace of the per-chunk kernel (see qla_set_trace_buffer), NULL in normal use
  int num_seqs, seq_len, num_k_heads, num_v_heads;
  int beta_dtype;
  int transpose_state;
  int dht_kv;                   // dht is [K, V] whatever transpose_state says for dh0 (segment end gradients)
  float scale;
};

// The reverse scan by itself, over `num_seqs` token intervals `cu_seqlens` (sequences, or the segments of a
// context-parallel plan), with the switches of its state-only passes.
struct BwdScanMode {
  const int32_t* chunk_limit;   // [num_seqs, Hv] or NULL: only the FIRST chunk_limit chunks of an interval (<= 0: none)
  const int32_t* out_map;       // [num_seqs] row of dh0 an interval writes (< 0: none) or NULL (identity)
  const int32_t* lead;          // [num_seqs, Hv] or NULL: chunks BEHIND an interval (same sequence) that are scanned first
                                // from a zero gradient, nothing of them stored: the warm-up of a segment inside its own scan
  int chunks_upper;             // rows of the dh / du workspace in chunks (extent of the store maps); unused when state_only
  int state_only;               // no du / dh: only the state gradient leaving the interval on the left
  int dual;                     // second half of the grid: transition pass (identity start, dO treated as zero) with
  const int32_t* chunk_limit_b; //   its limits,
  const int32_t* out_map_b;     //   its output rows
  float* out_b;                 //   and its output [rows, Hv, 128, 128]
};
int launch_bwd_scan(const BwdParams& p, const BwdScanMode& mode, int64_t total_tokens, bool is_bf16,
                    cudaStream_t stream);
int launch_chunk_bwd(const BwdParams& p, int64_t total_tokens, int total_chunks_upper, bool is_bf16,
                     cudaStream_t stream);

// Trace layout: [role 0..2][chunk 4..7][16 events] clock64 stamps of CTA 0.
constexpr int kTraceRoles = 3, kTraceChunks = 4, kTraceEvents = 16, kTraceFirstChunk = 4;
long long* current_trace_buffer();
long long current_trace_count();

int launch_chunk_tables(const int32_t* cu, int n, int32_t* pair_offsets, int32_t* chunk_offsets,
                        cudaStream_t stream);
int launch_kkt_solve(const KktParams& p, const void* k, const void* q, int64_t total_tokens, int pairs_upper,
                     bool is_bf16, cudaStream_t stream);
int launch_chunk_fwd(const FwdParams& p, const void* q, const void* k, const void* v, const void* A,
                     const void* w, int64_t total_tokens, bool is_bf16, bool state_only, cudaStream_t stream);

}  // namespace qla
