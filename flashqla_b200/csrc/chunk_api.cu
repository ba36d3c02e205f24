// C-ABI entry points of the chunked prefill path: argument checks, workspace carving, launch order
//   [chunk tables] -> kkt_solve (g_cumsum, A, w) -> chunk forward scan.
// Mirrors the launch sequence of chunk_gated_delta_rule_fwd,
// flash_qla/ops/gated_delta_rule/chunk/__init__.py:23-86.
#include "chunk_params.cuh"

namespace qla {



namespace {
long long* g_trace = nullptr;
long long g_trace_count = 0;
size_t table_bytes(int num_seqs) { return ((static_cast<size_t>(num_seqs) + 1) * sizeof(int32_t) + 15) & ~size_t(15); }
}  // namespace

long long* current_trace_buffer() { return g_trace; }
long long current_trace_count() { return g_trace_count; }

}  // namespace qla

extern "C" QLA_API int qla_set_trace_buffer(long long* device_buffer, size_t count) {
  using namespace qla;
  if (device_buffer != nullptr && count < static_cast<size_t>(kTraceRoles * kTraceChunks * kTraceEvents)) {
    set_last_error("trace buffer needs %d entries", kTraceRoles * kTraceChunks * kTraceEvents);
    return QLA_ERR_INVALID_ARG;
  }
  g_trace = device_buffer;
  g_trace_count = device_buffer ? static_cast<long long>(count) : 0;
  return QLA_OK;
}

extern "C" QLA_API size_t qla_chunk_fwd_workspace_bytes(const QlaChunkFwdArgs* a) {
  if (a == nullptr || a->cu_seqlens == nullptr || a->num_seqs <= 0) return 0;
  return 2 * qla::table_bytes(a->num_seqs);
}

extern "C" QLA_API int qla_chunk_fwd(const QlaChunkFwdArgs* args, void* stream_) {
  using namespace qla;
  QLA_CHECK_ARG(args != nullptr, "args is NULL");
  const QlaChunkFwdArgs& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  QLA_CHECK_ARG(a.batch > 0 && a.seq_len >= 0 && a.num_seqs > 0, "batch, seq_len, num_seqs must be positive");
  QLA_CHECK_ARG(a.num_k_heads > 0 && a.num_v_heads > 0 && a.num_v_heads % a.num_k_heads == 0,
                "num_v_heads must be a multiple of num_k_heads");
  QLA_CHECK_SUPPORTED(a.qkv_dtype == QLA_DT_BF16 || a.qkv_dtype == QLA_DT_F16, "q, k, v must be bf16 or fp16");
  const bool varlen = a.cu_seqlens != nullptr;
  QLA_CHECK_ARG(!varlen || a.batch == 1, "with cu_seqlens the batch size must be 1");
  QLA_CHECK_ARG(varlen || a.num_seqs == a.batch, "num_seqs must equal batch without cu_seqlens");
  const bool state_only = (a.flags & QLA_CHUNK_STATE_ONLY) != 0;
  const bool skip_prepare = (a.flags & QLA_CHUNK_SKIP_PREPARE) != 0;
  QLA_CHECK_ARG(a.k && a.beta && a.g_cumsum && a.A && a.w && a.status,
                "k, beta, g_cumsum, A, w, status are required");
  QLA_CHECK_ARG((a.flags & (QLA_CHUNK_ZERO_V | QLA_CHUNK_PREPARE_ONLY)) || a.v, "v is required");
  const bool a_given = (a.flags & QLA_CHUNK_A_GIVEN) != 0;
  QLA_CHECK_ARG(skip_prepare || a_given || a.g, "g is required");
  QLA_CHECK_ARG(!(skip_prepare && a_given), "QLA_CHUNK_SKIP_PREPARE and QLA_CHUNK_A_GIVEN exclude each other");
  QLA_CHECK_ARG(state_only || (a.flags & QLA_CHUNK_PREPARE_ONLY) || (a.q && a.o),
                "q and o are required unless QLA_CHUNK_STATE_ONLY");
  const bool l2norm = (a.flags & QLA_CHUNK_QK_L2NORM) != 0;
  QLA_CHECK_ARG(!l2norm || a.qk_rnorm, "QLA_CHUNK_QK_L2NORM needs the qk_rnorm buffer");
  QLA_CHECK_ARG(!l2norm || skip_prepare || a.q, "QLA_CHUNK_QK_L2NORM needs q in the preparation step");
  QLA_CHECK_SUPPORTED(!l2norm || !(a.flags & QLA_CHUNK_A_GIVEN), "QLA_CHUNK_QK_L2NORM with QLA_CHUNK_A_GIVEN");
  QLA_CHECK_SUPPORTED(!(a.flags & QLA_CHUNK_ZERO_V) || state_only, "QLA_CHUNK_ZERO_V needs QLA_CHUNK_STATE_ONLY");
  const bool gate_act = (a.flags & QLA_CHUNK_GATE_ACT) != 0, beta_logit = (a.flags & QLA_CHUNK_BETA_LOGIT) != 0;
  QLA_CHECK_ARG(!gate_act || (a.A_log && a.dt_bias), "QLA_CHUNK_GATE_ACT needs A_log and dt_bias");
  QLA_CHECK_ARG(!beta_logit || a.beta_out, "QLA_CHUNK_BETA_LOGIT needs the beta_out buffer");
  QLA_CHECK_ARG(!(gate_act || beta_logit) || !(skip_prepare || a_given),
                "gate / beta activation belongs to the preparation step: not with SKIP_PREPARE or A_GIVEN");
  const int64_t total_tokens = static_cast<int64_t>(a.batch) * a.seq_len;
  if (total_tokens == 0) return QLA_OK;
  QLA_CHECK_ARG(total_tokens < (int64_t(1) << 31), "too many tokens");
  const bool is_bf16 = a.qkv_dtype == QLA_DT_BF16;
  QLA_CHECK_SUPPORTED(a.state_dtype == QLA_DT_F32 || a.state_dtype == QLA_DT_BF16, "states must be fp32 or bf16");
  QLA_CHECK_ARG(!(a.flags & QLA_CHUNK_DUAL_TRANSITION) ||
                    (state_only && a.chunk_limit && a.chunk_limit_b && a.seq_map_b && a.final_state_b),
                "QLA_CHUNK_DUAL_TRANSITION needs QLA_CHUNK_STATE_ONLY, chunk_limit(_b), seq_map_b and final_state_b");

  int32_t* pair_offsets = nullptr;
  int32_t* chunk_offsets = nullptr;
  if (varlen) {
    const size_t need = 2 * table_bytes(a.num_seqs);
    if (a.workspace == nullptr || a.workspace_bytes < need) {
      set_last_error("workspace of %zu bytes required, %zu given", need, a.workspace_bytes);
      return QLA_ERR_WORKSPACE;
    }
    QLA_CHECK_ARG((reinterpret_cast<uintptr_t>(a.workspace) & 15u) == 0, "workspace must be 16-byte aligned");
    pair_offsets = static_cast<int32_t*>(a.workspace);
    chunk_offsets = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(a.workspace) + table_bytes(a.num_seqs));
    if (!(a.flags & QLA_CHUNK_TABLES_READY)) {
      int rc = launch_chunk_tables(a.cu_seqlens, a.num_seqs, pair_offsets, chunk_offsets, stream);
      if (rc != QLA_OK) return rc;
    }
  }

  if (!skip_prepare) {
    KktParams kp{};
    kp.g = a_given ? static_cast<const void*>(a.g_cumsum) : a.g; kp.beta = a.beta; kp.g_cumsum = a.g_cumsum;
    kp.A = a.A; kp.A_in = a_given ? a.A : nullptr; kp.w = a.w;
    kp.rnorm = l2norm ? a.qk_rnorm : nullptr; kp.norm_eps = 1e-6f;
    kp.A_log = gate_act ? a.A_log : nullptr; kp.dt_bias = gate_act ? a.dt_bias : nullptr;
    kp.beta_out = beta_logit ? a.beta_out : nullptr;
    kp.cu_seqlens = a.cu_seqlens; kp.pair_offsets = pair_offsets; kp.status = a.status;
    kp.num_seqs = a.num_seqs; kp.seq_len = a.seq_len; kp.num_k_heads = a.num_k_heads; kp.num_v_heads = a.num_v_heads;
    kp.gate_dtype = a_given ? QLA_DT_F32 : a.gate_dtype; kp.beta_dtype = a.beta_dtype;
    const int pairs_upper = varlen ? static_cast<int>(total_tokens / 128 + a.num_seqs)
                                   : a.batch * ((a.seq_len + 127) / 128);
    int rc = launch_kkt_solve(kp, a.k, a.q, total_tokens, pairs_upper, is_bf16, stream);
    if (rc != QLA_OK) return rc;
  }

  if (a.flags & QLA_CHUNK_PREPARE_ONLY) return QLA_OK;

  FwdParams fp{};
  fp.g_cumsum = a.g_cumsum; fp.beta = a.beta; fp.h0 = a.h0; fp.h0_map = a.h0_map;
  fp.state_dtype = a.state_dtype; fp.h0_kv = (a.flags & QLA_CHUNK_H0_KV_F32) ? 1 : 0;
  fp.cu_seqlens = a.cu_seqlens; fp.seq_map = a.seq_map; fp.seq_order = a.seq_order;
  fp.rnorm = l2norm ? a.qk_rnorm : nullptr; fp.chunk_offsets = chunk_offsets;
  fp.lead = a.lead;
  fp.chunk_limit = a.chunk_limit; fp.o = a.o; fp.v_new = a.v_new; fp.h = a.h; fp.final_state = a.final_state;
  fp.status = a.status; fp.num_seqs = a.num_seqs; fp.seq_len = a.seq_len;
  fp.num_k_heads = a.num_k_heads; fp.num_v_heads = a.num_v_heads; fp.beta_dtype = a.beta_dtype;
  fp.transpose_state = (a.flags & QLA_CHUNK_TRANSPOSE_STATE) ? 1 : 0;
  fp.init_identity = (a.flags & QLA_CHUNK_INIT_IDENTITY) ? 1 : 0;
  fp.zero_v = (a.flags & QLA_CHUNK_ZERO_V) ? 1 : 0;
  const bool out_norm = (a.flags & QLA_CHUNK_OUT_GATED_RMSNORM) != 0;
  QLA_CHECK_ARG(!out_norm || (a.norm_gate && a.norm_weight), "QLA_CHUNK_OUT_GATED_RMSNORM needs norm_gate and norm_weight");
  QLA_CHECK_SUPPORTED(!out_norm || (!state_only && a.h == nullptr && a.v_new == nullptr),
                      "the output norm is an inference epilogue: not with QLA_CHUNK_STATE_ONLY, h or v_new");
  QLA_CHECK_SUPPORTED(a.state_dtype != QLA_DT_BF16 || (!state_only && !out_norm && a.h == nullptr && a.v_new == nullptr),
                      "bf16 states are an inference path: not with QLA_CHUNK_STATE_ONLY, h, v_new or the output norm");
  fp.norm_gate = out_norm ? a.norm_gate : nullptr; fp.norm_weight = a.norm_weight; fp.norm_eps = a.norm_eps;
  fp.dual = (a.flags & QLA_CHUNK_DUAL_TRANSITION) ? 1 : 0;
  fp.chunk_limit_b = a.chunk_limit_b; fp.seq_map_b = a.seq_map_b; fp.final_state_b = a.final_state_b;
  fp.scale = a.scale;
  if (beta_logit) {  // the scan reads the activated values the preparation step just wrote
    fp.beta = a.beta_out;
    fp.beta_dtype = QLA_DT_F32;
  }
  fp.trace = current_trace_buffer();
  fp.trace_count = current_trace_count();
  const void* v = a.v ? a.v : a.k;  // never dereferenced with QLA_CHUNK_ZERO_V, only used for the tensor map
  return launch_chunk_fwd(fp, a.q, a.k, v, a.A, a.w, total_tokens, is_bf16, state_only, stream);
}

namespace qla {
namespace {
struct BwdWorkspace {
  size_t tables, dh, du, total;
  int chunks_upper;
};
BwdWorkspace bwd_workspace(const QlaChunkBwdArgs& a) {
  BwdWorkspace w{};
  const int64_t nt = static_cast<int64_t>(a.batch) * a.seq_len;
  const bool varlen = a.cu_seqlens != nullptr;
  w.chunks_upper = varlen ? static_cast<int>(nt / kChunk + a.num_seqs) : a.batch * ((a.seq_len + kChunk - 1) / kChunk);
  w.tables = varlen ? 2 * table_bytes(a.num_seqs) : 0;
  w.dh = ((static_cast<size_t>(w.chunks_upper) * a.num_v_heads * kHeadDim * kHeadDim * 2) + 15) & ~size_t(15);
  w.du = ((static_cast<size_t>(w.chunks_upper) * a.num_v_heads * kHeadDim * kChunk * 2) + 15) & ~size_t(15);
  w.total = w.tables + w.dh + w.du + (a.num_segments > 0 ? 2 * table_bytes(a.num_segments) : 0);
  return w;
}
}  // namespace
}  // namespace qla

extern "C" QLA_API size_t qla_chunk_bwd_workspace_bytes(const QlaChunkBwdArgs* a) {
  if (a == nullptr || a->batch <= 0 || a->num_seqs <= 0 || a->num_v_heads <= 0) return 0;
  return qla::bwd_workspace(*a).total;
}

extern "C" QLA_API int qla_chunk_bwd(const QlaChunkBwdArgs* args, void* stream_) {
  using namespace qla;
  QLA_CHECK_ARG(args != nullptr, "args is NULL");
  const QlaChunkBwdArgs& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  QLA_CHECK_ARG(a.batch > 0 && a.seq_len >= 0 && a.num_seqs > 0, "batch, seq_len, num_seqs must be positive");
  QLA_CHECK_ARG(a.num_k_heads > 0 && a.num_v_heads > 0 && a.num_v_heads % a.num_k_heads == 0,
                "num_v_heads must be a multiple of num_k_heads");
  QLA_CHECK_SUPPORTED(a.qkv_dtype == QLA_DT_BF16 || a.qkv_dtype == QLA_DT_F16, "q, k, v must be bf16 or fp16");
  const bool varlen = a.cu_seqlens != nullptr;
  const bool state_only = (a.flags & QLA_CHUNK_STATE_ONLY) != 0;
  QLA_CHECK_ARG(!varlen || a.batch == 1, "with cu_seqlens the batch size must be 1");
  QLA_CHECK_ARG(varlen || a.num_seqs == a.batch, "num_seqs must equal batch without cu_seqlens");
  QLA_CHECK_ARG(a.q && a.k && a.g_cumsum && a.d_o && a.w, "NULL input tensor");
  const int64_t total_tokens = static_cast<int64_t>(a.batch) * a.seq_len;
  if (total_tokens == 0) return QLA_OK;
  const bool is_bf16 = a.qkv_dtype == QLA_DT_BF16;

  BwdParams p{};
  p.q = a.q; p.k = a.k; p.v = a.v; p.v_new = a.v_new; p.d_o = a.d_o; p.A = a.A; p.h = a.h; p.w = a.w;
  p.g_cumsum = a.g_cumsum; p.beta = a.beta; p.dht = a.dht; p.cu_seqlens = a.cu_seqlens;
  p.dq = a.dq; p.dk = a.dk; p.dv = a.dv; p.dbeta = a.dbeta; p.dg = a.dg; p.dh0 = a.dh0;
  p.num_seqs = a.num_seqs; p.seq_len = a.seq_len; p.num_k_heads = a.num_k_heads; p.num_v_heads = a.num_v_heads;
  p.beta_dtype = a.beta_dtype; p.transpose_state = (a.flags & QLA_CHUNK_TRANSPOSE_STATE) ? 1 : 0;
  p.scale = a.scale; p.status = a.status;
  p.trace = current_trace_buffer();

  if (state_only) {
    // A state-only pass of the reverse scan (context parallelism): over the first chunk_limit chunks of every
    // interval, from a zero gradient (or dht), writing only the gradient that leaves the interval on the left
    // to row out_map[n] of dh0; optionally the transition-matrix pass in the same launch.
    QLA_CHECK_ARG(a.dh0 != nullptr, "a state-only pass writes dh0");
    QLA_CHECK_ARG(varlen, "a state-only pass works on intervals given by cu_seqlens");
    const bool dual = (a.flags & QLA_CHUNK_DUAL_TRANSITION) != 0;
    QLA_CHECK_ARG(!dual || (a.chunk_limit && a.chunk_limit_b && a.out_map_b && a.out_b),
                  "QLA_CHUNK_DUAL_TRANSITION needs chunk_limit(_b), out_map_b and out_b");
    BwdScanMode mode{};
    mode.chunk_limit = a.chunk_limit; mode.out_map = a.out_map; mode.state_only = 1; mode.dual = dual ? 1 : 0;
    mode.chunk_limit_b = a.chunk_limit_b; mode.out_map_b = a.out_map_b; mode.out_b = a.out_b;
    return launch_bwd_scan(p, mode, total_tokens, is_bf16, stream);
  }

  QLA_CHECK_ARG(a.v && a.beta && a.A, "NULL input tensor");
  QLA_CHECK_SUPPORTED(a.h && a.v_new, "h and v_new from the forward are required");
  QLA_CHECK_ARG(a.dq && a.dk && a.dv && a.dbeta && a.dg, "NULL output tensor");
  const BwdWorkspace w = bwd_workspace(a);
  if (a.workspace == nullptr || a.workspace_bytes < w.total) {
    set_last_error("workspace of %zu bytes required, %zu given", w.total, a.workspace_bytes);
    return QLA_ERR_WORKSPACE;
  }
  QLA_CHECK_ARG((reinterpret_cast<uintptr_t>(a.workspace) & 15u) == 0, "workspace must be 16-byte aligned");
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  int32_t* chunk_offsets = nullptr;
  if (varlen) {
    int32_t* pair_offsets = reinterpret_cast<int32_t*>(ws);
    chunk_offsets = reinterpret_cast<int32_t*>(ws + table_bytes(a.num_seqs));
    int rc = launch_chunk_tables(a.cu_seqlens, a.num_seqs, pair_offsets, chunk_offsets, stream);
    if (rc != QLA_OK) return rc;
  }
  p.chunk_offsets = chunk_offsets; p.dh = ws + w.tables; p.du = ws + w.tables + w.dh;

  // reverse scan: over whole sequences, or over the segments of a context-parallel plan (segments are whole
  // chunks, so the chunk numbering of the workspace is that of the sequences)
  BwdParams sp = p;
  BwdScanMode mode{};
  mode.chunks_upper = w.chunks_upper;
  if (a.num_segments > 0) {
    QLA_CHECK_ARG(a.seg_cu && a.seg_dht && a.seg_dh0_map, "segments need seg_cu, seg_dht and seg_dh0_map");
    int32_t* seg_tables = reinterpret_cast<int32_t*>(ws + w.tables + w.dh + w.du);
    int32_t* seg_chunk_offsets = reinterpret_cast<int32_t*>(ws + w.tables + w.dh + w.du + table_bytes(a.num_segments));
    int rc = launch_chunk_tables(a.seg_cu, a.num_segments, seg_tables, seg_chunk_offsets, stream);
    if (rc != QLA_OK) return rc;
    sp.cu_seqlens = a.seg_cu; sp.num_seqs = a.num_segments; sp.chunk_offsets = seg_chunk_offsets;
    sp.dht = a.seg_dht; sp.dht_kv = 1;
    mode.out_map = a.seg_dh0_map;
    mode.lead = a.seg_lead;
  }
  int rc = launch_bwd_scan(sp, mode, total_tokens, is_bf16, stream);
  if (rc != QLA_OK) return rc;
  return launch_chunk_bwd(p, total_tokens, w.chunks_upper, is_bf16, stream);
}
