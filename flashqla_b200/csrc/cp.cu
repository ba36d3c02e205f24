// Intra-card context parallelism for the chunked forward: a long sequence is cut into segments that
// run as independent CTAs; each non-final segment first produces the state it hands to its successor.
// Reference: flash_qla/ops/gated_delta_rule/chunk/cp_context.py:117-176 (orchestration),
// chunk/hopper/cp_fwd.py:7-63 (warm-up lengths) and :102-250 (chaining of the initial states).
//
//   plan  : per (segment, head) walk the chunk-end gates backwards from the segment end until the
//           accumulated log decay drops below `threshold`; that many trailing chunks, started from a
//           zero state, reproduce the segment-end state to exp(threshold).  If the whole segment does
//           not decay that far the (segment, head) is a "fallback": all chunks are run and the exact
//           K x K transition matrix M of the segment is needed as well.
//   chain : for fallback entries  h0[seg + 1] += M[seg] * h0[seg], in segment order.
#include "chunk_params.cuh"

namespace qla {
namespace {

// One CTA per (segment, head): thread 0 walks the chunk-end gates; all threads write the segment's start state.
__global__ void __launch_bounds__(256) cp_plan_kernel(const QlaCpPlanArgs a) {
  grid_dep_wait();    // earlier kernels of the stream have completed (see launch_dependent)
  grid_dep_launch();
  const int seg = blockIdx.x, h = blockIdx.y;
  const int num_heads = a.num_v_heads;
  if (threadIdx.x == 0) {
    const int start = a.cu_seqlens[seg], end = a.cu_seqlens[seg + 1];
    const int nchunks = (end - start + kChunk - 1) / kChunk;
    int warm = 0, ml = 0;
    if (a.seg_next[seg] >= 0 && nchunks > 0) {
      float acc = 0.f;
      bool reached = false;
      for (int i = 0; i < nchunks; ++i) {
        const int c = a.reverse ? i : nchunks - 1 - i;  // backward: the decay accumulates from the segment's start
        const int last = min(end, start + (c + 1) * kChunk) - 1;
        acc += a.g_cumsum[static_cast<int64_t>(last) * num_heads + h];
        ++warm;
        if (acc < a.threshold) { reached = true; break; }
      }
      if (!reached) ml = nchunks;  // warm == nchunks here
    }
    a.warm_limit[seg * num_heads + h] = warm;
    a.m_limit[seg * num_heads + h] = ml;
  }
  if (a.cp_h0 == nullptr) return;
  constexpr int kElems = kHeadDim * kHeadDim;
  float* dst = a.cp_h0 + (static_cast<int64_t>(seg) * num_heads + h) * kElems;
  const int raw = a.seg_start_of[seg];
  int row = -1;
  if (raw >= 0 && a.h0 != nullptr) row = a.h0_map != nullptr ? a.h0_map[raw] : raw;
  if (row < 0) {
    for (int i = threadIdx.x * 4; i < kElems; i += 256 * 4) *reinterpret_cast<float4*>(dst + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    return;
  }
  const int64_t off = (static_cast<int64_t>(row) * num_heads + h) * kElems;
  const float* s32 = static_cast<const float*>(a.h0) + off;
  const __nv_bfloat16* s16 = static_cast<const __nv_bfloat16*>(a.h0) + off;
  for (int i = threadIdx.x; i < kElems; i += 256) {
    // destination [K][V]; a transposed source is read along its rows by consecutive threads
    const int di = a.h0_transposed ? (i & (kHeadDim - 1)) * kHeadDim + (i >> 7) : i;
    dst[di] = a.h0_dtype == QLA_DT_BF16 ? __bfloat162float(s16[i]) : s32[i];
  }
}

// The plan with the warm-up folded into the main scan (forward, or reverse for the backward scan): one CTA per
// (original sequence, head), a thread per segment.  A (sequence, head) in which every segment decays below the threshold needs no state-only pass:
// the main scan's CTA of segment s simply starts lead[s] = warm(s - 1) chunks early, from a zero state.  If some
// segment never decays that far the limits are those of cp_plan_kernel (state-only pass, transition matrices,
// chain) and lead is 0.  Only the row of cp_h0 that starts the sequence is written here.
__global__ void __launch_bounds__(256) cp_plan_lead_kernel(const QlaCpPlanArgs a) {
  grid_dep_wait();
  grid_dep_launch();
  const int r = blockIdx.x, h = blockIdx.y;
  const int num_heads = a.num_v_heads;
  const int s0 = a.raw_first_seg[r], s1 = a.raw_first_seg[r + 1];
  int any = 0;
  for (int seg = s0 + threadIdx.x; seg < s1; seg += 256) {
    const int start = a.cu_seqlens[seg], end = a.cu_seqlens[seg + 1];
    const int nchunks = (end - start + kChunk - 1) / kChunk;
    int warm = 0, ml = 0;
    if (a.seg_next[seg] >= 0 && nchunks > 0) {
      float acc = 0.f;
      bool reached = false;
      for (int i = 0; i < nchunks; ++i) {
        const int c = a.reverse ? i : nchunks - 1 - i;  // backward: the decay accumulates from the segment's start
        const int last = min(end, start + (c + 1) * kChunk) - 1;
        acc += a.g_cumsum[static_cast<int64_t>(last) * num_heads + h];
        ++warm;
        if (acc < a.threshold) { reached = true; break; }
      }
      if (!reached) ml = nchunks;
    }
    a.warm_limit[seg * num_heads + h] = warm;
    a.m_limit[seg * num_heads + h] = ml;
    any |= ml;
  }
  any = __syncthreads_or(any);  // (also orders the limits written above before the reads below)
  // the neighbour whose warm-up this segment's scan runs itself: the segment before it (forward), behind it (backward)
  for (int seg = s0 + threadIdx.x; seg < s1; seg += 256) {
    const int nb = a.reverse ? seg + 1 : seg - 1;
    a.lead[seg * num_heads + h] = (!any && nb >= s0 && nb < s1) ? a.warm_limit[nb * num_heads + h] : 0;
  }
  __syncthreads();
  if (!any)
    for (int seg = s0 + threadIdx.x; seg < s1; seg += 256) a.warm_limit[seg * num_heads + h] = 0;
  // start state of the sequence (backward: the gradient of its final state, into the last segment's row): the
  // caller's (any dtype / layout, through h0_map) or zero
  constexpr int kElems = kHeadDim * kHeadDim;
  float* dst = a.cp_h0 + (static_cast<int64_t>(a.reverse ? s1 - 1 : s0) * num_heads + h) * kElems;
  int row = -1;
  if (a.h0 != nullptr) row = a.h0_map != nullptr ? a.h0_map[r] : r;
  if (row < 0) {
    for (int i = threadIdx.x * 4; i < kElems; i += 256 * 4) *reinterpret_cast<float4*>(dst + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    return;
  }
  const int64_t off = (static_cast<int64_t>(row) * num_heads + h) * kElems;
  const float* s32 = static_cast<const float*>(a.h0) + off;
  const __nv_bfloat16* s16 = static_cast<const __nv_bfloat16*>(a.h0) + off;
  if (!a.h0_transposed && a.h0_dtype != QLA_DT_BF16) {
    // the common case (a carried fp32 [K, V] state): 16-byte copies, four in flight per thread
#pragma unroll 4
    for (int i = threadIdx.x * 4; i < kElems; i += 256 * 4)
      *reinterpret_cast<float4*>(dst + i) = *reinterpret_cast<const float4*>(s32 + i);
    return;
  }
#pragma unroll 4
  for (int i = threadIdx.x; i < kElems; i += 256) {
    const int di = a.h0_transposed ? (i & (kHeadDim - 1)) * kHeadDim + (i >> 7) : i;
    dst[di] = a.h0_dtype == QLA_DT_BF16 ? __bfloat162float(s16[i]) : s32[i];
  }
}

// One CTA: one (raw sequence, head, 32-column slab of the state).  Thread t owns row k = t of the slab.
__global__ void __launch_bounds__(128) cp_chain_kernel(float* __restrict__ h0, const float* __restrict__ M,
                                                       const int32_t* __restrict__ m_limit,
                                                       const int32_t* __restrict__ raw_first_seg, int num_heads,
                                                       int reverse) {
  grid_dep_wait();
  grid_dep_launch();
  const int vt = blockIdx.x, h = blockIdx.y, r = blockIdx.z;
  const int s0 = raw_first_seg[r], s1 = raw_first_seg[r + 1];
  const int k = threadIdx.x;
  __shared__ float sh[kHeadDim][33];
  // the usual case (every segment decays below the threshold) has nothing to chain: find that out with one
  // parallel look at the flags instead of a serial walk
  int mine = 0;
  for (int seg = s0 + threadIdx.x; seg < s1; seg += 128) mine |= m_limit[seg * num_heads + h];
  if (__syncthreads_or(mine) == 0) return;
  for (int i = 0; i + 1 < s1 - s0; ++i) {
    // forward: segment s0 + i feeds s0 + i + 1; backward: segment s1 - 1 - i feeds s1 - 2 - i
    const int seg = reverse ? s1 - 1 - i : s0 + i;
    const int to = reverse ? seg - 1 : seg + 1;
    if (m_limit[seg * num_heads + h] == 0) continue;  // uniform across the CTA
    const float* src = h0 + (static_cast<int64_t>(seg) * num_heads + h) * kHeadDim * kHeadDim + vt * 32;
    float* dst = h0 + (static_cast<int64_t>(to) * num_heads + h) * kHeadDim * kHeadDim + vt * 32;
    const float* m = M + (static_cast<int64_t>(seg) * num_heads + h) * kHeadDim * kHeadDim;
    __syncthreads();
    for (int e = threadIdx.x; e < kHeadDim * 32; e += 128) sh[e >> 5][e & 31] = src[(e >> 5) * kHeadDim + (e & 31)];
    __syncthreads();
    float acc[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) acc[j] = 0.f;
    for (int j = 0; j < kHeadDim; ++j) {
      const float mk = m[k * kHeadDim + j];
#pragma unroll
      for (int c = 0; c < 32; ++c) acc[c] = fmaf(mk, sh[j][c], acc[c]);
    }
#pragma unroll
    for (int c = 0; c < 32; ++c) dst[k * kHeadDim + c] += acc[c];
    __threadfence();  // the next iteration of THIS CTA reads dst (same slab, same CTA): ordering only
  }
}

}  // namespace
}  // namespace qla

extern "C" QLA_API int qla_cp_plan(const QlaCpPlanArgs* a, void* stream) {
  using namespace qla;
  QLA_CHECK_ARG(a != nullptr && a->g_cumsum && a->cu_seqlens && a->seg_next && a->warm_limit && a->m_limit,
                "NULL pointer in QlaCpPlanArgs");
  QLA_CHECK_ARG(a->num_segments > 0 && a->num_v_heads > 0 && a->num_v_heads <= 65535, "bad sizes");
  QLA_CHECK_ARG(a->cp_h0 == nullptr || a->seg_start_of != nullptr, "cp_h0 needs seg_start_of");
  QLA_CHECK_SUPPORTED(a->h0 == nullptr || a->h0_dtype == QLA_DT_F32 || a->h0_dtype == QLA_DT_BF16,
                      "initial states must be fp32 or bf16");
  if (a->lead != nullptr) {
    QLA_CHECK_ARG(a->cp_h0 != nullptr && a->raw_first_seg != nullptr && a->num_raw_seqs > 0,
                  "lead needs cp_h0, raw_first_seg and num_raw_seqs");
    dim3 grid_lead(a->num_raw_seqs, a->num_v_heads);
    QLA_CHECK_CUDA(launch_dependent(cp_plan_lead_kernel, grid_lead, dim3(256), 0, static_cast<cudaStream_t>(stream), *a));
    return QLA_OK;
  }
  dim3 grid(a->num_segments, a->num_v_heads);
  QLA_CHECK_CUDA(launch_dependent(cp_plan_kernel, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), *a));
  return QLA_OK;
}

extern "C" QLA_API int qla_cp_chain(const QlaCpChainArgs* a, void* stream) {
  using namespace qla;
  QLA_CHECK_ARG(a != nullptr && a->h0 && a->M && a->m_limit && a->raw_first_seg, "NULL pointer in QlaCpChainArgs");
  QLA_CHECK_ARG(a->num_raw_seqs > 0 && a->num_v_heads > 0, "bad sizes");
  dim3 grid(kHeadDim / 32, a->num_v_heads, a->num_raw_seqs);
  QLA_CHECK_CUDA(launch_dependent(cp_chain_kernel, grid, dim3(128), 0, static_cast<cudaStream_t>(stream), a->h0, a->M,
                                  a->m_limit, a->raw_first_seg, a->num_v_heads, a->reverse));
  return QLA_OK;
}
