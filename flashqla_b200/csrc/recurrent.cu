// Recurrent gated-delta-rule step(s): decode (1 token), spec-decode verify (T draft tokens with a
// cached state per step), tree verify (a step may restart from the cached state of its parent)
// and ragged sequences (cu_seqlens).  One kernel covers what the reference spreads over 29
// generated kernels (flash_qla/ops/gated_delta_rule/recurrent_fused.py:290-6249); the per-token
// math follows the canonical body at :346-487 and the reload rule of the warp kernels at
// :5803-5836 (a parent equal to the previous step is not reloaded).
//
// The op is HBM-bound: every (sequence, v-head) streams a 64 KiB fp32 state in and out.
// Mapping: the state of one head is [V=128 rows][K=128 floats]; a row is 512 B.  Eight lanes share
// a row, each lane owning four float4 (columns j*32 + sub*4 .. +3, j = 0..3), so one warp
// instruction moves four whole rows = 2 KiB, fully coalesced, 128-bit per lane.  A thread keeps R
// rows in registers for the whole call (R*16 floats); the K-reductions (S.k and S.q) are three
// xor-shuffles over the eight lanes of a row.  A CTA of 128 threads covers 16*R rows.
#include "common.cuh"
#include "mma_sync.cuh"

namespace qla {
namespace {

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&out)[4]);

template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&out)[4]) {
  uint2 raw = *reinterpret_cast<const uint2*>(p);
  __nv_bfloat162 lo = *reinterpret_cast<__nv_bfloat162*>(&raw.x);
  __nv_bfloat162 hi = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
  float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
  out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
}
template <>
__device__ __forceinline__ void load4<__half>(const __half* p, float (&out)[4]) {
  uint2 raw = *reinterpret_cast<const uint2*>(p);
  __half2 lo = *reinterpret_cast<__half2*>(&raw.x);
  __half2 hi = *reinterpret_cast<__half2*>(&raw.y);
  float2 a = __half22float2(lo), b = __half22float2(hi);
  out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
}
template <typename T>
__device__ __forceinline__ void unpack4(uint2 raw, float (&out)[4]);
template <>
__device__ __forceinline__ void unpack4<__nv_bfloat16>(uint2 raw, float (&out)[4]) {
  float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw.x));
  float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw.y));
  out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
}
template <>
__device__ __forceinline__ void unpack4<__half>(uint2 raw, float (&out)[4]) {
  float2 a = __half22float2(*reinterpret_cast<__half2*>(&raw.x));
  float2 b = __half22float2(*reinterpret_cast<__half2*>(&raw.y));
  out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
}
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&out)[4]) {
  float4 raw = *reinterpret_cast<const float4*>(p);
  out[0] = raw.x; out[1] = raw.y; out[2] = raw.z; out[3] = raw.w;
}

__device__ __forceinline__ void store4(float* p, const float (&x)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&x)[4]) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]);
  __nv_bfloat162 hi = __floats2bfloat162_rn(x[2], x[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&lo);
  raw.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

__device__ __forceinline__ float group8_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  return x;
}

#ifndef QLA_REC_STAGES
#define QLA_REC_STAGES 2
#endif
constexpr int kRecStages = QLA_REC_STAGES;  // state tiles staged per CTA: the current one and kRecStages - 1 ahead

// One 16-byte (fp32 pool) or 8-byte (16-bit pool) piece of a state row: the four values a lane owns.
template <typename StateT>
struct StatePiece;
template <>
struct StatePiece<float> {
  using Raw = float4;
  static __device__ __forceinline__ void copy_async(Raw* dst, const float* src) { mm::cp_async16(dst, src, true); }
  static __device__ __forceinline__ void unpack(const Raw& x, float (&out)[4]) {
    out[0] = x.x; out[1] = x.y; out[2] = x.z; out[3] = x.w;
  }
};
template <>
struct StatePiece<__nv_bfloat16> {
  using Raw = uint2;
  static __device__ __forceinline__ void copy_async(Raw* dst, const __nv_bfloat16* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(mm::smem_addr(dst)), "l"(src) : "memory");
  }
  static __device__ __forceinline__ void unpack(const Raw& x, float (&out)[4]) { unpack4<__nv_bfloat16>(x, out); }
};

template <typename T, typename InterT, typename StateT, int R>
__global__ void __launch_bounds__(128) recurrent_kernel(const QlaRecurrentArgs p, const int64_t total_items) {
  constexpr int D = kHeadDim;
  constexpr int BV = 16 * R;
  constexpr int kTiles = D / BV;
  // [kRecStages][R * 4 pieces][128 threads] float4: every thread stages exactly the 16-byte pieces it owns, so
  // no barrier is needed between the copy and its use
  using Piece = StatePiece<StateT>;
  extern __shared__ __align__(16) uint8_t s_stage_raw[];
  typename Piece::Raw* s_stage = reinterpret_cast<typename Piece::Raw*>(s_stage_raw);
  grid_dep_wait();    // earlier kernels of the stream have completed (see launch_dependent)
  grid_dep_launch();  // the next one may be scheduled; it waits the same way
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane & 7, grp = lane >> 3;
  const int col0 = sub * 4;  // first owned column of j = 0; j-th is col0 + 32 j

  // A slot outside the pool is never touched: the sequence runs from a zero state without write-back, and
  // the status word says that an index was bad.
  auto bad_index = [&]() {
    if (p.status != nullptr && threadIdx.x == 0) atomicCAS(p.status, 0, kStatusBadIndex);
  };
  auto pool_slot = [&](int n) -> int64_t {
    int64_t sidx = p.state_indices ? p.state_indices[n] : n;
    return sidx >= p.state_slots ? -1 : sidx;
  };
  // The state tile of an item is requested one item ahead (cp.async, L2 only): the copy of the next tile is
  // in flight while this one is computed and written back, which keeps reads queued at the memory the whole
  // time instead of only at the start of every CTA.
  auto prefetch = [&](int64_t item, int stage) {
    const int tile = static_cast<int>(item % kTiles);
    const int64_t nh = item / kTiles;
    const int h = static_cast<int>(nh % p.num_v_heads), n = static_cast<int>(nh / p.num_v_heads);
    const int64_t sidx = pool_slot(n);
    if (sidx < 0) return;
    const int row0 = tile * BV + warp * 4 + grp;
    const StateT* sp = static_cast<const StateT*>(p.state) + ((sidx * p.num_v_heads + h) * D + row0) * D + col0;
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        Piece::copy_async(&s_stage[(stage * R * 4 + r * 4 + j) * 128 + threadIdx.x], sp + (r * 16) * D + j * 32);
  };

  const T* qb = static_cast<const T*>(p.q);
  const T* kb = static_cast<const T*>(p.k);
  const T* vb = static_cast<const T*>(p.v);
  T* ob = static_cast<T*>(p.o);
  InterT* ib = static_cast<InterT*>(p.inter);
  const bool l2norm = (p.flags & QLA_REC_QK_L2NORM) != 0;

  int64_t item = blockIdx.x;
#pragma unroll
  for (int a = 0; a < kRecStages - 1; ++a) {
    if (item + a * static_cast<int64_t>(gridDim.x) < total_items) prefetch(item + a * static_cast<int64_t>(gridDim.x), a);
    mm::cp_async_commit();
  }
  for (int it = 0; item < total_items; item += gridDim.x, ++it) {
  {
    const int64_t ahead = item + (kRecStages - 1) * static_cast<int64_t>(gridDim.x);
    if (ahead < total_items) prefetch(ahead, (it + kRecStages - 1) % kRecStages);
    mm::cp_async_commit();
  }
  mm::cp_async_wait<kRecStages - 1>();  // all but the newest kRecStages - 1 groups: this item's tile has landed

  const int tile = static_cast<int>(item % kTiles);
  const int64_t nh = item / kTiles;
  const int h = static_cast<int>(nh % p.num_v_heads);
  const int n = static_cast<int>(nh / p.num_v_heads);
  const int hk = h / (p.num_v_heads / p.num_k_heads);

  int t0, len;
  if (p.tokens_per_seq > 0) {
    t0 = n * p.tokens_per_seq;
    len = p.tokens_per_seq;
  } else {
    t0 = p.cu_seqlens[n];
    len = p.cu_seqlens[n + 1] - t0;
    // boundaries that leave the token range would read q / k / v and write o out of bounds
    if (t0 < 0 || len < 0 || t0 > p.total_tokens || len > p.total_tokens - t0) {
      bad_index();
      t0 = max(0, min(t0, p.total_tokens));
      len = max(0, min(len, p.total_tokens - t0));
    }
  }
  const int64_t sidx = pool_slot(n);
  if (p.state_indices != nullptr && p.state_indices[n] >= p.state_slots) bad_index();
  int64_t cidx = -1;
  if (p.inter != nullptr) {
    cidx = p.inter_indices ? p.inter_indices[n] : n;
    if (cidx >= p.inter_slots) {
      bad_index();
      cidx = -1;
    }
  }

  const int row0 = tile * BV + warp * 4 + grp;  // row of r = 0; r-th row is row0 + 16 r

  float S[R][4][4];
  if (sidx >= 0) {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        Piece::unpack(s_stage[((it % kRecStages) * R * 4 + r * 4 + j) * 128 + threadIdx.x], S[r][j]);
      }
  } else {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) S[r][j][i] = 0.f;
  }

  float a_coef = 0.f, dt_b = 0.f;
  if (!(p.flags & QLA_REC_A_IS_LOG_DECAY)) {
    a_coef = -expf(load_scalar(p.A_log, p.a_log_dtype, h));
    dt_b = load_scalar(p.dt_bias, p.dt_bias_dtype, h);
  }

  // Inputs of a step (q, k row pieces, v, gate, beta) are requested one step ahead, so that with several draft
  // tokens their global-memory latency overlaps the previous step's arithmetic instead of heading every step.
  uint2 q_raw[4], k_raw[4];
  T v_raw[R];
  float a_in = 0.f, b_in = 0.f;
  auto fetch_inputs = [&](int64_t t) {
    const T* qp = qb + (t * p.num_k_heads + hk) * D + col0;
    const T* kp = kb + (t * p.num_k_heads + hk) * D + col0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      q_raw[j] = *reinterpret_cast<const uint2*>(qp + j * 32);
      k_raw[j] = *reinterpret_cast<const uint2*>(kp + j * 32);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) v_raw[r] = vb[(t * p.num_v_heads + h) * D + row0 + 16 * r];
    a_in = load_scalar(p.a, p.a_dtype, t * p.num_v_heads + h);
    b_in = load_scalar(p.b, p.a_dtype, t * p.num_v_heads + h);
  };
  if (len > 0) fetch_inputs(t0);

  for (int step = 0; step < len; ++step) {
    const int64_t t = t0 + step;

    if (p.parents != nullptr && step > 0 && cidx >= 0) {
      if (step >= p.parents_steps) bad_index();  // the parents table is narrower than this sequence
      const int par = step < p.parents_steps ? p.parents[static_cast<int64_t>(n) * p.parents_stride + step] : step - 1;
      if (par != step - 1 && (par < 0 || par >= p.inter_steps)) bad_index();
      if (par != step - 1 && par >= 0 && par < p.inter_steps) {
        const InterT* src =
            ib + (((cidx * p.inter_steps + par) * p.num_v_heads + h) * D + row0) * D + col0;
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
          for (int j = 0; j < 4; ++j) load4<InterT>(src + (r * 16) * D + j * 32, S[r][j]);
      }
    }

    float qv[4][4], kv[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      unpack4<T>(q_raw[j], qv[j]);
      unpack4<T>(k_raw[j], kv[j]);
    }
    float vrow[R];
#pragma unroll
    for (int r = 0; r < R; ++r) vrow[r] = Cvt<T>::to_f32(v_raw[r]);
    const float a_raw = a_in, b_raw = b_in;
    if (step + 1 < len) fetch_inputs(t + 1);

    // q and k stay as loaded: the factors scale / |q| and 1 / |k| are folded into the three scalars that use them
    // (the k . S product, the update coefficient, the output), which saves 32 multiplies per thread and step
    float qs = p.scale, ks = 1.f;
    if (l2norm) {
      float qq = 0.f, kk = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          qq = fmaf(qv[j][i], qv[j][i], qq);
          kk = fmaf(kv[j][i], kv[j][i], kk);
        }
      qq = group8_sum(qq);
      kk = group8_sum(kk);
      qs *= rsqrtf(qq + 1e-6f);
      ks = rsqrtf(kk + 1e-6f);
    }

    float g;
    if (p.flags & QLA_REC_A_IS_LOG_DECAY) {
      g = a_raw;
    } else {
      const float x = a_raw + dt_b;
      const float bx = p.softplus_beta * x;
      const float sp = (bx <= p.softplus_threshold) ? log1pf(expf(bx)) / p.softplus_beta : x;
      g = a_coef * sp;
    }
    const float decay = expf(g);
    const float beta = (p.flags & QLA_REC_B_IS_BETA) ? b_raw : 1.f / (1.f + expf(-b_raw));

    // four partial sums per row (one per owned piece): the dependent chain of a row is 4 deep instead of 16
    float dot[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          S[r][j][i] *= decay;
          acc[j] = fmaf(S[r][j][i], kv[j][i], acc[j]);
        }
      dot[r] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) dot[r] = group8_sum(dot[r]) * ks;

    float out[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float delta = (vrow[r] - dot[r]) * beta * ks;  // times k / |k| below: one factor here
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          S[r][j][i] = fmaf(kv[j][i], delta, S[r][j][i]);
          acc[j] = fmaf(S[r][j][i], qv[j][i], acc[j]);
        }
      out[r] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) out[r] = group8_sum(out[r]) * qs;
    if (sub == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r)
        ob[(t * p.num_v_heads + h) * D + row0 + 16 * r] = Cvt<T>::from_f32(out[r]);
    }

    if (cidx >= 0 && step < p.inter_steps) {
      InterT* dst = ib + (((cidx * p.inter_steps + step) * p.num_v_heads + h) * D + row0) * D + col0;
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) store4(dst + (r * 16) * D + j * 32, S[r][j]);
    }
  }

  if (!(p.flags & QLA_REC_DISABLE_STATE_UPDATE) && sidx >= 0) {
    StateT* sp = static_cast<StateT*>(p.state) + ((sidx * p.num_v_heads + h) * D + row0) * D + col0;
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int j = 0; j < 4; ++j) store4(sp + (r * 16) * D + j * 32, S[r][j]);
  }
  }  // items
}

// Resident CTAs of `Fn` on the current device (SMs x CTAs per SM), looked up once per device.
template <auto Fn>
int resident_ctas(size_t smem, int* out) {
  static int cached[64] = {};
  int dev = 0;
  QLA_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && cached[dev] > 0) {
    *out = cached[dev];
    return QLA_OK;
  }
  int sms = 0, per_sm = 0;
  QLA_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  QLA_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, Fn, 128, smem));
  *out = sms * (per_sm > 0 ? per_sm : 1);
  if (dev >= 0 && dev < 64) cached[dev] = *out;
  return QLA_OK;
}

template <typename T, typename InterT, typename StateT, int R>
int launch_recurrent_rows(const QlaRecurrentArgs& a, cudaStream_t stream) {
  const int64_t items = static_cast<int64_t>(a.num_seqs) * a.num_v_heads * (kHeadDim / (16 * R));
  constexpr size_t smem = kRecStages * R * 4 * 128 * sizeof(typename StatePiece<StateT>::Raw);
  int resident = 0;
  int rc = ensure_dynamic_smem<recurrent_kernel<T, InterT, StateT, R>>(smem);
  if (rc != QLA_OK) return rc;
  rc = resident_ctas<recurrent_kernel<T, InterT, StateT, R>>(smem, &resident);
  if (rc != QLA_OK) return rc;
  // one CTA per item while they all fit at once; otherwise as many CTAs as are resident, each walking the
  // items with stride gridDim.x
  const unsigned grid = static_cast<unsigned>(items < resident ? items : resident);
  QLA_CHECK_CUDA(launch_dependent(recurrent_kernel<T, InterT, StateT, R>, dim3(grid), dim3(128), smem, stream, a, items));
  QLA_CHECK_CUDA(cudaGetLastError());
  return QLA_OK;
}

template <typename T, typename InterT>
int launch_recurrent(const QlaRecurrentArgs& a, int rows, cudaStream_t stream) {
  if (a.state_dtype == QLA_DT_BF16)
    return rows == 16 ? launch_recurrent_rows<T, InterT, __nv_bfloat16, 1>(a, stream)
                      : launch_recurrent_rows<T, InterT, __nv_bfloat16, 2>(a, stream);
  return rows == 16 ? launch_recurrent_rows<T, InterT, float, 1>(a, stream)
                    : launch_recurrent_rows<T, InterT, float, 2>(a, stream);
}

}  // namespace
}  // namespace qla

namespace qla {
namespace {
// One CTA per (sequence, v-head): 128 x 128 values = 64 KiB of fp32 state, 128-bit accesses.
template <typename InterT>
__global__ void __launch_bounds__(256) state_commit_kernel(const QlaStateCommitArgs a) {
  const int n = blockIdx.x, hv = blockIdx.y;
  const int acc = a.accepted[n];
  if (acc <= 0) return;
  const int64_t sslot = a.state_indices ? a.state_indices[n] : n;
  const int64_t islot = a.inter_indices ? a.inter_indices[n] : n;
  if (acc > a.inter_steps || sslot < 0 || sslot >= a.state_slots || islot < 0 || islot >= a.inter_slots) {
    if (a.status != nullptr && threadIdx.x == 0) atomicCAS(a.status, 0, kStatusBadIndex);
    return;
  }
  constexpr int kElems = kHeadDim * kHeadDim;
  const InterT* src = static_cast<const InterT*>(a.inter) +
                      ((islot * a.inter_steps + (acc - 1)) * a.num_v_heads + hv) * static_cast<int64_t>(kElems);
  const int64_t dst_off = (sslot * a.num_v_heads + hv) * static_cast<int64_t>(kElems);
  float* dst = static_cast<float*>(a.state) + dst_off;
  __nv_bfloat16* dst16 = static_cast<__nv_bfloat16*>(a.state) + dst_off;
  for (int i = threadIdx.x * 8; i < kElems; i += 256 * 8) {
    float x[8];
    if (sizeof(InterT) == 4) {
      const float4 lo = *reinterpret_cast<const float4*>(src + i), hi = *reinterpret_cast<const float4*>(src + i + 4);
      x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w; x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
    } else {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + i);
      const InterT* e = reinterpret_cast<const InterT*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = Cvt<InterT>::to_f32(e[j]);
    }
    if (a.state_dtype == QLA_DT_BF16) {
      const float lo[4] = {x[0], x[1], x[2], x[3]}, hi[4] = {x[4], x[5], x[6], x[7]};
      store4(dst16 + i, lo);
      store4(dst16 + i + 4, hi);
    } else {
      *reinterpret_cast<float4*>(dst + i) = make_float4(x[0], x[1], x[2], x[3]);
      *reinterpret_cast<float4*>(dst + i + 4) = make_float4(x[4], x[5], x[6], x[7]);
    }
  }
}
}  // namespace
}  // namespace qla

namespace qla {
// (32-row tiles of an fp32 pool: the largest variant; 16-row tiles and bf16 pools use a half / a quarter)
void launch_info_recurrent_kernel(int* block_threads, size_t* dynamic_smem_bytes) {
  *block_threads = 128;
  *dynamic_smem_bytes = kRecStages * 2 * 4 * 128 * sizeof(float4);
}
}  // namespace qla

extern "C" QLA_API int qla_state_commit(const QlaStateCommitArgs* args, void* stream) {
  using namespace qla;
  QLA_CHECK_ARG(args != nullptr, "args is NULL");
  const QlaStateCommitArgs& a = *args;
  QLA_CHECK_ARG(a.num_seqs >= 0 && a.num_v_heads > 0, "bad sizes");
  if (a.num_seqs == 0) return QLA_OK;
  QLA_CHECK_ARG(a.inter && a.accepted && a.state, "NULL tensor pointer");
  QLA_CHECK_ARG(a.inter_slots > 0 && a.inter_steps > 0 && a.state_slots > 0, "extents must be positive");
  QLA_CHECK_SUPPORTED(a.inter_dtype == QLA_DT_F32 || a.inter_dtype == QLA_DT_BF16,
                      "intermediate_states_buffer must be fp32 or bf16");
  QLA_CHECK_SUPPORTED(a.state_dtype == QLA_DT_F32 || a.state_dtype == QLA_DT_BF16, "the state pool must be fp32 or bf16");
  dim3 grid(a.num_seqs, a.num_v_heads);
  if (a.inter_dtype == QLA_DT_F32) state_commit_kernel<float><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  else state_commit_kernel<__nv_bfloat16><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  QLA_CHECK_CUDA(cudaGetLastError());
  return QLA_OK;
}

extern "C" QLA_API int qla_recurrent_update(const QlaRecurrentArgs* args, void* stream) {
  using namespace qla;
  QLA_CHECK_ARG(args != nullptr, "args is NULL");
  const QlaRecurrentArgs& a = *args;
  QLA_CHECK_ARG(a.num_seqs >= 0 && a.total_tokens >= 0, "negative sizes");
  if (a.num_seqs == 0 || a.total_tokens == 0) return QLA_OK;
  QLA_CHECK_ARG(a.num_k_heads > 0 && a.num_v_heads > 0 && a.num_v_heads % a.num_k_heads == 0,
                "num_value_heads must be divisible by num_key_heads");
  QLA_CHECK_ARG(a.q && a.k && a.v && a.a && a.b && a.o && a.state, "NULL tensor pointer");
  QLA_CHECK_ARG((a.flags & QLA_REC_A_IS_LOG_DECAY) || (a.A_log && a.dt_bias),
                "A_log and dt_bias are required unless a_is_log_decay");
  QLA_CHECK_ARG(a.tokens_per_seq > 0 || a.cu_seqlens != nullptr,
                "either tokens_per_seq > 0 or cu_seqlens must be given");
  QLA_CHECK_ARG(a.tokens_per_seq == 0 ||
                    static_cast<int64_t>(a.tokens_per_seq) * a.num_seqs == a.total_tokens,
                "total_tokens must equal num_seqs * tokens_per_seq");
  QLA_CHECK_SUPPORTED(a.qkv_dtype == QLA_DT_BF16 || a.qkv_dtype == QLA_DT_F16,
                      "q, k, v must be bf16 or fp16");
  QLA_CHECK_ARG(a.state_slots > 0, "state_slots must be positive");
  QLA_CHECK_SUPPORTED(a.state_dtype == QLA_DT_F32 || a.state_dtype == QLA_DT_BF16,
                      "initial_state_source must be fp32 or bf16");
  QLA_CHECK_ARG(a.parents == nullptr || a.parents_steps > 0, "parents_steps (second extent of parents) must be positive");
  QLA_CHECK_ARG(a.parents == nullptr || a.tokens_per_seq <= a.parents_steps,
                "retrieve_parent_token has fewer columns than tokens per sequence");
  if (a.inter != nullptr) {
    QLA_CHECK_ARG(a.inter_slots > 0 && a.inter_steps > 0, "inter extents must be positive");
    QLA_CHECK_SUPPORTED(a.inter_dtype == QLA_DT_F32 || a.inter_dtype == QLA_DT_BF16,
                        "intermediate_states_buffer must be fp32 or bf16");
  }
  QLA_CHECK_ARG(a.parents == nullptr || a.inter != nullptr,
                "retrieve_parent_token needs intermediate_states_buffer");
  QLA_CHECK_ARG(a.rows_per_cta == 0 || a.rows_per_cta == 16 || a.rows_per_cta == 32,
                "rows_per_cta must be 0, 16 or 32");
  int rows = a.rows_per_cta;
  if (rows == 0) {
    // 32 rows per CTA keeps two independent rows in flight per thread; fall back to 16 rows while
    // the grid would otherwise leave SMs idle (148 SMs, several CTAs each).
    rows = (static_cast<int64_t>(a.num_seqs) * a.num_v_heads * 4 >= 4 * 148) ? 32 : 16;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool inter_bf16 = a.inter != nullptr && a.inter_dtype == QLA_DT_BF16;
  if (a.qkv_dtype == QLA_DT_BF16) {
    return inter_bf16 ? launch_recurrent<__nv_bfloat16, __nv_bfloat16>(a, rows, s)
                      : launch_recurrent<__nv_bfloat16, float>(a, rows, s);
  }
  return inter_bf16 ? launch_recurrent<__half, __nv_bfloat16>(a, rows, s)
                    : launch_recurrent<__half, float>(a, rows, s);
}
