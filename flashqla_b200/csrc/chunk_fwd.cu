// Chunked gated-delta-rule forward for sm_100a: the serial scan over 64-token chunks of one
// (sequence, v-head) with the recurrent state resident in tensor memory.
// Reference: fused_gdr_fwd (flash_qla/ops/gated_delta_rule/chunk/hopper/fused_fwd.py:19-656; the gated-A
// variant chunk/blackwell/fused_fwd.py:383-393) and the state-only pass fused_gdr_h
// (chunk/hopper/prepare_h.py:13-556); math as in tests/ref_gdr.py:107-260.
//
// Per chunk (S0 = state entering the chunk, g = chunk-local cumulative gate, gL its last value):
//   Vd = A diag(beta) (V - exp(g) .* (K S0)) = Ab V - Wt S0           (= "v_new")
//        Ab = A diag(beta),  Wt = A diag(beta exp(g)) K  (both state independent; Wt comes, negated,
//        from the preparation kernel)
//   O  = s exp(g) .* (Q S0) + (s G .* Q K^T) Vd                      G[c,d] = exp(g_c - g_d), c >= d
//   S1 = exp(gL) S0 + K^T (exp(gL - g) .* Vd)
//
// Everything is computed TRANSPOSED so that each tcgen05.mma has M = 128 (the V dimension on the 128
// TMEM lanes) and every dependent operand can stay in tensor memory:
//   MMA0  D0[128,64]  = [K;Q] K^T          (SS)  rows 64..127 are P = Q K^T; state independent
//   MMAu  D2[128,64]  = V^T Ab^T           (SS)  state independent part of Vd^T
//   MMA2  D2[128,64] += S0^T_bf16 (-Wt)^T  (TS)  D2 = Vd^T; the only product between two state updates
//                                                besides MMA3
//   MMAq  Dq[128,64]  = S0^T_bf16 Q^T      (TS)  (Q S0)^T for the output, off the chain
//   MMA3  S^T[128,128] += V'^T K           (TS, B operand MN-major straight from the K tile)
//   MMA4  D4[128,64] += Vd^T Pg^T          (SS)  Pg = s G .* P and Vd^T are swizzled smem tiles; off the chain
// Thread v of a compute warpgroup owns TMEM lane v = column v of the state: it reads Vd^T rows
// with tcgen05.ld, applies the gates, and writes the bf16 operand of the next MMA back with
// tcgen05.st.  The fp32 state never leaves tensor memory between chunks.
//
// Warp roles (384 threads): warps 0-3 "chain" (Vd, state convert of columns 0..63), warps 4-7 "side"
// (output epilogue, state convert of columns 64..127), warp 8 TMA producer + gate vectors, warp 9 MMA
// issuer, warps 10-11 "aux" (operand tiles A diag(beta) and Pg).  Two smem stages of {K,Q,V,A,Wt,gates};
// all waits are bounded mbarrier waits that raise a status word instead of hanging.
#include "chunk_params.cuh"

namespace qla {


namespace {

// ---- tensor-memory column map (512 columns)
constexpr uint32_t kColS = 0;      // fp32 state S^T, 128 columns
constexpr uint32_t kColSbf = 128;  // bf16 copy of S^T (A operand of MMA1), 64 columns
constexpr uint32_t kColD2 = 192;   // Vd^T; columns 192..223 are overwritten in place by V' bf16 (A operand of MMA3)
constexpr uint32_t kColDq = 256;   // (Q S0)^T
constexpr uint32_t kColD4 = 320;   // output accumulator: s gamma .* (Q S0)^T, then += Vd^T Pg^T
constexpr uint32_t kColD0 = 384;   // [K;Q] K^T

// ---- shared-memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kStageKQ = 0;         // 32 KiB: half 0 [K rows | Q rows] (16 KiB), half 1 (16 KiB); SW128
constexpr uint32_t kStageV = 32768;      // 16 KiB: V tile as two [64][64] halves (columns 0..63 | 64..127), SW128
constexpr uint32_t kStageA = 49152;      // 8 KiB: A tile [64][64], SW128; scaled in place to A diag(beta)
constexpr uint32_t kStageW = 57344;      // 16 KiB: -Wt tile as two [64][64] halves (columns 0..63 | 64..127), SW128
constexpr uint32_t kStageGate = 73728;   // 1 KiB + : g[64], gamma[64], rho[64], beta[64], egl
constexpr uint32_t kStageBytes = 75776;  // 74 KiB, multiple of 1024
constexpr uint32_t kOffPg = 2 * kStageBytes;         // 8 KiB Pg tile, SW128
constexpr uint32_t kOffO = kOffPg + 8192;            // 2 x 16 KiB output tiles [64][128]
constexpr uint32_t kOffVd = kOffO + 2 * 16384;       // 2 x 16 KiB Vd^T tiles [128 v][64 d], SW128 (A of MMA4)
constexpr uint32_t kSmemBytes = kOffVd + 2 * 16384 + 1024;

struct Gates {
  float g[64];
  float gamma[64];
  float rho[64];
  float beta[64];
  float egl;
  int valid;  // number of valid tokens in the chunk
};

enum Bar {
  kFull0 = 0, kFull1, kEmpty0, kEmpty1,
  kPDone, kPFree, kPgReady, kDqDone, kQsStored, kD2Done, kVdReady, kSDone, kSbfReady, kSScaled, kAbReady0, kAbReady1, kD4Done, kOFree, kOReady,
  kNumBars
};

constexpr int kThreads = 384;

// One arrival per warp: every lane has finished (and fenced) its own writes, the warp converges, and
// lane 0 signals the barrier.
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) ptx::mbar_arrive(bar);
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 x = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&x);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 x = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&x);
}

template <typename T, bool kStateOnly, bool kTrace>
__global__ void __launch_bounds__(kThreads, 1)
chunk_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_a,
                 const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_o,
                 const FwdParams p) {
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? ptx::kFmtBF16 : ptx::kFmtF16;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hv = blockIdx.x % p.num_v_heads;
  const int seq = blockIdx.x / p.num_v_heads;
  const int hk = hv / (p.num_v_heads / p.num_k_heads);

  int seq_start, seq_end;
  if (p.cu_seqlens != nullptr) {
    seq_start = p.cu_seqlens[seq];
    seq_end = p.cu_seqlens[seq + 1];
  } else {
    seq_start = seq * p.seq_len;
    seq_end = seq_start + p.seq_len;
  }
  int nchunks = (seq_end - seq_start + kChunk - 1) / kChunk;
  int first_chunk = 0;
  if (p.chunk_limit != nullptr) {
    const int lim = p.chunk_limit[seq * p.num_v_heads + hv];
    if (lim <= 0) return;  // nothing asked of this (sequence, head); uniform for the whole CTA
    if (lim < nchunks) first_chunk = nchunks - lim;
  }
  const int nproc = nchunks - first_chunk;
  const int out_row = p.seq_map ? p.seq_map[seq] : seq;
  const int64_t chunk_base =
      p.chunk_offsets ? p.chunk_offsets[seq] : static_cast<int64_t>(seq) * ((p.seq_len + kChunk - 1) / kChunk);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // align up with pointer arithmetic on the shared array so that the compiler keeps the address space
  uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint64_t bars[kNumBars];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(16) float aux_g[2 * 2 * 64];  // [aux warp][chunk parity][64] cumulative gates

  if (tid == 0) {
    ptx::mbar_init(&bars[kFull0], 33);
    ptx::mbar_init(&bars[kFull1], 33);
    ptx::mbar_init(&bars[kEmpty0], 11);
    ptx::mbar_init(&bars[kEmpty1], 11);
    ptx::mbar_init(&bars[kPDone], 1);
    ptx::mbar_init(&bars[kPFree], 2);
    ptx::mbar_init(&bars[kPgReady], 2);
    ptx::mbar_init(&bars[kDqDone], 1);
    ptx::mbar_init(&bars[kQsStored], 4);
    ptx::mbar_init(&bars[kD2Done], 1);
    ptx::mbar_init(&bars[kVdReady], 4);
    ptx::mbar_init(&bars[kSDone], 1);
    ptx::mbar_init(&bars[kSbfReady], 8);
    ptx::mbar_init(&bars[kSScaled], 8);
    ptx::mbar_init(&bars[kAbReady0], 2);
    ptx::mbar_init(&bars[kAbReady1], 2);
    ptx::mbar_init(&bars[kD4Done], 1);
    ptx::mbar_init(&bars[kOFree], 1);
    ptx::mbar_init(&bars[kOReady], 4);
    ptx::fence_mbar_init();
  }
  if (warp == 8) {
    ptx::tmem_alloc(&tmem_base_s, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  int* status = p.status;
  constexpr int kTimeout = kStatusBarrierTimeout;

  // phase trace: leaders of CTA 0 stamp clock64() for chunks kTraceFirstChunk.. (off when p.trace is NULL)
  // the traced CTA is chosen by the host through the last slot of the phase region (0 by default)
  const bool tracing = kTrace && p.trace != nullptr &&
                       static_cast<long long>(blockIdx.x) == p.trace[kTraceRoles * kTraceChunks * kTraceEvents - 1];
  auto trace = [&](int role, int i, int ev) {
    if (kTrace && tracing && i >= kTraceFirstChunk && i < kTraceFirstChunk + kTraceChunks)
      p.trace[(role * kTraceChunks + (i - kTraceFirstChunk)) * kTraceEvents + ev] = clock64();
  };

  // per-CTA residency record (start, end in ns, SM id) after the phase trace, when the buffer is large enough
  const long long cta_slot = kTraceRoles * kTraceChunks * kTraceEvents + 3ll * blockIdx.x;
  const bool cta_trace = kTrace && p.trace != nullptr && cta_slot + 3 <= p.trace_count;
  if (cta_trace && tid == 0) {
    unsigned long long t;
    unsigned sm;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    asm volatile("mov.u32 %0, %smid;" : "=r"(sm));
    p.trace[cta_slot] = static_cast<long long>(t);
    p.trace[cta_slot + 2] = sm;
  }

  auto stage_ptr = [&](int s) { return smem + s * kStageBytes; };
  auto gates_of = [&](int s) { return reinterpret_cast<Gates*>(stage_ptr(s) + kStageGate); };

  if (warp == 8) {
    // =========================================================== producer: TMA + gate vectors
    // L2 prefetch runs kPrefetchAhead chunks ahead of the demand loads: with every SM streaming its own
    // sequence the DRAM latency of a tile exceeds one chunk period, and only two stages fit in shared
    // memory, so the tiles are pulled into L2 early and the demand TMA then hits L2.
    constexpr int kPrefetchAhead = 4;
    auto prefetch_chunk = [&](int j) {
      const int pt0 = seq_start + (first_chunk + j) * kChunk;
      ptx::tma_prefetch_l2_3d(&tm_k, 0, hk, pt0);
      ptx::tma_prefetch_l2_3d(&tm_k, 64, hk, pt0);
      if (!kStateOnly) {
        ptx::tma_prefetch_l2_3d(&tm_q, 0, hk, pt0);
        ptx::tma_prefetch_l2_3d(&tm_q, 64, hk, pt0);
      }
      if (!p.zero_v) {
        ptx::tma_prefetch_l2_3d(&tm_v, 0, hv, pt0);
        ptx::tma_prefetch_l2_3d(&tm_v, 64, hv, pt0);
      }
      ptx::tma_prefetch_l2_3d(&tm_a, 0, hv, pt0);
      ptx::tma_prefetch_l2_3d(&tm_w, 0, hv, pt0);
      ptx::tma_prefetch_l2_3d(&tm_w, 64, hv, pt0);
    };
    if (lane == 0)
      for (int j = 2; j < kPrefetchAhead && j < nproc; ++j) prefetch_chunk(j);
    for (int i = 0; i < nproc; ++i) {
      const int s = i & 1, use = i >> 1;
      if (lane == 0) trace(0, i, 9);
      const int chunk = first_chunk + i;
      const int t0 = seq_start + chunk * kChunk;
      const int valid = min(kChunk, seq_end - t0);
      // gate values are fetched into registers BEFORE waiting for the stage, so their global-memory
      // latency overlaps the wait
      const int64_t last_tok = static_cast<int64_t>(t0) + valid - 1;
      const float gl = p.g_cumsum[last_tok * p.num_v_heads + hv];
      float gcv[2], bcv[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int c = lane + 32 * r;
        const bool okc = c < valid;
        const int64_t tok = static_cast<int64_t>(t0) + c;
        gcv[r] = okc ? p.g_cumsum[tok * p.num_v_heads + hv] : gl;
        bcv[r] = okc ? load_scalar(p.beta, p.beta_dtype, tok * p.num_v_heads + hv) : 0.f;
      }
      if (use > 0 && !ptx::mbar_wait_warp(&bars[kEmpty0 + s], (use - 1) & 1, status, kTimeout | ((kEmpty0 + s) << 8))) break;
      if (lane == 0) trace(0, i, 10);
      uint8_t* st = stage_ptr(s);
      if (lane == 0) {
        if (i + kPrefetchAhead < nproc) prefetch_chunk(i + kPrefetchAhead);
        uint32_t bytes = 16384 + 8192 + 16384;  // K + A + Wt
        if (!kStateOnly) bytes += 16384;  // Q
        if (!p.zero_v) bytes += 16384;    // V
        ptx::mbar_expect_tx(&bars[kFull0 + s], bytes);
        ptx::tma_load_3d(st + kStageKQ, &tm_k, &bars[kFull0 + s], 0, hk, t0);
        ptx::tma_load_3d(st + kStageKQ + 16384, &tm_k, &bars[kFull0 + s], 64, hk, t0);
        if (!kStateOnly) {
          ptx::tma_load_3d(st + kStageKQ + 8192, &tm_q, &bars[kFull0 + s], 0, hk, t0);
          ptx::tma_load_3d(st + kStageKQ + 16384 + 8192, &tm_q, &bars[kFull0 + s], 64, hk, t0);
        }
        if (!p.zero_v) {
          ptx::tma_load_3d(st + kStageV, &tm_v, &bars[kFull0 + s], 0, hv, t0);
          ptx::tma_load_3d(st + kStageV + 8192, &tm_v, &bars[kFull0 + s], 64, hv, t0);
        }
        ptx::tma_load_3d(st + kStageA, &tm_a, &bars[kFull0 + s], 0, hv, t0);
        ptx::tma_load_3d(st + kStageW, &tm_w, &bars[kFull0 + s], 0, hv, t0);
        ptx::tma_load_3d(st + kStageW + 8192, &tm_w, &bars[kFull0 + s], 64, hv, t0);
      }
      Gates* gs = gates_of(s);
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int c = lane + 32 * r;
        const bool ok = c < valid;
        const float gc = gcv[r], bc = bcv[r];
        gs->g[c] = gc;
        gs->gamma[c] = __expf(gc);
        gs->rho[c] = ok ? __expf(gl - gc) : 0.f;
        gs->beta[c] = bc;
      }
      if (lane == 0) {
        gs->egl = __expf(gl);
        gs->valid = valid;
      }
      ptx::mbar_arrive(&bars[kFull0 + s]);  // 32 arrivals + the expect_tx arrival of lane 0
      if (lane == 0) trace(0, i, 11);
    }
  } else if (warp == 9) {
    // =========================================================== MMA issuer (one thread)
    if (lane == 0) {
      const uint32_t id_n64 = ptx::mma_idesc(128, 64, fmt, ptx::kMajorK, ptx::kMajorK);
      const uint32_t id_mn128 = ptx::mma_idesc(128, 128, fmt, ptx::kMajorK, ptx::kMajorMN);
      const uint32_t id_u = ptx::mma_idesc(128, 64, fmt, ptx::kMajorMN, ptx::kMajorK);
      // Descriptors are built once; inside the loop an operand step is one 64-bit add of
      // (byte offset >> 4) so that the single issuing thread spends its cycles on tcgen05.mma only.
      uint64_t d_kq[2], d_kmn[2], d_a[2], d_v[2], d_w[2];
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        d_kq[s] = ptx::smem_desc_sw128(ptx::smem_u32(stage_ptr(s) + kStageKQ), 16, 1024);      // K-major rows
        d_kmn[s] = ptx::smem_desc_sw128(ptx::smem_u32(stage_ptr(s) + kStageKQ), 16384, 1024);  // K tile, MN-major
        d_a[s] = ptx::smem_desc_sw128(ptx::smem_u32(stage_ptr(s) + kStageA), 16, 1024);
        d_v[s] = ptx::smem_desc_sw128(ptx::smem_u32(stage_ptr(s) + kStageV), 8192, 1024);      // V tile, MN-major
        d_w[s] = ptx::smem_desc_sw128(ptx::smem_u32(stage_ptr(s) + kStageW), 16, 1024);
      }
      const uint64_t d_pg = ptx::smem_desc_sw128(ptx::smem_u32(smem + kOffPg), 16, 1024);
      const uint64_t d_vd0 = ptx::smem_desc_sw128(ptx::smem_u32(smem + kOffVd), 16, 1024);
      const uint64_t d_vd1 = ptx::smem_desc_sw128(ptx::smem_u32(smem + kOffVd + 16384), 16, 1024);
      // Issue order (software pipelined).  Between two state updates only MMA2 -> (chain warpgroup: Vd)
      // -> MMA3 -> (both warpgroups: 16-bit state copy) are serial.  Everything else is issued in the
      // tail of a chunk, behind MMA3, so that the tensor pipe executes it while the state is converted:
      // MMAu and MMA0 of the NEXT chunk (state independent) and MMA4 of this chunk.
      // MMAu of chunk j: D2 = V^T (A diag(beta))^T.  A operand = V tile read MN-major (two 64-column halves
      // 8 KiB apart), B operand = the A tile after the aux warps scaled its columns by beta in place.
      auto issue_u = [&](int j) -> bool {
        const int s = j & 1;
        if (!ptx::mbar_spin(&bars[kFull0 + s], (j >> 1) & 1, status, kTimeout | ((kFull0 + s) << 8))) return false;
        if (!ptx::mbar_spin(&bars[kAbReady0 + s], (j >> 1) & 1, status, kTimeout | ((kAbReady0 + s) << 8))) return false;
        if (!p.zero_v) {
          const uint64_t vv = s ? d_v[1] : d_v[0], aa = s ? d_a[1] : d_a[0];
          ptx::tc_fence_after_sync();
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            ptx::mma_ss(tmem + kColD2, vv + ks * (2048 >> 4), aa + ks * (32 >> 4), id_u, ks > 0);
        }
        return true;
      };
      // MMA0 of chunk j: D0 = [K;Q] K^T (A = 128 rows, B = first 64 rows of the tile)
      auto issue_p = [&](int j) {
        const uint64_t kq = (j & 1) ? d_kq[1] : d_kq[0];
        ptx::tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t d = kq + ((ks >> 2) * (16384 >> 4) + (ks & 3) * (32 >> 4));
          ptx::mma_ss(tmem + kColD0, d, d, id_n64, ks > 0);
        }
        ptx::mma_commit(&bars[kPDone]);
      };
      // MMA4 of chunk j: D4 += Vd^T Pg^T on top of s gamma .* (Q S0)^T which the side warpgroup stored
      // there; both operands from shared memory (Vd tile j & 1)
      auto issue_mma4 = [&](int j) {
        const uint64_t dv = (j & 1) ? d_vd1 : d_vd0;
        ptx::tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          ptx::mma_ss(tmem + kColD4, dv + ks * (32 >> 4), d_pg + ks * (32 >> 4), id_n64, true);
        ptx::mma_commit(&bars[kD4Done]);
      };
      bool ok = true;
      if (nproc > 0) {
        ok = issue_u(0);
        if (ok && !kStateOnly) issue_p(0);
      }
      for (int i = 0; ok && i < nproc; ++i) {
        const int s = i & 1, ph = i & 1;
        // selects instead of dynamic indexing keep the descriptors in registers
        const uint64_t kq = s ? d_kq[1] : d_kq[0], kmn = s ? d_kmn[1] : d_kmn[0], ww = s ? d_w[1] : d_w[0];
        trace(0, i, 0);
        // MMA2: D2 += S0^T_bf16 (-Wt)^T  (B = the Wt tile, two 64-column halves 8 KiB apart)
        if (!(ok = ptx::mbar_spin(&bars[kSbfReady], ph, status, kTimeout | ((kSbfReady) << 8)))) break;
        trace(0, i, 2);
        ptx::tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          ptx::mma_ts(tmem + kColD2, tmem + kColSbf + ks * 8, ww + ((ks >> 2) * (8192 >> 4) + (ks & 3) * (32 >> 4)),
                      id_n64, ks > 0 || !p.zero_v);
        ptx::mma_commit(&bars[kD2Done]);
        trace(0, i, 3);
        // MMAq: Dq = S0^T_bf16 Q^T  (Q rows sit 8 KiB into each half of the stacked [K;Q] tile).  Dq is
        // free: the side warpgroup read the previous chunk's before MMA4 of that chunk was issued.
        if (!kStateOnly) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            ptx::mma_ts(tmem + kColDq, tmem + kColSbf + ks * 8,
                        kq + ((8192 >> 4) + (ks >> 2) * (16384 >> 4) + (ks & 3) * (32 >> 4)), id_n64, ks > 0);
          ptx::mma_commit(&bars[kDqDone]);
        }
        // MMA3: S^T += V'^T K   (B = K tile read MN-major: 64-column halves are 16 KiB apart)
        if (!(ok = ptx::mbar_spin(&bars[kVdReady], ph, status, kTimeout | ((kVdReady) << 8)))) break;
        if (!(ok = ptx::mbar_spin(&bars[kSScaled], ph, status, kTimeout | ((kSScaled) << 8)))) break;
        trace(0, i, 6);
        ptx::tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          ptx::mma_ts(tmem + kColS, tmem + kColD2 + ks * 8, kmn + ks * (2048 >> 4), id_mn128, true);
        ptx::mma_commit(&bars[kSDone]);
        ptx::mma_commit(&bars[kEmpty0 + s]);  // every MMA that reads this stage has been issued and tracked
        trace(0, i, 7);
        // tail: D2 is free again (the chain read Vd before VdReady, MMA3 precedes in the pipe)
        if (i + 1 < nproc && !(ok = issue_u(i + 1))) break;
        if (!kStateOnly) {
          if (!(ok = ptx::mbar_spin(&bars[kPgReady], ph, status, kTimeout | ((kPgReady) << 8)))) break;
          if (!(ok = ptx::mbar_spin(&bars[kQsStored], ph, status, kTimeout | ((kQsStored) << 8)))) break;
          issue_mma4(i);
          if (i + 1 < nproc) {
            if (!(ok = ptx::mbar_spin(&bars[kPFree], ph, status, kTimeout | ((kPFree) << 8)))) break;
            issue_p(i + 1);
          }
        }
        trace(0, i, 8);
      }
    }
  } else if (warp >= 10) {
    // =========================================================== aux warps 10, 11: operand tiles
    // (a) Ab = A diag(beta), in place in the stage's A tile (B operand of MMAu);
    // (b) Pg = s * G .* P from D0 rows 64..127 (TMEM quadrants 2, 3 = warps 10, 11) into a swizzled tile.
    const int r = tid - 320;  // 0..63: row of A / row c of P
    const uint32_t tm = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    // per-warp private copy of the chunk's cumulative gates (two chunks deep) so that the stage can be
    // released right after the A tile is scaled, long before Pg of that chunk is produced
    float* my_g = aux_g + (warp - 10) * 128;
    auto scale_a_tile = [&](int s, int chunk_parity) {
      const Gates* gs = gates_of(s);
      my_g[chunk_parity * 64 + lane] = gs->g[lane];
      my_g[chunk_parity * 64 + 32 + lane] = gs->g[32 + lane];
      uint8_t* at = stage_ptr(s) + kStageA;
#pragma unroll 1
      for (int c16 = 0; c16 < 8; ++c16) {
        uint4* ptr = reinterpret_cast<uint4*>(at + ptx::sw128_offset(r, c16));
        uint4 raw = *ptr;
        const float4 b0 = *reinterpret_cast<const float4*>(&gs->beta[c16 * 8]);
        const float4 b1 = *reinterpret_cast<const float4*>(&gs->beta[c16 * 8 + 4]);
        const T* e = reinterpret_cast<const T*>(&raw);
        raw = make_uint4(pack2<T>(Cvt<T>::to_f32(e[0]) * b0.x, Cvt<T>::to_f32(e[1]) * b0.y),
                         pack2<T>(Cvt<T>::to_f32(e[2]) * b0.z, Cvt<T>::to_f32(e[3]) * b0.w),
                         pack2<T>(Cvt<T>::to_f32(e[4]) * b1.x, Cvt<T>::to_f32(e[5]) * b1.y),
                         pack2<T>(Cvt<T>::to_f32(e[6]) * b1.z, Cvt<T>::to_f32(e[7]) * b1.w));
        *ptr = raw;
      }
      ptx::fence_proxy_async_smem();
      // one barrier per stage: the aux warps run one chunk ahead, and a waiter must never fall two
      // phases behind a barrier
      warp_arrive(&bars[kAbReady0 + s], lane);
      warp_arrive(&bars[kEmpty0 + s], lane);  // aux no longer touches stage s
    };
    bool ok = true;
    if (nproc > 0) {
      ok = ptx::mbar_wait_warp(&bars[kFull0], 0, status, kTimeout | ((kFull0) << 8));
      if (ok) scale_a_tile(0, 0);
    }
    for (int i = 0; ok && i < nproc; ++i) {
      const int s = i & 1, ph = i & 1;
      const float* gsg = my_g + (i & 1) * 64;
      // the A tile of the NEXT chunk first: MMAu of that chunk is issued in the tail of this one
      if (i + 1 < nproc) {
        if (!(ok = ptx::mbar_wait_warp(&bars[kFull0 + (s ^ 1)], ((i + 1) >> 1) & 1, status, kTimeout | ((kFull0 + (s ^ 1)) << 8)))) break;
        scale_a_tile(s ^ 1, (i + 1) & 1);
      }
      if (!kStateOnly) {
        if (tid == 320) trace(2, i, 8);
        if (!(ok = ptx::mbar_wait_warp(&bars[kPDone], ph, status, kTimeout | ((kPDone) << 8)))) break;
        // MMA4 of the previous chunk must have finished reading the Pg tile
        if (i > 0 && !(ok = ptx::mbar_wait_warp(&bars[kD4Done], (i - 1) & 1, status, kTimeout | ((kD4Done) << 8)))) break;
        ptx::tc_fence_after_sync();
        if (tid == 320) trace(2, i, 9);
        const int c = r;
        const float gc = gsg[c];
        uint8_t* pg = smem + kOffPg;
        // loops over 16-column groups are kept rolled: the per-chunk code of all roles has to stay
        // resident in the instruction cache
#pragma unroll 1
        for (int db = 0; db < 64; db += 16) {
          uint32_t pr[16];
          ptx::tmem_ld16(tm + kColD0 + db, pr);
          ptx::tmem_wait_ld();
          if (db == 48) {
            ptx::tc_fence_before_sync();
            warp_arrive(&bars[kPFree], lane);
          }
          // branch-free: every lane evaluates all entries, the causal mask is a select
#pragma unroll
          for (int j8 = 0; j8 < 16; j8 += 8) {
            const float4 ga = *reinterpret_cast<const float4*>(&gsg[db + j8]);
            const float4 gb = *reinterpret_cast<const float4*>(&gsg[db + j8 + 4]);
            const float gd[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float e = __expf(fminf(gc - gd[j], 0.f));
              const float val = p.scale * e * __uint_as_float(pr[j8 + j]);
              x[j] = (db + j8 + j <= c) ? val : 0.f;
            }
            *reinterpret_cast<uint4*>(pg + ptx::sw128_offset(c, (db + j8) >> 3)) =
                make_uint4(pack2<T>(x[0], x[1]), pack2<T>(x[2], x[3]), pack2<T>(x[4], x[5]), pack2<T>(x[6], x[7]));
          }
        }
        ptx::fence_proxy_async_smem();
        warp_arrive(&bars[kPgReady], lane);
        if (tid == 320) trace(2, i, 10);
      }
    }
  } else {
    // =========================================================== compute warpgroups
    // All loops over TMEM columns run in rolled groups of 16 columns (#pragma unroll 1): with four
    // roles executing different code every chunk, fully unrolled 64-column bodies overflow the
    // instruction cache and every SM stalls on instruction fetch.
    const int wg = warp >> 2;              // 0 = chain, 1 = side
    const int v = tid & 127;               // TMEM lane = state column
    const uint32_t tm = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const int col_half = wg * 64;          // this warpgroup converts state columns [col_half, col_half + 64)
    bool alive = true;
    // element (k, v) of a state tensor sits at k * st_k + v * st_v
    const int st_k = p.transpose_state ? 1 : kHeadDim, st_v = p.transpose_state ? kHeadDim : 1;
    float* fs_out = (p.final_state != nullptr && out_row >= 0)
                        ? p.final_state + (static_cast<int64_t>(out_row) * p.num_v_heads + hv) * kHeadDim * kHeadDim
                        : nullptr;
    const float* h0p = (!p.init_identity && p.h0 != nullptr)
                           ? p.h0 + (static_cast<int64_t>(seq) * p.num_v_heads + hv) * kHeadDim * kHeadDim
                           : nullptr;

    // ---- initial state: S = exp(gL_0) * S_init (fp32) and its 16-bit copy
    {
      float egl0 = 1.f;
      if (nproc > 0) {
        alive = ptx::mbar_wait_warp(&bars[kFull0], 0, status, kTimeout | ((kFull0) << 8));
        egl0 = gates_of(0)->egl;
      }
#pragma unroll 1
      for (int kb = 0; kb < 64; kb += 16) {
        float x[16];
        uint32_t sf[16], sb[8];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int k = col_half + kb + j;
          x[j] = 0.f;
          if (p.init_identity) x[j] = (k == v) ? 1.f : 0.f;
          else if (h0p != nullptr) x[j] = h0p[k * st_k + v * st_v];
        }
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          sf[j] = __float_as_uint(x[j] * egl0);
          sf[j + 1] = __float_as_uint(x[j + 1] * egl0);
          sb[j >> 1] = pack2<T>(x[j], x[j + 1]);
        }
        ptx::tmem_st16(tm + kColS + col_half + kb, sf);
        ptx::tmem_st8(tm + kColSbf + (col_half + kb) / 2, sb);
        if (nproc == 0 && fs_out != nullptr) {
#pragma unroll
          for (int j = 0; j < 16; ++j) fs_out[(col_half + kb + j) * st_k + v * st_v] = x[j];
        }
      }
      ptx::tmem_wait_st();
      ptx::tc_fence_before_sync();
      warp_arrive(&bars[kSbfReady], lane);
      warp_arrive(&bars[kSScaled], lane);
    }

    // Output epilogue of chunk j (side warpgroup): D4 holds O^T = s gamma .* (Q S0)^T + Vd^T Pg^T; it is
    // transposed through a shared-memory tile and written with one TMA store (row-masked stores for a
    // ragged tail).
    auto epilogue = [&](int j, int valid_j, int t0_j) -> bool {
      if (!ptx::mbar_wait_warp(&bars[kD4Done], j & 1, status, kTimeout | ((kD4Done) << 8))) return false;
      ptx::tc_fence_after_sync();
      if (tid == 128) trace(2, j, 6);
      T* so = reinterpret_cast<T*>(smem + kOffO + (j & 1) * 16384);
      // Two output tiles alternate: tile (j & 1) was last used by the TMA store of chunk j - 2, which
      // must have finished reading it.  Only mbarriers (bounded waits), never a CTA / named barrier.
      if (j >= 2) {
        if (tid == 128) {
          asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          ptx::mbar_arrive(&bars[kOFree]);
        }
        if (!ptx::mbar_wait_warp(&bars[kOFree], j & 1, status, kTimeout | ((kOFree) << 8))) return false;
      }
#pragma unroll 1
      for (int cb = 0; cb < 64; cb += 16) {
        uint32_t r[16];
        ptx::tmem_ld16(tm + kColD4 + cb, r);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 16; ++e) so[(cb + e) * kHeadDim + v] = Cvt<T>::from_f32(__uint_as_float(r[e]));
      }
      ptx::tc_fence_before_sync();
      if (tid == 128) trace(2, j, 12);
      ptx::fence_proxy_async_smem();
      warp_arrive(&bars[kOReady], lane);
      if (valid_j == kChunk) {
        if (warp == 4) {  // only the issuing warp waits for the tile to be complete
          if (!ptx::mbar_wait_warp(&bars[kOReady], j & 1, status, kTimeout | ((kOReady) << 8))) return false;
          if (tid == 128) {
            ptx::tma_store_3d(&tm_o, so, 0, hv, t0_j);
            ptx::tma_store_commit();
          }
        }
      } else {
        if (!ptx::mbar_wait_warp(&bars[kOReady], j & 1, status, kTimeout | ((kOReady) << 8))) return false;
        // ragged tail (always the last chunk of a sequence): row-masked 16-byte stores
        T* ob = static_cast<T*>(p.o);
        const int tl = tid - 128;  // 16 threads per row (8 elements each), 8 rows per pass
        for (int r0 = 0; r0 < valid_j; r0 += 8) {
          const int row = r0 + (tl >> 4);
          if (row < valid_j) {
            const uint4 x = *reinterpret_cast<const uint4*>(so + row * kHeadDim + (tl & 15) * 8);
            *reinterpret_cast<uint4*>(ob + (static_cast<int64_t>(t0_j + row) * p.num_v_heads + hv) * kHeadDim + (tl & 15) * 8) = x;
          }
        }
      }
      return true;
    };
    int prev_valid = 0, prev_t0 = 0;

    for (int i = 0; alive && i < nproc; ++i) {
      const int s = i & 1, ph = i & 1;
      const int chunk = first_chunk + i;
      const int t0 = seq_start + chunk * kChunk;
      const Gates* gs = gates_of(s);
      if (i > 0) alive = ptx::mbar_wait_warp(&bars[kFull0 + s], (i >> 1) & 1, status, kTimeout | ((kFull0 + s) << 8));
      if (!alive) break;
      if (tid == 128) trace(2, i, 0);
      const int valid = gs->valid;
      // the previous chunk's output first: its MMA4 was issued right after this chunk's MMA1
      if (!kStateOnly && wg == 1 && i > 0 && !(alive = epilogue(i - 1, prev_valid, prev_t0))) break;

      if (wg == 0) {
        // ---------------- chain: Vd (to the shared-memory tile of MMA4, and v_new) and V' = rho .* Vd
        if (!(alive = ptx::mbar_wait_warp(&bars[kD2Done], ph, status, kTimeout | ((kD2Done) << 8)))) break;
        ptx::tc_fence_after_sync();
        if (tid == 0) trace(1, i, 2);
        T* vn = static_cast<T*>(p.v_new);
        T* vn_dst = vn ? vn + (static_cast<int64_t>(t0) * p.num_v_heads + hv) * kHeadDim + v : nullptr;
        const int64_t vn_stride = static_cast<int64_t>(p.num_v_heads) * kHeadDim;
        uint8_t* vt = smem + kOffVd + (i & 1) * 16384;
#pragma unroll 1
        for (int cb = 0; cb < 64; cb += 16) {
          uint32_t d[16], vd[8], vp[8];
          ptx::tmem_ld16(tm + kColD2 + cb, d);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            const float4 r4 = *reinterpret_cast<const float4*>(&gs->rho[cb + j]);
            const float a0 = __uint_as_float(d[j]), a1 = __uint_as_float(d[j + 1]);
            const float a2 = __uint_as_float(d[j + 2]), a3 = __uint_as_float(d[j + 3]);
            vd[j >> 1] = pack2<T>(a0, a1);
            vd[(j >> 1) + 1] = pack2<T>(a2, a3);
            vp[j >> 1] = pack2<T>(a0 * r4.x, a1 * r4.y);
            vp[(j >> 1) + 1] = pack2<T>(a2 * r4.z, a3 * r4.w);
          }
          ptx::tmem_st8(tm + kColD2 + cb / 2, vp);  // V' in place (A operand of MMA3, on the chain)
          if (!kStateOnly) {
            *reinterpret_cast<uint4*>(vt + ptx::sw128_offset(v, cb >> 3)) = make_uint4(vd[0], vd[1], vd[2], vd[3]);
            *reinterpret_cast<uint4*>(vt + ptx::sw128_offset(v, (cb >> 3) + 1)) = make_uint4(vd[4], vd[5], vd[6], vd[7]);
          }
          if (vn_dst != nullptr) {
            const T* vdt = reinterpret_cast<const T*>(vd);
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (cb + j < valid) vn_dst[(cb + j) * vn_stride] = vdt[j];
          }
        }
        if (!kStateOnly) ptx::fence_proxy_async_smem();
        ptx::tmem_wait_st();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kVdReady], lane);
        if (tid == 0) trace(1, i, 3);
      } else if (!kStateOnly) {
        // ---------------- side: D4 <- s gamma .* (Q S0)^T; MMA4 accumulates Vd^T Pg^T on top later
        if (tid == 128) trace(2, i, 1);
        if (!(alive = ptx::mbar_wait_warp(&bars[kDqDone], ph, status, kTimeout | ((kDqDone) << 8)))) break;
        ptx::tc_fence_after_sync();
        if (tid == 128) trace(2, i, 2);
#pragma unroll 1
        for (int cb = 0; cb < 64; cb += 16) {
          uint32_t r[16];
          ptx::tmem_ld16(tm + kColDq + cb, r);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            const float4 g4 = *reinterpret_cast<const float4*>(&gs->gamma[cb + j]);
            r[j] = __float_as_uint(p.scale * g4.x * __uint_as_float(r[j]));
            r[j + 1] = __float_as_uint(p.scale * g4.y * __uint_as_float(r[j + 1]));
            r[j + 2] = __float_as_uint(p.scale * g4.z * __uint_as_float(r[j + 2]));
            r[j + 3] = __float_as_uint(p.scale * g4.w * __uint_as_float(r[j + 3]));
          }
          ptx::tmem_st16(tm + kColD4 + cb, r);
        }
        ptx::tmem_wait_st();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kQsStored], lane);
        if (tid == 128) trace(2, i, 3);
      }

      // ---------------- both: state convert after MMA3 (this warpgroup's 64 columns)
      if (!(alive = ptx::mbar_wait_warp(&bars[kSDone], ph, status, kTimeout | ((kSDone) << 8)))) break;
      ptx::tc_fence_after_sync();
      if (tid == 0) trace(1, i, 4);
      if (tid == 128) trace(2, i, 4);
      const bool last = (i + 1 == nproc);
      if (last) {
        if (fs_out != nullptr) {
#pragma unroll 1
          for (int kb = 0; kb < 64; kb += 16) {
            uint32_t sf[16];
            ptx::tmem_ld16(tm + kColS + col_half + kb, sf);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) fs_out[(col_half + kb + j) * st_k + v * st_v] = __uint_as_float(sf[j]);
          }
        }
      } else {
        if (!(alive = ptx::mbar_wait_warp(&bars[kFull0 + (s ^ 1)], ((i + 1) >> 1) & 1, status, kTimeout | ((kFull0 + (s ^ 1)) << 8)))) break;
        const float egl_next = gates_of(s ^ 1)->egl;
        T* hp = p.h ? static_cast<T*>(p.h) + ((chunk_base + chunk + 1) * p.num_v_heads + hv) * kHeadDim * kHeadDim + v
                    : nullptr;
        // (a) critical: 16-bit copy of the new state -> MMA1 of the next chunk may start
#pragma unroll 1
        for (int kb = 0; kb < 64; kb += 16) {
          uint32_t sf[16], sb[8];
          ptx::tmem_ld16(tm + kColS + col_half + kb, sf);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; j += 2) sb[j >> 1] = pack2<T>(__uint_as_float(sf[j]), __uint_as_float(sf[j + 1]));
          ptx::tmem_st8(tm + kColSbf + (col_half + kb) / 2, sb);
          if (hp != nullptr) {
            // h[chunk + 1] = state entering the next chunk, [K][V] layout
            const T* sbh = reinterpret_cast<const T*>(sb);
#pragma unroll
            for (int j = 0; j < 16; ++j) hp[(col_half + kb + j) * kHeadDim] = sbh[j];
          }
        }
        ptx::tmem_wait_st();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kSbfReady], lane);
        if (tid == 0) trace(1, i, 5);
        if (tid == 128) trace(2, i, 5);
        // (b) off the critical path: decay of the fp32 state for the next chunk (needed by MMA3 only)
#pragma unroll 1
        for (int kb = 0; kb < 64; kb += 16) {
          uint32_t sf[16];
          ptx::tmem_ld16(tm + kColS + col_half + kb, sf);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) sf[j] = __float_as_uint(__uint_as_float(sf[j]) * egl_next);
          ptx::tmem_st16(tm + kColS + col_half + kb, sf);
        }
        ptx::tmem_wait_st();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kSScaled], lane);
      }
      // The stage is released here: what follows for this chunk (MMA4, output store) only needs the
      // Vd / Pg tiles and tensor memory, so the producer can refill the stage already.
      warp_arrive(&bars[kEmpty0 + s], lane);
      prev_valid = valid;
      prev_t0 = t0;
    }
    if (!kStateOnly && wg == 1 && alive && nproc > 0) alive = epilogue(nproc - 1, prev_valid, prev_t0);
    if (!kStateOnly && tid == 128) ptx::tma_store_wait_all();
    // h[first chunk] = initial state
    if (p.h != nullptr && nproc > 0 && wg == 0) {
      T* hp = static_cast<T*>(p.h) + ((chunk_base + first_chunk) * p.num_v_heads + hv) * kHeadDim * kHeadDim;
#pragma unroll 4
      for (int k = 0; k < kHeadDim; ++k) {
        float x = 0.f;
        if (p.init_identity) x = (k == v) ? 1.f : 0.f;
        else if (h0p != nullptr) x = h0p[k * st_k + v * st_v];
        hp[k * kHeadDim + v] = Cvt<T>::from_f32(x);
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) ptx::tmem_dealloc(tmem, 512);
  if (cta_trace && tid == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    p.trace[cta_slot + 1] = static_cast<long long>(t);
  }
}

}  // namespace

int launch_chunk_fwd(const FwdParams& p, const void* q, const void* k, const void* v, const void* A,
                     const void* w, int64_t total_tokens, bool is_bf16, bool state_only, cudaStream_t stream) {
  CUtensorMap tm_q, tm_k, tm_v, tm_a, tm_w, tm_o;
  int rc;
  if ((rc = make_tmap_3d(&tm_k, k, total_tokens, p.num_k_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_q, state_only ? k : q, total_tokens, p.num_k_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_v, v, total_tokens, p.num_v_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_a, A, total_tokens, p.num_v_heads, 64, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_w, w, total_tokens, p.num_v_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_o, state_only ? v : p.o, total_tokens, p.num_v_heads, kHeadDim, 64, 128, false, is_bf16)) != QLA_OK) return rc;
  const unsigned grid = static_cast<unsigned>(p.num_seqs) * p.num_v_heads;
#define QLA_LAUNCH_FWD(T, SO, TR)                                                                          \
  do {                                                                                                     \
    QLA_CHECK_CUDA(cudaFuncSetAttribute(chunk_fwd_kernel<T, SO, TR>,                                       \
                                        cudaFuncAttributeMaxDynamicSharedMemorySize,                       \
                                        static_cast<int>(kSmemBytes)));                                    \
    chunk_fwd_kernel<T, SO, TR><<<grid, kThreads, kSmemBytes, stream>>>(tm_q, tm_k, tm_v, tm_a, tm_w, tm_o, p);  \
  } while (0)
  // the traced variant is a separate instantiation so that normal launches carry no tracing code
  const bool traced = p.trace != nullptr;
  if (is_bf16) {
    if (traced) { if (state_only) QLA_LAUNCH_FWD(__nv_bfloat16, true, true); else QLA_LAUNCH_FWD(__nv_bfloat16, false, true); }
    else if (state_only) QLA_LAUNCH_FWD(__nv_bfloat16, true, false);
    else QLA_LAUNCH_FWD(__nv_bfloat16, false, false);
  } else {
    if (traced) { if (state_only) QLA_LAUNCH_FWD(__half, true, true); else QLA_LAUNCH_FWD(__half, false, true); }
    else if (state_only) QLA_LAUNCH_FWD(__half, true, false);
    else QLA_LAUNCH_FWD(__half, false, false);
  }
#undef QLA_LAUNCH_FWD
  QLA_CHECK_CUDA(cudaGetLastError());
  return QLA_OK;
}

}  // namespace qla
