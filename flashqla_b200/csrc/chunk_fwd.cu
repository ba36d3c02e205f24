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
//   MMA0  D0[128,64]  = [-Wt;Q] K^T        (SS)  rows 64..127 are P = Q K^T; state independent
//   MMAu  D2[128,64]  = V^T Ab^T           (SS)  state independent part of Vd^T
//   MMA2  D2[128,64] += S0^T_bf16 (-Wt)^T  (TS)  D2 = Vd^T
//   MMAq  Dq[128,64]  = S0^T_bf16 Q^T      (TS)  (Q S0)^T for the output, off the chain
//   MMA3  S^T[128,128] += V'^T K           (TS, B operand MN-major straight from the K tile)
//   MMA4  D4[128,64] += Vd^T Pg^T          (SS)  Pg = s G .* P and Vd^T are swizzled smem tiles; off the chain
// Between two state updates only  MMA2 -> (V' = rho .* Vd) -> MMA3 -> (16-bit copy of the state)  are
// serial; the other products are issued into the two gaps and complete in their shadow.
// Thread v of a compute warpgroup owns TMEM lane v = column v of the state: it reads Vd^T rows
// with tcgen05.ld, applies the gates, and writes the bf16 operand of the next MMA back with
// tcgen05.st.  The fp32 state never leaves tensor memory between chunks.
//
// Warp roles (384 threads): warps 0-3 "chain" (Vd, state convert of columns 0..63), warps 4-7 "side"
// (output epilogue, state convert of columns 64..127), warp 8 TMA producer + gate vectors, warp 9 MMA
// issuer, warps 10-11 "aux" (operand tiles A diag(beta) and Pg).  Two smem stages of {Wt,Q,K,V,A}, a
// four-deep ring of gate vectors; all waits are bounded mbarrier waits that raise a status word instead
// of hanging.
#include "chunk_params.cuh"

namespace qla {


namespace {

// ---- tensor-memory column map (512 columns)
constexpr uint32_t kColS = 0;      // fp32 state S^T, 128 columns
constexpr uint32_t kColSbf = 128;  // bf16 copy of S^T (A operand of MMA2), 64 columns
constexpr uint32_t kColD2 = 192;   // Vd^T; columns 192..223 are overwritten in place by V' bf16 (A operand of MMA3)
constexpr uint32_t kColDq = 256;   // (Q S0)^T
constexpr uint32_t kColD4 = 320;   // output accumulator: s gamma .* (Q S0)^T, then += Vd^T Pg^T
constexpr uint32_t kColD0 = 384;   // [-Wt;Q] K^T, two buffers of 64 columns (chunk parity)

// ---- shared-memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kStageWQ = 0;         // 32 KiB: half 0 [-Wt rows | Q rows] (16 KiB), half 1 (16 KiB); SW128
constexpr uint32_t kStageK = 32768;      // 16 KiB: K tile as two [64][64] halves (columns 0..63 | 64..127), SW128
constexpr uint32_t kStageV = 49152;      // 16 KiB: V tile, same form
constexpr uint32_t kStageA = 65536;      // 8 KiB: A tile [64][64], SW128; scaled in place to A diag(beta)
constexpr uint32_t kStageBytes = 73728;  // 72 KiB, multiple of 1024
constexpr uint32_t kOffPg = 2 * kStageBytes;         // 2 x 8 KiB Pg tiles, SW128 (chunk parity)
constexpr uint32_t kOffO = kOffPg + 2 * 8192;        // 16 KiB output tile [64][128]
constexpr uint32_t kOffVd = kOffO + 16384;           // 2 x 16 KiB Vd^T tiles [128 v][64 d], SW128 (A of MMA4)
constexpr uint32_t kSmemBytes = kOffVd + 2 * 16384 + 1024;

struct alignas(16) Gates {
  // g * log2(e) in the two roles it plays for the aux warps, which form s exp(g_c - g_d) r_q[c] r_k[d] as
  // ex2(g2row[c] + log2 s - g2col[d]); r_q, r_k = 1 / |q_t|, 1 / |k_t| with in-kernel L2 norm, else 1
  float g2row[64];   // g log2(e) + log2 r_q
  float g2col[64];   // g log2(e) - log2 r_k
  float sgamma[64];  // scale * exp(g) * r_q
  float rho[64];
  float beta[64];
  float egl;
  int valid;  // number of valid tokens in the chunk
  int pad[2];
};
constexpr int kGateRing = 4;

enum Bar {
  kFull0 = 0, kFull1, kEmpty0, kEmpty1,
  kPDone0, kPDone1, kPgReady, kQsStored, kD2Done, kDqDone, kVdReady, kVdTile, kSDone, kSbfReady, kSScaled, kAbReady0, kAbReady1,
  kD4Done, kOFree, kOReady, kONormed,
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

// kAux: the launch stores h and / or v_new (training forward, backward recomputation).  A separate
// instantiation, so that the plain inference forward does not carry the 128 scattered stores per thread
// and chunk in its instruction stream: this kernel is bound by instruction fetch before anything else,
// and every loop below is shaped for a small per-chunk code footprint (32-column groups, rolled; every
// product issued from one place; barrier waits as real calls).
// kNorm: the output tile passes through the gated RMS norm that follows the op in a GDN layer
// (o <- o * rsqrt(mean_v(o^2) + eps) * weight[v] * silu(z[t, h, v])) before it is stored.
// kState16: h0 / final_state are bf16 (state pools); its own instantiation, like kNorm: the code of the plain
// forward must stay small (it is the instruction cache, not the work, that a few extra branches in the
// unrolled state loops cost: +20 % on the whole scan when they were part of the plain kernel).
template <typename T, bool kStateOnly, bool kAux, bool kTrace, bool kNorm = false, bool kState16 = false>
__global__ void __launch_bounds__(kThreads, 1)
chunk_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_a,
                 const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_o,
                 const FwdParams p) {
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? ptx::kFmtBF16 : ptx::kFmtF16;
  grid_dep_wait();    // earlier kernels of the stream have completed (see launch_dependent)
  grid_dep_launch();  // the next one may be scheduled; it waits the same way
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // A "dual" launch carries two passes over the same sequences in one grid: the CTAs of the second half run
  // the transition-matrix pass of context parallelism (start from the identity, V treated as zero) with their
  // own chunk limits and output rows (chunk_limit_b, seq_map_b, final_state_b).
  const bool pass_b = p.dual && blockIdx.x >= static_cast<unsigned>(p.num_seqs) * p.num_v_heads;
  const unsigned cta = pass_b ? blockIdx.x - static_cast<unsigned>(p.num_seqs) * p.num_v_heads : blockIdx.x;
  const bool zero_v = p.zero_v || pass_b, init_identity = p.init_identity || pass_b;
  const int32_t* chunk_limit = pass_b ? p.chunk_limit_b : p.chunk_limit;
  const int32_t* seq_map = pass_b ? p.seq_map_b : p.seq_map;
  void* final_state = pass_b ? p.final_state_b : p.final_state;
  const int hv = cta % p.num_v_heads;
  const int slot = cta / p.num_v_heads;
  const int seq = p.seq_order ? p.seq_order[slot] : slot;  // CTAs start in grid order: the caller's order of sequences
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
  if (chunk_limit != nullptr) {
    const int lim = chunk_limit[seq * p.num_v_heads + hv];
    if (lim <= 0) return;  // nothing asked of this (sequence, head); uniform for the whole CTA
    if (lim < nchunks) first_chunk = nchunks - lim;
  }
  // warm-up inside the scan: `lead` chunks of the interval in front (same sequence) are run first from a zero
  // state; nothing of them is stored (their own interval's CTA computes them exactly)
  const int lead = (p.lead != nullptr && !pass_b) ? p.lead[seq * p.num_v_heads + hv] : 0;
  first_chunk -= lead;
  const int nproc = nchunks - first_chunk;
  const int out_row = seq_map ? seq_map[seq] : seq;
  const int64_t chunk_base =
      p.chunk_offsets ? p.chunk_offsets[seq] : static_cast<int64_t>(seq) * ((p.seq_len + kChunk - 1) / kChunk);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // align up with pointer arithmetic on the shared array so that the compiler keeps the address space
  uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint64_t bars[kNumBars];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(16) float aux_g[2 * 2 * 128];  // [aux warp][chunk parity][row | column][64] cumulative gates
  // Gate vectors live in their own ring (indexed by chunk, not by stage): the compute warpgroups read
  // them long after the stage's tiles were consumed, and the stage must not wait for that.  Slot reuse
  // needs no barrier: chunk i + 2 is only loaded after MMA3 of chunk i was issued, which needs both
  // warpgroups to have left chunk i - 1, the last reader of the slot's previous tenant (chunk i - 2).
  __shared__ Gates gate_ring[kGateRing];

  if (tid == 0) {
#pragma unroll 1
    for (int b = 0; b < kNumBars; ++b) {
      int count = 1;  // kPDone*, kD2Done, kDqDone, kSDone, kD4Done, kOFree: one commit / one thread
      if (b == kFull0 || b == kFull1) count = 33;
      else if (b == kEmpty0 || b == kEmpty1) count = 3;
      else if (b == kPgReady || b == kAbReady0 || b == kAbReady1) count = 2;
      else if (b == kQsStored || b == kVdReady || b == kVdTile || b == kOReady || b == kONormed) count = 4;
      else if (b == kSbfReady || b == kSScaled) count = 8;
      ptx::mbar_init(&bars[b], count);
    }
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
  // every wait is a call: (barrier index, parity) -> warp-uniform verdict
  auto wait = [&](int b, uint32_t parity) {
    return ptx::mbar_wait_warp_call(&bars[b], parity, status, kStatusBarrierTimeout | (b << 8));
  };

  // phase trace: leaders of one CTA stamp clock64() for chunks kTraceFirstChunk.. (off when p.trace is NULL);
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
    unsigned sm;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
    p.trace[cta_slot] = static_cast<long long>(ptx::global_timer_ns());
    p.trace[cta_slot + 2] = sm;
  }

  auto stage_ptr = [&](int s) { return smem + s * kStageBytes; };
  auto gates_of = [&](int i) { return &gate_ring[i & (kGateRing - 1)]; };

  if (warp == 8) {
    // =========================================================== producer: TMA + gate vectors
    // L2 prefetch runs kPrefetchAhead chunks ahead of the demand loads: with every SM streaming its own
    // sequence the DRAM latency of a tile exceeds one chunk period, and only two stages fit in shared
    // memory, so the tiles are pulled into L2 early and the demand TMA then hits L2.  The loop starts
    // two iterations early so that the prefetch code exists once.
    constexpr int kPrefetchAhead = 4;
    for (int i = 2 - kPrefetchAhead; i < nproc; ++i) {
      if (lane == 0 && i + kPrefetchAhead < nproc) {
        const int pt0 = seq_start + (first_chunk + i + kPrefetchAhead) * kChunk;
#pragma unroll 1
        for (int x = 0; x < 128; x += 64) {
          ptx::tma_prefetch_l2_3d(&tm_k, x, hk, pt0);
          if (!kStateOnly) ptx::tma_prefetch_l2_3d(&tm_q, x, hk, pt0);
          if (!zero_v) ptx::tma_prefetch_l2_3d(&tm_v, x, hv, pt0);
          ptx::tma_prefetch_l2_3d(&tm_w, x, hv, pt0);
        }
        ptx::tma_prefetch_l2_3d(&tm_a, 0, hv, pt0);
      }
      if (i < 0) continue;
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
      float2 rn[2];  // (1 / |q|, 1 / |k|)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int c = lane + 32 * r;
        const bool okc = c < valid;
        const int64_t tok = static_cast<int64_t>(t0) + c;
        gcv[r] = okc ? p.g_cumsum[tok * p.num_v_heads + hv] : gl;
        bcv[r] = okc ? load_scalar(p.beta, p.beta_dtype, tok * p.num_v_heads + hv) : 0.f;
        rn[r] = (okc && p.rnorm != nullptr) ? *reinterpret_cast<const float2*>(p.rnorm + (tok * p.num_k_heads + hk) * 2)
                                           : make_float2(1.f, 1.f);
      }
      if (use > 0 && !wait(kEmpty0 + s, (use - 1) & 1)) break;
      if (lane == 0) trace(0, i, 10);
      uint8_t* st = stage_ptr(s);
      if (lane == 0) {
        uint32_t bytes = 16384 + 8192 + 16384;  // K + A + Wt
        if (!kStateOnly) bytes += 16384;  // Q
        if (!zero_v) bytes += 16384;    // V
        uint64_t* full = &bars[kFull0 + s];
        ptx::mbar_expect_tx(full, bytes);
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {  // the two 64-column halves of every 128-wide tile
          ptx::tma_load_3d(st + kStageWQ + h * 16384, &tm_w, full, h * 64, hv, t0);
          if (!kStateOnly) ptx::tma_load_3d(st + kStageWQ + h * 16384 + 8192, &tm_q, full, h * 64, hk, t0);
          ptx::tma_load_3d(st + kStageK + h * 8192, &tm_k, full, h * 64, hk, t0);
          if (!zero_v) ptx::tma_load_3d(st + kStageV + h * 8192, &tm_v, full, h * 64, hv, t0);
        }
        ptx::tma_load_3d(st + kStageA, &tm_a, full, 0, hv, t0);
      }
      Gates* gs = gates_of(i);
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int c = lane + 32 * r;
        const bool ok = c < valid;
        const float gc = gcv[r], bc = bcv[r];
        const float g2 = gc * 1.4426950408889634f;
        gs->g2row[c] = g2 + __log2f(rn[r].x);
        gs->g2col[c] = g2 - __log2f(rn[r].y);
        gs->sgamma[c] = p.scale * __expf(gc) * rn[r].x;
        gs->rho[c] = ok ? __expf(gl - gc) * rn[r].y : 0.f;
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
    // =========================================================== MMA issuer (whole warp, converged)
    // Every lane runs this loop and all waits; the tcgen05.mma / commit instructions are issued by one
    // elected lane inside the ptx::umma_* blocks.  Keeping the warp converged keeps descriptors and
    // addresses on the uniform datapath, which is what makes a product cost no more than its time on
    // the tensor pipe.  The loop is software pipelined over i = -1 .. nproc so that every product is
    // issued from exactly one place in the code:
    //   [MMA2(i)] [MMAq(i), MMA4(i-1)] [MMA3(i)] [MMAu(i+1), MMA0(i+1)]
    // Between two state updates only MMA2 -> (chain: V') -> MMA3 -> (both warpgroups: 16-bit state copy)
    // are serial; the other products sit in the two gaps and complete in their shadow.
    {
      const uint32_t id_n64 = ptx::mma_idesc(128, 64, fmt, ptx::kMajorK, ptx::kMajorK);
      const uint32_t id_mn128 = ptx::mma_idesc(128, 128, fmt, ptx::kMajorK, ptx::kMajorMN);
      const uint32_t id_u = ptx::mma_idesc(128, 64, fmt, ptx::kMajorMN, ptx::kMajorK);
      // operand descriptors of stage 0; stage 1 is kStageBytes further (added to the address field)
      const uint64_t d_wq = ptx::smem_desc_sw128(ptx::smem_u32(smem + kStageWQ), 16, 1024);    // [-Wt;Q], K-major
      const uint64_t d_k = ptx::smem_desc_sw128(ptx::smem_u32(smem + kStageK), 16, 1024);      // K tile, K-major
      const uint64_t d_kmn = ptx::smem_desc_sw128(ptx::smem_u32(smem + kStageK), 8192, 1024);  // K tile, MN-major
      const uint64_t d_a = ptx::smem_desc_sw128(ptx::smem_u32(smem + kStageA), 16, 1024);
      const uint64_t d_v = ptx::smem_desc_sw128(ptx::smem_u32(smem + kStageV), 8192, 1024);    // V tile, MN-major
      const uint64_t d_pg = ptx::smem_desc_sw128(ptx::smem_u32(smem + kOffPg), 16, 1024);
      const uint64_t d_vd = ptx::smem_desc_sw128(ptx::smem_u32(smem + kOffVd), 16, 1024);
      constexpr int kHalfWQ = (16384 >> 4) - 3 * 2;  // from k-step 3 to k-step 4 of the stacked tile
      constexpr int kHalfK = (8192 >> 4) - 3 * 2;
      // The CTA owns all 512 columns, so the allocation starts at column 0 of lane 0: tensor-memory
      // addresses are compile-time constants here (checked once; a value loaded from shared memory would
      // have to be moved to a uniform register for every instruction).  Barrier addresses for the commits
      // that the product blocks issue themselves.
      constexpr uint32_t tmem0 = 0;
      const uint32_t bar0 = ptx::smem_u32(&bars[0]);
      auto bar_addr = [&](int b) { return bar0 + 8u * static_cast<uint32_t>(b); };
      bool ok = tmem == tmem0;
      if (!ok) ptx::record_wait_failure(status, kStatusBadTmemBase, 0);
#pragma unroll 1
      for (int i = -1; ok && i <= nproc; ++i) {
        const int ph = i & 1, prev = (i - 1) & 1;
        const uint64_t so = static_cast<uint64_t>((i & 1) * (kStageBytes >> 4));
        const bool cur = i >= 0 && i < nproc;
        if (cur) {
          if (lane == 0) trace(0, i, 0);
          // MMA2: D2 += S0^T_bf16 (-Wt)^T on top of MMAu's product.  (The wait on the previous chunk's VdTile
          // sits before this chunk's MMA2 so that the barrier cannot complete its next phase first.)
          if (!kStateOnly && i > 0 && !(ok = wait(kVdTile, prev))) break;
          if (!(ok = wait(kSbfReady, ph))) break;
          if (lane == 0) trace(0, i, 2);
          ptx::tc_fence_after_sync();
          ptx::umma_ts_k128<2, kHalfWQ>(tmem0 + kColD2, tmem0 + kColSbf, d_wq + so, id_n64,
                                        kStateOnly ? !zero_v : true, bar_addr(kD2Done));
          if (lane == 0) trace(0, i, 3);
        }
        // gap 1 (the chain computes V'): MMAq(i): Dq = S0^T_bf16 Q^T (Q rows sit 8 KiB into each half of the
        // stacked tile; the side warpgroup has read the previous Dq before it arrived on QsStored), then
        // MMA4(i - 1): D4 += Vd^T Pg^T on top of s gamma .* (Q S0)^T which the side warpgroup stored there;
        // both operands from shared memory (tiles (i - 1) & 1)
        if (!kStateOnly && i >= 0) {
          if (i > 0) {
            if (i == nproc && !(ok = wait(kVdTile, prev))) break;
            if (!(ok = wait(kQsStored, prev))) break;
          }
          if (cur) {
            ptx::umma_ts_k128<2, kHalfWQ>(tmem0 + kColDq, tmem0 + kColSbf, d_wq + so + (8192 >> 4), id_n64, false,
                                          bar_addr(kDqDone));
          }
          if (i > 0) {
            if (!(ok = wait(kPgReady, prev))) break;
            ptx::tc_fence_after_sync();
            ptx::umma_ss_k64<2, 2>(tmem0 + kColD4, d_vd + static_cast<uint64_t>(prev * (16384 >> 4)),
                                   d_pg + static_cast<uint64_t>(prev * (8192 >> 4)), id_n64, true, bar_addr(kD4Done));
          }
        }
        if (cur) {
          if (lane == 0) trace(0, i, 4);
          // MMA3: S^T += V'^T K   (B = K tile read MN-major: 64-column halves are 8 KiB apart)
          if (!(ok = wait(kVdReady, ph))) break;
          if (!(ok = wait(kSScaled, ph))) break;
          if (lane == 0) trace(0, i, 6);
          ptx::tc_fence_after_sync();
          // (second commit: every MMA that reads this stage has been issued and tracked)
          ptx::umma_ts_k64<128>(tmem0 + kColS, tmem0 + kColD2, d_kmn + so, id_mn128, true, bar_addr(kSDone),
                                bar_addr(kEmpty0 + (i & 1)));
          if (lane == 0) trace(0, i, 7);
        }
        // gap 2 (both warpgroups convert the state): the state-independent products of the next chunk.
        // MMAu(i + 1): D2 = V^T (A diag(beta))^T; A operand = V tile read MN-major, B operand = the A tile after
        // the aux warps scaled its columns by beta in place.  D2 is free (the chain read Vd before VdReady,
        // MMA3 precedes in the pipe).  MMA0(i + 1): D0[(i + 1) & 1] = [-Wt;Q] K^T; that buffer was last read
        // for Pg of chunk i - 1, which preceded that chunk's MMA4.
        if (i + 1 < nproc) {
          const int j = i + 1, sj = j & 1;
          const uint64_t sn = static_cast<uint64_t>(sj * (kStageBytes >> 4));
          if (!(ok = wait(kFull0 + sj, (j >> 1) & 1))) break;
          if (!(ok = wait(kAbReady0 + sj, (j >> 1) & 1))) break;
          ptx::tc_fence_after_sync();
          if (!zero_v) ptx::umma_ss_k64<128, 2>(tmem0 + kColD2, d_v + sn, d_a + sn, id_u, false);
          if (!kStateOnly)  // (one PDone barrier per parity: the aux warps may lag a chunk)
            ptx::umma_ss_k128<2, kHalfWQ, 2, kHalfK>(tmem0 + kColD0 + sj * 64, d_wq + sn, d_k + sn, id_n64, false,
                                                     bar_addr(kPDone0 + sj));
        }
        if (cur && lane == 0) trace(0, i, 8);
      }
    }
  } else if (warp >= 10) {
    // =========================================================== aux warps 10, 11: operand tiles
    // (a) Ab = A diag(beta), in place in the stage's A tile (B operand of MMAu);
    // (b) Pg = s * G .* P from D0 rows 64..127 (TMEM quadrants 2, 3 = warps 10, 11) into a swizzled tile.
    // Software pipelined over i = -1 .. nproc - 1 so that the tile-scaling code exists once.
    const int r = tid - 320;  // 0..63: row of A / row c of P
    const uint32_t tm = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    // per-warp private copy of the chunk's cumulative gates (two chunks deep)
    float* my_g = aux_g + (warp - 10) * 256;
    const float log2_scale = __log2f(p.scale);
    bool ok = true;
#pragma unroll 1
    for (int i = -1; ok && i < nproc; ++i) {
      // the A tile of the NEXT chunk first: MMAu of that chunk is issued in the second half of this one
      if (i + 1 < nproc) {
        const int j = i + 1, sj = j & 1;
        if (!(ok = wait(kFull0 + sj, (j >> 1) & 1))) break;
        const Gates* gs = gates_of(j);
        my_g[sj * 128 + lane] = gs->g2row[lane];
        my_g[sj * 128 + 32 + lane] = gs->g2row[32 + lane];
        my_g[sj * 128 + 64 + lane] = gs->g2col[lane];
        my_g[sj * 128 + 96 + lane] = gs->g2col[32 + lane];
        uint8_t* at = stage_ptr(sj) + kStageA;
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
        warp_arrive(&bars[kAbReady0 + sj], lane);
        warp_arrive(&bars[kEmpty0 + sj], lane);  // aux no longer touches stage sj
      }
      if (!kStateOnly && i >= 0) {
        const int ph = i & 1;
        const float* gsg = my_g + ph * 128;
        if (tid == 320) trace(2, i, 8);
        if (!(ok = wait(kPDone0 + ph, (i >> 1) & 1))) break;
        ptx::tc_fence_after_sync();
        if (tid == 320) trace(2, i, 9);
        const int c = r;
        // s * exp(g_c - g_d) = 2^((g2_c + log2 s) - g2_d); above the diagonal the exponent may overflow, the
        // select below discards those entries
        const float gc = gsg[c] + log2_scale;
        const float* gcol = gsg + 64;
        // Pg tile i & 1 was last read by MMA4 of chunk i - 2; the wait for that is at the end of the previous
        // iteration
        uint8_t* pg = smem + kOffPg + ph * 8192;
#pragma unroll 1
        for (int db = 0; db < 64; db += 16) {
          uint32_t pr[16];
          ptx::tmem_ld16(tm + kColD0 + ph * 64 + db, pr);
          ptx::tmem_wait_ld();
          // branch-free: every lane evaluates all entries, the causal mask is a select
#pragma unroll
          for (int j8 = 0; j8 < 16; j8 += 8) {
            const float4 ga = *reinterpret_cast<const float4*>(&gcol[db + j8]);
            const float4 gb = *reinterpret_cast<const float4*>(&gcol[db + j8 + 4]);
            const float gd[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float val = ptx::ex2(gc - gd[j]) * __uint_as_float(pr[j8 + j]);
              x[j] = (db + j8 + j <= c) ? val : 0.f;
            }
            *reinterpret_cast<uint4*>(pg + ptx::sw128_offset(c, (db + j8) >> 3)) =
                make_uint4(pack2<T>(x[0], x[1]), pack2<T>(x[2], x[3]), pack2<T>(x[4], x[5]), pack2<T>(x[6], x[7]));
          }
        }
        ptx::fence_proxy_async_smem();
        ptx::tc_fence_before_sync();
        // Before announcing this tile, make sure MMA4 of the previous chunk has finished: the next
        // iteration overwrites the tile it read.  Waiting HERE (MMA4 of this chunk cannot be issued
        // before the arrival below) keeps this warp at most one phase behind the D4Done barrier.
        if (i > 0 && !(ok = wait(kD4Done, (i - 1) & 1))) break;
        warp_arrive(&bars[kPgReady], lane);
        if (tid == 320) trace(2, i, 10);
      }
    }
  } else {
    // =========================================================== compute warpgroups
    const int wg = warp >> 2;              // 0 = chain, 1 = side
    const int v = tid & 127;               // TMEM lane = state column
    const uint32_t tm = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const int col_half = wg * 64;          // this warpgroup converts state columns [col_half, col_half + 64)
    bool alive = true;
    // element (k, v) of a state tensor sits at k * st_k + v * st_v
    const int st_k = p.transpose_state ? 1 : kHeadDim, st_v = p.transpose_state ? kHeadDim : 1;
    // states are fp32 or bf16 (state pools of the recurrent op); the slot of a sequence comes from h0_map /
    // seq_map, so that a serving loop can prefill straight from and into its pool
    constexpr bool st16 = kState16;
    const int64_t fs_off = (static_cast<int64_t>(out_row) * p.num_v_heads + hv) * kHeadDim * kHeadDim;
    const bool fs16 = st16 && !pass_b;  // (transition matrices are always fp32)
    float* fs_out = (final_state != nullptr && out_row >= 0 && !fs16) ? static_cast<float*>(final_state) + fs_off : nullptr;
    __nv_bfloat16* fs_out16 =
        (final_state != nullptr && out_row >= 0 && fs16) ? static_cast<__nv_bfloat16*>(final_state) + fs_off : nullptr;
    const int h0_row = p.h0_map != nullptr ? p.h0_map[seq] : seq;
    const bool h0_16 = st16 && !p.h0_kv;
    const int h0_k = (p.transpose_state && !p.h0_kv) ? 1 : kHeadDim, h0_v = (p.transpose_state && !p.h0_kv) ? kHeadDim : 1;
    const int64_t h0_off = (static_cast<int64_t>(h0_row) * p.num_v_heads + hv) * kHeadDim * kHeadDim;
    const bool has_h0 = !init_identity && p.h0 != nullptr && h0_row >= 0 && lead == 0;
    const float* h0p = (has_h0 && !h0_16) ? static_cast<const float*>(p.h0) + h0_off : nullptr;
    const __nv_bfloat16* h0p16 = (has_h0 && h0_16) ? static_cast<const __nv_bfloat16*>(p.h0) + h0_off : nullptr;
    auto store_final = [&](int k, float x) {
      if (!kState16 || fs_out != nullptr) fs_out[k * st_k + v * st_v] = x;
      else if (fs_out16 != nullptr) fs_out16[k * st_k + v * st_v] = __float2bfloat16_rn(x);
    };
    const bool write_final = fs_out != nullptr || (kState16 && fs_out16 != nullptr);
    const int64_t vn_stride = static_cast<int64_t>(p.num_v_heads) * kHeadDim;

    // ---- initial state: S = exp(gL_0) * S_init (fp32) and its 16-bit copy.  This thread's 64 values are requested
    // before anything is waited for: their latency then overlaps the arrival of the first stage instead of
    // following it (with context-parallel segments of a dozen chunks a CTA's start-up is a tenth of its life).
    {
      float x[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        const int k = col_half + j;
        x[j] = 0.f;
        if (init_identity) x[j] = (k == v) ? 1.f : 0.f;
        else if (h0p != nullptr) x[j] = h0p[k * h0_k + v * h0_v];
        else if (kState16 && h0p16 != nullptr) x[j] = __bfloat162float(h0p16[k * h0_k + v * h0_v]);
      }
      float egl0 = 1.f;
      if (nproc > 0) {
        alive = wait(kFull0, 0);
        egl0 = gates_of(0)->egl;
      }
      T* hp0 = (kAux && p.h != nullptr && nproc > 0 && lead == 0)
                   ? static_cast<T*>(p.h) + ((chunk_base + first_chunk) * p.num_v_heads + hv) * kHeadDim * kHeadDim + v
                   : nullptr;
#pragma unroll
      for (int kb = 0; kb < 64; kb += 16) {
        uint32_t sf[16], sb[8];
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          sf[j] = __float_as_uint(x[kb + j] * egl0);
          sf[j + 1] = __float_as_uint(x[kb + j + 1] * egl0);
          sb[j >> 1] = pack2<T>(x[kb + j], x[kb + j + 1]);
        }
        ptx::tmem_st16(tm + kColS + col_half + kb, sf);
        ptx::tmem_st8(tm + kColSbf + (col_half + kb) / 2, sb);
        if (kAux && hp0 != nullptr) {  // h[first chunk] = initial state, [K][V] layout
          const T* sbh = reinterpret_cast<const T*>(sb);
#pragma unroll
          for (int j = 0; j < 16; ++j) hp0[(col_half + kb + j) * kHeadDim] = sbh[j];
        }
        if (nproc == 0 && write_final) {
#pragma unroll
          for (int j = 0; j < 16; ++j) store_final(col_half + kb + j, x[kb + j]);
        }
      }
      ptx::tmem_wait_st();
      ptx::tc_fence_before_sync();
      warp_arrive(&bars[kSbfReady], lane);
      warp_arrive(&bars[kSScaled], lane);
    }

    int prev_valid = 0, prev_t0 = 0;
    // The side warpgroup runs one extra iteration (i == nproc) for the last chunk's output.
    const int niter = (!kStateOnly && wg == 1 && nproc > 0) ? nproc + 1 : nproc;
#pragma unroll 1
    for (int i = 0; alive && i < niter; ++i) {
      const int s = i & 1, ph = i & 1;
      const int chunk = first_chunk + i;
      const int t0 = seq_start + chunk * kChunk;
      const Gates* gs = gates_of(i);
      const bool cur = i < nproc;
      // (the gates of chunk i are visible: convert (b) of the previous iteration waited for this stage's Full)
      if (tid == 128) trace(2, i, 0);
      const int valid = cur ? gs->valid : 0;

      if (wg == 0) {
        // ---------------- chain: V' = rho .* Vd back into tensor memory (MMA3 waits for it), Vd itself to the
        // shared-memory tile of MMA4 (and v_new).  32 columns at a time: V' of columns 32h.. lands in
        // columns 16h.. of D2, which the other half never reads.
        if (!(alive = wait(kD2Done, ph))) break;
        ptx::tc_fence_after_sync();
        if (tid == 0) trace(1, i, 2);
        uint8_t* vt = smem + kOffVd + (i & 1) * 16384;
        T* vn_dst = (kAux && p.v_new != nullptr && i >= lead)
                        ? static_cast<T*>(p.v_new) + (static_cast<int64_t>(t0) * p.num_v_heads + hv) * kHeadDim + v
                        : nullptr;
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          uint32_t d[32], vp[16];
          ptx::tmem_ld32(tm + kColD2 + 32 * h, d);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 r4 = *reinterpret_cast<const float4*>(&gs->rho[32 * h + j]);
            vp[j >> 1] = pack2<T>(__uint_as_float(d[j]) * r4.x, __uint_as_float(d[j + 1]) * r4.y);
            vp[(j >> 1) + 1] = pack2<T>(__uint_as_float(d[j + 2]) * r4.z, __uint_as_float(d[j + 3]) * r4.w);
          }
          ptx::tmem_st16(tm + kColD2 + 16 * h, vp);
          if (!kStateOnly || kAux) {
#pragma unroll
            for (int c8 = 0; c8 < 4; ++c8) {
              const uint4 pk = make_uint4(pack2<T>(__uint_as_float(d[c8 * 8]), __uint_as_float(d[c8 * 8 + 1])),
                                          pack2<T>(__uint_as_float(d[c8 * 8 + 2]), __uint_as_float(d[c8 * 8 + 3])),
                                          pack2<T>(__uint_as_float(d[c8 * 8 + 4]), __uint_as_float(d[c8 * 8 + 5])),
                                          pack2<T>(__uint_as_float(d[c8 * 8 + 6]), __uint_as_float(d[c8 * 8 + 7])));
              if (!kStateOnly) *reinterpret_cast<uint4*>(vt + ptx::sw128_offset(v, 4 * h + c8)) = pk;
              if (kAux && vn_dst != nullptr) {
                const T* vdt = reinterpret_cast<const T*>(&pk);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (32 * h + c8 * 8 + j < valid) vn_dst[(32 * h + c8 * 8 + j) * vn_stride] = vdt[j];
              }
            }
          }
        }
        ptx::tmem_wait_st();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kVdReady], lane);
        if (tid == 0) trace(1, i, 3);
        if (!kStateOnly) {
          ptx::fence_proxy_async_smem();
          warp_arrive(&bars[kVdTile], lane);
        }
      } else if (!kStateOnly) {
        // ---------------- side: output of the previous chunk (its MMA4 was issued right after this chunk's
        // MMA2).  D4 holds O^T = s gamma .* (Q S0)^T + Vd^T Pg^T; it is transposed through a shared-memory tile
        // and written with one TMA store (row-masked stores for a ragged tail).
        if (i > 0) {
          const int j = i - 1;
          T* so = reinterpret_cast<T*>(smem + kOffO);
          // One output tile: the TMA store of the chunk before (issued a whole chunk period ago) must have
          // finished reading it.  Only mbarriers (bounded waits), never a CTA / named barrier.
          if (j >= 1) {
            if (tid == 128) {
              ptx::tma_store_wait_read();
              ptx::mbar_arrive(&bars[kOFree]);
            }
            if (!(alive = wait(kOFree, (j - 1) & 1))) break;
          }
          if (!(alive = wait(kD4Done, j & 1))) break;
          ptx::tc_fence_after_sync();
          if (tid == 128) trace(2, j, 6);
#pragma unroll 1
          for (int cb = 0; cb < 64; cb += 32) {
            uint32_t r[32];
            ptx::tmem_ld32(tm + kColD4 + cb, r);
            ptx::tmem_wait_ld();
            T* dst = so + cb * kHeadDim + v;
#pragma unroll
            for (int e = 0; e < 32; ++e) dst[e * kHeadDim] = Cvt<T>::from_f32(__uint_as_float(r[e]));
          }
          ptx::tc_fence_before_sync();
          if (tid == 128) trace(2, j, 12);
          ptx::fence_proxy_async_smem();
          warp_arrive(&bars[kOReady], lane);
          if (kNorm) {
            // gated RMS norm of the finished tile, in place: 16 threads per token row (8 values each), 8 rows per pass
            if (!(alive = wait(kOReady, j & 1))) break;
            const int tl = tid - 128, c8 = (tl & 15) * 8;
            const T* zb = static_cast<const T*>(p.norm_gate);
            const float4 w0 = *reinterpret_cast<const float4*>(p.norm_weight + c8);
            const float4 w1 = *reinterpret_cast<const float4*>(p.norm_weight + c8 + 4);
            const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll 1
            for (int r8 = 0; r8 < kChunk; r8 += 8) {
              const int row = r8 + (tl >> 4);
              uint4* cell = reinterpret_cast<uint4*>(so + row * kHeadDim + c8);
              uint4 raw = *cell;
              uint4 zraw = make_uint4(0, 0, 0, 0);
              if (row < prev_valid)
                zraw = *reinterpret_cast<const uint4*>(zb + (static_cast<int64_t>(prev_t0 + row) * p.num_v_heads + hv) * kHeadDim + c8);
              const T* e = reinterpret_cast<const T*>(&raw);
              const T* ze = reinterpret_cast<const T*>(&zraw);
              float x[8], ss = 0.f;
#pragma unroll
              for (int q8 = 0; q8 < 8; ++q8) {
                x[q8] = Cvt<T>::to_f32(e[q8]);
                ss = fmaf(x[q8], x[q8], ss);
              }
#pragma unroll
              for (int off = 1; off < 16; off <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
              const float rstd = rsqrtf(ss * (1.f / kHeadDim) + p.norm_eps);
#pragma unroll
              for (int q8 = 0; q8 < 8; ++q8) {
                const float z = Cvt<T>::to_f32(ze[q8]);
                x[q8] = x[q8] * rstd * wv[q8] * (z / (1.f + __expf(-z)));
              }
              *cell = make_uint4(pack2<T>(x[0], x[1]), pack2<T>(x[2], x[3]), pack2<T>(x[4], x[5]), pack2<T>(x[6], x[7]));
            }
            ptx::fence_proxy_async_smem();
            warp_arrive(&bars[kONormed], lane);
          }
          constexpr int kTileDone = kNorm ? kONormed : kOReady;
          if (prev_valid == kChunk) {
            if (warp == 4) {  // only the issuing warp waits for the tile to be complete
              if (!(alive = wait(kTileDone, j & 1))) break;
              if (tid == 128) {
                ptx::tma_store_3d(&tm_o, so, 0, hv, prev_t0);
                ptx::tma_store_commit();
              }
            }
          } else {
            if (!(alive = wait(kTileDone, j & 1))) break;
            // ragged tail (always the last chunk of a sequence): row-masked 16-byte stores
            T* ob = static_cast<T*>(p.o);
            const int tl = tid - 128;  // 16 threads per row (8 elements each), 8 rows per pass
#pragma unroll 1
            for (int r0 = 0; r0 < prev_valid; r0 += 8) {
              const int row = r0 + (tl >> 4);
              if (row < prev_valid) {
                const uint4 x = *reinterpret_cast<const uint4*>(so + row * kHeadDim + (tl & 15) * 8);
                *reinterpret_cast<uint4*>(ob + (static_cast<int64_t>(prev_t0 + row) * p.num_v_heads + hv) * kHeadDim + (tl & 15) * 8) = x;
              }
            }
          }
        }
        if (!cur) break;
        // D4 <- s gamma .* (Q S0)^T (MMA4 accumulates Vd^T Pg^T on top later)
        if (tid == 128) trace(2, i, 1);
        if (!(alive = wait(kDqDone, ph))) break;
        ptx::tc_fence_after_sync();
        if (tid == 128) trace(2, i, 2);
#pragma unroll 1
        for (int cb = 0; cb < 64; cb += 32) {
          uint32_t r[32];
          ptx::tmem_ld32(tm + kColDq + cb, r);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 g4 = *reinterpret_cast<const float4*>(&gs->sgamma[cb + j]);
            r[j] = __float_as_uint(g4.x * __uint_as_float(r[j]));
            r[j + 1] = __float_as_uint(g4.y * __uint_as_float(r[j + 1]));
            r[j + 2] = __float_as_uint(g4.z * __uint_as_float(r[j + 2]));
            r[j + 3] = __float_as_uint(g4.w * __uint_as_float(r[j + 3]));
          }
          ptx::tmem_st32(tm + kColD4 + cb, r);
        }
        ptx::tmem_wait_st();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kQsStored], lane);
        if (tid == 128) trace(2, i, 3);
      }

      // ---------------- both: state convert after MMA3 (this warpgroup's 64 columns)
      if (!(alive = wait(kSDone, ph))) break;
      ptx::tc_fence_after_sync();
      if (tid == 0) trace(1, i, 4);
      if (tid == 128) trace(2, i, 4);
      const bool last = (i + 1 == nproc);
      if (last) {
        if (write_final) {
#pragma unroll 1
          for (int kb = 0; kb < 64; kb += 16) {
            uint32_t sf[16];
            ptx::tmem_ld16(tm + kColS + col_half + kb, sf);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) store_final(col_half + kb + j, __uint_as_float(sf[j]));
          }
        }
      } else {
        T* hp = (kAux && p.h != nullptr && i + 1 >= lead)
                    ? static_cast<T*>(p.h) + ((chunk_base + chunk + 1) * p.num_v_heads + hv) * kHeadDim * kHeadDim + v
                    : nullptr;
        // (a) critical: 16-bit copy of the new state -> MMA2 of the next chunk may start
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          uint32_t sf[32], sb[16];
          ptx::tmem_ld32(tm + kColS + col_half + 32 * h, sf);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j += 2) sb[j >> 1] = pack2<T>(__uint_as_float(sf[j]), __uint_as_float(sf[j + 1]));
          ptx::tmem_st16(tm + kColSbf + col_half / 2 + 16 * h, sb);
          if (kAux && hp != nullptr) {
            // h[chunk + 1] = state entering the next chunk, [K][V] layout
            const T* sbh = reinterpret_cast<const T*>(sb);
#pragma unroll
            for (int j = 0; j < 32; ++j) hp[(col_half + 32 * h + j) * kHeadDim] = sbh[j];
          }
        }
        ptx::tmem_wait_st();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kSbfReady], lane);
        if (tid == 0) trace(1, i, 5);
        if (tid == 128) trace(2, i, 5);
        // (b) off the critical path: decay of the fp32 state for the next chunk (needed by MMA3 only)
        if (!(alive = wait(kFull0 + (s ^ 1), ((i + 1) >> 1) & 1))) break;
        const float egl_next = gates_of(i + 1)->egl;
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          uint32_t sf[32];
          ptx::tmem_ld32(tm + kColS + col_half + 32 * h, sf);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) sf[j] = __float_as_uint(__uint_as_float(sf[j]) * egl_next);
          ptx::tmem_st32(tm + kColS + col_half + 32 * h, sf);
        }
        ptx::tmem_wait_st();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kSScaled], lane);
      }
      prev_valid = i < lead ? 0 : valid;  // nothing of a warm-up chunk is stored
      prev_t0 = t0;
    }
    if (!kStateOnly && tid == 128) ptx::tma_store_wait_all();
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) ptx::tmem_dealloc(tmem, 512);
  if (cta_trace && tid == 0) p.trace[cta_slot + 1] = static_cast<long long>(ptx::global_timer_ns());
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
  const unsigned grid = static_cast<unsigned>(p.num_seqs) * p.num_v_heads * (p.dual ? 2 : 1);
#define QLA_LAUNCH_FWD(T, SO, AUX, TR)                                                                          \
  do {                                                                                                          \
    { const int rc_ = ensure_dynamic_smem<chunk_fwd_kernel<T, SO, AUX, TR>>(kSmemBytes); if (rc_ != QLA_OK) return rc_; }  \
    QLA_CHECK_CUDA(launch_dependent(chunk_fwd_kernel<T, SO, AUX, TR>, dim3(grid), dim3(kThreads), kSmemBytes, stream, tm_q, tm_k, tm_v, tm_a, tm_w, tm_o, p)); \
  } while (0)
#define QLA_LAUNCH_FWD_NORM(T)                                                                                   \
  do {                                                                                                          \
    { const int rc_ = ensure_dynamic_smem<chunk_fwd_kernel<T, false, false, false, true>>(kSmemBytes); if (rc_ != QLA_OK) return rc_; }  \
    QLA_CHECK_CUDA(launch_dependent(chunk_fwd_kernel<T, false, false, false, true>, dim3(grid), dim3(kThreads), kSmemBytes, stream, tm_q, tm_k, tm_v, tm_a, tm_w, tm_o, p)); \
  } while (0)
#define QLA_LAUNCH_FWD_ST16(T)                                                                                   \
  do {                                                                                                          \
    { const int rc_ = ensure_dynamic_smem<chunk_fwd_kernel<T, false, false, false, false, true>>(kSmemBytes); if (rc_ != QLA_OK) return rc_; }  \
    QLA_CHECK_CUDA(launch_dependent(chunk_fwd_kernel<T, false, false, false, false, true>, dim3(grid), dim3(kThreads), kSmemBytes, stream, tm_q, tm_k, tm_v, tm_a, tm_w, tm_o, p)); \
  } while (0)
#define QLA_DISPATCH_FWD(T)                                                                  \
  do {                                                                                       \
    if (p.state_dtype == QLA_DT_BF16) QLA_LAUNCH_FWD_ST16(T);                                \
    else if (p.norm_gate != nullptr) QLA_LAUNCH_FWD_NORM(T);                                 \
    else if (traced) QLA_LAUNCH_FWD(T, false, false, true);                                  \
    else if (state_only && aux) QLA_LAUNCH_FWD(T, true, true, false);                        \
    else if (state_only) QLA_LAUNCH_FWD(T, true, false, false);                              \
    else if (aux) QLA_LAUNCH_FWD(T, false, true, false);                                     \
    else QLA_LAUNCH_FWD(T, false, false, false);                                             \
  } while (0)
  // the traced variant (plain full forward only) is a separate instantiation so that normal launches
  // carry no tracing code
  const bool aux = p.h != nullptr || p.v_new != nullptr;
  const bool traced = p.trace != nullptr && !state_only && !aux;
  if (is_bf16) QLA_DISPATCH_FWD(__nv_bfloat16);
  else QLA_DISPATCH_FWD(__half);
#undef QLA_DISPATCH_FWD
#undef QLA_LAUNCH_FWD_NORM
#undef QLA_LAUNCH_FWD_ST16
#undef QLA_LAUNCH_FWD
  QLA_CHECK_CUDA(cudaGetLastError());
  return QLA_OK;
}

void launch_info_chunk_fwd_kernel(int* block_threads, size_t* dynamic_smem_bytes) {
  *block_threads = kThreads;
  *dynamic_smem_bytes = kSmemBytes;
}

}  // namespace qla
