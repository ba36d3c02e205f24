// Chunked gated-delta-rule backward, part 1: the reverse scan over the chunks of one (sequence, v-head)
// with the gradient of the recurrent state resident in tensor memory.
// Reference: the reverse loop of fused_gdr_bwd (flash_qla/ops/gated_delta_rule/chunk/hopper/fused_bwd.py:287-361:
// dS update; :388-432: du and the product with A^T); math as in tests/ref_gdr.py:263-557.
//
// Per chunk, walking from the last chunk to the first (dS1 = gradient of the state leaving the chunk):
//   du  = Pg^T dO + rho .* (K dS1)                      Pg = s G .* (Q K^T), G[c,d] = exp(g_c - g_d), c >= d
//   dS0 = exp(gL) dS1 + (s gamma .* Q)^T dO + K^T X,    X = -(beta gamma) .* (A^T du)
//       = exp(gL) dS1 + (s gamma .* Q)^T dO + w^T du     -> dS1 of the chunk before; the last one is dh0
// with w = -(A diag(beta gamma) K), the operand the forward's preparation kernel produced for its own scan
// (K^T X = sum_i w_i^T du_i): one product on the serial chain instead of two with a conversion between them.
// du and the bf16 copy of every dS1 ("dh") go to the workspace the per-chunk kernel reads.
//
// The kernel mirrors the forward scan (chunk_fwd.cu): everything is computed TRANSPOSED so that each
// tcgen05.mma has M = 128 (the V dimension on the 128 TMEM lanes) and dependent operands stay in tensor memory:
//   MMA0  D0[128,64]  = [K;Q] K^T            (SS)  rows 64..127 are P = Q K^T; state independent
//   MMAu  Du0[128,64] = dO^T Pg              (SS)  A = dO tile read MN-major, B = Pg tile read MN-major
//   MMA2  D2[128,64]  = dS1^T_bf16 K^T       (TS)  chain
//   MMAq  dS^T[128,128] += dO^T (s gamma .* Q)              (SS, both operands MN-major)  off the chain
//   MMA3  dS^T[128,128] += du^T_bf16 w                     (TS, B = w tile read MN-major)  chain
// Thread v of a compute warpgroup owns TMEM lane v (column v of dS): it forms du = Du0 + rho .* D2, writes
// the 16-bit operand of the next product back with tcgen05.st and its 128 bytes of du^T to the workspace.
// Warp roles (416 threads): warps 0-7 compute (both warpgroups take half of the token columns of every
// chain phase and half of the state columns of the state conversion), warp 8 TMA producer + gate vectors,
// warp 9 MMA issuer, warps 10-11 operand tiles (Pg, s gamma .* Q in place), warp 12 sends du^T and dh^T of every
// chunk to the workspace with TMA stores from swizzled staging tiles (a thread owns a whole row of either: stored
// straight from registers, every 16-byte piece of a warp's store instruction would fall into a different
// 128-byte line).
// Every wait is a bounded mbarrier wait that raises the status word instead of hanging.
#include "chunk_params.cuh"

namespace qla {
namespace {

// ---- tensor-memory column map (512 columns)
constexpr uint32_t kColS = 0;       // fp32 dS^T, 128 columns
constexpr uint32_t kColSbf = 128;   // 16-bit copy of dS^T (A operand of MMA2), 64 columns
constexpr uint32_t kColD2 = 192;    // (K dS1)^T
constexpr uint32_t kColDu0 = 256;   // (Pg^T dO)^T
constexpr uint32_t kColDu16 = 320;  // 16-bit du^T (A operand of MMA3), 32 columns
constexpr uint32_t kColD0 = 384;    // [K;Q] K^T, two buffers of 64 columns (chunk parity)

// ---- shared-memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kStageKQ = 0;         // 32 KiB: half h (columns 64h..) = [K rows 8 KiB | Q rows 8 KiB]; SW128
constexpr uint32_t kStageDO = 32768;     // 16 KiB: dO tile as two [64][64] halves, SW128
constexpr uint32_t kStageW = 49152;      // 16 KiB: w tile as two [64][64] halves, SW128
constexpr uint32_t kStageBytes = 65536;  // 64 KiB
constexpr uint32_t kOffPg = 2 * kStageBytes;  // 2 x 8 KiB Pg tiles [c][d], SW128 (chunk parity)
constexpr uint32_t kOffDuT = kOffPg + 2 * 8192;   // 2 x 16 KiB du^T staging tiles [128 v][64 tokens], SW128 (chunk parity)
constexpr uint32_t kOffDhT = kOffDuT + 2 * 16384;  // 32 KiB dh^T staging tile [128 v][128 k] as two [128][64] halves, SW128
constexpr uint32_t kSmemBytes = kOffDhT + 32768 + 1024;

struct alignas(16) Gates {
  float g2[64];    // g log2(e)
  float rho[64];   // exp(gL - g), 0 on padded rows
  float sgam[64];  // scale * exp(g), 0 on padded rows
  float egl;
  int valid;
  int pad[2];
};
constexpr int kGateRing = 4;

enum Bar {
  kFull0 = 0, kFull1, kEmpty0, kEmpty1, kPDone0, kPDone1,
  kPgReady, kQsReady, kD2Done, kDu0Done, kDuReady, kSDone, kSbfReady, kSScaled,
  kTileReady,  // the compute warps have written this chunk's staging tiles (8 arrivals)
  kTileFree,   // the store warp's TMA stores of this chunk have read them (1 arrival)
  kNumBars
};
constexpr int kThreads = 416;

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

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
bwd_scan_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_do, const __grid_constant__ CUtensorMap tm_w,
                const __grid_constant__ CUtensorMap tm_dh, const __grid_constant__ CUtensorMap tm_du,
                const BwdParams p, const BwdScanMode mode) {
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? ptx::kFmtBF16 : ptx::kFmtF16;
  grid_dep_wait();    // earlier kernels of the stream have completed (see launch_dependent)
  grid_dep_launch();  // the next one may be scheduled; it waits the same way
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // context-parallel passes: the second half of a "dual" grid computes the K x K transition matrix of the reverse
  // recurrence over an interval's first chunks (identity start, dO treated as zero)
  const bool pass_b = mode.dual && blockIdx.x >= static_cast<unsigned>(p.num_seqs) * p.num_v_heads;
  const unsigned cta = pass_b ? blockIdx.x - static_cast<unsigned>(p.num_seqs) * p.num_v_heads : blockIdx.x;
  const bool zero_do = pass_b, init_identity = pass_b, state_only = mode.state_only || pass_b;
  const int32_t* chunk_limit = pass_b ? mode.chunk_limit_b : mode.chunk_limit;
  const int32_t* out_map = pass_b ? mode.out_map_b : mode.out_map;
  float* out_states = pass_b ? mode.out_b : p.dh0;
  const int hv = cta % p.num_v_heads;
  const int seq = cta / p.num_v_heads;
  const int hk = hv / (p.num_v_heads / p.num_k_heads);
  int seq_start, seq_end;
  if (p.cu_seqlens != nullptr) {
    seq_start = p.cu_seqlens[seq];
    seq_end = p.cu_seqlens[seq + 1];
  } else {
    seq_start = seq * p.seq_len;
    seq_end = seq_start + p.seq_len;
  }
  int nproc = (seq_end - seq_start + kChunk - 1) / kChunk;  // iteration i handles chunk nproc - 1 - i
  if (chunk_limit != nullptr) {
    const int lim = chunk_limit[seq * p.num_v_heads + hv];
    if (lim <= 0) return;  // nothing asked of this (interval, head); uniform for the whole CTA
    nproc = min(nproc, lim);
  }
  // warm-up inside the scan: `lead` chunks of the interval behind this one (same sequence: its end is the next
  // boundary) are scanned first from a zero gradient; nothing of them is stored
  const int lead = (mode.lead != nullptr && !state_only) ? mode.lead[seq * p.num_v_heads + hv] : 0;
  const int own_chunks = nproc;
  nproc += lead;
  const int tok_end = lead > 0 ? p.cu_seqlens[seq + 2] : seq_end;  // where the tokens of the scanned chunks end
  const int64_t chunk_base =
      p.chunk_offsets ? p.chunk_offsets[seq] : static_cast<int64_t>(seq) * ((p.seq_len + kChunk - 1) / kChunk);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint64_t bars[kNumBars];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(16) float aux_g[2 * 2 * 64];  // [aux warp][chunk parity][64] cumulative gates (log2 domain)
  __shared__ Gates gate_ring[kGateRing];

  if (tid == 0) {
#pragma unroll 1
    for (int b = 0; b < kNumBars; ++b) {
      int count = 1;  // commits: kPDone*, kD2Done, kDu0Done, kSDone
      if (b == kFull0 || b == kFull1) count = 33;
      else if (b == kEmpty0 || b == kEmpty1) count = 3;
      else if (b == kPgReady || b == kQsReady) count = 2;
      else if (b == kDuReady || b == kSbfReady || b == kSScaled || b == kTileReady) count = 8;
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
  auto wait = [&](int b, uint32_t parity) {
    return ptx::mbar_wait_warp_call(&bars[b], parity, status, kStatusBarrierTimeout | ((b + 64) << 8));  // + 64: the backward scan
  };
  auto stage_ptr = [&](int s) { return smem + s * kStageBytes; };
  auto gates_of = [&](int i) { return &gate_ring[i & (kGateRing - 1)]; };
  auto chunk_of = [&](int i) { return nproc - 1 - i; };

  if (warp == 8) {
    // =========================================================== producer: TMA + gate vectors
    constexpr int kPrefetchAhead = 4;
    for (int i = 2 - kPrefetchAhead; i < nproc; ++i) {
      if (lane == 0 && i + kPrefetchAhead < nproc) {
        const int pt0 = seq_start + chunk_of(i + kPrefetchAhead) * kChunk;
#pragma unroll 1
        for (int x = 0; x < 128; x += 64) {
          ptx::tma_prefetch_l2_3d(&tm_k, x, hk, pt0);
          ptx::tma_prefetch_l2_3d(&tm_q, x, hk, pt0);
          ptx::tma_prefetch_l2_3d(&tm_do, x, hv, pt0);
          ptx::tma_prefetch_l2_3d(&tm_w, x, hv, pt0);
        }
      }
      if (i < 0) continue;
      const int s = i & 1, use = i >> 1;
      const int t0 = seq_start + chunk_of(i) * kChunk;
      const int valid = min(kChunk, (chunk_of(i) >= own_chunks ? tok_end : seq_end) - t0);
      const int64_t last_tok = static_cast<int64_t>(t0) + valid - 1;
      const float gl = p.g_cumsum[last_tok * p.num_v_heads + hv];
      float gcv[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int c = lane + 32 * r;
        const int64_t tok = static_cast<int64_t>(t0) + c;
        gcv[r] = c < valid ? p.g_cumsum[tok * p.num_v_heads + hv] : gl;
      }
      if (use > 0 && !wait(kEmpty0 + s, (use - 1) & 1)) break;
      uint8_t* st = stage_ptr(s);
      if (lane == 0) {
        uint64_t* full = &bars[kFull0 + s];
        ptx::mbar_expect_tx(full, kStageBytes);
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          ptx::tma_load_3d(st + kStageKQ + h * 16384, &tm_k, full, h * 64, hk, t0);
          ptx::tma_load_3d(st + kStageKQ + h * 16384 + 8192, &tm_q, full, h * 64, hk, t0);
          ptx::tma_load_3d(st + kStageDO + h * 8192, &tm_do, full, h * 64, hv, t0);
          ptx::tma_load_3d(st + kStageW + h * 8192, &tm_w, full, h * 64, hv, t0);
        }
      }
      Gates* gs = gates_of(i);
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int c = lane + 32 * r;
        const bool ok = c < valid;
        const float gc = gcv[r];
        const float eg = __expf(gc);
        gs->g2[c] = gc * 1.4426950408889634f;
        gs->rho[c] = ok ? __expf(gl - gc) : 0.f;
        gs->sgam[c] = ok ? p.scale * eg : 0.f;
      }
      if (lane == 0) {
        gs->egl = __expf(gl);
        gs->valid = valid;
      }
      ptx::mbar_arrive(&bars[kFull0 + s]);
    }
  } else if (warp == 9) {
    // =========================================================== MMA issuer (whole warp, converged)
    const uint32_t id_n64 = ptx::mma_idesc(128, 64, fmt, ptx::kMajorK, ptx::kMajorK);        // MMA0, MMA2
    const uint32_t id_u = ptx::mma_idesc(128, 64, fmt, ptx::kMajorMN, ptx::kMajorMN);       // MMAu
    const uint32_t id_s = ptx::mma_idesc(128, 128, fmt, ptx::kMajorK, ptx::kMajorMN);       // MMA3
    const uint32_t id_q = ptx::mma_idesc(128, 128, fmt, ptx::kMajorMN, ptx::kMajorMN);      // MMAq
    // descriptors of stage 0; stage 1 is kStageBytes further
    const uint64_t d_kq = ptx::smem_desc_sw128(ptx::smem_u32(smem + kStageKQ), 16, 1024);           // [K;Q] 128 rows, K-major
    const uint64_t d_kmn = ptx::smem_desc_sw128(ptx::smem_u32(smem + kStageKQ), 16384, 1024);       // K rows, MN-major
    const uint64_t d_qmn = ptx::smem_desc_sw128(ptx::smem_u32(smem + kStageKQ + 8192), 16384, 1024);  // Q rows, MN-major
    const uint64_t d_do = ptx::smem_desc_sw128(ptx::smem_u32(smem + kStageDO), 8192, 1024);         // dO, MN-major
    const uint64_t d_wmn = ptx::smem_desc_sw128(ptx::smem_u32(smem + kStageW), 8192, 1024);         // w tile, MN-major
    const uint64_t d_pg = ptx::smem_desc_sw128(ptx::smem_u32(smem + kOffPg), 8192, 1024);           // Pg, MN-major
    constexpr int kHalf = (16384 >> 4) - 3 * 2;  // from k-step 3 to k-step 4: the second 64-column half
    constexpr uint32_t tmem0 = 0;
    const uint32_t bar0 = ptx::smem_u32(&bars[0]);
    auto bar_addr = [&](int b) { return bar0 + 8u * static_cast<uint32_t>(b); };
    bool ok = tmem == tmem0;
    if (!ok) ptx::record_wait_failure(status, kStatusBadTmemBase, 0);
    auto issue_mma0 = [&](int j) {  // D0[j & 1] = [K;Q] K^T of chunk j
      const uint64_t sn = static_cast<uint64_t>((j & 1) * (kStageBytes >> 4));
      ptx::tc_fence_after_sync();
      ptx::umma_ss_k128<2, kHalf, 2, kHalf>(tmem0 + kColD0 + (j & 1) * 64, d_kq + sn, d_kq + sn, id_n64, false,
                                            bar_addr(kPDone0 + (j & 1)));
    };
    bool p0_issued = false;  // MMA0 of the next chunk already issued in gap 1
#pragma unroll 1
    for (int i = -1; ok && i < nproc; ++i) {
      const int ph = i & 1;
      const uint64_t so = static_cast<uint64_t>((i & 1) * (kStageBytes >> 4));
      if (i >= 0) {
        // MMA2: D2 = dS1^T_bf16 K^T
        if (!(ok = wait(kSbfReady, ph))) break;
        ptx::tc_fence_after_sync();
        ptx::umma_ts_k128<2, kHalf>(tmem0 + kColD2, tmem0 + kColSbf, d_kq + so, id_n64, false, bar_addr(kD2Done));
        // gap 1 (the compute warps form du): MMAq, off the chain, and - when its tiles have landed - MMA0 of
        // the next chunk, so that Pg of that chunk is ready long before its MMAu
        if (!(ok = wait(kQsReady, ph))) break;
        if (!(ok = wait(kSScaled, ph))) break;
        ptx::tc_fence_after_sync();
        if (!zero_do) ptx::umma_ss_k64<128, 128>(tmem0 + kColS, d_do + so, d_qmn + so, id_q, true);
        p0_issued = false;
        if (i + 1 < nproc) {
          const int j = i + 1;
          const bool landed =
              __all_sync(0xffffffffu, ptx::mbar_test_wait(&bars[kFull0 + (j & 1)], (j >> 1) & 1)) != 0;
          if (landed) {
            issue_mma0(j);
            p0_issued = true;
          }
        }
        // MMA3: dS^T += du^T_bf16 w; its completion also releases the stage
        if (!(ok = wait(kDuReady, ph))) break;
        ptx::tc_fence_after_sync();
        ptx::umma_ts_k64<128>(tmem0 + kColS, tmem0 + kColDu16, d_wmn + so, id_s, true, bar_addr(kSDone),
                              bar_addr(kEmpty0 + ph));
      }
      // gap 2 (the compute warps convert the state): the state-independent products of the next chunk
      if (i + 1 < nproc) {
        const int j = i + 1;
        const uint64_t sn = static_cast<uint64_t>((j & 1) * (kStageBytes >> 4));
        if (!p0_issued) {
          if (!(ok = wait(kFull0 + (j & 1), (j >> 1) & 1))) break;
          issue_mma0(j);
        }
        // MMAu: Du0 = dO^T Pg (the compute warps read Du0 of this chunk before DuReady, MMA3 precedes in the pipe)
        if (!(ok = wait(kPgReady, j & 1))) break;
        ptx::tc_fence_after_sync();
        if (!zero_do)
          ptx::umma_ss_k64<128, 128>(tmem0 + kColDu0, d_do + sn, d_pg + static_cast<uint64_t>((j & 1) * (8192 >> 4)),
                                     id_u, false, bar_addr(kDu0Done));
      }
    }
  } else if (warp == 12) {
    // =========================================================== store warp: du^T and dh^T tiles -> workspace
    if (!state_only) {
      bool ok = true;
#pragma unroll 1
      for (int i = 0; ok && i < nproc; ++i) {
        if (!(ok = wait(kTileReady, i & 1))) break;
        if (lane == 0) {
          const int chunk = chunk_of(i);
          const int row = static_cast<int>(((chunk_base + chunk) * p.num_v_heads + hv) * kHeadDim);
          // (chunks of the warm-up belong to the interval behind: nothing of theirs is stored, except that the
          // last of them produces dh of this interval's last chunk)
          if (chunk < own_chunks) ptx::tma_store_3d(&tm_du, smem + kOffDuT + (i & 1) * 16384, 0, 0, row);
          if (i + 1 < nproc && chunk - 1 < own_chunks) {  // dh of the chunk before: the state this chunk's update produced
            const int row2 = row - p.num_v_heads * kHeadDim;
            ptx::tma_store_3d(&tm_dh, smem + kOffDhT, 0, 0, row2);
            ptx::tma_store_3d(&tm_dh, smem + kOffDhT + 16384, 64, 0, row2);
          }
          ptx::tma_store_commit();
          ptx::tma_store_wait_read();
          ptx::mbar_arrive(&bars[kTileFree]);
        }
        __syncwarp();
      }
      if (lane == 0) ptx::tma_store_wait_all();
    }
  } else if (warp >= 10) {
    // =========================================================== aux warps 10, 11: operand tiles
    const int r = tid - 320;  // 0..63: row of the A / Pg / Q tiles
    const uint32_t tm = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    float* my_g = aux_g + (warp - 10) * 128;
    const float log2_scale = __log2f(p.scale);
    bool ok = true;
#pragma unroll 1
    for (int j = 0; ok && j < nproc; ++j) {
      const int sj = j & 1;
      if (!(ok = wait(kFull0 + sj, (j >> 1) & 1))) break;
      const Gates* gs = gates_of(j);
      my_g[sj * 64 + lane] = gs->g2[lane];
      my_g[sj * 64 + 32 + lane] = gs->g2[32 + lane];
      const int valid = gs->valid;
      // (a) Pg = s G .* P from D0 rows 64..127 (TMEM quadrants 2, 3), rows beyond the sequence end zeroed.
      // The Pg tile of this parity was last read by MMAu two chunks ago, which precedes this chunk's MMA0 in
      // the tensor pipe and therefore has completed when PDone fires.
      if (!(ok = wait(kPDone0 + sj, (j >> 1) & 1))) break;
      ptx::tc_fence_after_sync();
      const float* gsg = my_g + sj * 64;
      const int c = r;
      const float gc = gsg[c] + log2_scale;
      uint8_t* pg = smem + kOffPg + sj * 8192;
#pragma unroll 1
      for (int db = 0; db < 64; db += 16) {
        uint32_t pr[16];
        ptx::tmem_ld16(tm + kColD0 + sj * 64 + db, pr);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int j8 = 0; j8 < 16; j8 += 8) {
          const float4 ga = *reinterpret_cast<const float4*>(&gsg[db + j8]);
          const float4 gb = *reinterpret_cast<const float4*>(&gsg[db + j8 + 4]);
          const float gd[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
          float x[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float val = ptx::ex2(gc - gd[e]) * __uint_as_float(pr[j8 + e]);
            x[e] = (db + j8 + e <= c && c < valid) ? val : 0.f;
          }
          *reinterpret_cast<uint4*>(pg + ptx::sw128_offset(c, (db + j8) >> 3)) =
              make_uint4(pack2<T>(x[0], x[1]), pack2<T>(x[2], x[3]), pack2<T>(x[4], x[5]), pack2<T>(x[6], x[7]));
        }
      }
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before_sync();
      warp_arrive(&bars[kPgReady], lane);
      // (b) Q rows times s gamma (0 beyond the sequence end), in place: MMA0 has read the raw tile
      const float f = gs->sgam[r];
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        uint8_t* qt = stage_ptr(sj) + kStageKQ + h * 16384 + 8192;
#pragma unroll 2
        for (int c16 = 0; c16 < 8; ++c16) {
          uint4* ptr = reinterpret_cast<uint4*>(qt + ptx::sw128_offset(r, c16));
          uint4 raw = *ptr;
          const T* e = reinterpret_cast<const T*>(&raw);
          raw = make_uint4(pack2<T>(Cvt<T>::to_f32(e[0]) * f, Cvt<T>::to_f32(e[1]) * f),
                           pack2<T>(Cvt<T>::to_f32(e[2]) * f, Cvt<T>::to_f32(e[3]) * f),
                           pack2<T>(Cvt<T>::to_f32(e[4]) * f, Cvt<T>::to_f32(e[5]) * f),
                           pack2<T>(Cvt<T>::to_f32(e[6]) * f, Cvt<T>::to_f32(e[7]) * f));
          *ptr = raw;
        }
      }
      ptx::fence_proxy_async_smem();
      warp_arrive(&bars[kQsReady], lane);
      warp_arrive(&bars[kEmpty0 + sj], lane);  // aux no longer touches stage sj
    }
  } else {
    // =========================================================== compute warpgroups
    const int wg = warp >> 2;   // token columns [32 wg, 32 wg + 32) of the chain phases, state columns [64 wg, ..)
    const int v = tid & 127;    // TMEM lane = column v of dS
    const uint32_t tm = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const int col_half = wg * 64;
    bool alive = true;
    const int st_k = p.transpose_state ? 1 : kHeadDim, st_v = p.transpose_state ? kHeadDim : 1;
    const int ht_k = (p.transpose_state && !p.dht_kv) ? 1 : kHeadDim, ht_v = (p.transpose_state && !p.dht_kv) ? kHeadDim : 1;
    const float* dhtp = (p.dht != nullptr && !init_identity && lead == 0)
                            ? p.dht + (static_cast<int64_t>(seq) * p.num_v_heads + hv) * kHeadDim * kHeadDim
                            : nullptr;
    const int out_row = out_map != nullptr ? out_map[seq] : seq;
    float* dh0p = (out_states != nullptr && out_row >= 0)
                      ? out_states + (static_cast<int64_t>(out_row) * p.num_v_heads + hv) * kHeadDim * kHeadDim
                      : nullptr;
    T* dh_ws = static_cast<T*>(p.dh);  // [chunk][Hv][128 v][128 k]
    auto dh_row = [&](int chunk) {
      return dh_ws + (((chunk_base + chunk) * p.num_v_heads + hv) * kHeadDim + v) * kHeadDim;
    };

    // ---- initial state: dS = exp(gL) * dht (fp32), its 16-bit copy, and dh of the last chunk
    // (this thread's 64 values are requested before the first stage is waited for: the two latencies overlap)
    {
      float xs[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        const int k = col_half + j;
        xs[j] = dhtp != nullptr ? dhtp[k * ht_k + v * ht_v] : ((init_identity && k == v) ? 1.f : 0.f);
      }
      float egl0 = 1.f;
      if (nproc > 0) {
        alive = wait(kFull0, 0);
        egl0 = gates_of(0)->egl;
      }
      T* hp = (nproc > 0 && !state_only && lead == 0) ? dh_row(nproc - 1) : nullptr;
#pragma unroll
      for (int kb = 0; kb < 64; kb += 16) {
        const float* x = xs + kb;
        uint32_t sf[16], sb[8];
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          sf[j] = __float_as_uint(x[j] * egl0);
          sf[j + 1] = __float_as_uint(x[j + 1] * egl0);
          sb[j >> 1] = pack2<T>(x[j], x[j + 1]);
        }
        ptx::tmem_st16(tm + kColS + col_half + kb, sf);
        ptx::tmem_st8(tm + kColSbf + (col_half + kb) / 2, sb);
        if (hp != nullptr) {
          *reinterpret_cast<uint4*>(hp + col_half + kb) = make_uint4(sb[0], sb[1], sb[2], sb[3]);
          *reinterpret_cast<uint4*>(hp + col_half + kb + 8) = make_uint4(sb[4], sb[5], sb[6], sb[7]);
        }
        if (nproc == 0 && dh0p != nullptr) {
#pragma unroll
          for (int j = 0; j < 16; ++j) dh0p[(col_half + kb + j) * st_k + v * st_v] = x[j];
        }
      }
      ptx::tmem_wait_st();
      ptx::tc_fence_before_sync();
      warp_arrive(&bars[kSbfReady], lane);
      warp_arrive(&bars[kSScaled], lane);
    }

#pragma unroll 1
    for (int i = 0; alive && i < nproc; ++i) {
      const int ph = i & 1;
      const int chunk = chunk_of(i);
      const Gates* gs = gates_of(i);
      // ---------------- du^T = Du0 + rho .* D2 for this warpgroup's 32 tokens: 16-bit copy into tensor memory
      // (A operand of MMA3) and to the workspace
      if (!(alive = wait(kD2Done, ph))) break;
      if (!zero_do && !(alive = wait(kDu0Done, ph))) break;
      ptx::tc_fence_after_sync();
      {
        uint32_t d2[32], u0[32], pk[16];
        ptx::tmem_ld32(tm + kColD2 + 32 * wg, d2);
        if (!zero_do) {
          ptx::tmem_ld32(tm + kColDu0 + 32 * wg, u0);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) u0[j] = 0u;
        }
        ptx::tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 r4 = *reinterpret_cast<const float4*>(&gs->rho[32 * wg + j]);
          pk[j >> 1] = pack2<T>(fmaf(__uint_as_float(d2[j]), r4.x, __uint_as_float(u0[j])),
                                fmaf(__uint_as_float(d2[j + 1]), r4.y, __uint_as_float(u0[j + 1])));
          pk[(j >> 1) + 1] = pack2<T>(fmaf(__uint_as_float(d2[j + 2]), r4.z, __uint_as_float(u0[j + 2])),
                                      fmaf(__uint_as_float(d2[j + 3]), r4.w, __uint_as_float(u0[j + 3])));
        }
        ptx::tmem_st16(tm + kColDu16 + 16 * wg, pk);
        ptx::tmem_wait_st();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kDuReady], lane);
        if (!state_only) {
          // this thread's 32 tokens of du^T (64 bytes of row v) into the staging tile of this chunk's parity;
          // its last tenant (chunk i - 2) was stored before the compute warps passed TileFree of chunk i - 2
          uint8_t* dt = smem + kOffDuT + (i & 1) * 16384 + v * 128;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(dt + (((4 * wg + j) ^ (v & 7)) << 4)) =
                make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
        }
      }
      // ---------------- state conversion after MMA3 (this warpgroup's 64 columns)
      if (!(alive = wait(kSDone, ph))) break;
      ptx::tc_fence_after_sync();
      if (i + 1 == nproc) {
        if (dh0p != nullptr) {
#pragma unroll 1
          for (int kb = 0; kb < 64; kb += 16) {
            uint32_t sf[16];
            ptx::tmem_ld16(tm + kColS + col_half + kb, sf);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) dh0p[(col_half + kb + j) * st_k + v * st_v] = __uint_as_float(sf[j]);
          }
        }
        if (!state_only) {
          ptx::fence_proxy_async_smem();
          warp_arrive(&bars[kTileReady], lane);  // only du^T this time
        }
      } else {
        // the dh^T staging tile is single: the stores of the previous chunk (issued a chunk period ago) must
        // have read it
        if (!state_only && i > 0 && !(alive = wait(kTileFree, (i - 1) & 1))) break;
        // (a) critical: 16-bit copy of the new state -> MMA2 of the next chunk may start; the same values are dh
        uint8_t* ht = smem + kOffDhT + wg * 16384 + v * 128;  // this warpgroup's 64 columns = half wg of the tile
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          uint32_t sf[32], sb[16];
          ptx::tmem_ld32(tm + kColS + col_half + 32 * h, sf);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j += 2) sb[j >> 1] = pack2<T>(__uint_as_float(sf[j]), __uint_as_float(sf[j + 1]));
          ptx::tmem_st16(tm + kColSbf + col_half / 2 + 16 * h, sb);
          if (!state_only) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint4*>(ht + (((4 * h + j) ^ (v & 7)) << 4)) =
                  make_uint4(sb[4 * j], sb[4 * j + 1], sb[4 * j + 2], sb[4 * j + 3]);
          }
        }
        ptx::tmem_wait_st();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kSbfReady], lane);
        if (!state_only) {
          ptx::fence_proxy_async_smem();
          warp_arrive(&bars[kTileReady], lane);
        }
        // (b) off the critical path: decay of the fp32 state for the next chunk (needed by MMAq / MMA3 only)
        if (!(alive = wait(kFull0 + ((i + 1) & 1), ((i + 1) >> 1) & 1))) break;
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
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) ptx::tmem_dealloc(tmem, 512);
}

}  // namespace

int launch_bwd_scan(const BwdParams& p, const BwdScanMode& mode, int64_t total_tokens, bool is_bf16,
                    cudaStream_t stream) {
  CUtensorMap tm_q, tm_k, tm_do, tm_w;
  int rc;
  if ((rc = make_tmap_3d(&tm_k, p.k, total_tokens, p.num_k_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_q, p.q, total_tokens, p.num_k_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_do, p.d_o, total_tokens, p.num_v_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_w, p.w, total_tokens, p.num_v_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  // store maps of the workspace tensors dh^T [chunks * Hv * 128 rows][128] and du^T [... rows][64] (boxes of 128 rows
  // x 64 columns, 128B swizzle: the form bwd_chunk_kernel loads them in); a state-only pass stores nothing and
  // gets placeholder maps
  CUtensorMap tm_dh = tm_k, tm_du = tm_k;
  if (!mode.state_only) {
    const uint64_t rows = static_cast<uint64_t>(mode.chunks_upper) * p.num_v_heads * kHeadDim;
    if ((rc = make_tmap_3d(&tm_dh, p.dh, rows, 1, kHeadDim, 128, 64, true, is_bf16)) != QLA_OK) return rc;
    if ((rc = make_tmap_3d(&tm_du, p.du, rows, 1, kChunk, 128, 64, true, is_bf16)) != QLA_OK) return rc;
  }
  const unsigned grid = static_cast<unsigned>(p.num_seqs) * p.num_v_heads * (mode.dual ? 2 : 1);
  if (is_bf16) {
    if ((rc = ensure_dynamic_smem<bwd_scan_kernel<__nv_bfloat16>>(kSmemBytes)) != QLA_OK) return rc;
    QLA_CHECK_CUDA(launch_dependent(bwd_scan_kernel<__nv_bfloat16>, dim3(grid), dim3(kThreads), kSmemBytes, stream, tm_q, tm_k,
                                    tm_do, tm_w, tm_dh, tm_du, p, mode));
  } else {
    if ((rc = ensure_dynamic_smem<bwd_scan_kernel<__half>>(kSmemBytes)) != QLA_OK) return rc;
    QLA_CHECK_CUDA(launch_dependent(bwd_scan_kernel<__half>, dim3(grid), dim3(kThreads), kSmemBytes, stream, tm_q, tm_k, tm_do,
                                    tm_w, tm_dh, tm_du, p, mode));
  }
  QLA_CHECK_CUDA(cudaGetLastError());
  return QLA_OK;
}

void launch_info_bwd_scan_kernel(int* block_threads, size_t* dynamic_smem_bytes) {
  *block_threads = kThreads;
  *dynamic_smem_bytes = kSmemBytes;
}

}  // namespace qla
