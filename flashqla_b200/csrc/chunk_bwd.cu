// Chunked gated-delta-rule backward for sm_100a, part 2: everything that is local to one chunk.
// Reference: chunk_gated_delta_rule_bwd (flash_qla/ops/gated_delta_rule/chunk/__init__.py:89-182); the
// math is the decomposed form of tests/ref_gdr.py:263-557 / chunk/blackwell/bwd_sm12x.py (dv_local,
// dq/dk/dw/dg, WY backward), the fused original is chunk/hopper/fused_bwd.py:388-882.
//
// The backward is two kernels:
//  bwd_scan_kernel   (chunk_bwd_scan.cu) one CTA per (sequence, v-head), chunks in reverse order, dS resident
//                    in tensor memory; writes du^T [chunk][Hv][128 v][64 tokens], the state gradient
//                    leaving every chunk dh^T [chunk][Hv][128 v][128 k] and dh0.
//  bwd_chunk_kernel  (this file) persistent CTAs walk the (chunk, k-head) items and loop over the v-heads of the
//                    GQA group, so that dq and dk leave already reduced over the group: the sixteen remaining
//                    products of a chunk, the triangular-inverse backward, dbeta, and dg with its chunk-local
//                    reverse cumulative sum.
//
// Every product is a tcgen05.mma with M = 64 (the 64 tokens of the chunk; such an accumulator occupies 16
// lanes of each 32-lane partition of tensor memory, so two accumulators share a column range: "bank" 0 at
// lane offset 0, bank 1 at lane offset 16), operands are TMA-written or thread-written 128B-swizzled
// shared-memory tiles read K-major or MN-major as the product needs, so no tile is ever transposed.
// Accumulators are read back as 16 x 256 bit fragments, which hand warp w = (mt, nh) rows 16 mt .. 16 mt + 15
// and one quarter of the columns in the mma.sync accumulator layout: thread 4 g + c holds rows g, g + 8 and
// column pairs 8 nt + 2 c.  dq / dk accumulate in registers over the heads of the group.
//
//   level 0 (inputs only)   T1 = dO h^T   T2 = v_new dh^T   dw- = du h^T   x = A^T du   dO v_new^T   Q K^T
//                           du V^T   K K^T
//   level 1 (ds, dw)        ds K    ds^T Q    A^T dw    dw K^T
//   level 2 (dA)            M1 = A^T dA
//   level 3 (M1)            M1 A^T
//   level 4 (dL)            dL K    (beta dL)^T K
// Warp roles (576 threads): warps 0-15 epilogues (warp = row tile mt x column quarter nh), warp 16 TMA producer +
// gate vectors, warp 17 MMA issuer.  dv, dq and dk leave through shared-memory tiles and TMA stores.  The
// tiles only level 0 reads (dO, v_new, V, du, h, dh: 128 KiB) are refilled for the next head while levels 1-4
// run.  Rows beyond the end of a sequence hold the next sequence's tokens (TMA does not know about sequences);
// they never contribute because du, beta, rho and the ds rows of such tokens are exactly zero.
#include "chunk_params.cuh"

namespace qla {
namespace {

constexpr int kComputeWarps = 16;
constexpr int kThreads = 32 * (kComputeWarps + 2);
constexpr int kRedFloats = 800;  // per parity: dg rows [4][64], dbeta rows [4][64], dg columns [4][64], last [16], carry

// ---- shared-memory map (offsets from a 1024-byte aligned base; every tile 128B-swizzled)
constexpr uint32_t kOffQ = 0;        // [64][128] as two [64][64] halves
constexpr uint32_t kOffK = 16384;
constexpr uint32_t kOffA = 32768;    // [64][64]
constexpr uint32_t kOffDO = 40960;
constexpr uint32_t kOffVn = 57344;
constexpr uint32_t kOffV = 73728;
constexpr uint32_t kOffDu = 90112;   // du^T [128 v][64 tokens]
constexpr uint32_t kOffH = 106496;   // h [128 k][128 v] as two [128][64] halves
constexpr uint32_t kOffDh = 139264;  // dh^T [128 v][128 k] as two [128][64] halves
constexpr uint32_t kOffDw = 172032;  // dw [64][128], written by the epilogue
constexpr uint32_t kOffX = 188416;   // [64][64]: ds, then M1, then beta .* dL
constexpr uint32_t kOffY = 196608;   // [64][64]: dA, then dL
constexpr uint32_t kSmemBytes = 204800 + 1024;
constexpr uint32_t kEarlyBytes = 3 * 16384 + 16384 + 2 * 32768;  // dO, v_new, V, du^T, h, dh^T

// ---- tensor-memory columns; bank 1 = the same columns at lane offset 16
constexpr uint32_t kBank1 = 16u << 16;
constexpr uint32_t kColT = 0;      // T1 | T2           later M1 (0..63), M1 A^T (64..127)
constexpr uint32_t kColW = 128;    // dw- | x           later A^T dw (bank 0); dL K | (beta dL)^T K
constexpr uint32_t kColP = 256;    // dO v_new^T | Q K^T    later dw K^T (bank 0)
constexpr uint32_t kColR = 320;    // du V^T | K K^T
constexpr uint32_t kColQ = 384;    // ds K | ds^T Q

enum Bar {
  kEarlyFull = 0, kLateFull, kEarlyFree, kLateFree, kC45, kC3, kCB, kCT, kL1Ready, kCL1, kDaReady, kC12, kM1Ready,
  kC13, kDlReady, kC4, kNumBars
};

struct ChunkCoord {
  int seq, seq_start, seq_end, local_chunk;
};

// chunk index -> sequence (binary search over the exclusive scan of chunks per sequence)
__device__ __forceinline__ ChunkCoord locate_chunk(int chunk, const int32_t* cu, const int32_t* chunk_offsets,
                                                   int num_seqs, int seq_len) {
  ChunkCoord c;
  if (cu != nullptr) {
    int lo = 0, hi = num_seqs - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (chunk_offsets[mid] <= chunk) lo = mid; else hi = mid - 1;
    }
    c.seq = lo;
    c.seq_start = cu[lo];
    c.seq_end = cu[lo + 1];
    c.local_chunk = chunk - chunk_offsets[lo];
  } else {
    const int per = (seq_len + kChunk - 1) / kChunk;
    c.seq = chunk / per;
    c.local_chunk = chunk % per;
    c.seq_start = c.seq * seq_len;
    c.seq_end = c.seq_start + seq_len;
  }
  return c;
}

__device__ __forceinline__ float quad_sum(float x) {  // over the four lanes that share a row
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  return x;
}
__device__ __forceinline__ float oct_sum(float x) {  // over the eight lanes that share a column pair
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  x += __shfl_xor_sync(0xffffffffu, x, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 16);
  return x;
}
__device__ __forceinline__ void compute_sync() {  // the epilogue warps
  asm volatile("bar.sync 1, %0;" ::"n"(32 * kComputeWarps) : "memory");
}
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
__device__ __forceinline__ float2 unpack2(uint32_t raw) {
  const T* e = reinterpret_cast<const T*>(&raw);
  return make_float2(Cvt<T>::to_f32(e[0]), Cvt<T>::to_f32(e[1]));
}

// Two 16-bit elements (row, col), (row, col + 1) of a [rows][128] tile stored as two 64-column halves
// `half_bytes` apart; col is even.
__device__ __forceinline__ uint32_t ld_pair(const uint8_t* tile, uint32_t half_bytes, int row, int col) {
  return *reinterpret_cast<const uint32_t*>(tile + (col >> 6) * half_bytes + ptx::sw128_offset(row, (col & 63) >> 3) +
                                            (col & 7) * 2);
}
__device__ __forceinline__ void st_pair(uint8_t* tile, uint32_t half_bytes, int row, int col, uint32_t v) {
  *reinterpret_cast<uint32_t*>(tile + (col >> 6) * half_bytes + ptx::sw128_offset(row, (col & 63) >> 3) + (col & 7) * 2) = v;
}

// kTrace: a separate instantiation whose CTA 0 stamps clock64() at the phase boundaries of its fourth step into
// the buffer registered with qla_set_trace_buffer (events 0..19 epilogue warp 0, 20..31 the MMA issuer).
template <typename T, bool kTrace>
__global__ void __launch_bounds__(kThreads, 1)
bwd_chunk_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_vn,
                 const __grid_constant__ CUtensorMap tm_do, const __grid_constant__ CUtensorMap tm_a,
                 const __grid_constant__ CUtensorMap tm_h, const __grid_constant__ CUtensorMap tm_dh,
                 const __grid_constant__ CUtensorMap tm_du, const __grid_constant__ CUtensorMap tm_dq,
                 const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv, const BwdParams p,
                 const int total_items) {
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? ptx::kFmtBF16 : ptx::kFmtF16;
  grid_dep_wait();    // earlier kernels of the stream have completed (see launch_dependent)
  grid_dep_launch();  // the next one may be scheduled; it waits the same way
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = p.num_v_heads / p.num_k_heads;
  const int real_chunks = p.cu_seqlens != nullptr ? p.chunk_offsets[p.num_seqs] : 0x7fffffff;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint64_t bars[kNumBars];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(16) float sG[2][64];  // cumulative gates of the step (parity), padded rows = last valid
  __shared__ __align__(16) float sB[2][64];  // beta, 0 on padded rows
  __shared__ float red[2 * kRedFloats];

  if (tid == 0) {
#pragma unroll 1
    for (int b = 0; b < kNumBars; ++b) {
      int count = 1;  // tcgen05.commit, or the producer's expect_tx arrival
      if (b == kEarlyFull) count = 33;
      else if (b == kEarlyFree || b == kLateFree) count = kComputeWarps + 1;
      else if (b == kL1Ready || b == kDaReady || b == kM1Ready || b == kDlReady) count = kComputeWarps;
      ptx::mbar_init(&bars[b], count);
    }
    ptx::fence_mbar_init();
  }
  if (warp == kComputeWarps) {
    ptx::tmem_alloc(&tmem_base_s, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  int* status = p.status;
  auto wait = [&](int b, uint32_t parity) {  // (+ 128 in the recorded barrier index: this kernel)
    return ptx::mbar_wait_warp_call(&bars[b], parity, status, kStatusBarrierTimeout | ((b + 128) << 8));
  };
  auto trace = [&](int step, int ev) {
    if (kTrace && p.trace != nullptr && blockIdx.x == 0 && step == 3 && lane == 0) p.trace[ev] = clock64();
  };

  if (warp == kComputeWarps) {
    // =========================================================== producer: TMA + gate vectors
    int step = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
      const int chunk = item / p.num_k_heads, hk = item % p.num_k_heads;
      if (chunk >= real_chunks) continue;
      const ChunkCoord cc = locate_chunk(chunk, p.cu_seqlens, p.chunk_offsets, p.num_seqs, p.seq_len);
      const int t0 = cc.seq_start + cc.local_chunk * kChunk;
      const int valid = min(kChunk, cc.seq_end - t0);
      for (int hv = hk * group; ok && hv < (hk + 1) * group; ++hv, ++step) {
        const int ph = step & 1;
        // gates of this head into the step's parity slot (its previous reader finished two steps ago)
        const int64_t last_tok = static_cast<int64_t>(t0) + valid - 1;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int c = lane + 32 * r;
          const bool okc = c < valid;
          const int64_t tok = okc ? static_cast<int64_t>(t0) + c : last_tok;
          sG[ph][c] = p.g_cumsum[tok * p.num_v_heads + hv];
          sB[ph][c] = okc ? load_scalar(p.beta, p.beta_dtype, tok * p.num_v_heads + hv) : 0.f;
        }
        if (step > 0 && !(ok = wait(kEarlyFree, (step - 1) & 1))) break;
        if (lane == 0) {
          uint64_t* full = &bars[kEarlyFull];
          ptx::mbar_expect_tx(full, kEarlyBytes);
          const int row = (chunk * p.num_v_heads + hv) * kHeadDim;  // row of the [chunks * Hv * 128, width] views
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
            ptx::tma_load_3d(smem + kOffDO + h * 8192, &tm_do, full, h * 64, hv, t0);
            ptx::tma_load_3d(smem + kOffVn + h * 8192, &tm_vn, full, h * 64, hv, t0);
            ptx::tma_load_3d(smem + kOffV + h * 8192, &tm_v, full, h * 64, hv, t0);
            ptx::tma_load_3d(smem + kOffH + h * 16384, &tm_h, full, h * 64, 0, row);
            ptx::tma_load_3d(smem + kOffDh + h * 16384, &tm_dh, full, h * 64, 0, row);
          }
          ptx::tma_load_3d(smem + kOffDu, &tm_du, full, 0, 0, row);
        }
        ptx::mbar_arrive(&bars[kEarlyFull]);  // 32 arrivals (gates written) + the expect_tx arrival
        // the tiles of the NEXT step into L2, so that its demand loads (issued when this step's buffers are
        // released) find them there
        if (lane == 0) {
          int hv2 = hv + 1, item2 = item;
          if (hv2 == (hk + 1) * group) {
            item2 = item + gridDim.x;
            hv2 = (item2 % p.num_k_heads) * group;
          }
          const int chunk2 = item2 / p.num_k_heads;
          if (item2 < total_items && chunk2 < real_chunks) {
            int t2 = t0;
            if (item2 != item) {
              const ChunkCoord c2 = locate_chunk(chunk2, p.cu_seqlens, p.chunk_offsets, p.num_seqs, p.seq_len);
              t2 = c2.seq_start + c2.local_chunk * kChunk;
            }
            const int hk2 = hv2 / group;
            const int row2 = (chunk2 * p.num_v_heads + hv2) * kHeadDim;
#pragma unroll 1
            for (int x = 0; x < 128; x += 64) {
              ptx::tma_prefetch_l2_3d(&tm_do, x, hv2, t2);
              ptx::tma_prefetch_l2_3d(&tm_vn, x, hv2, t2);
              ptx::tma_prefetch_l2_3d(&tm_v, x, hv2, t2);
              ptx::tma_prefetch_l2_3d(&tm_h, x, 0, row2);
              ptx::tma_prefetch_l2_3d(&tm_dh, x, 0, row2);
              if (item2 != item) {
                ptx::tma_prefetch_l2_3d(&tm_q, x, hk2, t2);
                ptx::tma_prefetch_l2_3d(&tm_k, x, hk2, t2);
              }
            }
            ptx::tma_prefetch_l2_3d(&tm_du, 0, 0, row2);
            ptx::tma_prefetch_l2_3d(&tm_a, 0, hv2, t2);
          }
        }
        if (step > 0 && !(ok = wait(kLateFree, (step - 1) & 1))) break;
        if (lane == 0) {
          uint64_t* full = &bars[kLateFull];
          const bool first_head = hv == hk * group;
          ptx::mbar_expect_tx(full, first_head ? 8192 + 32768 : 8192);
          ptx::tma_load_3d(smem + kOffA, &tm_a, full, 0, hv, t0);
          if (first_head) {
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
              ptx::tma_load_3d(smem + kOffQ + h * 8192, &tm_q, full, h * 64, hk, t0);
              ptx::tma_load_3d(smem + kOffK + h * 8192, &tm_k, full, h * 64, hk, t0);
            }
          }
        }
      }
    }
  } else if (warp == kComputeWarps + 1) {
    // =========================================================== MMA issuer (whole warp, converged)
    using ptx::kMajorK;
    using ptx::kMajorMN;
    auto desc = [&](uint32_t off, uint32_t lbo) { return ptx::smem_desc_sw128(ptx::smem_u32(smem + off), lbo, 1024); };
    const uint64_t d_q = desc(kOffQ, 16), d_k = desc(kOffK, 16), d_a = desc(kOffA, 16), d_do = desc(kOffDO, 16);
    const uint64_t d_vn = desc(kOffVn, 16), d_v = desc(kOffV, 16), d_du = desc(kOffDu, 16), d_h = desc(kOffH, 16);
    const uint64_t d_dw = desc(kOffDw, 16), d_x = desc(kOffX, 16), d_y = desc(kOffY, 16);
    // the same tiles read MN-major (leading-dimension offset = distance of the two 64-wide halves)
    const uint64_t m_q = desc(kOffQ, 8192), m_k = desc(kOffK, 8192), m_a = desc(kOffA, 8192), m_du = desc(kOffDu, 8192);
    const uint64_t m_dh = desc(kOffDh, 16384), m_dw = desc(kOffDw, 8192), m_x = desc(kOffX, 8192), m_y = desc(kOffY, 8192);
    constexpr int kJ8 = (8192 >> 4) - 6, kJ16 = (16384 >> 4) - 6;  // to the second 64-column half of a K-major tile
    const uint32_t i_kk64 = ptx::mma_idesc(64, 64, fmt, kMajorK, kMajorK), i_mk64 = ptx::mma_idesc(64, 64, fmt, kMajorMN, kMajorK);
    const uint32_t i_mm64 = ptx::mma_idesc(64, 64, fmt, kMajorMN, kMajorMN);
    const uint32_t i_kk = ptx::mma_idesc(64, 128, fmt, kMajorK, kMajorK), i_km = ptx::mma_idesc(64, 128, fmt, kMajorK, kMajorMN);
    const uint32_t i_mk = ptx::mma_idesc(64, 128, fmt, kMajorMN, kMajorK), i_mm = ptx::mma_idesc(64, 128, fmt, kMajorMN, kMajorMN);
    constexpr uint32_t t0c = 0;  // the CTA owns all 512 columns: the allocation starts at column 0
    const uint32_t bar0 = ptx::smem_u32(&bars[0]);
    auto ba = [&](int b) { return bar0 + 8u * static_cast<uint32_t>(b); };
    bool ok = tmem == t0c;
    if (!ok) ptx::record_wait_failure(status, kStatusBadTmemBase, 0);
    int step = 0;
    for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
      if (item / p.num_k_heads >= real_chunks) continue;
      for (int hh = 0; ok && hh < group; ++hh, ++step) {
        const uint32_t ph = step & 1;
        if (!(ok = wait(kEarlyFull, ph))) break;
        trace(step, 30);
        if (!(ok = wait(kLateFull, ph))) break;
        ptx::tc_fence_after_sync();
        trace(step, 20);
        // ---- level 0
        ptx::umma_ss_k128<2, kJ8, 2, kJ8>(t0c + kColP, d_do, d_vn, i_kk64, false);                      // dO v_new^T
        ptx::umma_ss_k128<2, kJ8, 2, kJ8>(t0c + kColP + kBank1, d_q, d_k, i_kk64, false, ba(kC45));     // Q K^T
        ptx::umma_ss_k128<128, 128, 2, kJ16>(t0c + kColW, m_du, d_h, i_mk, false, ba(kC3));             // du h^T
        ptx::umma_ss_k64<128, 2>(t0c + kColW + kBank1, m_a, d_du, i_mk, false);                         // x = A^T du
        ptx::umma_ss_k128<128, 128, 2, kJ8>(t0c + kColR, m_du, d_v, i_mk64, false);                     // du V^T
        ptx::umma_ss_k128<2, kJ8, 2, kJ8>(t0c + kColR + kBank1, d_k, d_k, i_kk64, false, ba(kCB));      // K K^T
        ptx::umma_ss_k128<2, kJ8, 2, kJ16>(t0c + kColT, d_do, d_h, i_kk, false);                        // T1 = dO h^T
        ptx::umma_ss_k128<2, kJ8, 128, 128>(t0c + kColT + kBank1, d_vn, m_dh, i_km, false, ba(kCT), ba(kEarlyFree));  // T2
        trace(step, 21);
        // ---- level 1
        if (!(ok = wait(kL1Ready, ph))) break;
        ptx::tc_fence_after_sync();
        trace(step, 22);
        ptx::umma_ss_k64<2, 128>(t0c + kColQ, d_x, m_k, i_km, false);                                   // ds K
        ptx::umma_ss_k64<128, 128>(t0c + kColQ + kBank1, m_x, m_q, i_mm, false);                        // ds^T Q
        ptx::umma_ss_k64<128, 128>(t0c + kColW, m_a, m_dw, i_mm, false);                                // y = A^T dw
        ptx::umma_ss_k128<2, kJ8, 2, kJ8>(t0c + kColP, d_dw, d_k, i_kk64, false, ba(kCL1));             // dw K^T
        trace(step, 23);
        // ---- level 2
        if (!(ok = wait(kDaReady, ph))) break;
        ptx::tc_fence_after_sync();
        trace(step, 24);
        ptx::umma_ss_k64<128, 128>(t0c + kColT, m_a, m_y, i_mm64, false, ba(kC12));                     // M1 = A^T dA
        trace(step, 25);
        // ---- level 3
        if (!(ok = wait(kM1Ready, ph))) break;
        ptx::tc_fence_after_sync();
        trace(step, 26);
        ptx::umma_ss_k64<2, 2>(t0c + kColT + 64, d_x, d_a, i_kk64, false, ba(kC13));                    // M1 A^T
        trace(step, 27);
        // ---- level 4
        if (!(ok = wait(kDlReady, ph))) break;
        ptx::tc_fence_after_sync();
        trace(step, 28);
        ptx::umma_ss_k64<2, 128>(t0c + kColW, d_y, m_k, i_km, false);                                   // z = dL K
        ptx::umma_ss_k64<128, 128>(t0c + kColW + kBank1, m_x, m_k, i_mm, false, ba(kC4), ba(kLateFree));  // (beta dL)^T K
        trace(step, 29);
      }
    }
  } else if (warp < kComputeWarps) {
    // =========================================================== epilogue warps
    const int g = lane >> 2, c4 = lane & 3;
    const int mt = warp & 3, nh = warp >> 2;  // rows 16 mt .., column quarter nh
    const int r0 = mt * 16 + g, r1 = r0 + 8;  // the two rows this thread owns in every fragment
    const uint32_t tq = tmem + (static_cast<uint32_t>(mt * 32) << 16);  // bank 0 of this warp's partition
    uint8_t* sQ = smem + kOffQ;
    uint8_t* sK = smem + kOffK;
    uint8_t* sV = smem + kOffV;
    // wide fragment: 16 rows x 32 columns (a quarter of a 128-column product); narrow: 16 rows x 16 columns
    auto wide = [&](uint32_t col, float (&acc)[4][4]) {
      uint32_t r[16];
      ptx::tmem_ld_frag4(tq + col + 32 * nh, r);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j >> 2][j & 3] = __uint_as_float(r[j]);
    };
    auto wide2 = [&](uint32_t col_a, float (&a)[4][4], uint32_t col_b, float (&b)[4][4]) {  // two loads in flight
      uint32_t ra[16], rb[16];
      ptx::tmem_ld_frag4(tq + col_a + 32 * nh, ra);
      ptx::tmem_ld_frag4(tq + col_b + 32 * nh, rb);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        a[j >> 2][j & 3] = __uint_as_float(ra[j]);
        b[j >> 2][j & 3] = __uint_as_float(rb[j]);
      }
    };
    auto narrow2 = [&](uint32_t col_a, float (&a)[2][4], uint32_t col_b, float (&b)[2][4]) {
      uint32_t ra[8], rb[8];
      ptx::tmem_ld_frag2(tq + col_a + 16 * nh, ra);
      ptx::tmem_ld_frag2(tq + col_b + 16 * nh, rb);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a[j >> 2][j & 3] = __uint_as_float(ra[j]);
        b[j >> 2][j & 3] = __uint_as_float(rb[j]);
      }
    };
    auto narrow = [&](uint32_t col, float (&a)[2][4]) {
      uint32_t ra[8];
      ptx::tmem_ld_frag2(tq + col + 16 * nh, ra);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j >> 2][j & 3] = __uint_as_float(ra[j]);
    };
    // byte offsets of this thread's elements inside 128B-swizzled tiles (r0 & 7 = r1 & 7 = g)
    const uint32_t row_off0 = r0 * 128 + 4 * c4, row_off1 = r1 * 128 + 4 * c4;
    auto wide_off = [&](int nt) {  // column 32 nh + 8 nt + 2 c4 of a [64][128] tile (two halves 8192 apart)
      return static_cast<uint32_t>((nh >> 1) * 8192 + (((((nh & 1) * 4 + nt) ^ g)) << 4));
    };
    auto narrow_off = [&](int nt) {  // column 16 nh + 8 nt + 2 c4 of a [64][64] tile
      return static_cast<uint32_t>(((nh * 2 + nt) ^ g) << 4);
    };
    // sum over this thread's columns of acc .* M[rows r0 / r1][32 nh + ...]   (M = a [64][128] tile)
    auto dot_rows = [&](const float (&acc)[4][4], const uint8_t* M, float& s0, float& s1) {
      s0 = 0.f; s1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const uint32_t o = wide_off(nt);
        const float2 a = unpack2<T>(*reinterpret_cast<const uint32_t*>(M + row_off0 + o));
        const float2 b = unpack2<T>(*reinterpret_cast<const uint32_t*>(M + row_off1 + o));
        s0 += acc[nt][0] * a.x + acc[nt][1] * a.y;
        s1 += acc[nt][2] * b.x + acc[nt][3] * b.y;
      }
    };
    auto st_wide = [&](uint8_t* tile, const float (&acc)[4][4], float f0, float f1) {  // [64][128] tile
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const uint32_t o = wide_off(nt);
        *reinterpret_cast<uint32_t*>(tile + row_off0 + o) = pack2<T>(f0 * acc[nt][0], f0 * acc[nt][1]);
        *reinterpret_cast<uint32_t*>(tile + row_off1 + o) = pack2<T>(f1 * acc[nt][2], f1 * acc[nt][3]);
      }
    };
    auto st_narrow = [&](uint8_t* tile, const float (&acc)[2][4]) {  // [64][64] tile
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const uint32_t o = narrow_off(nt);
        *reinterpret_cast<uint32_t*>(tile + row_off0 + o) = pack2<T>(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<uint32_t*>(tile + row_off1 + o) = pack2<T>(acc[nt][2], acc[nt][3]);
      }
    };
    // rows r0 / r1 of a [64][128] result straight to global memory (ragged tail chunks)
    auto st_global_rows = [&](T* base, int heads, int head, int t0, int valid, const float (&acc)[4][4], float f0, float f1) {
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int col = nh * 32 + nt * 8 + 2 * c4;
        if (r0 < valid)
          *reinterpret_cast<uint32_t*>(base + (static_cast<int64_t>(t0 + r0) * heads + head) * kHeadDim + col) =
              pack2<T>(f0 * acc[nt][0], f0 * acc[nt][1]);
        if (r1 < valid)
          *reinterpret_cast<uint32_t*>(base + (static_cast<int64_t>(t0 + r1) * heads + head) * kHeadDim + col) =
              pack2<T>(f1 * acc[nt][2], f1 * acc[nt][3]);
      }
    };

    int step = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
      const int chunk = item / p.num_k_heads, hk = item % p.num_k_heads;
      if (chunk >= real_chunks) continue;
      const ChunkCoord cc = locate_chunk(chunk, p.cu_seqlens, p.chunk_offsets, p.num_seqs, p.seq_len);
      const int t0 = cc.seq_start + cc.local_chunk * kChunk;
      const int valid = min(kChunk, cc.seq_end - t0);
      float dq_acc[4][4], dk_acc[4][4];  // rows r0 / r1, columns 32 nh ..; summed over the v-heads of the group
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) dq_acc[nt][e] = dk_acc[nt][e] = 0.f;

      for (int hv = hk * group; ok && hv < (hk + 1) * group; ++hv, ++step) {
        const uint32_t ph = step & 1;
        if (!(ok = wait(kEarlyFull, ph))) break;
        if (warp == 0) trace(step, 0);
        const float* gs = sG[ph];
        const float* bs = sB[ph];
        const float gl = gs[valid - 1];
        const float g0 = gs[r0], g1 = gs[r1];
        const float gam0 = __expf(g0), gam1 = __expf(g1);
        const float rho0 = (r0 < valid) ? __expf(gl - g0) : 0.f, rho1 = (r1 < valid) ? __expf(gl - g1) : 0.f;
        const float be0 = bs[r0], be1 = bs[r1];
        float dg_row[2] = {0.f, 0.f}, db_row[2] = {0.f, 0.f};
        float dg_col[2][2];  // columns 16 nh + 8 nt + 2 c4 + {0, 1} of the 64 x 64 products
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) dg_col[nt][0] = dg_col[nt][1] = 0.f;
        float dg_last = 0.f;

        // ---- sum(h .* dh) straight from the tiles while level 0 runs: thread = (k, quarter of v)
        {
          const int k = tid & 127, vq = tid >> 7;
          const uint8_t* hrow = smem + kOffH + (vq >> 1) * 16384 + k * 128;
          const uint8_t* dcol = smem + kOffDh + (k >> 6) * 16384 + (k & 7) * 2;
          const int kc = (k & 63) >> 3;
          float hd = 0.f;
#pragma unroll 2
          for (int j = (vq & 1) * 4; j < (vq & 1) * 4 + 4; ++j) {
            const uint4 raw = *reinterpret_cast<const uint4*>(hrow + ((j ^ (k & 7)) << 4));
            const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              const int v = (vq >> 1) * 64 + j * 8 + x;
              const T d = *reinterpret_cast<const T*>(dcol + v * 128 + ((kc ^ (v & 7)) << 4));
              hd += Cvt<T>::to_f32(e[x]) * Cvt<T>::to_f32(d);
            }
          }
          dg_last += __expf(gl) * hd;
        }
        if (warp == 0) trace(step, 1);
        // the tiles the previous item's dq / dk left through (dw, ds / dA areas) are rewritten from here on
        if (tid == 0) ptx::tma_store_wait_read();
        compute_sync();

        // ---- level 0, first pair: ds = s G .* (dO v_new^T) (rows of the sequence only), ds2 = ds .* (Q K^T)
        if (!(ok = wait(kC45, ph))) break;
        ptx::tc_fence_after_sync();
        if (warp == 0) trace(step, 2);
        // decay factors of this thread's eight (row, column) pairs of the 64 x 64 products, exp(min(g_row - g_col, 0)),
        // and exp(g_col) of its four columns: formed once per head, used by levels 0, 1 and 3
        float gw[2][4], ecol[2][2];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float gc = gs[nh * 16 + nt * 8 + 2 * c4 + (e & 1)];
            gw[nt][e] = __expf(fminf(((e >> 1) ? g1 : g0) - gc, 0.f));
            if (e < 2) ecol[nt][e] = __expf(gc);
          }
        {
          float acc[2][4], pq[2][4];
          narrow2(kColP, acc, kColP + kBank1, pq);
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int row = (e >> 1) ? r1 : r0, col = nh * 16 + nt * 8 + 2 * c4 + (e & 1);
              const float w = p.scale * gw[nt][e];
              const float ds = (col <= row && row < valid) ? acc[nt][e] * w : 0.f;
              acc[nt][e] = ds;
              const float ds2 = ds * pq[nt][e];
              dg_row[e >> 1] += ds2;
              dg_col[nt][e & 1] -= ds2;
            }
          st_narrow(smem + kOffX, acc);
        }
        if (warp == 0) trace(step, 3);
        // ---- dw = -du h^T
        if (!(ok = wait(kC3, ph))) break;
        ptx::tc_fence_after_sync();
        if (warp == 0) trace(step, 4);
        {
          float acc[4][4];
          wide(kColW, acc);
          st_wide(smem + kOffDw, acc, -1.f, -1.f);
        }
        ptx::fence_proxy_async_smem();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kL1Ready], lane);
        if (warp == 0) trace(step, 5);

        // ---- x = A^T du: dv = beta .* x, dbeta += x . v; a2 = du V^T kept for dA
        if (!(ok = wait(kCB, ph))) break;
        ptx::tc_fence_after_sync();
        if (warp == 0) trace(step, 6);
        float a2[2][4];
        {
          float acc[4][4];
          wide(kColW + kBank1, acc);
          narrow(kColR, a2);
          float s0, s1;
          dot_rows(acc, sV, s0, s1);
          db_row[0] += s0; db_row[1] += s1;
          if (valid == kChunk) {
            // through the V tile (level 0 has read it, and so has every warp after the barrier) and one TMA store
            compute_sync();
            st_wide(sV, acc, be0, be1);
            ptx::fence_proxy_async_smem();
            compute_sync();
            if (tid == 0) {
              ptx::tma_store_3d(&tm_dv, sV, 0, hv, t0);
              ptx::tma_store_3d(&tm_dv, sV + 8192, 64, hv, t0);
              ptx::tma_store_commit();
            }
          } else {
            st_global_rows(static_cast<T*>(p.dv), p.num_v_heads, hv, t0, valid, acc, be0, be1);
          }
        }
        if (warp == 0) trace(step, 7);
        // ---- T1 = dO h^T: dq += s gamma .* T1, dg += q . that;  T2 = v_new dh^T: dk += rho .* T2, dg -= k . that
        if (!(ok = wait(kCT, ph))) break;
        if (!(ok = wait(kLateFull, ph))) break;  // Q, K rows are read below (they landed before level 0 was issued)
        ptx::tc_fence_after_sync();
        if (warp == 0) trace(step, 8);
        {
          float acc[4][4], acc2[4][4];
          wide2(kColT, acc, kColT + kBank1, acc2);
          const float f0 = p.scale * gam0, f1 = p.scale * gam1;
#pragma unroll
          for (int nt = 0; nt < 4; ++nt) {
            acc[nt][0] *= f0; acc[nt][1] *= f0; acc[nt][2] *= f1; acc[nt][3] *= f1;
            acc2[nt][0] *= rho0; acc2[nt][1] *= rho0; acc2[nt][2] *= rho1; acc2[nt][3] *= rho1;
          }
          float s0, s1;
          dot_rows(acc, sQ, s0, s1);
          dg_row[0] += s0; dg_row[1] += s1;
          dot_rows(acc2, sK, s0, s1);
          dg_row[0] -= s0; dg_row[1] -= s1;
          dg_last += s0 + s1;
#pragma unroll
          for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              dq_acc[nt][e] += acc[nt][e];
              dk_acc[nt][e] += acc2[nt][e];
            }
        }
        // this warp no longer reads the tiles only level 0 uses; the dv store must have read the V tile
        if (tid == 0) ptx::tma_store_wait_read();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kEarlyFree], lane);
        if (warp == 0) trace(step, 9);

        // ---- level 1: dq += ds K, dk += ds^T Q; y = A^T dw; dA from dw K^T and du V^T
        if (!(ok = wait(kCL1, ph))) break;
        ptx::tc_fence_after_sync();
        if (warp == 0) trace(step, 10);
        {
          float acc[4][4], acc2[4][4];
          wide2(kColQ, acc, kColQ + kBank1, acc2);
#pragma unroll
          for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              dq_acc[nt][e] += acc[nt][e];
              dk_acc[nt][e] += acc2[nt][e];
            }
          // y = A^T dw: dk += (beta gamma) .* y ; dbeta += gamma * (y . k) ; dg += beta gamma * (y . k)
          float a1[2][4];
          wide(kColW, acc);
          narrow(kColP, a1);
          float s0, s1;
          dot_rows(acc, sK, s0, s1);
          db_row[0] += gam0 * s0; db_row[1] += gam1 * s1;
          dg_row[0] += be0 * gam0 * s0; dg_row[1] += be1 * gam1 * s1;
          const float f0 = be0 * gam0, f1 = be1 * gam1;
#pragma unroll
          for (int nt = 0; nt < 4; ++nt) {
            dk_acc[nt][0] += f0 * acc[nt][0]; dk_acc[nt][1] += f0 * acc[nt][1];
            dk_acc[nt][2] += f1 * acc[nt][2]; dk_acc[nt][3] += f1 * acc[nt][3];
          }
          // dA = (beta gamma)_d (dw K^T) + beta_d (du V^T), strictly lower
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int row = (e >> 1) ? r1 : r0, col = nh * 16 + nt * 8 + 2 * c4 + (e & 1);
              const float val = bs[col] * (ecol[nt][e & 1] * a1[nt][e] + a2[nt][e]);
              a1[nt][e] = (col < row) ? val : 0.f;
            }
          st_narrow(smem + kOffY, a1);
        }
        ptx::fence_proxy_async_smem();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kDaReady], lane);
        if (warp == 0) trace(step, 11);

        // ---- level 2: M1 = A^T dA as the next operand (the ds tile it overwrites was read by level 1)
        if (!(ok = wait(kC12, ph))) break;
        ptx::tc_fence_after_sync();
        if (warp == 0) trace(step, 12);
        {
          float acc[2][4];
          narrow(kColT, acc);
          st_narrow(smem + kOffX, acc);
        }
        ptx::fence_proxy_async_smem();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kM1Ready], lane);
        if (warp == 0) trace(step, 13);

        // ---- level 3: dL = -(M1 A^T) .* G (strictly lower); t = dL .* (beta_row K K^T): dg += rowsum(t) - colsum(t)
        if (!(ok = wait(kC13, ph))) break;
        ptx::tc_fence_after_sync();
        if (warp == 0) trace(step, 14);
        {
          float acc[2][4], kk[2][4], lb[2][4];
          narrow2(kColT + 64, acc, kColR + kBank1, kk);
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int row = (e >> 1) ? r1 : r0, col = nh * 16 + nt * 8 + 2 * c4 + (e & 1);
              const float dl = (col < row) ? -acc[nt][e] * gw[nt][e] : 0.f;
              const float be = (e >> 1) ? be1 : be0;
              acc[nt][e] = dl;
              lb[nt][e] = be * dl;
              const float t = be * dl * kk[nt][e];
              dg_row[e >> 1] += t;
              dg_col[nt][e & 1] -= t;
            }
          st_narrow(smem + kOffY, acc);  // dL over dA (level 2 has read it)
          st_narrow(smem + kOffX, lb);   // beta .* dL over M1 (level 3 has read it)
        }
        ptx::fence_proxy_async_smem();
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kDlReady], lane);
        if (warp == 0) trace(step, 15);

        // ---- partial sums of this head that do not depend on level 4 (they overlap its products)
        float* rr = red + ph * kRedFloats;
        {
          const float a0 = quad_sum(dg_row[0]), a1 = quad_sum(dg_row[1]);
          if (c4 == 0) {
            rr[nh * 64 + r0] = a0;
            rr[nh * 64 + r1] = a1;
          }
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float s = oct_sum(dg_col[nt][e]);
              if (g == 0) rr[512 + mt * 64 + nh * 16 + nt * 8 + 2 * c4 + e] = s;
            }
          float s = dg_last;
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
          if (lane == 0) rr[768 + warp] = s;
        }

        // ---- level 4: z = dL K: dbeta += z . k ; dk += beta .* z ;  dk += (beta .* dL)^T K
        if (!(ok = wait(kC4, ph))) break;
        ptx::tc_fence_after_sync();
        if (warp == 0) trace(step, 16);
        {
          float acc[4][4], acc2[4][4];
          wide2(kColW, acc, kColW + kBank1, acc2);
          float s0, s1;
          dot_rows(acc, sK, s0, s1);
          db_row[0] += s0; db_row[1] += s1;
#pragma unroll
          for (int nt = 0; nt < 4; ++nt) {
            dk_acc[nt][0] += be0 * acc[nt][0] + acc2[nt][0]; dk_acc[nt][1] += be0 * acc[nt][1] + acc2[nt][1];
            dk_acc[nt][2] += be1 * acc[nt][2] + acc2[nt][2]; dk_acc[nt][3] += be1 * acc[nt][3] + acc2[nt][3];
          }
        }
        // this warp no longer reads Q, K, A or tensor memory of this head
        ptx::tc_fence_before_sync();
        warp_arrive(&bars[kLateFree], lane);
        if (warp == 0) trace(step, 17);

        // ---- reductions: dg (rows + columns + last), dbeta; chunk-local reverse cumulative sum of dg
        {
          const float b0 = quad_sum(db_row[0]), b1 = quad_sum(db_row[1]);
          if (c4 == 0) {
            rr[256 + nh * 64 + r0] = b0;
            rr[256 + nh * 64 + r1] = b1;
          }
        }
        compute_sync();
        if (tid < 64) {
          float dg_c = 0.f, db_c = 0.f;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            dg_c += rr[q * 64 + tid] + rr[512 + q * 64 + tid];
            db_c += rr[256 + q * 64 + tid];
          }
          if (tid == valid - 1) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < 16; ++w) s += rr[768 + w];
            dg_c += s;
          }
          if (tid >= valid) dg_c = 0.f;  // rows of the next sequence: they must not enter the suffix sum
          // suffix sum over the 64 tokens of the chunk (two warps): dg_raw[c] = sum_{c' >= c} dg_cum[c']
          float s = dg_c;
#pragma unroll
          for (int off = 1; off < 32; off <<= 1) {
            const float n = __shfl_down_sync(0xffffffffu, s, off);
            if (lane + off < 32) s += n;
          }
          if (tid == 32) rr[784] = s;  // total of tokens 32..63
          asm volatile("bar.sync 2, 64;" ::: "memory");
          if (tid < 32) s += rr[784];
          if (tid < valid) {
            p.dg[(static_cast<int64_t>(t0) + tid) * p.num_v_heads + hv] = s;
            p.dbeta[(static_cast<int64_t>(t0) + tid) * p.num_v_heads + hv] = db_c;
          }
        }
        if (warp == 0) trace(step, 18);
      }
      if (!ok) break;

      // dq, dk of the k-head (already summed over its v-heads): through the dw and ds / dA tile areas and TMA
      // stores when the chunk is complete, row by row for a ragged tail
      if (valid == kChunk) {
        st_wide(smem + kOffDw, dq_acc, 1.f, 1.f);
        st_wide(smem + kOffX, dk_acc, 1.f, 1.f);
        ptx::fence_proxy_async_smem();
        compute_sync();
        if (tid == 0) {
          ptx::tma_store_3d(&tm_dq, smem + kOffDw, 0, hk, t0);
          ptx::tma_store_3d(&tm_dq, smem + kOffDw + 8192, 64, hk, t0);
          ptx::tma_store_3d(&tm_dk, smem + kOffX, 0, hk, t0);
          ptx::tma_store_3d(&tm_dk, smem + kOffX + 8192, 64, hk, t0);
          ptx::tma_store_commit();
        }
      } else {
        st_global_rows(static_cast<T*>(p.dq), p.num_k_heads, hk, t0, valid, dq_acc, 1.f, 1.f);
        st_global_rows(static_cast<T*>(p.dk), p.num_k_heads, hk, t0, valid, dk_acc, 1.f, 1.f);
      }
    }
    if (tid == 0) ptx::tma_store_wait_all();
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == kComputeWarps) ptx::tmem_dealloc(tmem, 512);
}

// [rows, width] row-major tensor of 16-bit elements seen as a 3-D map with a unit middle extent
int make_tmap_rows(CUtensorMap* out, const void* base, uint64_t rows, uint64_t width, uint32_t box_rows, bool is_bf16) {
  return make_tmap_3d(out, base, rows, 1, width, box_rows, 64, true, is_bf16);
}

}  // namespace

int launch_chunk_bwd(const BwdParams& p, int64_t total_tokens, int total_chunks_upper, bool is_bf16,
                     cudaStream_t stream) {
  int rc;
  CUtensorMap tm_q, tm_k, tm_v, tm_vn, tm_do, tm_a, tm_h, tm_dh, tm_du, tm_dq, tm_dk, tm_dv;
  const uint64_t state_rows = static_cast<uint64_t>(total_chunks_upper) * p.num_v_heads * kHeadDim;
  if ((rc = make_tmap_3d(&tm_q, p.q, total_tokens, p.num_k_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_k, p.k, total_tokens, p.num_k_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_v, p.v, total_tokens, p.num_v_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_vn, p.v_new, total_tokens, p.num_v_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_do, p.d_o, total_tokens, p.num_v_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_a, p.A, total_tokens, p.num_v_heads, 64, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_rows(&tm_h, p.h, state_rows, kHeadDim, 128, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_rows(&tm_dh, p.dh, state_rows, kHeadDim, 128, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_rows(&tm_du, p.du, state_rows, kChunk, 128, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_dq, p.dq, total_tokens, p.num_k_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_dk, p.dk, total_tokens, p.num_k_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  if ((rc = make_tmap_3d(&tm_dv, p.dv, total_tokens, p.num_v_heads, kHeadDim, 64, 64, true, is_bf16)) != QLA_OK) return rc;
  const int total_items = total_chunks_upper * p.num_k_heads;
  int dev = 0, sms = 0;
  QLA_CHECK_CUDA(cudaGetDevice(&dev));
  QLA_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const unsigned grid = static_cast<unsigned>(total_items < sms ? total_items : sms);
#define QLA_LAUNCH_BWD_CHUNK(T, TR)                                                                         \
  do {                                                                                                     \
    if ((rc = ensure_dynamic_smem<bwd_chunk_kernel<T, TR>>(kSmemBytes)) != QLA_OK) return rc;              \
    QLA_CHECK_CUDA(launch_dependent(bwd_chunk_kernel<T, TR>, dim3(grid), dim3(kThreads), kSmemBytes, stream, tm_q, tm_k, tm_v, \
                                    tm_vn, tm_do, tm_a, tm_h, tm_dh, tm_du, tm_dq, tm_dk, tm_dv, p, total_items)); \
  } while (0)
  const bool traced = p.trace != nullptr;
  if (is_bf16) {
    if (traced) QLA_LAUNCH_BWD_CHUNK(__nv_bfloat16, true); else QLA_LAUNCH_BWD_CHUNK(__nv_bfloat16, false);
  } else {
    if (traced) QLA_LAUNCH_BWD_CHUNK(__half, true); else QLA_LAUNCH_BWD_CHUNK(__half, false);
  }
#undef QLA_LAUNCH_BWD_CHUNK
  QLA_CHECK_CUDA(cudaGetLastError());
  return QLA_OK;
}

void launch_info_bwd_chunk_kernel(int* block_threads, size_t* dynamic_smem_bytes) {
  *block_threads = kThreads;
  *dynamic_smem_bytes = kSmemBytes;
}

}  // namespace qla
