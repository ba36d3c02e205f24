// Chunked gated-delta-rule backward for sm_100a.
// Reference: chunk_gated_delta_rule_bwd (flash_qla/ops/gated_delta_rule/chunk/__init__.py:89-182); the
// math is the decomposed form of tests/ref_gdr.py:263-557 / chunk/blackwell/bwd_sm12x.py (dv_local,
// reverse state scan, dq/dk/dw/dg, WY backward), regrouped into two kernels:
//
//  bwd_scan_kernel   (chunk_bwd_scan.cu) one CTA per (sequence, v-head), chunks in reverse order, dS resident
//                    in tensor memory; writes du^T [chunk][Hv][128 v][64 tokens], the state gradient
//                    leaving every chunk dh^T [chunk][Hv][128 v][128 k] and dh0.
//  bwd_chunk_kernel  one CTA per (chunk, k-head), looping over the v-heads of the GQA group so that dq and
//                    dk leave already reduced over the group: every remaining product of the chunk
//                    (dq, dk, dw, dA, the triangular-inverse backward, dbeta, dg with its chunk-local
//                    reverse cumulative sum).
//
// This kernel runs its many small products (64 x 64 x 128, 64 x 128 x 64, ...) with mma.sync on padded
// shared-memory tiles; rows beyond the end of a sequence are zero-filled on load, which makes every
// contraction over the chunk dimension ignore them.
#include "chunk_params.cuh"
#include "mma_sync.cuh"

namespace qla {
namespace {

constexpr int kBwdThreads = 256;
constexpr int LD = 136;  // padded row stride (elements) of [*][128] tiles: conflict-free ldmatrix
constexpr int LS = 72;   // padded row stride of [*][64] tiles

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

// ============================================================================== per-chunk kernel
// Row sums over the columns a warp owns, reduced over the four lanes that share a row.
__device__ __forceinline__ float quad_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  return x;
}
// Column sums over the 16 rows a warp owns, reduced over the eight lanes that share a column pair.
__device__ __forceinline__ float oct_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  x += __shfl_xor_sync(0xffffffffu, x, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 16);
  return x;
}

template <typename T>
__global__ void __launch_bounds__(kBwdThreads, 1) bwd_chunk_kernel(const BwdParams p) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c4 = lane & 3;
  const int mt = warp & 3, nh = warp >> 2;
  const int hk = blockIdx.y;
  const int group = p.num_v_heads / p.num_k_heads;
  if (p.cu_seqlens != nullptr && static_cast<int>(blockIdx.x) >= p.chunk_offsets[p.num_seqs]) return;
  const ChunkCoord cc = locate_chunk(blockIdx.x, p.cu_seqlens, p.chunk_offsets, p.num_seqs, p.seq_len);
  const int t0 = cc.seq_start + cc.local_chunk * kChunk;
  const int valid = min(kChunk, cc.seq_end - t0);
  const int64_t chunk_global = blockIdx.x;

  extern __shared__ __align__(16) uint8_t smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);  // [64][LD]
  T* sK = sQ + 64 * LD;
  T* sV = sK + 64 * LD;
  T* sVn = sV + 64 * LD;
  T* sdO = sVn + 64 * LD;
  T* sDu = sdO + 64 * LD;       // du^T [128 v][LS]
  T* sDw = sDu + 128 * LS;
  T* sA = sDw + 64 * LD;        // [64][LS]
  T* sH = sA + 64 * LS;         // [128][LD]
  T* sDh = sH + 128 * LD;       // [128][LD]
  // 64 x 64 temporaries reuse the h / dh area once those are consumed
  T* sDs = sH;                  // ds            [64][LS]
  T* sDA = sDs + 64 * LS;       // masked dA
  T* sM1 = sDA + 64 * LS;       // A^T dA
  T* sDL = sM1 + 64 * LS;       // dL
  T* sDLb = sDL + 64 * LS;      // beta .* dL
  float* sG = reinterpret_cast<float*>(sDh + 128 * LD);  // [64]
  float* sB = sG + 64;                                   // [64]
  float* red = sB + 64;                                  // [4][64] cross-warp partials
  float* red2 = red + 256;                               // [8] scalar partials

  const int64_t qk_stride = static_cast<int64_t>(p.num_k_heads) * kHeadDim;
  const int64_t v_stride = static_cast<int64_t>(p.num_v_heads) * kHeadDim;
  const int64_t a_stride = static_cast<int64_t>(p.num_v_heads) * kChunk;
  const T* qg = static_cast<const T*>(p.q) + (static_cast<int64_t>(t0) * p.num_k_heads + hk) * kHeadDim;
  const T* kg = static_cast<const T*>(p.k) + (static_cast<int64_t>(t0) * p.num_k_heads + hk) * kHeadDim;
  mm::load_tile_async<T, 64, 128, kBwdThreads>(sQ, LD, qg, qk_stride, valid);
  mm::load_tile_async<T, 64, 128, kBwdThreads>(sK, LD, kg, qk_stride, valid);
  mm::cp_async_commit();

  float dq_acc[8][4], dk_acc[8][4];  // rows 16 mt.., columns 64 nh.. ; summed over the v-heads of the group
  mm::zero_acc(dq_acc);
  mm::zero_acc(dk_acc);

  for (int hv = hk * group; hv < (hk + 1) * group; ++hv) {
    __syncthreads();  // previous head's shared-memory readers are done
    {
      const int64_t vo = (static_cast<int64_t>(t0) * p.num_v_heads + hv) * kHeadDim;
      mm::load_tile_async<T, 64, 128, kBwdThreads>(sV, LD, static_cast<const T*>(p.v) + vo, v_stride, valid);
      mm::load_tile_async<T, 64, 128, kBwdThreads>(sVn, LD, static_cast<const T*>(p.v_new) + vo, v_stride, valid);
      mm::load_tile_async<T, 64, 128, kBwdThreads>(sdO, LD, static_cast<const T*>(p.d_o) + vo, v_stride, valid);
      mm::load_tile_async<T, 128, 64, kBwdThreads>(
          sDu, LS, static_cast<const T*>(p.du) + (chunk_global * p.num_v_heads + hv) * kHeadDim * kChunk, kChunk, 128);
      mm::load_tile_async<T, 64, 64, kBwdThreads>(sA, LS, static_cast<const T*>(p.A) + (static_cast<int64_t>(t0) * p.num_v_heads + hv) * kChunk, a_stride, valid);
      const int64_t ho = (chunk_global * p.num_v_heads + hv) * kHeadDim * kHeadDim;
      mm::load_tile_async<T, 128, 128, kBwdThreads>(sH, LD, static_cast<const T*>(p.h) + ho, kHeadDim, 128);
      mm::load_tile_async<T, 128, 128, kBwdThreads>(sDh, LD, static_cast<const T*>(p.dh) + ho, kHeadDim, 128);
      mm::cp_async_commit();
      if (tid < 64) {
        const int64_t last = static_cast<int64_t>(t0) + valid - 1;
        const bool ok = tid < valid;
        const int64_t tok = ok ? static_cast<int64_t>(t0) + tid : last;
        sG[tid] = p.g_cumsum[tok * p.num_v_heads + hv];
        sB[tid] = ok ? load_scalar(p.beta, p.beta_dtype, tok * p.num_v_heads + hv) : 0.f;
      }
    }
    mm::cp_async_wait<0>();
    __syncthreads();

    const int r0 = mt * 16 + g, r1 = r0 + 8;  // the two rows this thread owns in every 64-row product
    const float gl = sG[valid - 1];
    const float g0 = sG[r0], g1 = sG[r1];
    const float gam0 = __expf(g0), gam1 = __expf(g1);
    const float rho0 = (r0 < valid) ? __expf(gl - g0) : 0.f, rho1 = (r1 < valid) ? __expf(gl - g1) : 0.f;
    const float be0 = sB[r0], be1 = sB[r1];
    float dg_row[2] = {0.f, 0.f}, db_row[2] = {0.f, 0.f};
    float dg_col[4][2];  // columns 32 nh + 8 nt + 2 c4 + {0, 1} of the 64 x 64 products
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) dg_col[nt][0] = dg_col[nt][1] = 0.f;
    float dg_last = 0.f;

    // helper: sum over this thread's columns of acc .* M[rows r0 / r1][64 nh + ...]
    auto dot_rows = [&](const float (&acc)[8][4], const T* M, float& s0, float& s1) {
      s0 = 0.f; s1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int col = nh * 64 + nt * 8 + 2 * c4;
        const uint32_t a = *reinterpret_cast<const uint32_t*>(M + r0 * LD + col);
        const uint32_t b = *reinterpret_cast<const uint32_t*>(M + r1 * LD + col);
        const T* ea = reinterpret_cast<const T*>(&a);
        const T* eb = reinterpret_cast<const T*>(&b);
        s0 += acc[nt][0] * Cvt<T>::to_f32(ea[0]) + acc[nt][1] * Cvt<T>::to_f32(ea[1]);
        s1 += acc[nt][2] * Cvt<T>::to_f32(eb[0]) + acc[nt][3] * Cvt<T>::to_f32(eb[1]);
      }
    };  // per-thread partials: every use is linear, the quad reduction happens once at the end

    // ---- phase 1: products with the chunk states h (entering) and dh (gradient of the leaving state)
    {
      float acc[8][4];
      // dq += s gamma .* (dO h^T);  dg += q . that
      mm::zero_acc(acc);
      mm::warp_gemm<T, 8, false, false>(acc, sdO + mt * 16 * LD, LD, sH + nh * 64 * LD, LD, 128);
      const float f0 = p.scale * gam0, f1 = p.scale * gam1;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) { acc[nt][0] *= f0; acc[nt][1] *= f0; acc[nt][2] *= f1; acc[nt][3] *= f1; }
      float s0, s1;
      dot_rows(acc, sQ, s0, s1);
      dg_row[0] += s0; dg_row[1] += s1;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) dq_acc[nt][e] += acc[nt][e];
      // dk += rho .* (v_new dh^T);  dg -= k . that;  dg_last += sum of the same
      mm::zero_acc(acc);
      mm::warp_gemm<T, 8, false, true>(acc, sVn + mt * 16 * LD, LD, sDh + nh * 64, LD, 128);  // dh stored [v][k]
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) { acc[nt][0] *= rho0; acc[nt][1] *= rho0; acc[nt][2] *= rho1; acc[nt][3] *= rho1; }
      dot_rows(acc, sK, s0, s1);
      dg_row[0] -= s0; dg_row[1] -= s1;
      dg_last += s0 + s1;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) dk_acc[nt][e] += acc[nt][e];
      // dw = -du h^T
      mm::zero_acc(acc);
      mm::warp_gemm<T, 8, true, false>(acc, sDu + mt * 16, LS, sH + nh * 64 * LD, LD, 128);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nt][e] = -acc[nt][e];
      mm::store_acc<T, 8>(sDw + mt * 16 * LD + nh * 64, LD, acc);
      // dg_last += exp(gL) * sum(h .* dh)
      float hd = 0.f;
      for (int i = tid; i < 128 * 64; i += kBwdThreads) {
        const int r = i >> 6, c2 = (i & 63) * 2;
        const uint32_t a = *reinterpret_cast<const uint32_t*>(sH + r * LD + c2);
        const T* ea = reinterpret_cast<const T*>(&a);
        hd += Cvt<T>::to_f32(ea[0]) * Cvt<T>::to_f32(sDh[c2 * LD + r]) +
              Cvt<T>::to_f32(ea[1]) * Cvt<T>::to_f32(sDh[(c2 + 1) * LD + r]);
      }
      dg_last += __expf(gl) * hd;
    }
    __syncthreads();  // sDw complete; sH / sDh may be overwritten by the 64 x 64 temporaries

    // ---- phase 2: ds = s G .* (dO v_new^T), ds2 = ds .* (Q K^T)       rows 16 mt.., columns 32 nh..
    {
      float acc[4][4], pq[4][4];
      mm::zero_acc(acc);
      mm::zero_acc(pq);
      mm::warp_gemm<T, 4, false, false>(acc, sdO + mt * 16 * LD, LD, sVn + nh * 32 * LD, LD, 128);
      mm::warp_gemm<T, 4, false, false>(pq, sQ + mt * 16 * LD, LD, sK + nh * 32 * LD, LD, 128);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = (e >> 1) ? r1 : r0, col = nh * 32 + nt * 8 + 2 * c4 + (e & 1);
          const float w = p.scale * __expf(fminf(((e >> 1) ? g1 : g0) - sG[col], 0.f));
          const float ds = (col <= row) ? acc[nt][e] * w : 0.f;
          acc[nt][e] = ds;
          const float ds2 = ds * pq[nt][e];
          dg_row[e >> 1] += ds2;     // per-thread partial, reduced over the quad at the end
          dg_col[nt][e & 1] -= ds2;  // reduced over the rows at the end
        }
      mm::store_acc<T, 4>(sDs + mt * 16 * LS + nh * 32, LS, acc);
    }
    __syncthreads();
    {
      // dq += ds K ;  dk += ds^T Q
      mm::warp_gemm<T, 8, false, true>(dq_acc, sDs + mt * 16 * LS, LS, sK + nh * 64, LD, 64);
      mm::warp_gemm<T, 8, true, true>(dk_acc, sDs + mt * 16, LS, sQ + nh * 64, LD, 64);
    }

    // ---- phase 3: WY backward
    {
      // dA = (beta gamma)_d (dw K^T) + beta_d (du V^T), strictly lower
      float a1[4][4], a2[4][4];
      mm::zero_acc(a1);
      mm::zero_acc(a2);
      mm::warp_gemm<T, 4, false, false>(a1, sDw + mt * 16 * LD, LD, sK + nh * 32 * LD, LD, 128);
      mm::warp_gemm<T, 4, true, false>(a2, sDu + mt * 16, LS, sV + nh * 32 * LD, LD, 128);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = (e >> 1) ? r1 : r0, col = nh * 32 + nt * 8 + 2 * c4 + (e & 1);
          const float bd = sB[col];
          const float val = bd * (__expf(sG[col]) * a1[nt][e] + a2[nt][e]);
          a1[nt][e] = (col < row) ? val : 0.f;
        }
      mm::store_acc<T, 4>(sDA + mt * 16 * LS + nh * 32, LS, a1);
    }
    {
      // y = A^T dw: dk += (beta gamma) .* y ; dbeta += gamma * (y . k) ; dg += beta gamma * (y . k)
      float acc[8][4];
      mm::zero_acc(acc);
      mm::warp_gemm<T, 8, true, true>(acc, sA + mt * 16, LS, sDw + nh * 64, LD, 64);
      float s0, s1;
      dot_rows(acc, sK, s0, s1);
      db_row[0] += gam0 * s0; db_row[1] += gam1 * s1;
      dg_row[0] += be0 * gam0 * s0; dg_row[1] += be1 * gam1 * s1;
      const float f0 = be0 * gam0, f1 = be1 * gam1;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        dk_acc[nt][0] += f0 * acc[nt][0]; dk_acc[nt][1] += f0 * acc[nt][1];
        dk_acc[nt][2] += f1 * acc[nt][2]; dk_acc[nt][3] += f1 * acc[nt][3];
      }
      // x = A^T du: dv = beta .* x ; dbeta += x . v
      mm::zero_acc(acc);
      mm::warp_gemm<T, 8, true, false>(acc, sA + mt * 16, LS, sDu + nh * 64 * LS, LS, 64);
      dot_rows(acc, sV, s0, s1);
      db_row[0] += s0; db_row[1] += s1;
      T* dvg = static_cast<T*>(p.dv);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int col = nh * 64 + nt * 8 + 2 * c4;
        if (r0 < valid)
          *reinterpret_cast<uint32_t*>(dvg + (static_cast<int64_t>(t0 + r0) * p.num_v_heads + hv) * kHeadDim + col) =
              mm::pack_pair<T>(be0 * acc[nt][0], be0 * acc[nt][1]);
        if (r1 < valid)
          *reinterpret_cast<uint32_t*>(dvg + (static_cast<int64_t>(t0 + r1) * p.num_v_heads + hv) * kHeadDim + col) =
              mm::pack_pair<T>(be1 * acc[nt][2], be1 * acc[nt][3]);
      }
    }
    __syncthreads();  // sDA complete
    {
      float acc[4][4];
      mm::zero_acc(acc);
      mm::warp_gemm<T, 4, true, true>(acc, sA + mt * 16, LS, sDA + nh * 32, LS, 64);  // M1 = A^T dA
      mm::store_acc<T, 4>(sM1 + mt * 16 * LS + nh * 32, LS, acc);
    }
    __syncthreads();
    {
      // dL = -(M1 A^T) .* G (strictly lower); t = dL .* (beta_row K K^T): dg += rowsum(t) - colsum(t)
      float acc[4][4], kk[4][4], lb[4][4];
      mm::zero_acc(acc);
      mm::zero_acc(kk);
      mm::warp_gemm<T, 4, false, false>(acc, sM1 + mt * 16 * LS, LS, sA + nh * 32 * LS, LS, 64);
      mm::warp_gemm<T, 4, false, false>(kk, sK + mt * 16 * LD, LD, sK + nh * 32 * LD, LD, 128);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = (e >> 1) ? r1 : r0, col = nh * 32 + nt * 8 + 2 * c4 + (e & 1);
          const float w = __expf(fminf(((e >> 1) ? g1 : g0) - sG[col], 0.f));
          const float dl = (col < row) ? -acc[nt][e] * w : 0.f;
          const float be = (e >> 1) ? be1 : be0;
          acc[nt][e] = dl;
          lb[nt][e] = be * dl;
          const float t = be * dl * kk[nt][e];
          dg_row[e >> 1] += t;
          dg_col[nt][e & 1] -= t;
        }
      mm::store_acc<T, 4>(sDL + mt * 16 * LS + nh * 32, LS, acc);
      mm::store_acc<T, 4>(sDLb + mt * 16 * LS + nh * 32, LS, lb);
    }
    __syncthreads();
    {
      // z = dL K: dbeta += z . k ; dk += beta .* z ;  dk += (beta .* dL)^T K
      float acc[8][4];
      mm::zero_acc(acc);
      mm::warp_gemm<T, 8, false, true>(acc, sDL + mt * 16 * LS, LS, sK + nh * 64, LD, 64);
      float s0, s1;
      dot_rows(acc, sK, s0, s1);
      db_row[0] += s0; db_row[1] += s1;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        dk_acc[nt][0] += be0 * acc[nt][0]; dk_acc[nt][1] += be0 * acc[nt][1];
        dk_acc[nt][2] += be1 * acc[nt][2]; dk_acc[nt][3] += be1 * acc[nt][3];
      }
      mm::warp_gemm<T, 8, true, true>(dk_acc, sDLb + mt * 16, LS, sK + nh * 64, LD, 64);
    }

    // ---- reductions: dg (rows + columns + last), dbeta; chunk-local reverse cumulative sum of dg
    // red[0..1][64]: row partials of the two column halves; red[2..3] reused after a barrier for columns
    __syncthreads();
    {
      const float a0 = quad_sum(dg_row[0]), a1 = quad_sum(dg_row[1]);
      const float b0 = quad_sum(db_row[0]), b1 = quad_sum(db_row[1]);
      if (c4 == 0) {
        red[nh * 64 + r0] = a0; red[nh * 64 + r1] = a1;
        red[128 + nh * 64 + r0] = b0; red[128 + nh * 64 + r1] = b1;
      }
      float s = dg_last;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
      if (lane == 0) red2[warp] = s;
    }
    __syncthreads();
    float dg_c = 0.f, db_c = 0.f;
    if (tid < 64) {
      dg_c = red[tid] + red[64 + tid];
      db_c = red[128 + tid] + red[192 + tid];
      if (tid == valid - 1) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) s += red2[w];
        dg_c += s;
      }
    }
    __syncthreads();
    {
      // column partials: four row-tile warps per column
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float s = oct_sum(dg_col[nt][e]);
          if (g == 0) red[mt * 64 + nh * 32 + nt * 8 + 2 * c4 + e] = s;
        }
    }
    __syncthreads();
    if (tid < 64) {
      dg_c += red[tid] + red[64 + tid] + red[128 + tid] + red[192 + tid];
      red2[0] = 0.f;
    }
    __syncthreads();
    // suffix sum over the 64 tokens of the chunk (two warps): dg_raw[c] = sum_{c' >= c} dg_cum[c']
    if (tid < 64) {
      float s = dg_c;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float n = __shfl_down_sync(0xffffffffu, s, off);
        if (lane + off < 32) s += n;
      }
      if (tid == 32) red2[0] = s;  // total of tokens 32..63
      __syncwarp();
      red[tid] = s;
    }
    __syncthreads();
    if (tid < 64) {
      float s = red[tid];
      if (tid < 32) s += red2[0];
      if (tid < valid) {
        p.dg[(static_cast<int64_t>(t0) + tid) * p.num_v_heads + hv] = s;
        p.dbeta[(static_cast<int64_t>(t0) + tid) * p.num_v_heads + hv] = db_c;
      }
    }
  }

  // dq, dk of the k-head (already summed over its v-heads)
  T* dqg = static_cast<T*>(p.dq);
  T* dkg = static_cast<T*>(p.dk);
  const int r0 = mt * 16 + g, r1 = r0 + 8;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    const int col = nh * 64 + nt * 8 + 2 * c4;
    if (r0 < valid) {
      const int64_t o = (static_cast<int64_t>(t0 + r0) * p.num_k_heads + hk) * kHeadDim + col;
      *reinterpret_cast<uint32_t*>(dqg + o) = mm::pack_pair<T>(dq_acc[nt][0], dq_acc[nt][1]);
      *reinterpret_cast<uint32_t*>(dkg + o) = mm::pack_pair<T>(dk_acc[nt][0], dk_acc[nt][1]);
    }
    if (r1 < valid) {
      const int64_t o = (static_cast<int64_t>(t0 + r1) * p.num_k_heads + hk) * kHeadDim + col;
      *reinterpret_cast<uint32_t*>(dqg + o) = mm::pack_pair<T>(dq_acc[nt][2], dq_acc[nt][3]);
      *reinterpret_cast<uint32_t*>(dkg + o) = mm::pack_pair<T>(dk_acc[nt][2], dk_acc[nt][3]);
    }
  }
}

constexpr size_t kChunkSmem = (6 * 64 * LD + 128 * LS + 64 * LS + 2 * 128 * LD) * 2 + (64 + 64 + 256 + 8) * sizeof(float);

}  // namespace

int launch_chunk_bwd(const BwdParams& p, int64_t total_tokens, int total_chunks_upper, bool is_bf16,
                     cudaStream_t stream) {
  int rc = launch_bwd_scan(p, total_tokens, is_bf16, stream);
  if (rc != QLA_OK) return rc;
  dim3 chunk_grid(total_chunks_upper, p.num_k_heads);
  if (is_bf16) {
    if ((rc = ensure_dynamic_smem<bwd_chunk_kernel<__nv_bfloat16>>(kChunkSmem)) != QLA_OK) return rc;
    bwd_chunk_kernel<__nv_bfloat16><<<chunk_grid, kBwdThreads, kChunkSmem, stream>>>(p);
  } else {
    if ((rc = ensure_dynamic_smem<bwd_chunk_kernel<__half>>(kChunkSmem)) != QLA_OK) return rc;
    bwd_chunk_kernel<__half><<<chunk_grid, kBwdThreads, kChunkSmem, stream>>>(p);
  }
  QLA_CHECK_CUDA(cudaGetLastError());
  return QLA_OK;
}

}  // namespace qla
