// Chunk preparation for the prefill path: chunk-local cumulative gates and the gated WY matrix
//   A = (I + StrictLower(diag(beta) * (G .* K K^T)))^-1,   G[c,d] = exp(g_c - g_d),
// one 64x64 unit-lower-triangular inverse per (chunk, v-head), stored in the input dtype as
// A[token, v-head, 64].  Reference: chunk_local_cumsum (flash_qla/ops/utils/cumsum.py:17-168) and
// kkt_solve (chunk/hopper/kkt_solve.py:18-342; the gated form is chunk/blackwell/kkt_solve.py:118-136
// and tests/ref_gdr.py:42-104).
//
// One CTA (128 threads) owns 128 consecutive tokens (two chunks) of one k-head and loops over the
// v-heads that share it, so K is fetched once per group.  K K^T for both chunks is a single
// tcgen05.mma (M = N = K = 128, operands straight from the TMA-written 128B-swizzled tile,
// accumulator in tensor memory); thread t then owns row t of the product (TMEM lane t) and keeps its
// chunk's 64 columns in registers for every v-head.  It also produces, per v-head, the chunk operand
//   Wt = A diag(beta gamma) K      (the "w" of tests/ref_gdr.py:107-147, stored negated)
// that lets the scan kernel form Vd = A diag(beta) V - Wt S0 with a single state-dependent product:
// one more tcgen05.mma per chunk (the [128][64] tile of -A diag(beta gamma) rows times that chunk's K rows read
// MN-major) leaves row t of Wt in TMEM lane t; the rows leave through a swizzled staging tile and TMA stores
// (row by row for a ragged tail).  The inverse of the unit-lower-triangular I + L is
// blocked: the four 16 x 16 diagonal blocks by fp32 forward substitution (one thread per column), then
// X21 = -X22 (L21 X11) at block size 16 and again at block size 32 with mma.sync m16n8k8 products on
// fp32 shared-memory tiles; at block size 16 each operand is split into two TF32 parts (3xTF32), at block
// size 32 the products are plain TF32 (see kSplit32).
#include "chunk_params.cuh"

namespace qla {


namespace {

// The inverse is formed IN PLACE: every block of X = (I + L)^-1 overwrites the block of L it was computed from, and
// the products L21 X11 pass through the (never used) upper-right 32 x 32 block of the same tile.  One fp32 tile
// per chunk keeps a CTA at 67 KiB of shared memory and 128 tensor-memory columns: three CTAs per SM.
constexpr int kLStride = 68;  // floats per L row: 16-byte aligned rows, conflict-free float4 stores
constexpr int kXStride = kLStride;
// Product precision of the blocked inverse.  Block size 16 keeps 3xTF32; block size 32 uses single TF32
// products like the reference's fp32-tile gemm there (chunk/hopper/kkt_solve.py:181-183): against an fp64
// inverse the error of that block is 1.70e-3 relative rms instead of 1.68e-3 (the 16-bit rounding of A
// dominates both), and o / final state do not move in the fourth digit.
constexpr bool kSplit32 = false;
constexpr bool kSplit16 = true;
constexpr int kTStride = kLStride;  // the products live in columns 32..63 of rows 0..31 of the chunk's tile

__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// One warp: C[16 x 8*NT] = A[16 x K] * B[K x 8*NT] on fp32 shared-memory tiles (row-major, strides in
// floats).  A points at the first of the 16 rows, B at row 0 / first column of the K x N block.
// kLowerB: B is lower triangular (B[k][n] = 0 for n > k), so column tile nt starts at k0 = 8 nt.
// kSplit: 3xTF32 (fp32-level products); otherwise one TF32 product per term.
template <int NT, bool kLowerB = false, bool kSplit = true>
__device__ __forceinline__ void warp_gemm_tf32(float (&acc)[NT][4], const float* A, int lda, const float* B,
                                               int ldb, int K) {
  const int lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
#pragma unroll 2
  for (int k0 = 0; k0 < K; k0 += 8) {
    // 3xTF32: x = hi + lo with hi = tf32(x), lo = tf32(x - hi); hi*hi + hi*lo + lo*hi keeps the products
    // at fp32-level accuracy (the dropped lo*lo term is ~2^-22 relative)
    const float af[4] = {A[g * lda + k0 + c], A[(g + 8) * lda + k0 + c], A[g * lda + k0 + c + 4],
                         A[(g + 8) * lda + k0 + c + 4]};
    uint32_t ah[4], al[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      ah[e] = to_tf32(af[e]);
      if (kSplit) al[e] = to_tf32(af[e] - __uint_as_float(ah[e]));
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if (kLowerB && nt * 8 > k0) continue;
      const float bf0 = B[(k0 + c) * ldb + nt * 8 + g], bf1 = B[(k0 + c + 4) * ldb + nt * 8 + g];
      const uint32_t bh0 = to_tf32(bf0), bh1 = to_tf32(bf1);
      if (kSplit) {
        const uint32_t bl0 = to_tf32(bf0 - __uint_as_float(bh0)), bl1 = to_tf32(bf1 - __uint_as_float(bh1));
        mma_tf32(acc[nt], al, bh0, bh1);
        mma_tf32(acc[nt], ah, bl0, bl1);
      }
      mma_tf32(acc[nt], ah, bh0, bh1);
    }
  }
}
// Store a warp's 16 x 8*NT accumulator tile, negated or not, to a row-major fp32 tile.
template <int NT>
__device__ __forceinline__ void store_tile(float* D, int ldd, const float (&acc)[NT][4], float sign) {
  const int lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    *reinterpret_cast<float2*>(D + g * ldd + nt * 8 + 2 * c) = make_float2(sign * acc[nt][0], sign * acc[nt][1]);
    *reinterpret_cast<float2*>(D + (g + 8) * ldd + nt * 8 + 2 * c) = make_float2(sign * acc[nt][2], sign * acc[nt][3]);
  }
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
__device__ __forceinline__ void pair_sync(int ci) {  // the two warps that own one chunk
  asm volatile("bar.sync %0, 64;" ::"r"(ci + 1) : "memory");
}

// K tile 32 KiB + one fp32 L / X tile per chunk (later the Aw, A and w staging tiles)
constexpr size_t kKktSmemBytes = 1024 + 32768 + 2 * 64 * kLStride * sizeof(float);

template <typename T>
__global__ void __launch_bounds__(128, 3) kkt_solve_kernel(const __grid_constant__ CUtensorMap tm_k,
                                                        const __grid_constant__ CUtensorMap tm_q,
                                                        const __grid_constant__ CUtensorMap tm_a,
                                                        const __grid_constant__ CUtensorMap tm_w,
                                                        const KktParams p) {
  grid_dep_wait();    // earlier kernels of the stream have completed (see launch_dependent)
  grid_dep_launch();  // the next one may be scheduled; it waits the same way
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hk = blockIdx.y;
  const int group = p.num_v_heads / p.num_k_heads;

  // ---- which 128 tokens
  int seq_start, seq_end, local_pair;
  if (p.cu_seqlens != nullptr) {
    const int pair = blockIdx.x;
    if (pair >= p.pair_offsets[p.num_seqs]) return;
    int lo = 0, hi = p.num_seqs - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (p.pair_offsets[mid] <= pair) lo = mid; else hi = mid - 1;
    }
    seq_start = p.cu_seqlens[lo];
    seq_end = p.cu_seqlens[lo + 1];
    local_pair = pair - p.pair_offsets[lo];
  } else {
    const int pairs_per_seq = (p.seq_len + 127) / 128;
    const int b = blockIdx.x / pairs_per_seq;
    local_pair = blockIdx.x % pairs_per_seq;
    seq_start = b * p.seq_len;
    seq_end = seq_start + p.seq_len;
  }
  const int tok0 = seq_start + local_pair * 128;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* sK = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
  float* sL = reinterpret_cast<float*>(sK + 32768);  // [2][64][kLStride]: L, then X in place
  uint8_t* sAw = reinterpret_cast<uint8_t*>(sL);     // 16 KiB [128 tokens][64] tile -A diag(beta gamma) (SW128), overlays L once solved
  uint8_t* sAst = sAw + 16384;                       // 16 KiB [128 tokens][64] staging tile of A for the TMA store (SW128)
  uint8_t* sW = sAw;                                 // 32 KiB staging tile of w (two [128][64] halves, SW128), once both are consumed
  __shared__ __align__(16) float s_bg[128];          // -beta * gamma per token
  __shared__ __align__(16) float s_g[128];
  __shared__ __align__(16) float s_rk[128];          // 1 / |k_t| per token (in-kernel q/k L2 norm), else unused
  __shared__ float s_part[4];
  __shared__ uint64_t bar_tma, bar_mma;
  __shared__ uint32_t tmem_base_s;

  if (tid == 0) {
    ptx::mbar_init(&bar_tma, 1);
    ptx::mbar_init(&bar_mma, 1);
    ptx::fence_mbar_init();
  }
  if (warp == 0) {
    ptx::tmem_alloc(&tmem_base_s, 128);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;

  // gate / beta of the first v-head are requested before anything waits, those of the next head at the
  // top of every head iteration: their global-memory latency hides behind the work in between
  const int64_t tok = static_cast<int64_t>(tok0) + tid;
  const bool valid = tok < seq_end;
  float gv_n = 0.f, bv_n = 0.f, gin_n = 0.f;
  auto fetch_gates = [&](int hv) {
    gv_n = bv_n = gin_n = 0.f;
    if (valid && hv < (hk + 1) * group) {
      const int64_t idx = tok * p.num_v_heads + hv;
      bv_n = load_scalar(p.beta, p.beta_dtype, idx);
      if (p.beta_out != nullptr) {  // logits in: the activated value is what every later stage reads
        bv_n = 1.f / (1.f + __expf(-bv_n));
        p.beta_out[idx] = bv_n;
      }
      if (p.A_in != nullptr) gin_n = p.g_cumsum[idx];
      else gv_n = load_scalar(p.g, p.gate_dtype, idx);
      if (p.A_log != nullptr) {  // gate activation of the layer (recurrent op: recurrent_fused.py:346-487)
        const float x = gv_n + p.dt_bias[hv];
        gv_n = -expf(p.A_log[hv]) * (x <= 20.f ? log1pf(expf(x)) : x);
      }
    }
  };
  fetch_gates(hk * group);

  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? ptx::kFmtBF16 : ptx::kFmtF16;
  // Products are issued by warp 0 as a converged warp (one elected lane inside ptx::umma_*): operand
  // arithmetic then stays on the uniform datapath and an instruction costs its time on the tensor pipe.
  if (warp == 0) {
    if (lane == 0) {
      ptx::mbar_expect_tx(&bar_tma, p.rnorm != nullptr ? 65536 : 32768);
      ptx::tma_load_3d(sK, &tm_k, &bar_tma, 0, hk, tok0);           // columns 0..63 of 128 tokens
      ptx::tma_load_3d(sK + 16384, &tm_k, &bar_tma, 64, hk, tok0);  // columns 64..127
      if (p.rnorm != nullptr) {  // the Q tile visits the (still unused) X area, only for its row norms
        ptx::tma_load_3d(sK + 32768, &tm_q, &bar_tma, 0, hk, tok0);
        ptx::tma_load_3d(sK + 32768 + 16384, &tm_q, &bar_tma, 64, hk, tok0);
      }
    }
    __syncwarp();
    const bool got = __all_sync(0xffffffffu, ptx::mbar_wait(&bar_tma, 0, p.status, kStatusBarrierTimeout));
    if (got) {
      const uint64_t d = ptx::smem_desc_sw128(ptx::smem_u32(sK), 16, 1024);
      ptx::umma_ss_k128<2, 1024 - 6, 2, 1024 - 6>(tmem, d, d, ptx::mma_idesc(128, 128, fmt, ptx::kMajorK, ptx::kMajorK),
                                                  false);
    }
    ptx::umma_commit(&bar_mma);
  }
  // In-kernel L2 norm of q and k (reference: l2norm before the kernels, flash_qla/utils/math.py:14-21 via
  // chunk/__init__.py:332-334): thread t computes 1/sqrt(|row t|^2 + eps) of its K and Q rows while the
  // product runs.  Everything downstream uses the RAW tiles and folds the factors in: K K^T[c][d] r_c r_d
  // here, r_k into beta gamma for w; the scan folds r_k into rho, r_q into s gamma and both into Pg.
  float rk_c = 1.f;
  if (p.rnorm != nullptr) {
    const bool got = ptx::mbar_wait(&bar_tma, 0, p.status, kStatusBarrierTimeout);
    float sk = 0.f, sq = 0.f;
    if (got) {
#pragma unroll 1
      for (int h = 0; h < 2; ++h)
#pragma unroll 2
        for (int c16 = 0; c16 < 8; ++c16) {
          const uint32_t off = h * 16384 + ptx::sw128_offset(tid, c16);
          const uint4 kv = *reinterpret_cast<const uint4*>(sK + off);
          const uint4 qv = *reinterpret_cast<const uint4*>(sK + 32768 + off);
          const T* ke = reinterpret_cast<const T*>(&kv);
          const T* qe = reinterpret_cast<const T*>(&qv);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float a = Cvt<T>::to_f32(ke[e]), b = Cvt<T>::to_f32(qe[e]);
            sk += a * a;
            sq += b * b;
          }
        }
    }
    rk_c = rsqrtf(sk + p.norm_eps);
    const float rq_c = rsqrtf(sq + p.norm_eps);
    s_rk[tid] = rk_c;
    if (valid) *reinterpret_cast<float2*>(p.rnorm + (tok * p.num_k_heads + hk) * 2) = make_float2(rq_c, rk_c);
  }
  // every thread reaches this point; the AND makes the decision CTA-uniform so that the barriers
  // inside the head loop are never reached by only part of the CTA (it also orders s_rk and the last reads
  // of the Q tile before the head loop reuses that memory)
  const bool ok = __syncthreads_and(ptx::mbar_wait(&bar_mma, 0, p.status, kStatusBarrierTimeout)) != 0;
  ptx::tc_fence_after_sync();

  const int ci = tid >> 6, c = tid & 63;
  float kk[64];
  if (ok) {
    uint32_t r[32];
    const uint32_t taddr = tmem + (static_cast<uint32_t>(warp * 32) << 16) + ci * 64;
    ptx::tmem_ld32(taddr, r);
    ptx::tmem_wait_ld();
#pragma unroll
    for (int j = 0; j < 32; ++j) kk[j] = __uint_as_float(r[j]);
    ptx::tmem_ld32(taddr + 32, r);
    ptx::tmem_wait_ld();
#pragma unroll
    for (int j = 0; j < 32; ++j) kk[32 + j] = __uint_as_float(r[j]);
    if (p.rnorm != nullptr) {
      const float* rkc = s_rk + ci * 64;
#pragma unroll
      for (int j = 0; j < 64; ++j) kk[j] *= rk_c * rkc[j];
    }
  }

  float* Lc = sL + ci * 64 * kLStride;
  T* Ab = static_cast<T*>(p.A);

  int mma_uses = 0;  // completed phases of bar_mma after the first (K K^T)
  bool w_store_pending = false;
  for (int hv = hk * group; ok && hv < (hk + 1) * group; ++hv) {
    const float gv = gv_n, bv = bv_n, gin = gin_n;
    fetch_gates(hv + 1);
    // inclusive scan over the 64 tokens of the chunk (two warps)
    float gcs = gv;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, gcs, off);
      if (lane >= off) gcs += n;
    }
    if (lane == 31) s_part[warp] = gcs;
    __syncthreads();
    if (warp & 1) gcs += s_part[warp - 1];
    if (p.A_in != nullptr) gcs = gin;  // gates are cumulative already
    else if (valid) p.g_cumsum[tok * p.num_v_heads + hv] = gcs;
    const float gc2 = gcs * 1.4426950408889634f;  // exponents are formed in the log2 domain: one FADD + ex2 each
    s_g[tid] = gc2;
    s_bg[tid] = -bv * ptx::ex2(gc2) * rk_c;
    // the previous head's w tile lies where L is built next: its store must have read it by now
    if (tid == 0 && w_store_pending) ptx::tma_store_wait_read();
    __syncthreads();

    // L[c][d] = beta_c * exp(g_c - g_d) * (k_c . k_d) for d < c
    const float* gch = s_g + ci * 64;
    // branch-free (the causal mask is a select, so an overflowing exponent above the diagonal is harmless):
    // a data-dependent branch per entry would diverge
    // Only the lower block triangle of L is ever read, so the warp that owns rows 0..31 stops at column 32.
#pragma unroll
    for (int d4 = 0; d4 < 64; d4 += 4) {
      if (d4 >= 32 && (warp & 1) == 0) break;
      const float4 g4 = *reinterpret_cast<const float4*>(gch + d4);
      float4 l;
      l.x = bv * ptx::ex2(gc2 - g4.x) * kk[d4 + 0];
      l.y = bv * ptx::ex2(gc2 - g4.y) * kk[d4 + 1];
      l.z = bv * ptx::ex2(gc2 - g4.z) * kk[d4 + 2];
      l.w = bv * ptx::ex2(gc2 - g4.w) * kk[d4 + 3];
      l.x = (d4 + 0 < c) ? l.x : 0.f;
      l.y = (d4 + 1 < c) ? l.y : 0.f;
      l.z = (d4 + 2 < c) ? l.z : 0.f;
      l.w = (d4 + 3 < c) ? l.w : 0.f;
      *reinterpret_cast<float4*>(Lc + c * kLStride + d4) = l;
    }
    __syncthreads();

    float* Xc = Lc;  // in place
    if (p.A_in != nullptr) {
      // A comes from an earlier call: row c of this chunk straight into the X tile
      const T* arow = static_cast<const T*>(p.A_in) + ((static_cast<int64_t>(tok0) + tid) * p.num_v_heads + hv) * 64;
#pragma unroll 1
      for (int j = 0; j < 64; j += 8) {
        uint4 raw = valid ? *reinterpret_cast<const uint4*>(arow + j) : make_uint4(0, 0, 0, 0);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int x = 0; x < 8; ++x) Xc[c * kXStride + j + x] = Cvt<T>::to_f32(e[x]);
      }
      pair_sync(ci);
    } else {
    // ---- blocked inverse of I + L for this chunk (64 threads = warps 2 ci, 2 ci + 1)
    float* Tc = Lc + 32;  // rows 0..31, columns 32..63 of the tile
    const int wl = warp & 1;  // warp within the chunk
    {
      // the four 16 x 16 diagonal blocks: thread = (block, column)
      const int b0 = (c >> 4) * 16, cc = c & 15;
      float x[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float acc = (i == cc) ? 1.f : 0.f;
#pragma unroll
        for (int j = 0; j < i; ++j) acc -= Lc[(b0 + i) * kLStride + b0 + j] * x[j];
        x[i] = acc;
      }
      __syncwarp();  // a block's 16 threads sit in one warp: all have read the block before it is overwritten
#pragma unroll
      for (int i = 0; i < 16; ++i) Xc[(b0 + i) * kXStride + b0 + cc] = x[i];
    }
    pair_sync(ci);
    {
      // block size 16: X[R, C] = -X[R, R] (L[R, C] X[C, C]) for (R, C) = (16, 0) and (48, 32); one per warp
      const int C0 = 32 * wl, R0 = C0 + 16;
      float acc[2][4];
      warp_gemm_tf32<2, true, kSplit16>(acc, Lc + R0 * kLStride + C0, kLStride, Xc + C0 * kXStride + C0, kXStride, 16);
      float* Tw = Tc + wl * 16 * kTStride;
      store_tile<2>(Tw, kTStride, acc, 1.f);
      __syncwarp();
      warp_gemm_tf32<2, false, kSplit16>(acc, Xc + R0 * kXStride + R0, kXStride, Tw, kTStride, 16);
      store_tile<2>(Xc + R0 * kXStride + C0, kXStride, acc, -1.f);
    }
    pair_sync(ci);
    {
      // block size 32: X[32:64, 0:32] = -X[32:64, 32:64] (L[32:64, 0:32] X[0:32, 0:32]); 16 rows per warp
      const int R0 = 32 + 16 * wl;
      float acc[4][4];
      // X[0:32, 0:32] is lower triangular: column tile nt has nothing above row 8 nt.  X[32:64, 32:64] is too:
      // its rows 0..15 (warp 0) end at column 15.
      warp_gemm_tf32<4, true, kSplit32>(acc, Lc + R0 * kLStride, kLStride, Xc, kXStride, 32);
      store_tile<4>(Tc + wl * 16 * kTStride, kTStride, acc, 1.f);
      pair_sync(ci);
      warp_gemm_tf32<4, false, kSplit32>(acc, Xc + R0 * kXStride + 32, kXStride, Tc, kTStride, 16 * (wl + 1));
      store_tile<4>(Xc + R0 * kXStride, kXStride, acc, -1.f);
    }
    pair_sync(ci);
    }  // A_in
    // ---- w = -A diag(beta gamma) K.  Row t of the [128][64] tile holds -A[t][:] .* (beta gamma) of t's own
    // chunk; one tcgen05.mma per chunk multiplies the WHOLE tile with that chunk's 64 K rows (read MN-major),
    // so rows 0..63 of the first product and rows 64..127 of the second are the wanted ones and no zero
    // padding is needed.  The same pass writes A itself (16-bit) into a staging tile for one TMA store.
    // The upper triangle of X is exactly zero (zeroed once per CTA and never written; forward substitution yields exact zeros inside the diagonal blocks),
    // and rows / columns of tokens past the sequence end carry beta = 0, so no mask is applied here.
    __syncthreads();
    const bool full_pair = tok0 + 128 <= seq_end;
    {
      // The staging tiles overlay the fp32 tile they are built from: every thread first takes its whole row into
      // registers (both 16-bit forms), and writes after a barrier.  Columns 32..63 of rows 0..31 hold the scratch
      // products, not zeros: they are skipped.
      const float* xr = Xc + c * kXStride;
      const float* bg = s_bg + ci * 64;
      uint32_t aw[32], av[32];
#pragma unroll
      for (int c16 = 0; c16 < 8; ++c16) {
        float4 x0 = *reinterpret_cast<const float4*>(xr + c16 * 8);
        float4 x1 = *reinterpret_cast<const float4*>(xr + c16 * 8 + 4);
        if (c16 >= 4 && c < 32) x0 = x1 = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 b0 = *reinterpret_cast<const float4*>(bg + c16 * 8);
        const float4 b1 = *reinterpret_cast<const float4*>(bg + c16 * 8 + 4);
        aw[4 * c16 + 0] = pack2<T>(x0.x * b0.x, x0.y * b0.y);
        aw[4 * c16 + 1] = pack2<T>(x0.z * b0.z, x0.w * b0.w);
        aw[4 * c16 + 2] = pack2<T>(x1.x * b1.x, x1.y * b1.y);
        aw[4 * c16 + 3] = pack2<T>(x1.z * b1.z, x1.w * b1.w);
        av[4 * c16 + 0] = pack2<T>(x0.x, x0.y);
        av[4 * c16 + 1] = pack2<T>(x0.z, x0.w);
        av[4 * c16 + 2] = pack2<T>(x1.x, x1.y);
        av[4 * c16 + 3] = pack2<T>(x1.z, x1.w);
      }
      __syncthreads();
      T* arow = Ab + (tok * p.num_v_heads + hv) * 64;
#pragma unroll
      for (int c16 = 0; c16 < 8; ++c16) {
        const uint32_t off = ptx::sw128_offset(tid, c16);  // row = token within the pair
        *reinterpret_cast<uint4*>(sAw + off) = make_uint4(aw[4 * c16], aw[4 * c16 + 1], aw[4 * c16 + 2], aw[4 * c16 + 3]);
        if (p.A_in == nullptr) {
          const uint4 a4 = make_uint4(av[4 * c16], av[4 * c16 + 1], av[4 * c16 + 2], av[4 * c16 + 3]);
          if (full_pair) *reinterpret_cast<uint4*>(sAst + off) = a4;
          else if (valid) *reinterpret_cast<uint4*>(arow + c16 * 8) = a4;  // ragged tail: the next sequence owns the rest
        }
      }
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
      if (lane == 0 && p.A_in == nullptr && full_pair) {
        ptx::tma_store_3d(&tm_a, sAst, 0, hv, tok0);
        ptx::tma_store_commit();
      }
      __syncwarp();
      ptx::tc_fence_after_sync();
      // two M = 64 products into the same 128 columns: row r of chunk 0 lands in lane (r % 16) + 32 (r / 16), the
      // rows of chunk 1 in the 16 lanes above them
      const uint32_t idesc = ptx::mma_idesc(64, 128, fmt, ptx::kMajorK, ptx::kMajorMN);
      const uint64_t da = ptx::smem_desc_sw128(ptx::smem_u32(sAw), 16, 1024);
      const uint64_t db = ptx::smem_desc_sw128(ptx::smem_u32(sK), 16384, 1024);
      ptx::umma_ss_k64<2, 128>(tmem, da, db, idesc, false);                                            // chunk 0: K rows 0..63
      ptx::umma_ss_k64<2, 128>(tmem + (16u << 16), da + (8192 >> 4), db + (8192 >> 4), idesc, false);  // chunk 1: K rows 64..127
      ptx::umma_commit(&bar_mma);
      // the w rows are staged where the A tile sits: its store has to have read it before anybody passes
      // the barrier below
      if (lane == 0) ptx::tma_store_wait_read();
      __syncwarp();
    }
    ++mma_uses;
    const bool ok2 = __syncthreads_and(ptx::mbar_wait(&bar_mma, mma_uses & 1, p.status, kStatusBarrierTimeout)) != 0;
    ptx::tc_fence_after_sync();
    if (ok2) {
      // One row of w per thread: 128 values; lane l of warp w holds row 16 w + (l & 15) of chunk l >> 4.  A full
      // pair goes through a swizzled staging tile and two TMA stores (whole 128-byte lines per token row); a ragged
      // tail is written row by row, only by lanes with a valid token.  tcgen05.ld is warp-collective: every lane
      // runs the loop.
      const int tp = (lane >> 4) * 64 + warp * 16 + (lane & 15);  // token within the pair
      const bool valid_w = static_cast<int64_t>(tok0) + tp < seq_end;
      T* wrow = static_cast<T*>(p.w) + ((static_cast<int64_t>(tok0) + tp) * p.num_v_heads + hv) * kHeadDim;
      const uint32_t taddr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
#pragma unroll 1
      for (int kb = 0; kb < 128; kb += 32) {
        uint32_t r[32];
        ptx::tmem_ld32(taddr + kb, r);
        ptx::tmem_wait_ld();
        uint8_t* half = sW + (kb >> 6) * 16384;
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          const uint4 val = make_uint4(pack2<T>(__uint_as_float(r[e]), __uint_as_float(r[e + 1])),
                                       pack2<T>(__uint_as_float(r[e + 2]), __uint_as_float(r[e + 3])),
                                       pack2<T>(__uint_as_float(r[e + 4]), __uint_as_float(r[e + 5])),
                                       pack2<T>(__uint_as_float(r[e + 6]), __uint_as_float(r[e + 7])));
          if (full_pair) *reinterpret_cast<uint4*>(half + ptx::sw128_offset(tp, ((kb & 63) + e) >> 3)) = val;
          else if (valid_w) *reinterpret_cast<uint4*>(wrow + kb + e) = val;
        }
      }
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before_sync();
    __syncthreads();  // s_g / s_bg are rewritten for the next head; the w tile is complete
    if (tid == 0 && ok2 && full_pair) {
      ptx::tma_store_3d(&tm_w, sW, 0, hv, tok0);
      ptx::tma_store_3d(&tm_w, sW + 16384, 64, hv, tok0);
      ptx::tma_store_commit();
    }
    w_store_pending = true;
  }
  if (tid == 0) ptx::tma_store_wait_read();  // shared memory stays allocated until the last store has read it

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) ptx::tmem_dealloc(tmem, 128);
}

// pair_offsets[n] = sum_{m<n} ceil(len_m / 128), chunk_offsets[n] = sum_{m<n} ceil(len_m / 64).
__global__ void chunk_tables_kernel(const int32_t* cu, int n, int32_t* pair_offsets, int32_t* chunk_offsets) {
  grid_dep_wait();
  grid_dep_launch();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int po = 0, co = 0;
    for (int i = 0; i < n; ++i) {
      pair_offsets[i] = po;
      chunk_offsets[i] = co;
      const int len = cu[i + 1] - cu[i];
      po += (len + 127) / 128;
      co += (len + 63) / 64;
    }
    pair_offsets[n] = po;
    chunk_offsets[n] = co;
  }
}

}  // namespace

int launch_chunk_tables(const int32_t* cu, int n, int32_t* pair_offsets, int32_t* chunk_offsets,
                        cudaStream_t stream) {
  QLA_CHECK_CUDA(launch_dependent(chunk_tables_kernel, dim3(1), dim3(32), 0, stream, cu, n, pair_offsets, chunk_offsets));
  QLA_CHECK_CUDA(cudaGetLastError());
  return QLA_OK;
}

int launch_kkt_solve(const KktParams& p, const void* k, const void* q, int64_t total_tokens, int pairs_upper,
                     bool is_bf16, cudaStream_t stream) {
  CUtensorMap tm_k, tm_q, tm_a, tm_w;
  int rc = make_tmap_3d(&tm_k, k, total_tokens, p.num_k_heads, kHeadDim, 128, 64, true, is_bf16);
  if (rc != QLA_OK) return rc;
  // q is only read for the in-kernel L2 norm (p.rnorm set); otherwise the map is made over k and unused
  rc = make_tmap_3d(&tm_q, p.rnorm != nullptr ? q : k, total_tokens, p.num_k_heads, kHeadDim, 128, 64, true, is_bf16);
  if (rc != QLA_OK) return rc;
  // A leaves through a [128 tokens][64] staging tile; in rebuild mode (A given) the map is made but unused
  rc = make_tmap_3d(&tm_a, p.A, total_tokens, p.num_v_heads, 64, 128, 64, true, is_bf16);
  if (rc != QLA_OK) return rc;
  // w leaves through two [128 tokens][64] staging tiles per (pair, head)
  rc = make_tmap_3d(&tm_w, p.w, total_tokens, p.num_v_heads, kHeadDim, 128, 64, true, is_bf16);
  if (rc != QLA_OK) return rc;
  const size_t smem = kKktSmemBytes;
  dim3 grid(pairs_upper, p.num_k_heads);
  if (is_bf16) {
    if ((rc = ensure_dynamic_smem<kkt_solve_kernel<__nv_bfloat16>>(smem)) != QLA_OK) return rc;
    QLA_CHECK_CUDA(launch_dependent(kkt_solve_kernel<__nv_bfloat16>, grid, dim3(128), smem, stream, tm_k, tm_q, tm_a, tm_w, p));
  } else {
    if ((rc = ensure_dynamic_smem<kkt_solve_kernel<__half>>(smem)) != QLA_OK) return rc;
    QLA_CHECK_CUDA(launch_dependent(kkt_solve_kernel<__half>, grid, dim3(128), smem, stream, tm_k, tm_q, tm_a, tm_w, p));
  }
  QLA_CHECK_CUDA(cudaGetLastError());
  return QLA_OK;
}

void launch_info_kkt_solve_kernel(int* block_threads, size_t* dynamic_smem_bytes) {
  *block_threads = 128;
  *dynamic_smem_bytes = kKktSmemBytes;
}

}  // namespace qla
