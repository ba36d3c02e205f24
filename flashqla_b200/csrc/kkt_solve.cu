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
// chunk's 64 columns in registers for every v-head.  The triangular inverse runs on CUDA cores in
// fp32: L goes to shared memory and thread `col` computes column `col` of the inverse by forward
// substitution with the L entries broadcast from shared memory.
#include "chunk_params.cuh"

namespace qla {


namespace {

constexpr int kLStride = 68;  // floats per L row: 16-byte aligned rows, conflict-free float4 stores

template <int BASE>
__device__ __forceinline__ void solve_column(const float* __restrict__ L, int col, float (&X)[64]) {
  // X = column `col` of (I + L)^-1 restricted to rows >= BASE (rows < BASE are zero for col >= BASE).
#pragma unroll
  for (int i = 0; i < 64; ++i) X[i] = (i == col) ? 1.f : 0.f;
#pragma unroll
  for (int i = BASE + 1; i < 64; ++i) {
    float acc0 = 0.f, acc1 = 0.f;
    const float* row = L + i * kLStride;
#pragma unroll
    for (int j4 = BASE; j4 < i; j4 += 4) {
      const float4 l = *reinterpret_cast<const float4*>(row + j4);
      acc0 = fmaf(l.x, X[j4], acc0);
      if (j4 + 1 < i) acc1 = fmaf(l.y, X[j4 + 1], acc1);
      if (j4 + 2 < i) acc0 = fmaf(l.z, X[j4 + 2], acc0);
      if (j4 + 3 < i) acc1 = fmaf(l.w, X[j4 + 3], acc1);
    }
    X[i] -= acc0 + acc1;
  }
}

template <typename T>
__global__ void __launch_bounds__(128) kkt_solve_kernel(const __grid_constant__ CUtensorMap tm_k,
                                                        const KktParams p) {
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
  float* sL = reinterpret_cast<float*>(sK + 32768);  // [2][64][kLStride]
  __shared__ __align__(16) float s_g[128];
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

  if (tid == 0) {
    ptx::mbar_expect_tx(&bar_tma, 32768);
    ptx::tma_load_3d(sK, &tm_k, &bar_tma, 0, hk, tok0);           // columns 0..63 of 128 tokens
    ptx::tma_load_3d(sK + 16384, &tm_k, &bar_tma, 64, hk, tok0);  // columns 64..127
    bool ok = ptx::mbar_wait(&bar_tma, 0, p.status, kStatusBarrierTimeout);
    if (ok) {
      constexpr uint32_t fmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? ptx::kFmtBF16 : ptx::kFmtF16;
      const uint32_t idesc = ptx::mma_idesc(128, 128, fmt, ptx::kMajorK, ptx::kMajorK);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t d = ptx::smem_desc_sw128(ptx::smem_u32(sK) + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024);
        ptx::mma_ss(tmem, d, d, idesc, ks > 0);
      }
    }
    ptx::mma_commit(&bar_mma);
  }
  // every thread reaches this point; the AND makes the decision CTA-uniform so that the barriers
  // inside the head loop are never reached by only part of the CTA
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
  }

  const int64_t tok = static_cast<int64_t>(tok0) + tid;
  const bool valid = tok < seq_end;
  float* Lc = sL + ci * 64 * kLStride;
  T* Ab = static_cast<T*>(p.A);

  for (int hv = hk * group; ok && hv < (hk + 1) * group; ++hv) {
    float gv = 0.f, bv = 0.f;
    if (valid) {
      gv = load_scalar(p.g, p.gate_dtype, tok * p.num_v_heads + hv);
      bv = load_scalar(p.beta, p.beta_dtype, tok * p.num_v_heads + hv);
    }
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
    if (valid) p.g_cumsum[tok * p.num_v_heads + hv] = gcs;
    s_g[tid] = gcs;
    __syncthreads();

    // L[c][d] = beta_c * exp(g_c - g_d) * (k_c . k_d) for d < c
    const float* gch = s_g + ci * 64;
    // branch-free (the causal mask is a select): a data-dependent branch per entry would diverge
#pragma unroll
    for (int d4 = 0; d4 < 64; d4 += 4) {
      const float4 g4 = *reinterpret_cast<const float4*>(gch + d4);
      float4 l;
      l.x = bv * __expf(fminf(gcs - g4.x, 0.f)) * kk[d4 + 0];
      l.y = bv * __expf(fminf(gcs - g4.y, 0.f)) * kk[d4 + 1];
      l.z = bv * __expf(fminf(gcs - g4.z, 0.f)) * kk[d4 + 2];
      l.w = bv * __expf(fminf(gcs - g4.w, 0.f)) * kk[d4 + 3];
      l.x = (d4 + 0 < c) ? l.x : 0.f;
      l.y = (d4 + 1 < c) ? l.y : 0.f;
      l.z = (d4 + 2 < c) ? l.z : 0.f;
      l.w = (d4 + 3 < c) ? l.w : 0.f;
      *reinterpret_cast<float4*>(Lc + c * kLStride + d4) = l;
    }
    __syncthreads();

    float X[64];
    if (warp & 1) solve_column<32>(Lc, c, X); else solve_column<0>(Lc, c, X);

    const int64_t row_tok0 = static_cast<int64_t>(tok0) + ci * 64;
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      if (row_tok0 + i < seq_end)
        Ab[((row_tok0 + i) * p.num_v_heads + hv) * 64 + c] = Cvt<T>::from_f32(X[i]);
    }
    __syncthreads();  // s_g / sL are rewritten for the next head
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) ptx::tmem_dealloc(tmem, 128);
}

// pair_offsets[n] = sum_{m<n} ceil(len_m / 128), chunk_offsets[n] = sum_{m<n} ceil(len_m / 64).
__global__ void chunk_tables_kernel(const int32_t* cu, int n, int32_t* pair_offsets, int32_t* chunk_offsets) {
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
  chunk_tables_kernel<<<1, 32, 0, stream>>>(cu, n, pair_offsets, chunk_offsets);
  QLA_CHECK_CUDA(cudaGetLastError());
  return QLA_OK;
}

int launch_kkt_solve(const KktParams& p, const void* k, int64_t total_tokens, int pairs_upper, bool is_bf16,
                     cudaStream_t stream) {
  CUtensorMap tm_k;
  int rc = make_tmap_3d(&tm_k, k, total_tokens, p.num_k_heads, kHeadDim, 128, 64, true, is_bf16);
  if (rc != QLA_OK) return rc;
  const size_t smem = 1024 + 32768 + 2 * 64 * kLStride * sizeof(float);
  dim3 grid(pairs_upper, p.num_k_heads);
  if (is_bf16) {
    QLA_CHECK_CUDA(cudaFuncSetAttribute(kkt_solve_kernel<__nv_bfloat16>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    kkt_solve_kernel<__nv_bfloat16><<<grid, 128, smem, stream>>>(tm_k, p);
  } else {
    QLA_CHECK_CUDA(cudaFuncSetAttribute(kkt_solve_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(smem)));
    kkt_solve_kernel<__half><<<grid, 128, smem, stream>>>(tm_k, p);
  }
  QLA_CHECK_CUDA(cudaGetLastError());
  return QLA_OK;
}

}  // namespace qla
