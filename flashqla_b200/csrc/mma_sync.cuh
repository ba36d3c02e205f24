// Warp-level tensor-core tiles (mma.sync m16n8k16, 16-bit inputs, fp32 accumulate) on padded
// shared-memory operands, plus cp.async tile loads.  Used by the backward kernels, whose many small
// (64 x 64 / 64 x 128) products per chunk are independent across thousands of CTAs, so throughput
// comes from occupancy rather than from one large asynchronous tile.
#pragma once

#include "common.cuh"

namespace qla {
namespace mm {

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr(p)));
}

template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One warp: C[16 x 8*NT] += A[16 x K] * B[K x 8*NT]   (NT even).
//   A_TRANS = false: A(m, k) = A[m * lda + k]          A_TRANS = true: A(m, k) = A[k * lda + m]
//   B_NMAJOR = false: B(k, n) = B[n * ldb + k]         B_NMAJOR = true: B(k, n) = B[k * ldb + n]
// `A` points at the warp's first row (column of the stored matrix when transposed), `B` at its first n.
// Accumulator element layout (lane = 4 g + c): acc[nt][0..1] = row g, columns 8 nt + 2c, +1;
// acc[nt][2..3] = row g + 8, same columns.  All row strides must be multiples of 8 elements.
template <typename T, int NT, bool A_TRANS, bool B_NMAJOR>
__device__ __forceinline__ void warp_gemm(float (&acc)[NT][4], const T* A, int lda, const T* B, int ldb, int K) {
  static_assert(NT % 2 == 0, "NT must be even");
  const int lane = threadIdx.x & 31;
  const int j = lane >> 3, r = lane & 7;
#pragma unroll 4
  for (int k0 = 0; k0 < K; k0 += 16) {
    uint32_t a[4];
    if (!A_TRANS) {
      ldsm_x4(a, A + (lane & 15) * lda + k0 + (lane >> 4) * 8);
    } else {
      ldsm_x4_trans(a, A + (k0 + r + (j >> 1) * 8) * lda + (j & 1) * 8);
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt += 2) {
      uint32_t b[4];
      if (!B_NMAJOR) {
        ldsm_x4(b, B + (nt * 8 + r + (j >> 1) * 8) * ldb + k0 + (j & 1) * 8);
      } else {
        ldsm_x4_trans(b, B + (k0 + r + (j & 1) * 8) * ldb + nt * 8 + (j >> 1) * 8);
      }
      mma_16816<T>(acc[nt], a, b[0], b[1]);
      mma_16816<T>(acc[nt + 1], a, b[2], b[3]);
    }
  }
}

template <int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[NT][4]) {
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
}

// ---- cp.async (16-byte, L2 only); src_bytes = 0 zero-fills the destination
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Load ROWS x COLS 16-bit elements: row r from `src + r * src_stride` (elements) into `dst + r * ld`;
// rows >= valid_rows are zero-filled.  All threads of the CTA (NTHREADS) take part.
template <typename T, int ROWS, int COLS, int NTHREADS>
__device__ __forceinline__ void load_tile_async(T* dst, int ld, const T* src, int64_t src_stride, int valid_rows) {
  constexpr int kChunksPerRow = COLS / 8;
  constexpr int kTotal = ROWS * kChunksPerRow;
  for (int i = threadIdx.x; i < kTotal; i += NTHREADS) {
    const int r = i / kChunksPerRow, c = (i % kChunksPerRow) * 8;
    const bool ok = r < valid_rows;
    cp_async16(dst + r * ld + c, ok ? src + r * src_stride + c : src, ok);
  }
}

template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 x = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&x);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float a, float b) {
  __half2 x = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&x);
}

// Store a warp's accumulator tile (16 x 8*NT) as 16-bit values into shared memory (row stride ld).
template <typename T, int NT>
__device__ __forceinline__ void store_acc(T* dst, int ld, const float (&acc)[NT][4]) {
  const int lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    *reinterpret_cast<uint32_t*>(dst + g * ld + nt * 8 + 2 * c) = pack_pair<T>(acc[nt][0], acc[nt][1]);
    *reinterpret_cast<uint32_t*>(dst + (g + 8) * ld + nt * 8 + 2 * c) = pack_pair<T>(acc[nt][2], acc[nt][3]);
  }
}

}  // namespace mm
}  // namespace qla
