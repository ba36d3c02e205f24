// Shared host/device helpers for the flashqla_b200 kernels (sm_100a only).
#pragma once

#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/flashqla_b200.h"

namespace qla {

constexpr int kHeadDim = 128;  // K = V = 128 (recurrent_fused.py:6484, chunk/__init__.py:308-315)
constexpr int kChunk = 64;     // chunk size of the prefill path

// Codes written to the device status word by kernels (0 = fine).
enum DeviceStatus : int {
  kStatusOk = 0,
  kStatusBarrierTimeout = 1,  // a bounded mbarrier wait gave up
  kStatusBadIndex = 2,        // an index tensor pointed outside its buffer
  kStatusBadTmemBase = 3,     // a full tensor-memory allocation did not start at column 0
};

void set_last_error(const char* fmt, ...);

#define QLA_CHECK_ARG(cond, ...)            \
  do {                                      \
    if (!(cond)) {                          \
      ::qla::set_last_error(__VA_ARGS__);   \
      return QLA_ERR_INVALID_ARG;           \
    }                                       \
  } while (0)

#define QLA_CHECK_SUPPORTED(cond, ...)      \
  do {                                      \
    if (!(cond)) {                          \
      ::qla::set_last_error(__VA_ARGS__);   \
      return QLA_ERR_UNSUPPORTED;           \
    }                                       \
  } while (0)

#define QLA_CHECK_CUDA(expr)                                                              \
  do {                                                                                    \
    cudaError_t err__ = (expr);                                                           \
    if (err__ != cudaSuccess) {                                                           \
      ::qla::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__),    \
                            __FILE__, __LINE__);                                          \
      return QLA_ERR_CUDA;                                                                \
    }                                                                                     \
  } while (0)

// Raise the dynamic shared-memory limit of kernel `Fn` once per device instead of on every launch (the
// attribute belongs to the function in that device's context).  `Fn` is a template argument so that every
// kernel instantiation has its own flags.
template <auto Fn>
inline int ensure_dynamic_smem(size_t bytes) {
  static bool done[64] = {};
  int dev = 0;
  QLA_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && done[dev]) return QLA_OK;
  QLA_CHECK_CUDA(cudaFuncSetAttribute(Fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
  if (dev >= 0 && dev < 64) done[dev] = true;
  return QLA_OK;
}

// Programmatic dependent launch: the kernels of one forward call are launched with this attribute, so that the
// CTAs of a kernel are scheduled while the kernel before it in the stream drains; every kernel of the library
// executes grid_dep_wait() as its first statement (before any global-memory access and before any early exit),
// which returns when all earlier grids have completed and their writes are visible, so ordering is unchanged.
// QLA_PDL=0 in the environment turns the attribute off (plain stream-ordered launches).
inline bool pdl_enabled() {
  static const bool on = []() {
    const char* e = std::getenv("QLA_PDL");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Load one scalar of a runtime dtype (gates, biases: tiny tensors whose dtype varies by caller).
__device__ __forceinline__ float load_scalar(const void* p, int dtype, int64_t i) {
  if (dtype == QLA_DT_F32) return static_cast<const float*>(p)[i];
  if (dtype == QLA_DT_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}

template <typename T>
struct Cvt;
template <>
struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float x) { return __float2bfloat16_rn(x); }
};
template <>
struct Cvt<__half> {
  static __device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f32(float x) { return __float2half_rn(x); }
};
template <>
struct Cvt<float> {
  static __device__ __forceinline__ float to_f32(float x) { return x; }
  static __device__ __forceinline__ float from_f32(float x) { return x; }
};

}  // namespace qla
