// Status / error reporting of the C ABI (include/flashqla_b200.h).
#include <stdarg.h>

#include <string>

#include "ptx_sm100.cuh"

namespace qla {
namespace {
thread_local char g_last_error[512] = "";
}

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}
}  // namespace qla

extern "C" QLA_API const char* qla_status_string(int code) {
  switch (code) {
    case QLA_OK: return "ok";
    case QLA_ERR_INVALID_ARG: return "invalid argument";
    case QLA_ERR_UNSUPPORTED: return "unsupported configuration";
    case QLA_ERR_CUDA: return "CUDA call failed";
    case QLA_ERR_WORKSPACE: return "workspace missing or too small";
    case QLA_ERR_DEVICE: return "device reported a fault";
    default: return "unknown status";
  }
}

extern "C" QLA_API const char* qla_last_error(void) { return qla::g_last_error; }

extern "C" QLA_API int qla_abi_version(void) { return QLA_ABI_VERSION; }

namespace qla {
namespace {
// One warp waits, with the bounded wait every kernel of the library uses, for a barrier phase that nothing
// will ever complete: the wait gives up after `limit_ns`, records barrier / parity / warp in the status word
// and the kernel returns normally.
__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    ptx::fence_mbar_init();
  }
  __syncthreads();
  const bool ok = ptx::mbar_wait_polling(&bar, 0, status, kStatusBarrierTimeout | (255 << 8), limit_ns);
  if (ok && status != nullptr) atomicCAS(status, 0, kStatusBadIndex);  // cannot happen: nobody arrives
}
}  // namespace
}  // namespace qla

extern "C" QLA_API int qla_selftest_bounded_wait(int32_t* status, uint64_t limit_ns, void* stream) {
  using namespace qla;
  QLA_CHECK_ARG(status != nullptr, "status is NULL");
  QLA_CHECK_ARG(limit_ns > 0 && limit_ns <= 1000000000ull, "limit_ns must be in (0, 1e9]");
  bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, limit_ns);
  QLA_CHECK_CUDA(cudaGetLastError());
  return QLA_OK;
}

namespace qla {
void launch_info_chunk_fwd_kernel(int*, size_t*);
void launch_info_bwd_scan_kernel(int*, size_t*);
void launch_info_bwd_chunk_kernel(int*, size_t*);
void launch_info_kkt_solve_kernel(int*, size_t*);
void launch_info_recurrent_kernel(int*, size_t*);
}  // namespace qla

extern "C" QLA_API int qla_kernel_launch_info(const char* kernel, int32_t* block_threads, size_t* dynamic_smem_bytes) {
  using namespace qla;
  QLA_CHECK_ARG(kernel != nullptr && block_threads != nullptr && dynamic_smem_bytes != nullptr, "NULL argument");
  int block = 0;
  size_t smem = 0;
  const std::string name(kernel);
  if (name == "chunk_fwd_kernel") launch_info_chunk_fwd_kernel(&block, &smem);
  else if (name == "bwd_scan_kernel") launch_info_bwd_scan_kernel(&block, &smem);
  else if (name == "bwd_chunk_kernel") launch_info_bwd_chunk_kernel(&block, &smem);
  else if (name == "kkt_solve_kernel") launch_info_kkt_solve_kernel(&block, &smem);
  else if (name == "recurrent_kernel") launch_info_recurrent_kernel(&block, &smem);
  else {
    set_last_error("unknown kernel '%s'", kernel);
    return QLA_ERR_INVALID_ARG;
  }
  *block_threads = block;
  *dynamic_smem_bytes = smem;
  return QLA_OK;
}
