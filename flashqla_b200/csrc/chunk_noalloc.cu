// qla_chunk_fwd_noalloc: the chunked forward for callers that may not allocate device memory.
//
// Some hosts of this library hand out all device memory at start-up (state pools, activation arenas)
// and then forbid cudaMalloc on the request path: an allocation there can fail when the pool owns the
// whole card, and it stalls every stream of the process while the driver serves it.  Such a caller
// cannot provide the workspace qla_chunk_fwd asks for when sequences are packed with cu_seqlens (two
// small int32 tables: first 128-token pair and first chunk of every sequence).  This entry point keeps
// those tables in a fixed array that lives in the library's device image instead.
//
// Limits and rules:
//   * at most QLA_NOALLOC_MAX_SEQS sequences per call (larger calls are rejected);
//   * the array exists once per GPU that loads the library and stays allocated until the process exits
//     (about 32 KiB);
//   * every call on a GPU uses the same array, so two calls that may overlap on the GPU (different
//     streams) race on it - serialise them;
//   * the tables are rewritten completely by each call before they are read, nothing in the array has
//     to be cleared between calls; for the same reason QLA_CHUNK_TABLES_READY is ignored here (another
//     call may have rewritten the shared array since the caller last filled it);
//   * the first call on each GPU looks the array's device address up (cudaGetSymbolAddress) and, like
//     qla_chunk_fwd, raises the dynamic shared-memory limit of the kernels it launches
//     (cudaFuncSetAttribute); make that first call outside of any stream capture.
// It calls no cudaMalloc / cudaFree and no allocating library routine; inputs, outputs and the status
// word are still the caller's.
#include <mutex>

#include "common.cuh"

namespace qla {
namespace {

constexpr size_t kTableBytes = ((static_cast<size_t>(QLA_NOALLOC_MAX_SEQS) + 1) * sizeof(int32_t) + 15) & ~size_t(15);
constexpr size_t kScratchBytes = 2 * kTableBytes;

// In host code this name is only a stand-in for the device object: its device address has to be asked
// from the runtime (per device) before it can be given to a kernel.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

int scratch_for_current_device(void** out) {
  int dev = -1;
  QLA_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    set_last_error("device index %d outside the supported range [0, %d)", dev, kMaxDevices);
    return QLA_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    QLA_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return QLA_OK;
}

}  // namespace
}  // namespace qla

extern "C" QLA_API int qla_chunk_fwd_noalloc(const QlaChunkFwdArgs* args, void* stream) {
  using namespace qla;
  QLA_CHECK_ARG(args != nullptr, "args is NULL");
  if (args->cu_seqlens != nullptr && args->num_seqs > QLA_NOALLOC_MAX_SEQS) {
    set_last_error("qla_chunk_fwd_noalloc handles at most %d sequences per call, got %d; use qla_chunk_fwd with a "
                   "caller-provided workspace for larger batches",
                   QLA_NOALLOC_MAX_SEQS, args->num_seqs);
    return QLA_ERR_INVALID_ARG;
  }
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != QLA_OK) return rc;
  QlaChunkFwdArgs a = *args;
  a.workspace = scratch;
  a.workspace_bytes = kScratchBytes;
  a.flags &= ~QLA_CHUNK_TABLES_READY;  // the shared array may hold another call's tables
  return qla_chunk_fwd(&a, stream);
}
