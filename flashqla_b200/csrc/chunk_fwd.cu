// placeholder, replaced by the chunked forward
#include "common.cuh"
extern "C" QLA_API size_t qla_chunk_fwd_workspace_bytes(const QlaChunkFwdArgs*) { return 0; }
extern "C" QLA_API int qla_chunk_fwd(const QlaChunkFwdArgs*, void*) {
  qla::set_last_error("chunk forward not built yet");
  return QLA_ERR_UNSUPPORTED;
}
