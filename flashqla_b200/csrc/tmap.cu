// Host side of TMA: tensor-map encoding through the driver entry point obtained from the runtime.
#include "ptx_sm100.cuh"

namespace qla {

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int make_tmap_3d(CUtensorMap* out, const void* base, uint64_t tokens, uint64_t heads, uint64_t width,
                 uint32_t box_rows, uint32_t box_width, bool swizzle128, bool is_bf16) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) {
    set_last_error("cuTensorMapEncodeTiled is not available from the driver");
    return QLA_ERR_CUDA;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) {
    set_last_error("tensor base address must be 16-byte aligned for TMA");
    return QLA_ERR_INVALID_ARG;
  }
  cuuint64_t dims[3] = {width, heads, tokens};
  cuuint64_t strides[2] = {width * 2, heads * width * 2};
  cuuint32_t box[3] = {box_width, 1, box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed with CUresult %d (tokens=%llu heads=%llu width=%llu)",
                   static_cast<int>(r), static_cast<unsigned long long>(tokens),
                   static_cast<unsigned long long>(heads), static_cast<unsigned long long>(width));
    return QLA_ERR_CUDA;
  }
  return QLA_OK;
}

}  // namespace qla
