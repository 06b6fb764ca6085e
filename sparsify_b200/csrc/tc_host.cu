// Host-side creation of TMA tensor maps through the driver entry point
// (no link-time dependency on libcuda).
#include "tc.cuh"

#include <mutex>

namespace sc {
namespace tc {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
std::once_flag g_once;
EncodeTiledFn g_encode = nullptr;
}  // namespace

int make_tensor_map_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                         uint32_t box_rows) {
  std::call_once(g_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  });
  if (g_encode == nullptr) return sc::fail(SC_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return sc::fail(SC_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return SC_OK;
}

}  // namespace tc
}  // namespace sc

