// Host-side construction of TMA tensor maps. cuTensorMapEncodeTiled is looked up through the
// runtime's driver-entry-point query, so the library has no link-time dependency on libcuda.
#include <mutex>

#include "kernels.h"

namespace wb200 {
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *entry = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &query) ==
            cudaSuccess &&
        query == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(entry);
  });
  return fn;
}

wb200_status encode(CUtensorMap *map, const void *base, int format, uint32_t rank,
                    const cuuint64_t *dims, const cuuint64_t *strides, const cuuint32_t *box) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return fail(WB200_ERR_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
  if (format != WB200_BF16 && format != WB200_F16)
    return fail(WB200_ERR_UNSUPPORTED, "TMA maps are built for 16-bit float formats only");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return fail(WB200_ERR_INVALID_ARGUMENT, "TMA base address must be 16-byte aligned");
  for (uint32_t i = 0; i + 1 < rank; ++i)
    if (strides[i] % 16 != 0)
      return fail(WB200_ERR_INVALID_ARGUMENT, "TMA strides must be multiples of 16 bytes");
  const cuuint32_t element_strides[3] = {1, 1, 1};
  CUresult result =
      fn(map, format == WB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
         rank, const_cast<void *>(base), dims, strides, box, element_strides,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (result != CUDA_SUCCESS)
    return fail(WB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(result));
  return WB200_OK;
}

}  // namespace

wb200_status encode_tmap_2d(CUtensorMap *map, const void *base, int format, uint64_t inner,
                            uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner,
                            uint32_t box_outer) {
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_pitch_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  return encode(map, base, format, 2, dims, strides, box);
}

wb200_status encode_tmap_3d(CUtensorMap *map, const void *base, int format, uint64_t inner,
                            uint64_t outer, uint64_t batch, uint64_t row_pitch_bytes,
                            uint64_t batch_pitch_bytes, uint32_t box_inner, uint32_t box_outer) {
  const cuuint64_t dims[3] = {inner, outer, batch};
  const cuuint64_t strides[2] = {row_pitch_bytes, batch_pitch_bytes};
  const cuuint32_t box[3] = {box_inner, box_outer, 1};
  return encode(map, base, format, 3, dims, strides, box);
}

}  // namespace wb200
