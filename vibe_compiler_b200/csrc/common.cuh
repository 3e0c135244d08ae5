// Shared host/device helpers: scalar formats, IEEE conversions, error plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>

#include <string>

#include "../../include/wb200.h"

namespace wb200 {

// ---------------------------------------------------------------- errors
void set_last_error(const std::string &message);
wb200_status fail(wb200_status status, const std::string &message);

#define WB200_CUDA_CHECK(expr)                                                              \
  do {                                                                                      \
    cudaError_t err__ = (expr);                                                             \
    if (err__ != cudaSuccess)                                                               \
      return ::wb200::fail(WB200_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(err__)); \
  } while (0)

// ---------------------------------------------------------------- formats
__host__ __device__ inline int format_bits(int format) {
  switch (format) {
    case WB200_I8: case WB200_U8: return 8;
    case WB200_I16: case WB200_U16: case WB200_F16: case WB200_BF16: return 16;
    case WB200_I32: case WB200_U32: case WB200_F32: case WB200_TF32: return 32;
    case WB200_I64: case WB200_U64: return 64;
    case WB200_BOOL: return 1;
    default: return 0;
  }
}
__host__ __device__ inline bool is_float_format(int format) {
  return format == WB200_F16 || format == WB200_BF16 || format == WB200_F32;
}

// Widening is exact for f16 / bf16 -> f32 (OneDNNGemmAdapter.cpp:42-92 of the reference does the
// same bit manipulation on the host).
__device__ __forceinline__ float widen_bits(uint32_t bits, int format) {
  if (format == WB200_F32) return __uint_as_float(bits);
  if (format == WB200_BF16) return __uint_as_float(bits << 16);
  return __half2float(__ushort_as_half(static_cast<unsigned short>(bits)));
}
// Round-to-nearest-even narrowing. NaN becomes the canonical positive quiet NaN of the destination
// (0x7fc00000 / 0x7e00 / 0x7fc0), as the reference's formal finalize does
// (lib/Wafer/Simulator/Reference/Formal/FormalNumericGemm.cpp:131-139).
__device__ __forceinline__ uint32_t narrow_bits(float value, int format) {
  if (format == WB200_F32) return (value != value) ? 0x7fc00000u : __float_as_uint(value);
  if (format == WB200_BF16) {
    if (value != value) return 0x7fc0u;
    return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(value)));
  }
  if (value != value) return 0x7e00u;
  return static_cast<uint32_t>(__half_as_ushort(__float2half_rn(value)));
}

__device__ __forceinline__ uint32_t load_element_bits(const uint8_t *base, int64_t index, int format) {
  if (format == WB200_F32) return reinterpret_cast<const uint32_t *>(base)[index];
  return reinterpret_cast<const uint16_t *>(base)[index];
}
__device__ __forceinline__ void store_element_bits(uint8_t *base, int64_t index, int format,
                                                   uint32_t bits) {
  if (format == WB200_F32)
    reinterpret_cast<uint32_t *>(base)[index] = bits;
  else
    reinterpret_cast<uint16_t *>(base)[index] = static_cast<uint16_t>(bits);
}

// ---------------------------------------------------------------- physical layout
// Plain-data form of the reference's PhysicalTensorGeometry + offset calculator
// (lib/Wafer/Target/PhysicalTensor/PhysicalLayout.cpp:111-310), usable on host and device.
struct LayoutMap {
  int layout;                   // wb200_layout
  int rank;
  int64_t shape[WB200_MAX_RANK];
  int64_t c_block;              // 64 (128 for 8-bit integers)
  int64_t cx_blocks;            // full channel blocks after the tail decision
  int64_t c0;                   // kept tail width (0 when none)
  int64_t block_outer_elements; // product of the dims between the leading slice and C
  int64_t outer_slice_stride;   // physical elements between NCx leading slices
  int64_t physical_elements;
  int64_t element_count;
};

// Physical element index of compact row-major element `linear`.
__host__ __device__ inline int64_t physical_index(const LayoutMap &map, int64_t linear) {
  if (map.layout == WB200_LAYOUT_TENSOR || map.layout == WB200_LAYOUT_NTENSOR) return linear;
  const int64_t channels = map.shape[map.rank - 1];
  const int64_t c = linear % channels;
  int64_t outer = linear / channels;  // row-major index over all non-channel dims
  int64_t base = 0;
  if (map.layout == WB200_LAYOUT_NCX && map.rank > 1) {
    const int64_t slice = outer / map.block_outer_elements;
    outer = outer % map.block_outer_elements;
    base = slice * map.outer_slice_stride;
  }
  const int64_t full_c = map.cx_blocks * map.c_block;
  if (c < full_c)
    return base + (c / map.c_block) * (map.block_outer_elements * map.c_block) + outer * map.c_block +
           c % map.c_block;
  return base + map.cx_blocks * map.block_outer_elements * map.c_block + outer * map.c0 + (c - full_c);
}

wb200_status make_layout_map(const wb200_tensor_desc &desc, LayoutMap *map, wb200_geometry *geometry);

}  // namespace wb200
