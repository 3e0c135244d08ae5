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
  if (format == WB200_F32 || format == WB200_TF32) return reinterpret_cast<const uint32_t *>(base)[index];
  return reinterpret_cast<const uint16_t *>(base)[index];
}
__device__ __forceinline__ void store_element_bits(uint8_t *base, int64_t index, int format,
                                                   uint32_t bits) {
  if (format == WB200_F32 || format == WB200_TF32)
    reinterpret_cast<uint32_t *>(base)[index] = bits;
  else
    reinterpret_cast<uint16_t *>(base)[index] = static_cast<uint16_t>(bits);
}

// Eight consecutive elements of `bytes` bytes each, starting at element 8 * group of a 16-byte aligned base, moved
// with 128-bit accesses (two for 4-byte elements, one for 2-byte elements, a 64-bit one for bytes).
__device__ __forceinline__ void load_group8(const uint8_t *base, int64_t group, int bytes, uint32_t (&v)[8]) {
  if (bytes == 4) {
    const uint4 lo = reinterpret_cast<const uint4 *>(base)[2 * group], hi = reinterpret_cast<const uint4 *>(base)[2 * group + 1];
    v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
  } else if (bytes == 2) {
    const uint4 w = reinterpret_cast<const uint4 *>(base)[group];
    v[0] = w.x & 0xffffu; v[1] = w.x >> 16; v[2] = w.y & 0xffffu; v[3] = w.y >> 16;
    v[4] = w.z & 0xffffu; v[5] = w.z >> 16; v[6] = w.w & 0xffffu; v[7] = w.w >> 16;
  } else {
    const uint2 w = reinterpret_cast<const uint2 *>(base)[group];
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[i] = (w.x >> (8 * i)) & 0xffu; v[4 + i] = (w.y >> (8 * i)) & 0xffu; }
  }
}
__device__ __forceinline__ void store_group8(uint8_t *base, int64_t group, int bytes, const uint32_t (&v)[8]) {
  if (bytes == 4) {
    reinterpret_cast<uint4 *>(base)[2 * group] = make_uint4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<uint4 *>(base)[2 * group + 1] = make_uint4(v[4], v[5], v[6], v[7]);
  } else if (bytes == 2) {
    reinterpret_cast<uint4 *>(base)[group] = make_uint4((v[0] & 0xffffu) | (v[1] << 16), (v[2] & 0xffffu) | (v[3] << 16),
                                                        (v[4] & 0xffffu) | (v[5] << 16), (v[6] & 0xffffu) | (v[7] << 16));
  } else {
    uint2 w = make_uint2(0u, 0u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { w.x |= (v[i] & 0xffu) << (8 * i); w.y |= (v[4 + i] & 0xffu) << (8 * i); }
    reinterpret_cast<uint2 *>(base)[group] = w;
  }
}
// True when every pointer is 16-byte aligned (null pointers count as aligned).
inline bool all_aligned16(const void *a, const void *b = nullptr, const void *c = nullptr) {
  return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15) == 0;
}

// ORs every thread's `flags` into *word with one global atomic per block (a single hot word would otherwise serialise
// one atomic per thread). Every thread of the block must reach the call.
__device__ __forceinline__ void merge_block_flags(uint32_t *word, uint32_t flags) {
  __shared__ uint32_t block_flags;
  if (threadIdx.x == 0) block_flags = 0;
  __syncthreads();
  flags = __reduce_or_sync(0xffffffffu, flags);
  if ((threadIdx.x & 31) == 0 && flags) atomicOr(&block_flags, flags);
  __syncthreads();
  if (threadIdx.x == 0 && block_flags) atomicOr(word, block_flags);
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

// The same placement for a rank-4 NCx tensor [n, h, w, c] from its coordinates, without the divisions by the shape:
// `outer` = h * W + w. Agrees with physical_index(map, ((n * H + h) * W + w) * C + c).
__host__ __device__ inline int64_t physical_index_nhwc(const LayoutMap &map, int64_t n, int64_t outer, int64_t c) {
  const int64_t full_c = map.cx_blocks * map.c_block;
  const int64_t base = n * map.outer_slice_stride;
  if (c < full_c) {
    const uint32_t block = static_cast<uint32_t>(c) / static_cast<uint32_t>(map.c_block);   // channel counts fit 32 bits
    return base + block * (map.block_outer_elements * map.c_block) + outer * map.c_block + (c - block * map.c_block);
  }
  return base + map.cx_blocks * map.block_outer_elements * map.c_block + outer * map.c0 + (c - full_c);
}

wb200_status make_layout_map(const wb200_tensor_desc &desc, LayoutMap *map, wb200_geometry *geometry);

}  // namespace wb200
