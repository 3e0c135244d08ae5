// Movement commands of the TargetCall ABI on device-resident memory images: strided DMA (DDR <-> scratch-pad),
// gather / scatter inside a scratch-pad, element fill. A strided byte layout is {inner_bytes, strides[3],
// iterations[3]}; its segments are enumerated with dimension 0 fastest and the payload is their concatenation
// (lib/Wafer/Simulator/Memory/TargetModelStridedMemory.cpp:121-152). A copy pairs payload byte p of the source
// layout with payload byte p of the destination layout (lib/Wafer/Simulator/Kernel/TargetModelMovement.cpp:52-146).
// HBM-bound byte work: algorithmic bytes = payload read once + written once.
#include "kernels.h"

namespace wb200 {
namespace {

template <typename Unit>
__global__ void __launch_bounds__(256) strided_copy_kernel(const uint8_t *src, uint8_t *dst, StridedLayout from, StridedLayout to,
                                                            uint32_t units_per_segment, uint64_t total_units) {
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  for (uint64_t u = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; u < total_units; u += stride) {
    // a command moves at most 4 GiB, so 32-bit division is enough (64-bit division is several times slower)
    const uint32_t unit = static_cast<uint32_t>(u);
    const uint32_t segment = unit / units_per_segment;
    const uint64_t within = static_cast<uint64_t>(unit - segment * units_per_segment) * sizeof(Unit);
    uint32_t s = segment, t = segment;
    uint64_t from_offset = within, to_offset = within;
#pragma unroll
    for (int d = 0; d < 3; ++d) {
      const uint32_t s_next = s / from.iterations[d], t_next = t / to.iterations[d];
      from_offset += static_cast<uint64_t>(s - s_next * from.iterations[d]) * from.strides[d];
      to_offset += static_cast<uint64_t>(t - t_next * to.iterations[d]) * to.strides[d];
      s = s_next;
      t = t_next;
    }
    *reinterpret_cast<Unit *>(dst + to_offset) = *reinterpret_cast<const Unit *>(src + from_offset);
  }
}

template <typename Element>
__global__ void __launch_bounds__(256) fill_kernel(Element *dst, Element value, uint64_t count) {
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) dst[i] = value;
}

// wafer_tx81_bit2fp (lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:198-236): bit i of the packed Bool source
// (least significant bit first) becomes 1.0 or +0 of the destination format.
template <typename T>
__global__ void __launch_bounds__(256) bit2fp_kernel(const uint8_t *src, T *dst, uint32_t count, T one) {
  const uint32_t stride = gridDim.x * blockDim.x;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) dst[i] = ((src[i >> 3] >> (i & 7)) & 1u) ? one : static_cast<T>(0);
}

// wafer_tx81_mask_move (:238-286): destination elements whose mask element is exactly 1.0 take the source element, a
// zero mask keeps them; any other mask value refuses the command. `store` = 0 only validates; the smallest refused
// element is reported as (element << 8 | 4).
template <typename T>
__global__ void __launch_bounds__(256) mask_move_kernel(const T *src, const T *mask, T *dst, uint32_t count, T one, int store,
                                                        unsigned long long *first_refused) {
  const uint32_t stride = gridDim.x * blockDim.x;
  unsigned long long refused = ~0ull;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
    const T predicate = mask[i];
    if (predicate == one) {
      if (store) dst[i] = src[i];
    } else if (predicate != 0) {
      const unsigned long long key = (static_cast<unsigned long long>(i) << 8) | 4ull;
      refused = key < refused ? key : refused;
    }
  }
  if (refused != ~0ull) atomicMin(first_refused, refused);
}

int grid_for(uint64_t items) {
  uint64_t blocks = (items + 255) / 256;
  if (blocks > 148u * 8u) blocks = 148u * 8u;
  return blocks == 0 ? 1 : static_cast<int>(blocks);
}

bool layout_aligned(const StridedLayout &layout, uint32_t unit) {
  if (layout.inner_bytes % unit) return false;
  for (int d = 0; d < 3; ++d)
    if (layout.iterations[d] > 1 && layout.strides[d] % unit) return false;
  return true;
}

}  // namespace

uint64_t strided_segments(const StridedLayout &layout) {
  return static_cast<uint64_t>(layout.iterations[0]) * layout.iterations[1] * layout.iterations[2];
}

uint64_t strided_span(const StridedLayout &layout) {
  uint64_t span = layout.inner_bytes;
  for (int d = 0; d < 3; ++d)
    if (layout.iterations[d] > 1) span += static_cast<uint64_t>(layout.iterations[d] - 1) * layout.strides[d];
  return span;
}

wb200_status launch_strided_copy(const uint8_t *src, const StridedLayout &from, uint8_t *dst, const StridedLayout &to,
                                 cudaStream_t stream) {
  if (from.inner_bytes == 0 || from.inner_bytes != to.inner_bytes)
    return fail(WB200_ERR_INVALID_ARGUMENT, "strided copy needs equal, non-zero inner byte counts");
  for (int d = 0; d < 3; ++d)
    if (from.iterations[d] == 0 || to.iterations[d] == 0) return fail(WB200_ERR_INVALID_ARGUMENT, "strided copy iteration counts must be positive");
  const uint64_t segments = strided_segments(from);
  if (segments != strided_segments(to)) return fail(WB200_ERR_INVALID_ARGUMENT, "source and destination segment counts differ");
  const uint64_t bytes = segments * from.inner_bytes;
  const uintptr_t bases = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst);
  if (bases % 16 == 0 && layout_aligned(from, 16) && layout_aligned(to, 16)) {
    strided_copy_kernel<uint4><<<grid_for(bytes / 16), 256, 0, stream>>>(src, dst, from, to, from.inner_bytes / 16, bytes / 16);
  } else if (bases % 4 == 0 && layout_aligned(from, 4) && layout_aligned(to, 4)) {
    strided_copy_kernel<uint32_t><<<grid_for(bytes / 4), 256, 0, stream>>>(src, dst, from, to, from.inner_bytes / 4, bytes / 4);
  } else {
    strided_copy_kernel<uint8_t><<<grid_for(bytes), 256, 0, stream>>>(src, dst, from, to, from.inner_bytes, bytes);
  }
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

wb200_status launch_fill(uint8_t *dst, uint32_t value_bits, uint64_t count, int element_bytes, cudaStream_t stream) {
  if (count == 0) return WB200_OK;
  if (reinterpret_cast<uintptr_t>(dst) % element_bytes) return fail(WB200_ERR_INVALID_ARGUMENT, "fill destination is not element aligned");
  switch (element_bytes) {
    case 1: fill_kernel<uint8_t><<<grid_for(count), 256, 0, stream>>>(dst, static_cast<uint8_t>(value_bits), count); break;
    case 2: fill_kernel<uint16_t><<<grid_for(count), 256, 0, stream>>>(reinterpret_cast<uint16_t *>(dst), static_cast<uint16_t>(value_bits), count); break;
    case 4: fill_kernel<uint32_t><<<grid_for(count), 256, 0, stream>>>(reinterpret_cast<uint32_t *>(dst), value_bits, count); break;
    default: return fail(WB200_ERR_UNSUPPORTED, "fill takes 1, 2 or 4 byte elements");
  }
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

wb200_status launch_bit2fp(const uint8_t *src, uint8_t *dst, uint32_t count, int format, cudaStream_t stream) {
  if (count == 0) return WB200_OK;
  const int grid = grid_for(count);
  if (format == WB200_F32) bit2fp_kernel<uint32_t><<<grid, 256, 0, stream>>>(src, reinterpret_cast<uint32_t *>(dst), count, 0x3f800000u);
  else if (format == WB200_BF16) bit2fp_kernel<uint16_t><<<grid, 256, 0, stream>>>(src, reinterpret_cast<uint16_t *>(dst), count, static_cast<uint16_t>(0x3f80));
  else if (format == WB200_F16) bit2fp_kernel<uint16_t><<<grid, 256, 0, stream>>>(src, reinterpret_cast<uint16_t *>(dst), count, static_cast<uint16_t>(0x3c00));
  else return fail(WB200_ERR_UNSUPPORTED, "Bit2FP requires F16, BF16 or F32 output");
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

wb200_status launch_mask_move(const uint8_t *src, const uint8_t *mask, uint8_t *dst, uint32_t count, int format, int store,
                              unsigned long long *first_refused, cudaStream_t stream) {
  if (count == 0) return WB200_OK;
  const int grid = grid_for(count);
  if (format == WB200_F32)
    mask_move_kernel<uint32_t><<<grid, 256, 0, stream>>>(reinterpret_cast<const uint32_t *>(src), reinterpret_cast<const uint32_t *>(mask),
                                                         reinterpret_cast<uint32_t *>(dst), count, 0x3f800000u, store, first_refused);
  else if (format == WB200_BF16 || format == WB200_F16)
    mask_move_kernel<uint16_t><<<grid, 256, 0, stream>>>(reinterpret_cast<const uint16_t *>(src), reinterpret_cast<const uint16_t *>(mask),
                                                         reinterpret_cast<uint16_t *>(dst), count,
                                                         static_cast<uint16_t>(format == WB200_BF16 ? 0x3f80 : 0x3c00), store, first_refused);
  else return fail(WB200_ERR_UNSUPPORTED, "MaskMove requires F16, BF16 or F32");
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

}  // namespace wb200
