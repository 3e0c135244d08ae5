// Managed-reference tensor commands on the device: elementwise, convert, reduce, and the physical
// tensor codec. Semantics follow lib/Wafer/Simulator/Reference/ManagedReferenceTargetModel.cpp:
// decode every operand to f32 (:137-155), apply one f32 operation (:230-299), encode with
// round-to-nearest-even (:157-185); NaN inputs or results are reported, not produced. Arithmetic
// uses the explicitly rounded intrinsics so the compiler cannot contract or reassociate.
#include "kernels.h"

namespace wb200 {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float apply_elementwise(int op, float x, float y) {
  switch (op) {
    case WB200_EW_ABS: return fabsf(x);
    case WB200_EW_NEG: return -x;
    case WB200_EW_RECIP: return __fdiv_rn(1.0f, x);
    case WB200_EW_SQUARE: return __fmul_rn(x, x);
    case WB200_EW_MAX: return fmaxf(x, y);
    case WB200_EW_MIN: return fminf(x, y);
    case WB200_EW_ADD: return __fadd_rn(x, y);
    case WB200_EW_SUB: return __fsub_rn(x, y);
    case WB200_EW_MUL: return __fmul_rn(x, y);
    case WB200_EW_RELU: return x < 0.0f ? 0.0f : x;
    case WB200_EW_SQRT: return __fsqrt_rn(x);
    case WB200_EW_RSQRT: return __fdiv_rn(1.0f, __fsqrt_rn(x));
    case WB200_EW_LOG2: return log2f(x);
    case WB200_EW_LN: return logf(x);
    case WB200_EW_POW2: return exp2f(x);
    case WB200_EW_EXP: return expf(x);
    case WB200_EW_EXPLP: return exp2f(__fmul_rn(x, 0x1.715476p+0f));
    case WB200_EW_SIN: return sinf(x);
    case WB200_EW_COS: return cosf(x);
    case WB200_EW_TANH: return tanhf(x);
    case WB200_EW_SIGMOID:
      if (x >= 0.0f) return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x)));
      return __fdiv_rn(expf(x), __fadd_rn(1.0f, expf(x)));
    case WB200_EW_SOFTPLUS: return __fadd_rn(fmaxf(x, 0.0f), log1pf(expf(-fabsf(x))));
    default: return x;
  }
}

__global__ void __launch_bounds__(kThreads)
elementwise_kernel(int op, int format, int input_count, const uint8_t *in0, const uint8_t *in1, uint8_t *dst,
                   const LayoutMap map, int *nan_flag) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  bool saw_nan = false;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < map.element_count; i += stride) {
    const int64_t phys = physical_index(map, i);
    const float x = widen_bits(load_element_bits(in0, phys, format), format);
    const float y = input_count > 1 ? widen_bits(load_element_bits(in1, phys, format), format) : 0.0f;
    const float result = apply_elementwise(op, x, y);
    saw_nan |= (x != x) | (y != y) | (result != result);
    store_element_bits(dst, phys, format, narrow_bits(result, format));
  }
  if (saw_nan) atomicExch(nan_flag, 1);
}

__global__ void __launch_bounds__(kThreads)
convert_kernel(int src_format, int dst_format, const uint8_t *src, uint8_t *dst, const LayoutMap src_map,
               const LayoutMap dst_map, int *nan_flag) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  bool saw_nan = false;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < src_map.element_count; i += stride) {
    const float x = widen_bits(load_element_bits(src, physical_index(src_map, i), src_format), src_format);
    saw_nan |= (x != x);
    store_element_bits(dst, physical_index(dst_map, i), dst_format, narrow_bits(x, dst_format));
  }
  if (saw_nan) atomicExch(nan_flag, 1);
}

// One thread per output element; the reduced coordinates are visited in row-major input order, which
// is the order the reference's running accumulator sees them (:412-447).
__global__ void __launch_bounds__(kThreads)
reduce_kernel(int op, int format, const uint8_t *src, uint8_t *dst, const LayoutMap src_map,
              const LayoutMap dst_map, uint32_t reduced_mask, int *nan_flag) {
  const int64_t out_index = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (out_index >= dst_map.element_count) return;
  const int rank = src_map.rank;
  int64_t coord[WB200_MAX_RANK];
  int64_t stride[WB200_MAX_RANK];
  {
    int64_t s = 1;
    for (int d = rank - 1; d >= 0; --d) { stride[d] = s; s *= src_map.shape[d]; }
    int64_t remaining = out_index;
    for (int d = rank - 1; d >= 0; --d) {
      if (reduced_mask & (1u << d)) { coord[d] = 0; continue; }
      coord[d] = remaining % src_map.shape[d];
      remaining /= src_map.shape[d];
    }
  }
  int64_t reduced_count = 1;
  for (int d = 0; d < rank; ++d)
    if (reduced_mask & (1u << d)) reduced_count *= src_map.shape[d];
  float acc = op == WB200_RED_MAX ? -INFINITY : (op == WB200_RED_MIN ? INFINITY : 0.0f);
  bool saw_nan = false;
  for (int64_t r = 0; r < reduced_count; ++r) {
    int64_t remaining = r;
    for (int d = rank - 1; d >= 0; --d) {
      if (!(reduced_mask & (1u << d))) continue;
      coord[d] = remaining % src_map.shape[d];
      remaining /= src_map.shape[d];
    }
    int64_t linear = 0;
    for (int d = 0; d < rank; ++d) linear += coord[d] * stride[d];
    const float value = widen_bits(load_element_bits(src, physical_index(src_map, linear), format), format);
    saw_nan |= (value != value);
    if (op == WB200_RED_SUM) {
      acc = __fadd_rn(acc, value);
    } else if (acc == 0.0f && value == 0.0f) {
      const bool negative = op == WB200_RED_MAX ? (signbit(acc) && signbit(value)) : (signbit(acc) || signbit(value));
      acc = negative ? -0.0f : 0.0f;
    } else {
      acc = op == WB200_RED_MAX ? fmaxf(acc, value) : fminf(acc, value);
    }
    saw_nan |= (acc != acc);
  }
  store_element_bits(dst, physical_index(dst_map, out_index), format, narrow_bits(acc, format));
  if (saw_nan) atomicExch(nan_flag, 1);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
codec_kernel(const T *src, T *dst, const LayoutMap map, int pack) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < map.element_count; i += stride) {
    const int64_t phys = physical_index(map, i);
    if (pack) dst[phys] = src[i];
    else dst[i] = src[phys];
  }
}

int grid_for(int64_t elements) {
  int64_t blocks = (elements + kThreads - 1) / kThreads;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return static_cast<int>(blocks);
}

wb200_status launch_codec(const uint8_t *src, uint8_t *dst, const LayoutMap &map, int element_bytes, int pack,
                          cudaStream_t stream) {
  const int grid = grid_for(map.element_count);
  switch (element_bytes) {
    case 1: codec_kernel<uint8_t><<<grid, kThreads, 0, stream>>>(src, dst, map, pack); break;
    case 2: codec_kernel<uint16_t><<<grid, kThreads, 0, stream>>>(reinterpret_cast<const uint16_t *>(src), reinterpret_cast<uint16_t *>(dst), map, pack); break;
    case 4: codec_kernel<uint32_t><<<grid, kThreads, 0, stream>>>(reinterpret_cast<const uint32_t *>(src), reinterpret_cast<uint32_t *>(dst), map, pack); break;
    case 8: codec_kernel<uint64_t><<<grid, kThreads, 0, stream>>>(reinterpret_cast<const uint64_t *>(src), reinterpret_cast<uint64_t *>(dst), map, pack); break;
    default: return fail(WB200_ERR_UNSUPPORTED, "codec supports byte-addressable element types only");
  }
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

}  // namespace

wb200_status launch_elementwise(int op, int format, int input_count, const uint8_t *in0, const uint8_t *in1,
                                uint8_t *dst, const LayoutMap &map, int *nan_flag, cudaStream_t stream) {
  elementwise_kernel<<<grid_for(map.element_count), kThreads, 0, stream>>>(op, format, input_count, in0, in1, dst, map, nan_flag);
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

wb200_status launch_convert(int src_format, int dst_format, const uint8_t *src, uint8_t *dst,
                            const LayoutMap &src_map, const LayoutMap &dst_map, int *nan_flag, cudaStream_t stream) {
  convert_kernel<<<grid_for(src_map.element_count), kThreads, 0, stream>>>(src_format, dst_format, src, dst, src_map, dst_map, nan_flag);
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

wb200_status launch_reduce(int op, int format, const uint8_t *src, uint8_t *dst, const LayoutMap &src_map,
                           const LayoutMap &dst_map, uint32_t reduced_mask, int *nan_flag, cudaStream_t stream) {
  const int64_t blocks = (dst_map.element_count + kThreads - 1) / kThreads;
  reduce_kernel<<<static_cast<int>(blocks < 1 ? 1 : blocks), kThreads, 0, stream>>>(op, format, src, dst, src_map, dst_map, reduced_mask, nan_flag);
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

wb200_status launch_unpack(const uint8_t *storage, uint8_t *compact, const LayoutMap &map, int element_bytes, cudaStream_t stream) {
  return launch_codec(storage, compact, map, element_bytes, 0, stream);
}
wb200_status launch_pack(const uint8_t *compact, uint8_t *storage, const LayoutMap &map, int element_bytes, cudaStream_t stream) {
  return launch_codec(compact, storage, map, element_bytes, 1, stream);
}

}  // namespace wb200
