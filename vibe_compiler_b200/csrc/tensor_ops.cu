// Managed-reference tensor commands on the device: elementwise, convert, reduce, and the physical
// tensor codec. Semantics follow lib/Wafer/Simulator/Reference/ManagedReferenceTargetModel.cpp:
// decode every operand to f32 (:137-155), apply one f32 operation (:230-299), encode with
// round-to-nearest-even (:157-185); NaN inputs or results are reported, not produced. Arithmetic
// uses the explicitly rounded intrinsics so the compiler cannot contract or reassociate.
#include "gemm_formal.cuh"
#include "kernels.h"
#include "formal_functions_f32.cuh"

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

// Linear (Tensor / NTensor) layouts with 16-byte aligned operands: eight elements per thread with 128-bit accesses,
// the operation and the format fixed at compile time.
template <int kOp, int kFormat>
__global__ void __launch_bounds__(kThreads)
elementwise_linear_kernel(int input_count, const uint8_t *in0, const uint8_t *in1, uint8_t *dst, int64_t total, int *nan_flag) {
  constexpr int bytes = kFormat == WB200_F32 ? 4 : 2;
  const int64_t groups = total / 8, stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  bool saw_nan = false;
  for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < groups; g += stride) {
    uint32_t a[8], b[8], r[8];
    load_group8(in0, g, bytes, a);
    if (input_count > 1) load_group8(in1, g, bytes, b);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float x = widen_bits(a[e], kFormat), y = input_count > 1 ? widen_bits(b[e], kFormat) : 0.0f;
      const float result = apply_elementwise(kOp, x, y);
      saw_nan |= (x != x) | (y != y) | (result != result);
      r[e] = narrow_bits(result, kFormat);
    }
    store_group8(dst, g, bytes, r);
  }
  if (blockIdx.x == 0 && threadIdx.x < total - groups * 8) {   // ragged tail
    const int64_t i = groups * 8 + threadIdx.x;
    const float x = widen_bits(load_element_bits(in0, i, kFormat), kFormat);
    const float y = input_count > 1 ? widen_bits(load_element_bits(in1, i, kFormat), kFormat) : 0.0f;
    const float result = apply_elementwise(kOp, x, y);
    saw_nan |= (x != x) | (y != y) | (result != result);
    store_element_bits(dst, i, kFormat, narrow_bits(result, kFormat));
  }
  if (saw_nan) atomicExch(nan_flag, 1);
}

template <int kSrc, int kDst>
__global__ void __launch_bounds__(kThreads)
convert_linear_kernel(const uint8_t *src, uint8_t *dst, int64_t total, int *nan_flag) {
  constexpr int src_bytes = kSrc == WB200_F32 ? 4 : 2, dst_bytes = kDst == WB200_F32 ? 4 : 2;
  const int64_t groups = total / 8, stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  bool saw_nan = false;
  for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < groups; g += stride) {
    uint32_t a[8], r[8];
    load_group8(src, g, src_bytes, a);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float x = widen_bits(a[e], kSrc);
      saw_nan |= (x != x);
      r[e] = narrow_bits(x, kDst);
    }
    store_group8(dst, g, dst_bytes, r);
  }
  if (blockIdx.x == 0 && threadIdx.x < total - groups * 8) {
    const int64_t i = groups * 8 + threadIdx.x;
    const float x = widen_bits(load_element_bits(src, i, kSrc), kSrc);
    saw_nan |= (x != x);
    store_element_bits(dst, i, kDst, narrow_bits(x, kDst));
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

// The same reduction for rank-4 NCx tensors [n, h, w, c] (every TargetCall-level reduce): the output index is split
// once with 32-bit divisions, and while the channel is kept the fold walks constant strides along n, h and w.
template <int kOp, int kFormat>
__global__ void __launch_bounds__(kThreads)
reduce_nhwc_kernel(const uint8_t *src, uint8_t *dst, const LayoutMap src_map, const LayoutMap dst_map, uint32_t reduced_mask, int *nan_flag) {
  const int64_t out_index = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (out_index >= dst_map.element_count) return;
  const uint32_t out_c = static_cast<uint32_t>(dst_map.shape[3]), out_w = static_cast<uint32_t>(dst_map.shape[2]), out_h = static_cast<uint32_t>(dst_map.shape[1]);
  const uint32_t index = static_cast<uint32_t>(out_index);
  const uint32_t pixel = index / out_c, c0 = index - pixel * out_c;
  const uint32_t row = pixel / out_w, w0 = pixel - row * out_w;
  const uint32_t n0 = row / out_h, h0 = row - n0 * out_h;
  const uint32_t n_count = (reduced_mask & 1u) ? static_cast<uint32_t>(src_map.shape[0]) : 1u, h_count = (reduced_mask & 2u) ? static_cast<uint32_t>(src_map.shape[1]) : 1u;
  const uint32_t w_count = (reduced_mask & 4u) ? static_cast<uint32_t>(src_map.shape[2]) : 1u, c_count = (reduced_mask & 8u) ? static_cast<uint32_t>(src_map.shape[3]) : 1u;
  const uint32_t in_w = static_cast<uint32_t>(src_map.shape[2]);
  float acc = kOp == WB200_RED_MAX ? -INFINITY : (kOp == WB200_RED_MIN ? INFINITY : 0.0f);
  bool saw_nan = false;
  auto step = [&](float value) {
    saw_nan |= (value != value);
    if (kOp == WB200_RED_SUM) {
      acc = __fadd_rn(acc, value);
    } else if (acc == 0.0f && value == 0.0f) {
      const bool negative = kOp == WB200_RED_MAX ? (signbit(acc) && signbit(value)) : (signbit(acc) || signbit(value));
      acc = negative ? -0.0f : 0.0f;
    } else {
      acc = kOp == WB200_RED_MAX ? fmaxf(acc, value) : fminf(acc, value);
    }
    saw_nan |= (acc != acc);
  };
  if (!(reduced_mask & 8u)) {
    const int64_t full_c = src_map.cx_blocks * src_map.c_block;
    const int64_t width = static_cast<int64_t>(c0) < full_c ? src_map.c_block : src_map.c0;
    const int64_t stride_h = width * in_w, stride_n = src_map.outer_slice_stride;
    const int64_t base = physical_index_nhwc(src_map, (reduced_mask & 1u) ? 0 : n0,
                                             static_cast<int64_t>((reduced_mask & 2u) ? 0u : h0) * in_w + ((reduced_mask & 4u) ? 0u : w0), c0);
    for (uint32_t n = 0; n < n_count; ++n)
      for (uint32_t h = 0; h < h_count; ++h) {
        const int64_t line = base + n * stride_n + h * stride_h;
#pragma unroll 8
        for (uint32_t w = 0; w < w_count; ++w) step(widen_bits(load_element_bits(src, line + w * width, kFormat), kFormat));
      }
  } else {
    for (uint32_t n = 0; n < n_count; ++n)
      for (uint32_t h = 0; h < h_count; ++h)
        for (uint32_t w = 0; w < w_count; ++w)
          for (uint32_t c = 0; c < c_count; ++c) {
            const int64_t in_n = (reduced_mask & 1u) ? n : n0;
            const uint32_t in_h = (reduced_mask & 2u) ? h : h0, in_wi = (reduced_mask & 4u) ? w : w0;
            step(widen_bits(load_element_bits(src, physical_index_nhwc(src_map, in_n, static_cast<int64_t>(in_h) * in_w + in_wi, c), kFormat), kFormat));
          }
  }
  store_element_bits(dst, physical_index_nhwc(dst_map, n0, static_cast<int64_t>(h0) * out_w + w0, c0), kFormat, narrow_bits(acc, kFormat));
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

// ------------------------------------------------------------------------------------------------ formal elementwise
// Bit-exact evaluation of the reference's formal elementwise family
// (lib/Wafer/Simulator/Reference/Formal/FormalNumericElementwise.cpp:23-248): arithmetic in the operand format with
// one RNE rounding, NaN results canonicalised (not rejected), relations to Bool or to 1.0 / 0.0, logic on "bits != 0",
// and the IEEE exception flags. Arithmetic runs in f32 and is narrowed once: for f16 / bf16 the double rounding is
// innocuous (24 >= 2 * 11 + 2), for f32 the hardware operation is the RNE operation. Inexactness comes from
// error-free transformations, not from a wider re-computation.
constexpr uint32_t kFlagInvalid = 1u, kFlagDivByZero = 2u, kFlagOverflow = 4u, kFlagUnderflow = 8u, kFlagInexact = 16u;

struct FormatTraits { uint32_t sign, exp_mask, mant_mask, quiet_bit, canonical_nan, one; int precision; float min_normal; };
// Folds (reduce, pooling): their chained f32 add steps take the early-return path too. Measured on 2^27 elements: NCx sum
// over w 0.418 ms with it, 0.458 ms without; 2x2 sum pooling 0.254 ms against 0.338 ms.
constexpr bool kFoldCommonCase = true;
__device__ __forceinline__ FormatTraits traits_of(int format) {
  if (format == WB200_F32) return {0x80000000u, 0x7f800000u, 0x007fffffu, 0x00400000u, 0x7fc00000u, 0x3f800000u, 24, 1.17549435e-38f};
  if (format == WB200_BF16) return {0x8000u, 0x7f80u, 0x007fu, 0x0040u, 0x7fc0u, 0x3f80u, 8, 1.17549435e-38f};
  return {0x8000u, 0x7c00u, 0x03ffu, 0x0200u, 0x7e00u, 0x3c00u, 11, 6.10351562e-05f};
}

// |value| rounded to `precision` bits with an unbounded exponent range is below the smallest normal number.
__device__ __forceinline__ bool tiny_after_rounding(double value, int precision, float min_normal) {
  if (value == 0.0) return false;
  int exponent;
  const double mantissa = frexp(fabs(value), &exponent);                 // [0.5, 1)
  const double rounded = ldexp(rint(ldexp(mantissa, precision)), exponent - precision);
  return rounded < static_cast<double>(min_normal);
}

// `common_case` false leaves out the early-return path of f32 add / sub / mul / square (see kFoldCommonCase).
__device__ __forceinline__ uint32_t formal_scalar(int op, int format, int out_format, uint32_t a, uint32_t b, uint32_t *flags_out,
                                                  bool common_case = true) {
  if (common_case && format == WB200_F32 && out_format == WB200_F32 && (op == WB200_EW_ADD || op == WB200_EW_SUB || op == WB200_EW_MUL || op == WB200_EW_SQUARE)) {
    // The common f32 case first: finite operands and a finite result that cannot be tiny. The arithmetic is the general
    // path's (same sum / product, same error-free residual), with its NaN, infinity, narrowing and underflow decisions
    // known in advance: a finite sum that is subnormal or zero is exact, and a product of at least 2^-100 is normal and
    // has a residual that one fused multiply-add yields exactly.
    const uint32_t second = op == WB200_EW_SQUARE ? a : b;
    if ((a & 0x7f800000u) != 0x7f800000u && (second & 0x7f800000u) != 0x7f800000u) {
      const float x = __uint_as_float(a);
      float r, residual;
      bool decided;
      if (op == WB200_EW_MUL || op == WB200_EW_SQUARE) {
        const float y = __uint_as_float(second);
        r = __fmul_rn(x, y);
        residual = __fmaf_rn(x, y, -r);
        decided = fabsf(r) >= 7.8886090522101181e-31f;
      } else {
        const float y = op == WB200_EW_SUB ? -__uint_as_float(second) : __uint_as_float(second);
        r = __fadd_rn(x, y);
        const float part = __fsub_rn(r, x);
        residual = __fadd_rn(__fsub_rn(x, __fsub_rn(r, part)), __fsub_rn(y, part));
        decided = true;
      }
      if (decided && fabsf(r) < __uint_as_float(0x7f800000u)) {
        *flags_out = residual != 0.f ? kFlagInexact : 0u;
        return __float_as_uint(r);
      }
    }
  }
  const FormatTraits t = traits_of(format);
  if (common_case && (format == WB200_F16 || format == WB200_BF16) && out_format == format &&
      (op == WB200_EW_ADD || op == WB200_EW_SUB || op == WB200_EW_MUL || op == WB200_EW_SQUARE)) {
    // The 16-bit common case: finite operands and a normal result. Same f32 sum / product, residual and single narrowing
    // as the general path. A small sum of two 16-bit values is exact, so only a product can be tiny after rounding, and
    // one of at least twice the smallest normal number (and at least 2^-100, for the exact residual) is not.
    const uint32_t second = op == WB200_EW_SQUARE ? a : b;
    if ((a & t.exp_mask) != t.exp_mask && (second & t.exp_mask) != t.exp_mask) {
      const float x = widen_bits(a, format);
      float r, residual;
      bool decided;
      if (op == WB200_EW_MUL || op == WB200_EW_SQUARE) {
        const float y = widen_bits(second, format);
        r = __fmul_rn(x, y);
        residual = __fmaf_rn(x, y, -r);
        decided = fabsf(r) >= 7.8886090522101181e-31f && fabsf(r) >= 2.0f * t.min_normal;
      } else {
        const float y = op == WB200_EW_SUB ? -widen_bits(second, format) : widen_bits(second, format);
        r = __fadd_rn(x, y);
        const float part = __fsub_rn(r, x);
        residual = __fadd_rn(__fsub_rn(x, __fsub_rn(r, part)), __fsub_rn(y, part));
        decided = true;
      }
      const uint32_t narrowed = narrow_bits(r, format);   // r is not a NaN: the operands are finite
      const uint32_t exponent = narrowed & t.exp_mask;
      if (decided && exponent != 0 && exponent != t.exp_mask) {
        *flags_out = (residual != 0.f || widen_bits(narrowed, format) != r) ? kFlagInexact : 0u;
        return narrowed;
      }
    }
  }
  if (op == WB200_EW_MAX || op == WB200_EW_MIN) {
    // Maximum / minimum as straight-line selects (no branch, so a fold's independent loads stay ahead of its chain):
    // a NaN operand gives the canonical NaN (invalid when it signals), two zeros give -0 only when the sign rule says
    // so, otherwise the operand the comparison picks. No rounding.
    const uint32_t magnitude_a = a & ~t.sign, magnitude_b = b & ~t.sign;
    const bool nan_a = magnitude_a > t.exp_mask, nan_b = magnitude_b > t.exp_mask;
    const bool signalling = (nan_a && !(a & t.quiet_bit)) || (nan_b && !(b & t.quiet_bit));
    const float x = widen_bits(a, format), y = widen_bits(b, format);
    const uint32_t picked = (op == WB200_EW_MAX ? x < y : x > y) ? b : a;
    const uint32_t zero = (op == WB200_EW_MAX ? (a & b) : (a | b)) & t.sign;
    *flags_out = signalling ? kFlagInvalid : 0u;
    return (nan_a || nan_b) ? t.canonical_nan : ((magnitude_a | magnitude_b) == 0 ? zero : picked);
  }
  uint32_t flags = 0;
  const bool binary = !(op == WB200_EW_ABS || op == WB200_EW_NEG || op == WB200_EW_RECIP || op == WB200_EW_SQUARE || op == WB200_EW_RELU);
  auto is_nan = [&](uint32_t v) { return (v & t.exp_mask) == t.exp_mask && (v & t.mant_mask) != 0; };
  auto is_snan = [&](uint32_t v) { return is_nan(v) && (v & t.quiet_bit) == 0; };
  auto is_zero = [&](uint32_t v) { return (v & ~t.sign) == 0; };
  auto is_inf = [&](uint32_t v) { return (v & ~t.sign) == t.exp_mask; };
  const bool nan = is_nan(a) || (binary && is_nan(b));
  if (is_snan(a) || (binary && is_snan(b))) flags |= kFlagInvalid;
  const float x = widen_bits(a, format), y = binary ? widen_bits(b, format) : 0.f;
  uint32_t result;
  if (op >= WB200_EW_EQ && op <= WB200_EW_LT) {
    bool truth;
    if (nan) truth = op == WB200_EW_NE;
    else switch (op) {
      case WB200_EW_EQ: truth = x == y; break;
      case WB200_EW_NE: truth = x != y; break;
      case WB200_EW_GE: truth = x >= y; break;
      case WB200_EW_GT: truth = x > y; break;
      case WB200_EW_LE: truth = x <= y; break;
      default: truth = x < y; break;
    }
    *flags_out = flags;
    if (out_format == WB200_BOOL) return truth ? 1u : 0u;
    return truth ? traits_of(out_format).one : 0u;
  }
  if (nan && (op == WB200_EW_ABS || op == WB200_EW_NEG || op == WB200_EW_MAX || op == WB200_EW_MIN || op == WB200_EW_RELU)) {
    *flags_out = flags;
    return t.canonical_nan;
  }
  switch (op) {
    case WB200_EW_ABS: result = a & ~t.sign; break;
    case WB200_EW_NEG: result = a ^ t.sign; break;
    case WB200_EW_RELU: result = ((a & t.sign) && !is_zero(a)) ? 0u : a; break;
    case WB200_EW_MAX:
    case WB200_EW_MIN:
      if (is_zero(a) && is_zero(b)) {
        const bool negative = op == WB200_EW_MAX ? ((a & t.sign) && (b & t.sign)) : ((a & t.sign) || (b & t.sign));
        result = negative ? t.sign : 0u;
      } else {
        const bool choose_rhs = op == WB200_EW_MAX ? x < y : x > y;
        result = choose_rhs ? b : a;
      }
      break;
    default: {
      // recip, square, add, sub, mul: one RNE rounding in the operand format
      float r32;
      double small_product = 0.0;   // the exact product where it is small enough to be tiny after rounding
      bool maybe_tiny = false;
      bool inexact32 = false, finite_inputs = !is_inf(a) && !(binary && is_inf(b)) && !nan;
      if (op == WB200_EW_RECIP) {
        r32 = __fdiv_rn(1.0f, x);
        if (!nan && is_zero(a)) flags |= kFlagDivByZero;
        // 1 / x is representable only when x is a power of two
        if (finite_inputs && !is_zero(a)) inexact32 = (__float_as_uint(fabsf(x)) & 0x007fffffu) != 0 && (__float_as_uint(fabsf(x)) & 0x7f800000u) != 0;
        if (finite_inputs && !is_zero(a) && (__float_as_uint(fabsf(x)) & 0x7f800000u) == 0)   // subnormal f32 operand: power of two iff one bit set
          inexact32 = (__float_as_uint(fabsf(x)) & (__float_as_uint(fabsf(x)) - 1u)) != 0;
      } else if (op == WB200_EW_ADD || op == WB200_EW_SUB) {
        const float yy = op == WB200_EW_SUB ? -y : y;
        r32 = __fadd_rn(x, yy);
        if (finite_inputs && isfinite(r32)) {
          const float bb = __fsub_rn(r32, x);
          const float err = __fadd_rn(__fsub_rn(x, __fsub_rn(r32, bb)), __fsub_rn(yy, bb));
          inexact32 = err != 0.f;
        }
      } else {
        const float yy = op == WB200_EW_SQUARE ? x : y;
        r32 = __fmul_rn(x, yy);
        const float magnitude = fabsf(r32);
        if (magnitude >= 7.8886090522101181e-31f && magnitude >= 2.0f * t.min_normal) {
          // |r32| >= 2^-100: the residual x * yy - r32 is a multiple of 2^-149, so one fused multiply-add yields it
          // exactly; and a product of at least twice the smallest normal number is never tiny after rounding.
          if (finite_inputs) inexact32 = __fmaf_rn(x, yy, -r32) != 0.f;
        } else {
          if (finite_inputs) inexact32 = static_cast<double>(r32) != static_cast<double>(x) * static_cast<double>(yy);
          // only a product below twice the smallest normal number can still be tiny after rounding; whether it is also
          // inexact is known once the result is narrowed (a 16-bit product is exact in f32 and inexact only after that)
          small_product = static_cast<double>(x) * static_cast<double>(yy);
          maybe_tiny = finite_inputs && fabs(small_product) < 2.0 * static_cast<double>(t.min_normal);
        }
      }
      if (r32 != r32) {
        if (!nan) flags |= kFlagInvalid;   // inf - inf, 0 * inf
        result = t.canonical_nan;
        break;
      }
      result = narrow_bits(r32, format);
      const bool inexact = inexact32 || widen_bits(result, format) != r32;
      if (finite_inputs && !(flags & kFlagDivByZero)) {
        if (is_inf(result)) flags |= kFlagOverflow | kFlagInexact;
        else if (inexact) {
          flags |= kFlagInexact;
          if ((result & t.exp_mask) == 0) flags |= kFlagUnderflow;   // subnormal or zero after rounding, and inexact
          else if (maybe_tiny && tiny_after_rounding(small_product, t.precision, t.min_normal)) flags |= kFlagUnderflow;   // rounded up to the smallest normal
        }
      }
      break;
    }
  }
  *flags_out = flags;
  return result;
}

// Correctly rounded unary functions of the reference's MPFR family for the 16-bit formats
// (lib/Wafer/Simulator/Reference/Numeric/MPFRNumeric.cpp:560-682: the function evaluated exactly, rounded once to
// nearest-even with gradual underflow; sigmoid and softplus as whole functions, :372-470). The value is computed in
// f64 (a few ulp of f64) and narrowed with a single rounding (f64 -> f32 with round-to-odd, then RNE to 11 or 8 bits);
// a misrounding needs the true value within 2^-50 of a rounding boundary of a 16-bit format, and the complete input
// space (65 536 operands per function and format) is checked against a 200-bit evaluation. binary32 and TF32 operands
// take the two-step evaluation of formal_functions_f32.cuh.
__device__ __forceinline__ uint32_t narrow_from_double(double value, int format) {
  float f = __double2float_rz(value);
  if (static_cast<double>(f) != value && isfinite(f)) f = __uint_as_float(__float_as_uint(f) | 1u);   // sticky bit: round to odd
  return narrow_bits(f, format);
}

__device__ uint32_t formal_mpfr_scalar(int op, int format, uint32_t a, uint32_t *flags_out) {
  if (format == WB200_F32 || format == WB200_TF32) {
    // binary32 and TF32 operands: binary64 evaluation with a rounding test and a double-double second step
    // (formal_functions_f32.cuh). TF32 keeps its 19 significant bits in storage bits 31..13; the low bits are ignored.
    int function;
    switch (op) {
      case WB200_EW_SQRT: function = ff32::kSqrt; break;
      case WB200_EW_RSQRT: function = ff32::kRsqrt; break;
      case WB200_EW_LOG2: function = ff32::kLog2; break;
      case WB200_EW_LN: function = ff32::kLn; break;
      case WB200_EW_POW2: function = ff32::kPow2; break;
      case WB200_EW_EXP: function = ff32::kExp; break;
      case WB200_EW_SIN: function = ff32::kSin; break;
      case WB200_EW_COS: function = ff32::kCos; break;
      case WB200_EW_TANH: function = ff32::kTanh; break;
      case WB200_EW_SIGMOID: function = ff32::kSigmoid; break;
      default: function = ff32::kSoftplus; break;
    }
    const bool tf32 = format == WB200_TF32;
    return ff32::correctly_rounded(function, tf32, tf32 ? (a & 0xffffe000u) : a, flags_out, nullptr);
  }
  const FormatTraits t = traits_of(format);
  uint32_t flags = 0;
  const bool nan = (a & t.exp_mask) == t.exp_mask && (a & t.mant_mask) != 0;
  if (nan) {
    *flags_out = (a & t.quiet_bit) ? 0u : kFlagInvalid;
    return t.canonical_nan;
  }
  const bool negative = (a & t.sign) != 0, zero = (a & ~t.sign) == 0, inf = (a & ~t.sign) == t.exp_mask;
  const double x = static_cast<double>(widen_bits(a, format));
  const uint32_t pos_inf = t.exp_mask, neg_inf = t.exp_mask | t.sign;
  auto finish = [&](uint32_t bits, uint32_t f) { *flags_out = f; return bits; };
  double value;
  bool exact = false;
  switch (op) {
    case WB200_EW_SQRT:
      if (zero) return finish(a, 0);                                   // sqrt(-0) = -0
      if (negative) return finish(t.canonical_nan, kFlagInvalid);
      if (inf) return finish(pos_inf, 0);
      value = sqrt(x);
      exact = fma(value, value, -x) == 0.0;
      break;
    case WB200_EW_RSQRT:
      if (zero) return finish(negative ? neg_inf : pos_inf, kFlagDivByZero);
      if (negative) return finish(t.canonical_nan, kFlagInvalid);
      if (inf) return finish(0u, 0);
      value = 1.0 / sqrt(x);
      { int e; exact = frexp(x, &e) == 0.5 && ((e - 1) & 1) == 0; }      // x = 4^k
      break;
    case WB200_EW_LOG2:
    case WB200_EW_LN:
      if (zero) return finish(neg_inf, kFlagDivByZero);
      if (negative) return finish(t.canonical_nan, kFlagInvalid);
      if (inf) return finish(pos_inf, 0);
      if (op == WB200_EW_LOG2) { int e; const bool power = frexp(x, &e) == 0.5; value = power ? static_cast<double>(e - 1) : log2(x); exact = power; }
      else { value = log(x); exact = x == 1.0; }
      break;
    case WB200_EW_POW2:
    case WB200_EW_EXP:
      if (inf) return finish(negative ? 0u : pos_inf, 0);
      value = op == WB200_EW_POW2 ? exp2(x) : exp(x);
      exact = op == WB200_EW_POW2 ? (x == rint(x)) : zero;
      break;
    case WB200_EW_SIN:
    case WB200_EW_COS:
      if (inf) return finish(t.canonical_nan, kFlagInvalid);
      if (zero) return finish(op == WB200_EW_SIN ? a : t.one, 0);
      value = op == WB200_EW_SIN ? sin(x) : cos(x);
      break;
    case WB200_EW_TANH:
      if (zero) return finish(a, 0);
      if (inf) return finish(negative ? (t.one | t.sign) : t.one, 0);
      value = tanh(x);
      break;
    case WB200_EW_SIGMOID:
      if (inf) return finish(negative ? 0u : t.one, 0);
      if (zero) return finish(narrow_bits(0.5f, format), 0);
      value = x >= 0.0 ? 1.0 / (1.0 + exp(-x)) : exp(x) / (1.0 + exp(x));
      break;
    default:   // softplus = ln(1 + e^x)
      if (inf) return finish(negative ? 0u : pos_inf, 0);
      value = x > 0.0 ? x + log1p(exp(-x)) : log1p(exp(x));
      break;
  }
  const uint32_t bits = narrow_from_double(value, format);
  // Every exactly infinite result was returned above, so an infinite result here is an overflow; 2^x, e^x, sigmoid
  // and softplus are never exactly zero, so a zero result of theirs is an underflow (this also covers an f64
  // evaluation that saturated, e.g. 2^1904 or 2^-2000 with an integer operand).
  const bool never_zero = op == WB200_EW_POW2 || op == WB200_EW_EXP || op == WB200_EW_SIGMOID || op == WB200_EW_SOFTPLUS;
  if ((bits & ~t.sign) == t.exp_mask) flags |= kFlagOverflow | kFlagInexact;
  else if ((bits & ~t.sign) == 0 && never_zero) flags |= kFlagUnderflow | kFlagInexact;
  else if (!exact || static_cast<double>(widen_bits(bits, format)) != value) {
    flags |= kFlagInexact;
    if (tiny_after_rounding(value, t.precision, t.min_normal)) flags |= kFlagUnderflow;
  }
  return finish(bits, flags);
}

__device__ __forceinline__ uint32_t formal_load(const uint8_t *base, int format, const LayoutMap &map, int64_t i) {
  if (format == WB200_BOOL) return (base[i >> 3] >> (i & 7)) & 1u;   // bit-packed, least significant bit first
  return load_element_bits(base, physical_index(map, i), format);
}

// One thread per 8 consecutive logical elements, so that a bit-packed Bool destination byte has a single writer.
// kLinear: every tensor is in Tensor / NTensor layout (physical index == logical index); with `vector` set (all
// pointers 16-byte aligned) full groups then move with 128-bit accesses and no layout arithmetic at all.
// kOp >= 0 fixes the operation and the operand format at compile time (the arithmetic and relation families in linear
// layout): the generic evaluator then folds to a few dozen instructions instead of its whole decision tree.
// The groups first_group, first_group + group_stride, ... of one command; returns the OR of the elements' flags. The
// command's own kernel walks the groups with its whole grid, a command run (formal_run_kernel) with one block.
template <bool kLinear, int kOp, int kFormat>
__device__ __forceinline__ uint32_t
formal_elementwise_groups(int runtime_op, int runtime_format, int out_format, int input_count, const uint8_t *in0, const uint8_t *in1, uint8_t *dst,
                          const LayoutMap &in_map, const LayoutMap &out_map, const RhsBroadcast rhs, int vector, int64_t first_group,
                          int64_t group_stride) {
  const int op = kOp >= 0 ? kOp : runtime_op, in_format = kOp >= 0 ? kFormat : runtime_format;
  const int64_t total = out_map.element_count;
  const int64_t groups = (total + 7) / 8;
  const int64_t stride = group_stride;
  uint32_t flags = 0;
  const bool logic = op >= WB200_EW_LOGIC_NOT && op <= WB200_EW_LOGIC_XOR;
  const bool mpfr_family = op == WB200_EW_SQRT || op == WB200_EW_RSQRT || (op >= WB200_EW_LOG2 && op <= WB200_EW_EXP) ||
                           (op >= WB200_EW_SIN && op <= WB200_EW_SIGMOID) || op == WB200_EW_SOFTPLUS;
  const int in_bytes = format_bits(in_format) / 8, out_bytes = format_bits(out_format) / 8;   // 0 for Bool
  const bool same_rhs = input_count > 1 && rhs.mode == WB200_RHS_SAME;
  const bool scalar_rhs = input_count > 1 && rhs.mode == WB200_RHS_SCALAR;   // decided once, not per element
  if (kOp < 0 && mpfr_family) {
    // The correctly rounded functions cost hundreds to thousands of instructions per element: one element per thread
    // and step (first_group / group_stride are then the thread's index and the thread count), so that a short vector
    // spreads over as many threads as it has elements. Unary, float in and out: no Bool packing to respect.
    for (int64_t i = first_group; i < total; i += stride) {
      const uint32_t a = kLinear ? load_element_bits(in0, i, in_format) : formal_load(in0, in_format, in_map, i);
      uint32_t element_flags = 0;
      const uint32_t value = formal_mpfr_scalar(op, in_format, a, &element_flags);
      flags |= element_flags;
      store_element_bits(dst, kLinear ? i : physical_index(out_map, i), out_format, value);
    }
    return flags;
  }
  for (int64_t g = first_group; g < groups; g += stride) {
    const int64_t first = g * 8;
    const int count = total - first < 8 ? static_cast<int>(total - first) : 8;
    const bool wide = kLinear && vector && count == 8;
    uint32_t a[8], b[8], value[8];
    if (wide && in_bytes) {
      load_group8(in0, g, in_bytes, a);
      if (same_rhs) load_group8(in1, g, in_bytes, b);
    } else if (wide) {   // packed Bool operands: one byte holds the group
      const uint32_t byte_a = in0[g], byte_b = same_rhs ? in1[g] : 0u;
#pragma unroll
      for (int e = 0; e < 8; ++e) { a[e] = (byte_a >> e) & 1u; b[e] = (byte_b >> e) & 1u; }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (e >= count) break;
      const int64_t i = first + e;
      if (!wide) a[e] = kLinear ? (in_format == WB200_BOOL ? (in0[i >> 3] >> (i & 7)) & 1u : load_element_bits(in0, i, in_format))
                                : formal_load(in0, in_format, in_map, i);
      if (scalar_rhs) {
        b[e] = rhs.parameter;
      } else if (input_count > 1 && !(wide && same_rhs)) {
        // Second-operand forms of lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:347-372.
        int64_t j = i;
        if (rhs.mode == WB200_RHS_UNIT) j = i % rhs.parameter;
        else if (rhs.mode == WB200_RHS_GROUP) j = i / rhs.parameter * 64 + i % 64;
        b[e] = kLinear ? (in_format == WB200_BOOL ? (in1[j >> 3] >> (j & 7)) & 1u : load_element_bits(in1, j, in_format))
                       : formal_load(in1, in_format, in_map, j);
      } else if (input_count <= 1) {
        b[e] = 0u;
      }
      uint32_t element_flags = 0;
      if (logic) {
        const bool lhs = a[e] != 0, rhs_bit = b[e] != 0;
        value[e] = op == WB200_EW_LOGIC_NOT ? !lhs : op == WB200_EW_LOGIC_AND ? (lhs && rhs_bit) : op == WB200_EW_LOGIC_OR ? (lhs || rhs_bit) : (lhs != rhs_bit);
      } else if (mpfr_family) {
        value[e] = formal_mpfr_scalar(op, in_format, a[e], &element_flags);
      } else {
        value[e] = formal_scalar(op, in_format, out_format, a[e], b[e], &element_flags);
      }
      flags |= element_flags;
    }
    if (out_format == WB200_BOOL) {
      uint32_t packed = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (e < count) packed |= (value[e] & 1u) << e;
      const uint32_t keep = count == 8 ? 0u : (0xffu << count) & 0xffu;   // bits past the tensor keep the template's value
      dst[g] = static_cast<uint8_t>(keep ? ((dst[g] & keep) | packed) : packed);
    } else if (wide) {
      store_group8(dst, g, out_bytes, value);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (e < count) store_element_bits(dst, kLinear ? first + e : physical_index(out_map, first + e), out_format, value[e]);
    }
  }
  return flags;
}

template <bool kLinear, int kOp, int kFormat>
__global__ void __launch_bounds__(kThreads)
formal_elementwise_kernel(int runtime_op, int runtime_format, int out_format, int input_count, const uint8_t *in0, const uint8_t *in1, uint8_t *dst,
                          const LayoutMap in_map, const LayoutMap out_map, const RhsBroadcast rhs, int vector, uint32_t *flags_word) {
  const uint32_t flags = formal_elementwise_groups<kLinear, kOp, kFormat>(
      runtime_op, runtime_format, out_format, input_count, in0, in1, dst, in_map, out_map, rhs, vector,
      static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x, static_cast<int64_t>(gridDim.x) * blockDim.x);
  merge_block_flags(flags_word, flags);
}

// One step of a chain on a thread's eight values. The switch gives every arithmetic operation its own copy of the scalar
// evaluator with the operation and format fixed at compile time (a few dozen instructions each); only the cases a chain
// uses are ever fetched. The correctly rounded function family is one out-of-line call.
template <int kFormat>
__device__ __forceinline__ void chain_step(int op, uint32_t (&value)[8], const uint32_t (&b)[8], int count, uint32_t &flags) {
#define WB200_CHAIN_CASE(OP)                                                             \
  case OP:                                                                               \
    _Pragma("unroll") for (int e = 0; e < 8; ++e) {                                      \
      if (e < count) {                                                                   \
        uint32_t element_flags = 0;                                                      \
        value[e] = formal_scalar(OP, kFormat, kFormat, value[e], b[e], &element_flags);  \
        flags |= element_flags;                                                          \
      }                                                                                  \
    }                                                                                    \
    break;
  switch (op) {
    WB200_CHAIN_CASE(WB200_EW_ABS) WB200_CHAIN_CASE(WB200_EW_NEG) WB200_CHAIN_CASE(WB200_EW_RELU) WB200_CHAIN_CASE(WB200_EW_RECIP)
    WB200_CHAIN_CASE(WB200_EW_SQUARE) WB200_CHAIN_CASE(WB200_EW_MAX) WB200_CHAIN_CASE(WB200_EW_MIN) WB200_CHAIN_CASE(WB200_EW_ADD)
    WB200_CHAIN_CASE(WB200_EW_SUB) WB200_CHAIN_CASE(WB200_EW_MUL)
    default:
#pragma unroll 1
      for (int e = 0; e < count; ++e) {
        uint32_t element_flags = 0;
        value[e] = formal_mpfr_scalar(op, kFormat, value[e], &element_flags);
        flags |= element_flags;
      }
      break;
  }
#undef WB200_CHAIN_CASE
}

// A chain of formal elementwise commands (see ElementwiseChain): the running value stays in registers, every step's
// destination is still written, second operands are read where the step names one. A thread owns the same eight
// elements of every vector, so a step may read what an earlier step of the chain wrote at the same address.
template <int kFormat>
__global__ void __launch_bounds__(kThreads)
formal_chain_kernel(const ElementwiseChain chain, int vector, uint32_t *flags_word) {
  constexpr int format = kFormat, bytes = kFormat == WB200_F32 ? 4 : 2;
  const int64_t total = chain.count, groups = (total + 7) / 8;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  uint32_t flags = 0;
  for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < groups; g += stride) {
    const int64_t first = g * 8;
    const int count = total - first < 8 ? static_cast<int>(total - first) : 8;
    const bool wide = vector && count == 8;
    uint32_t value[8], b[8];
    if (wide) {
      load_group8(chain.lhs, g, bytes, value);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) value[e] = e < count ? load_element_bits(chain.lhs, first + e, format) : 0u;
    }
#pragma unroll 1
    for (int s = 0; s < chain.steps; ++s) {
      const uint8_t *rhs = chain.step[s].rhs;
      uint8_t *dst = chain.step[s].dst;
      if (chain.step[s].rhs_mode == WB200_RHS_SAME) {
        if (wide) {
          load_group8(rhs, g, bytes, b);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) b[e] = e < count ? load_element_bits(rhs, first + e, format) : 0u;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) b[e] = chain.step[s].scalar;
      }
      chain_step<kFormat>(chain.step[s].op, value, b, count, flags);
      if (wide) {
        store_group8(dst, g, bytes, value);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (e < count) store_element_bits(dst, first + e, format, value[e]);
      }
    }
  }
  merge_block_flags(flags_word, flags);
}

// The same fold for rank-4 NCx tensors [n, h, w, c] (every TargetCall-level reduce): coordinates are carried as loop
// counters, so the only divisions are the three that split the output index.
template <int kCombine, int kFormat>
__device__ __forceinline__ uint32_t formal_reduce_nhwc_output(const uint8_t *src, uint8_t *dst, const LayoutMap &src_map, const LayoutMap &dst_map,
                                                              uint32_t reduced_mask, int64_t out_index) {
  constexpr int format = kFormat, combine = kCombine;
  uint32_t block_flags_in = 0;
  if (out_index < dst_map.element_count) {
  const uint32_t out_c = static_cast<uint32_t>(dst_map.shape[3]), out_w = static_cast<uint32_t>(dst_map.shape[2]), out_h = static_cast<uint32_t>(dst_map.shape[1]);
  const uint32_t index = static_cast<uint32_t>(out_index);    // the launcher admits at most 2^32 - 1 outputs
  const uint32_t pixel = index / out_c, c0 = index - pixel * out_c;
  const uint32_t row = pixel / out_w, w0 = pixel - row * out_w;
  const uint32_t n0 = row / out_h, h0 = row - n0 * out_h;
  // dimension d is bit d of the mask; a reduced dimension runs over its whole input extent from 0
  const uint32_t n_count = (reduced_mask & 1u) ? static_cast<uint32_t>(src_map.shape[0]) : 1u, h_count = (reduced_mask & 2u) ? static_cast<uint32_t>(src_map.shape[1]) : 1u;
  const uint32_t w_count = (reduced_mask & 4u) ? static_cast<uint32_t>(src_map.shape[2]) : 1u, c_count = (reduced_mask & 8u) ? static_cast<uint32_t>(src_map.shape[3]) : 1u;
  const uint32_t in_w = static_cast<uint32_t>(src_map.shape[2]);
  const uint32_t infinity = format == WB200_F32 ? 0x7f800000u : format == WB200_BF16 ? 0x7f80u : 0x7c00u;
  const uint32_t sign = format == WB200_F32 ? 0x80000000u : 0x8000u;
  uint32_t accumulator = combine == WB200_EW_ADD ? 0u : combine == WB200_EW_MAX ? (infinity | sign) : infinity;
  uint32_t flags = 0;
  if (!(reduced_mask & 8u)) {
    // The channel is kept: along n, h and w the physical address moves by constant strides (one channel block is
    // `width` elements wide), so the fold is three strided loops whose loads do not depend on one another.
    const int64_t full_c = src_map.cx_blocks * src_map.c_block;
    const int64_t width = static_cast<int64_t>(c0) < full_c ? src_map.c_block : src_map.c0;
    const int64_t stride_w = width, stride_h = width * in_w, stride_n = src_map.outer_slice_stride;
    const int64_t base = physical_index_nhwc(src_map, (reduced_mask & 1u) ? 0 : n0,
                                             static_cast<int64_t>((reduced_mask & 2u) ? 0u : h0) * in_w + ((reduced_mask & 4u) ? 0u : w0), c0);
    for (uint32_t n = 0; n < n_count; ++n)
      for (uint32_t h = 0; h < h_count; ++h) {
        const int64_t row = base + n * stride_n + h * stride_h;
#pragma unroll 8
        for (uint32_t w = 0; w < w_count; ++w) {
          uint32_t step_flags = 0;
          accumulator = formal_scalar(combine, format, format, accumulator, load_element_bits(src, row + w * stride_w, format), &step_flags, kFoldCommonCase);
          flags |= step_flags;
        }
      }
  } else {
    for (uint32_t n = 0; n < n_count; ++n)
      for (uint32_t h = 0; h < h_count; ++h)
        for (uint32_t w = 0; w < w_count; ++w)
          for (uint32_t c = 0; c < c_count; ++c) {
            const int64_t in_n = (reduced_mask & 1u) ? n : n0;
            const uint32_t in_h = (reduced_mask & 2u) ? h : h0, in_wi = (reduced_mask & 4u) ? w : w0;
            uint32_t step_flags = 0;
            const uint32_t value = load_element_bits(src, physical_index_nhwc(src_map, in_n, static_cast<int64_t>(in_h) * in_w + in_wi, c), format);
            accumulator = formal_scalar(combine, format, format, accumulator, value, &step_flags, kFoldCommonCase);
            flags |= step_flags;
          }
  }
  store_element_bits(dst, physical_index_nhwc(dst_map, n0, static_cast<int64_t>(h0) * out_w + w0, c0), format, accumulator);
  block_flags_in = flags;
  }
  return block_flags_in;
}
template <int kCombine, int kFormat>
__global__ void __launch_bounds__(kThreads)
formal_reduce_nhwc_kernel(const uint8_t *src, uint8_t *dst, const LayoutMap src_map, const LayoutMap dst_map,
                          uint32_t reduced_mask, uint32_t *flags_word) {
  const uint32_t flags = formal_reduce_nhwc_output<kCombine, kFormat>(src, dst, src_map, dst_map, reduced_mask,
                                                                     static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x);
  merge_block_flags(flags_word, flags);
}

// Formal reduction (lib/Wafer/Simulator/Reference/Numeric/FormalTensorNumeric.cpp:363-425 with the step of
// Reference/Formal/FormalNumericReduce.cpp:12-67): every output starts from +0 (sum) or -inf / +inf (max / min) and folds
// its inputs in row-major input order with the formal add / maximum / minimum, so NaNs are canonicalised instead of
// refused and the IEEE flags of every step are collected. One thread per output element.
__global__ void __launch_bounds__(kThreads)
formal_reduce_kernel(int op, int format, const uint8_t *src, uint8_t *dst, const LayoutMap src_map, const LayoutMap dst_map,
                     uint32_t reduced_mask, uint32_t *flags_word) {
  const int64_t out_index = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  uint32_t block_flags_in = 0;
  if (out_index < dst_map.element_count) {
  const int rank = src_map.rank;
  int64_t coord[WB200_MAX_RANK];
  int64_t stride[WB200_MAX_RANK];
  int64_t s = 1;
  for (int d = rank - 1; d >= 0; --d) { stride[d] = s; s *= src_map.shape[d]; }
  int64_t remaining = out_index;
  int64_t reduced_count = 1;
  for (int d = rank - 1; d >= 0; --d) {
    if (reduced_mask & (1u << d)) { coord[d] = 0; reduced_count *= src_map.shape[d]; continue; }
    coord[d] = remaining % src_map.shape[d];
    remaining /= src_map.shape[d];
  }
  const uint32_t infinity = format == WB200_F32 ? 0x7f800000u : format == WB200_BF16 ? 0x7f80u : 0x7c00u;
  const uint32_t sign = format == WB200_F32 ? 0x80000000u : 0x8000u;
  uint32_t accumulator = op == WB200_RED_SUM ? 0u : op == WB200_RED_MAX ? (infinity | sign) : infinity;
  const int combine = op == WB200_RED_SUM ? WB200_EW_ADD : op == WB200_RED_MAX ? WB200_EW_MAX : WB200_EW_MIN;
  uint32_t flags = 0;
  for (int64_t r = 0; r < reduced_count; ++r) {
    int64_t rest = r;
    for (int d = rank - 1; d >= 0; --d) {
      if (!(reduced_mask & (1u << d))) continue;
      coord[d] = rest % src_map.shape[d];
      rest /= src_map.shape[d];
    }
    int64_t linear = 0;
    for (int d = 0; d < rank; ++d) linear += coord[d] * stride[d];
    uint32_t step_flags = 0;
    accumulator = formal_scalar(combine, format, format, accumulator, load_element_bits(src, physical_index(src_map, linear), format), &step_flags, kFoldCommonCase);
    flags |= step_flags;
  }
  store_element_bits(dst, physical_index(dst_map, out_index), format, accumulator);
  block_flags_in = flags;
  }
  merge_block_flags(flags_word, block_flags_in);
}

// ------------------------------------------------------------------------------------------------ command runs
// One launch for a run of formal commands of one Tile (FormalRun). A cluster of kRunCtas thread blocks of kRunThreads
// threads executes the commands in issue order with a cluster barrier (release / acquire at cluster scope) after each,
// so a command reads what earlier commands of the run wrote, whichever block wrote it. A cluster is co-scheduled by the
// hardware, so its blocks may wait for one another. Elementwise commands and reductions go through the very device
// functions of their own kernels, spread over the cluster's threads; the GEMM is the formal chain of gemm_formal.cu written for one thread per output:
//   acc = +0; for k ascending: acc = fma(widen(lhs), widen(rhs), acc); [acc = acc + psum;] dst = narrow(acc)
// (lib/Wafer/Simulator/Reference/Numeric/FormalTensorNumeric.cpp:271-361) through the tile function of gemm_formal.cuh, so
// every destination gets the bits the command-by-command replay gives it.
constexpr int kRunThreads = 512;   // 128 registers per thread: the formal evaluators need them
constexpr int kRunCtas = 8;        // one cluster (the portable maximum)
__device__ __forceinline__ uint32_t run_cta_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}
__device__ __forceinline__ void run_cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The GEMM of a run: 64 x 64 output tiles, sixteen at a time (one per group of 256 threads of the cluster, each group with
// shared-memory panels of its own), through the tile function of the command's own kernel, so every output sees the same k-ascending
// chain. `variant` was chosen on the host (gemm_formal_variant).
struct RunPanels {
  float lhs[kRunThreads / 256][kPanelK][kBlockM + 4];
  float rhs[kRunThreads / 256][kPanelK][kBlockN + 4];
};
__device__ __forceinline__ void run_gemm(const GemmFormalArgs &a, int variant, RunPanels &panels) {
  const int group = threadIdx.x >> 8, tid = threadIdx.x & 255;
  const int cluster_group = static_cast<int>(run_cta_rank()) * (kRunThreads / 256) + group;
  const int tiles_n = (a.n + kBlockN - 1) / kBlockN, tiles = ((a.m + kBlockM - 1) / kBlockM) * tiles_n;
  for (int first = 0; first < tiles; first += kRunCtas * (kRunThreads / 256)) {
    const int tile = first + cluster_group;
    const bool active = tile < tiles;
    const int row0 = active ? (tile / tiles_n) * kBlockM : 0, col0 = active ? (tile % tiles_n) * kBlockN : 0;
    if (variant == 3) gemm_formal_tile<true, true, true>(a, 0, row0, col0, tid, active, panels.lhs[group], panels.rhs[group]);
    else if (variant == 2) gemm_formal_tile<true, true, false>(a, 0, row0, col0, tid, active, panels.lhs[group], panels.rhs[group]);
    else gemm_formal_tile<false, false, false>(a, 0, row0, col0, tid, active, panels.lhs[group], panels.rhs[group]);
  }
}

// An elementwise command of a run. The arithmetic family on float operands takes the instantiation with the operation
// and format fixed at compile time, as in the command's own kernel (a few dozen instructions per element instead of the
// generic evaluator's decision tree); everything else takes the generic one.
template <int kOp>
__device__ __noinline__ uint32_t run_elementwise_op(const RunElementwise &e, int vector) {
  if (e.in_format == WB200_F32)
    return formal_elementwise_groups<true, kOp, WB200_F32>(e.op, e.in_format, e.out_format, e.input_count, e.in0, e.in1, e.dst, e.in_map, e.out_map,
                                                           e.rhs, vector, run_cta_rank() * kRunThreads + threadIdx.x, kRunCtas * kRunThreads);
  if (e.in_format == WB200_BF16)
    return formal_elementwise_groups<true, kOp, WB200_BF16>(e.op, e.in_format, e.out_format, e.input_count, e.in0, e.in1, e.dst, e.in_map, e.out_map,
                                                            e.rhs, vector, run_cta_rank() * kRunThreads + threadIdx.x, kRunCtas * kRunThreads);
  return formal_elementwise_groups<true, kOp, WB200_F16>(e.op, e.in_format, e.out_format, e.input_count, e.in0, e.in1, e.dst, e.in_map, e.out_map,
                                                         e.rhs, vector, run_cta_rank() * kRunThreads + threadIdx.x, kRunCtas * kRunThreads);
}
__device__ __noinline__ uint32_t run_elementwise_generic(const RunElementwise &e, int vector) {
  return formal_elementwise_groups<true, -1, 0>(e.op, e.in_format, e.out_format, e.input_count, e.in0, e.in1, e.dst, e.in_map, e.out_map, e.rhs,
                                                vector, run_cta_rank() * kRunThreads + threadIdx.x, kRunCtas * kRunThreads);
}
__device__ __forceinline__ uint32_t run_elementwise(const RunElementwise &e, int vector) {
  if (is_float_format(e.in_format)) {
    switch (e.op) {
      case WB200_EW_MAX: return run_elementwise_op<WB200_EW_MAX>(e, vector);
      case WB200_EW_MIN: return run_elementwise_op<WB200_EW_MIN>(e, vector);
      case WB200_EW_ADD: return run_elementwise_op<WB200_EW_ADD>(e, vector);
      case WB200_EW_SUB: return run_elementwise_op<WB200_EW_SUB>(e, vector);
      case WB200_EW_MUL: return run_elementwise_op<WB200_EW_MUL>(e, vector);
      default: break;
    }
  }
  return run_elementwise_generic(e, vector);
}

__device__ __forceinline__ uint32_t run_reduce(const RunReduce &r) {
  uint32_t flags = 0;
  const bool nhwc = r.src_map.layout == WB200_LAYOUT_NCX && r.dst_map.layout == WB200_LAYOUT_NCX && r.src_map.rank == 4 && r.dst_map.rank == 4;
  if (!nhwc) return flags;   // formal_run_admits lets nothing else in
  for (int64_t out = run_cta_rank() * kRunThreads + threadIdx.x; out < r.dst_map.element_count; out += kRunCtas * kRunThreads) {
#define WB200_RUN_REDUCE(COMBINE)                                                                                                  \
    if (r.format == WB200_F32) flags |= formal_reduce_nhwc_output<COMBINE, WB200_F32>(r.src, r.dst, r.src_map, r.dst_map, r.reduced_mask, out);   \
    else if (r.format == WB200_BF16) flags |= formal_reduce_nhwc_output<COMBINE, WB200_BF16>(r.src, r.dst, r.src_map, r.dst_map, r.reduced_mask, out); \
    else flags |= formal_reduce_nhwc_output<COMBINE, WB200_F16>(r.src, r.dst, r.src_map, r.dst_map, r.reduced_mask, out)
    if (r.op == WB200_RED_SUM) { WB200_RUN_REDUCE(WB200_EW_ADD); }
    else if (r.op == WB200_RED_MAX) { WB200_RUN_REDUCE(WB200_EW_MAX); }
    else { WB200_RUN_REDUCE(WB200_EW_MIN); }
#undef WB200_RUN_REDUCE
  }
  return flags;
}

__global__ void __cluster_dims__(kRunCtas, 1, 1) __launch_bounds__(kRunThreads) formal_run_kernel(const __grid_constant__ FormalRun run, uint32_t *flags_word) {
  __shared__ __align__(16) RunPanels panels;
  // The command being executed, copied from the parameter space: its fields are read inside the inner loops, and a
  // dynamically indexed kernel parameter costs a constant-bank load per use.
  __shared__ __align__(16) unsigned char command_storage[sizeof(RunCommand)];
  const RunCommand &command = *reinterpret_cast<const RunCommand *>(command_storage);
  static_assert(sizeof(RunCommand) % 4 == 0, "copied as 32-bit words");
  uint32_t flags = 0;
#pragma unroll 1
  for (int c = 0; c < run.count; ++c) {
    {
      const uint32_t *from = reinterpret_cast<const uint32_t *>(&run.command[c]);
      uint32_t *to = reinterpret_cast<uint32_t *>(command_storage);
      for (int w = threadIdx.x; w < static_cast<int>(sizeof(RunCommand) / 4); w += kRunThreads) to[w] = from[w];
    }
    __syncthreads();
    if (command.kind == WB200_RUN_ELEMENTWISE) {
      const RunElementwise &e = command.u.elementwise;
      const int vector = ((reinterpret_cast<uintptr_t>(e.in0) | reinterpret_cast<uintptr_t>(e.in1) | reinterpret_cast<uintptr_t>(e.dst)) & 15) == 0;
      flags |= run_elementwise(e, vector);
    } else if (command.kind == WB200_RUN_REDUCE) {
      flags |= run_reduce(command.u.reduce);
    } else {
      run_gemm(command.u.gemm, command.variant, panels);
    }
    run_cluster_barrier();   // the next command may read anything this one wrote, in any block
  }
  merge_block_flags(flags_word, flags);
}

// Plain pooling (lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:466-583): every output folds its window in
// (kh, kw) order with the formal max / min / add, so the roundings and the raised flags are those of the reference's
// window-by-window elementwise passes. Sum starts from +0 and adds every tap; max / min start from the first tap.
// kVec consecutive channels per thread (1 or 4): with 4 the taps move as one 16-byte (f32) or 8-byte (16-bit) access and
// the index arithmetic is shared; the launcher picks it when channel counts, strides and pointers allow it.
template <int kVec>
__device__ __forceinline__ void load_channels(const uint8_t *base, int64_t index, int format, uint32_t (&v)[kVec]) {
  if (kVec == 1) {
    v[0] = load_element_bits(base, index, format);
  } else if (format == WB200_F32) {
    const uint4 w = *reinterpret_cast<const uint4 *>(base + index * 4);
    v[0] = w.x; v[1 % kVec] = w.y; v[2 % kVec] = w.z; v[3 % kVec] = w.w;
  } else {
    const uint2 w = *reinterpret_cast<const uint2 *>(base + index * 2);
    v[0] = w.x & 0xffffu; v[1 % kVec] = w.x >> 16; v[2 % kVec] = w.y & 0xffffu; v[3 % kVec] = w.y >> 16;
  }
}
template <int kVec>
__device__ __forceinline__ void store_channels(uint8_t *base, int64_t index, int format, const uint32_t (&v)[kVec]) {
  if (kVec == 1) {
    store_element_bits(base, index, format, v[0]);
  } else if (format == WB200_F32) {
    *reinterpret_cast<uint4 *>(base + index * 4) = make_uint4(v[0], v[1 % kVec], v[2 % kVec], v[3 % kVec]);
  } else {
    *reinterpret_cast<uint2 *>(base + index * 2) = make_uint2((v[0] & 0xffffu) | (v[1 % kVec] << 16), (v[2 % kVec] & 0xffffu) | (v[3 % kVec] << 16));
  }
}

template <int kCombine, int kFormat, int kVec>
__global__ void __launch_bounds__(kThreads)
formal_pool_kernel(const uint8_t *src, uint8_t *dst, const LayoutMap src_map, const LayoutMap dst_map,
                   const PoolWindow window, uint32_t *flags_word) {
  constexpr int combine = kCombine, format = kFormat;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  uint32_t flags = 0;
  const uint32_t out_h = static_cast<uint32_t>(dst_map.shape[1]), out_w = static_cast<uint32_t>(dst_map.shape[2]);
  const uint32_t channel_groups = static_cast<uint32_t>(dst_map.shape[3]) / kVec, in_w = static_cast<uint32_t>(src_map.shape[2]);
  const int64_t total = dst_map.element_count / kVec;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const uint32_t index = static_cast<uint32_t>(i);          // the launcher admits at most 2^32 - 1 outputs
    const uint32_t pixel = index / channel_groups, c = (index - pixel * channel_groups) * kVec;
    const uint32_t row = pixel / out_w, w = pixel - row * out_w;
    const uint32_t n = row / out_h, h = row - n * out_h;
    uint32_t result[kVec];
    const int64_t full_c = src_map.cx_blocks * src_map.c_block;
    const int64_t width = static_cast<int64_t>(c) < full_c ? src_map.c_block : src_map.c0;   // taps of one channel move by constant strides
    const int64_t corner = physical_index_nhwc(src_map, n, static_cast<int64_t>(h * window.stride_h) * in_w + w * window.stride_w, c);
    for (uint32_t kh = 0; kh < window.kernel_h; ++kh)
      for (uint32_t kw = 0; kw < window.kernel_w; ++kw) {
        uint32_t tap[kVec];
        load_channels<kVec>(src, corner + (static_cast<int64_t>(kh) * in_w + kw) * width, format, tap);
#pragma unroll
        for (int v = 0; v < kVec; ++v) {
          if (kh == 0 && kw == 0) {
            if (combine != WB200_EW_ADD) { result[v] = tap[v]; continue; }
            result[v] = 0u;
          }
          uint32_t element_flags = 0;
          result[v] = formal_scalar(combine, format, format, result[v], tap[v], &element_flags, kFoldCommonCase);
          flags |= element_flags;
        }
      }
    store_channels<kVec>(dst, physical_index_nhwc(dst_map, n, static_cast<int64_t>(h) * out_w + w, c), format, result);
  }
  merge_block_flags(flags_word, flags);
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
  const bool linear = (map.layout == WB200_LAYOUT_TENSOR || map.layout == WB200_LAYOUT_NTENSOR) && all_aligned16(in0, in1, dst);
  const int64_t groups = map.element_count / 8;
  int64_t blocks = (groups + kThreads - 1) / kThreads;
  const int grid = static_cast<int>(blocks < 1 ? 1 : blocks > 148 * 32 ? 148 * 32 : blocks);
#define WB200_MEW(OP)                                                                                                                     \
  case OP:                                                                                                                                \
    if (format == WB200_F32) elementwise_linear_kernel<OP, WB200_F32><<<grid, kThreads, 0, stream>>>(input_count, in0, in1, dst, map.element_count, nan_flag);        \
    else if (format == WB200_BF16) elementwise_linear_kernel<OP, WB200_BF16><<<grid, kThreads, 0, stream>>>(input_count, in0, in1, dst, map.element_count, nan_flag); \
    else elementwise_linear_kernel<OP, WB200_F16><<<grid, kThreads, 0, stream>>>(input_count, in0, in1, dst, map.element_count, nan_flag);                          \
    break;
  switch (linear ? op : -1) {
    WB200_MEW(WB200_EW_ABS) WB200_MEW(WB200_EW_NEG) WB200_MEW(WB200_EW_RECIP) WB200_MEW(WB200_EW_SQUARE) WB200_MEW(WB200_EW_MAX)
    WB200_MEW(WB200_EW_MIN) WB200_MEW(WB200_EW_ADD) WB200_MEW(WB200_EW_SUB) WB200_MEW(WB200_EW_MUL) WB200_MEW(WB200_EW_RELU)
    WB200_MEW(WB200_EW_SQRT) WB200_MEW(WB200_EW_RSQRT) WB200_MEW(WB200_EW_LOG2) WB200_MEW(WB200_EW_LN) WB200_MEW(WB200_EW_POW2)
    WB200_MEW(WB200_EW_EXP) WB200_MEW(WB200_EW_EXPLP) WB200_MEW(WB200_EW_SIN) WB200_MEW(WB200_EW_COS) WB200_MEW(WB200_EW_TANH)
    WB200_MEW(WB200_EW_SIGMOID) WB200_MEW(WB200_EW_SOFTPLUS)
    default:
      elementwise_kernel<<<grid_for(map.element_count), kThreads, 0, stream>>>(op, format, input_count, in0, in1, dst, map, nan_flag);
      break;
  }
#undef WB200_MEW
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

wb200_status launch_elementwise_formal(int op, int in_format, int out_format, int input_count, const uint8_t *in0, const uint8_t *in1,
                                       uint8_t *dst, const LayoutMap &in_map, const LayoutMap &out_map, uint32_t *flags_word,
                                       cudaStream_t stream, RhsBroadcast rhs) {
  auto linear_layout = [](const LayoutMap &m) { return m.layout == WB200_LAYOUT_TENSOR || m.layout == WB200_LAYOUT_NTENSOR; };
  const bool function_family = op == WB200_EW_SQRT || op == WB200_EW_RSQRT || (op >= WB200_EW_LOG2 && op <= WB200_EW_EXP) ||
                               (op >= WB200_EW_SIN && op <= WB200_EW_SIGMOID) || op == WB200_EW_SOFTPLUS;
  // a thread takes eight consecutive elements, or one at a time for the correctly rounded functions
  const int64_t groups = function_family ? out_map.element_count : (out_map.element_count + 7) / 8;
  int64_t blocks = (groups + kThreads - 1) / kThreads;
  blocks = blocks < 1 ? 1 : blocks > 148 * 32 ? 148 * 32 : blocks;
  const int grid = static_cast<int>(blocks);
#define WB200_EW_LAUNCH(LINEAR, OP, FORMAT)                                                                                              \
  formal_elementwise_kernel<LINEAR, OP, FORMAT><<<grid, kThreads, 0, stream>>>(op, in_format, out_format, input_count, in0, in1, dst, in_map, \
                                                                              out_map, rhs, vector, flags_word)
#define WB200_EW_FORMATS(OP)                                            \
  case OP:                                                              \
    if (in_format == WB200_F32) WB200_EW_LAUNCH(true, OP, WB200_F32);   \
    else if (in_format == WB200_BF16) WB200_EW_LAUNCH(true, OP, WB200_BF16); \
    else WB200_EW_LAUNCH(true, OP, WB200_F16);                          \
    break;
  if (linear_layout(in_map) && linear_layout(out_map)) {
    const int vector = all_aligned16(in0, in1, dst);
    const bool specialised = is_float_format(in_format);
    switch (specialised ? op : -1) {
      WB200_EW_FORMATS(WB200_EW_ABS) WB200_EW_FORMATS(WB200_EW_NEG) WB200_EW_FORMATS(WB200_EW_RELU) WB200_EW_FORMATS(WB200_EW_RECIP)
      WB200_EW_FORMATS(WB200_EW_SQUARE) WB200_EW_FORMATS(WB200_EW_MAX) WB200_EW_FORMATS(WB200_EW_MIN) WB200_EW_FORMATS(WB200_EW_ADD)
      WB200_EW_FORMATS(WB200_EW_SUB) WB200_EW_FORMATS(WB200_EW_MUL) WB200_EW_FORMATS(WB200_EW_EQ) WB200_EW_FORMATS(WB200_EW_NE)
      WB200_EW_FORMATS(WB200_EW_GE) WB200_EW_FORMATS(WB200_EW_GT) WB200_EW_FORMATS(WB200_EW_LE) WB200_EW_FORMATS(WB200_EW_LT)
      default: WB200_EW_LAUNCH(true, -1, 0); break;
    }
  } else {
    const int vector = 0;
    WB200_EW_LAUNCH(false, -1, 0);
  }
#undef WB200_EW_FORMATS
#undef WB200_EW_LAUNCH
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

wb200_status launch_elementwise_chain(const ElementwiseChain &chain, uint32_t *flags_word, cudaStream_t stream) {
  if (chain.steps < 1 || chain.steps > kMaxChainSteps || chain.count < 1 || !is_float_format(chain.format))
    return fail(WB200_ERR_INVALID_ARGUMENT, "malformed elementwise chain");
  uintptr_t low_bits = reinterpret_cast<uintptr_t>(chain.lhs);
  for (int s = 0; s < chain.steps; ++s)
    low_bits |= reinterpret_cast<uintptr_t>(chain.step[s].dst) | (chain.step[s].rhs_mode == WB200_RHS_SAME ? reinterpret_cast<uintptr_t>(chain.step[s].rhs) : 0);
  const int64_t groups = (chain.count + 7) / 8;
  int64_t blocks = (groups + kThreads - 1) / kThreads;
  blocks = blocks < 1 ? 1 : blocks > 148 * 32 ? 148 * 32 : blocks;
  const int grid = static_cast<int>(blocks), vector = (low_bits & 15) == 0;
  if (chain.format == WB200_F32) formal_chain_kernel<WB200_F32><<<grid, kThreads, 0, stream>>>(chain, vector, flags_word);
  else if (chain.format == WB200_BF16) formal_chain_kernel<WB200_BF16><<<grid, kThreads, 0, stream>>>(chain, vector, flags_word);
  else formal_chain_kernel<WB200_F16><<<grid, kThreads, 0, stream>>>(chain, vector, flags_word);
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

// Commands small enough for one thread block: one block is 1 / 148 of the machine, so a large command is faster in its
// own kernel. Elementwise: linear 1-D vectors of at most 2^17 elements; reduce: NCx rank 4 with at most 2^18 inputs;
// GEMM: one matrix of at most 2^20 multiply-adds.
bool formal_run_admits(const RunCommand &command) {
  auto linear = [](const LayoutMap &m) { return m.layout == WB200_LAYOUT_TENSOR || m.layout == WB200_LAYOUT_NTENSOR; };
  if (command.kind == WB200_RUN_ELEMENTWISE) {
    const RunElementwise &e = command.u.elementwise;
    return linear(e.in_map) && linear(e.out_map) && e.out_map.element_count <= (1 << 17);
  }
  if (command.kind == WB200_RUN_REDUCE) {
    const RunReduce &r = command.u.reduce;
    return r.src_map.layout == WB200_LAYOUT_NCX && r.dst_map.layout == WB200_LAYOUT_NCX && r.src_map.rank == 4 && r.dst_map.rank == 4 &&
           r.src_map.element_count <= (1 << 18);
  }
  const GemmFormalArgs &g = command.u.gemm;
  return g.batch == 1 && static_cast<int64_t>(g.m) * g.n * g.k <= (1 << 20) && is_float_format(g.in_format) && is_float_format(g.out_format);
}

wb200_status launch_formal_run(const FormalRun &run, uint32_t *flags_word, cudaStream_t stream) {
  if (run.count < 1 || run.count > kMaxRunCommands) return fail(WB200_ERR_INVALID_ARGUMENT, "malformed command run");
  for (int c = 0; c < run.count; ++c)
    if (!formal_run_admits(run.command[c])) return fail(WB200_ERR_INVALID_ARGUMENT, "command outside the domain of a command run");
  formal_run_kernel<<<kRunCtas, kRunThreads, 0, stream>>>(run, flags_word);
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

wb200_status launch_reduce_formal(int op, int format, const uint8_t *src, uint8_t *dst, const LayoutMap &src_map, const LayoutMap &dst_map,
                                  uint32_t reduced_mask, uint32_t *flags_word, cudaStream_t stream) {
  const int64_t blocks = (dst_map.element_count + kThreads - 1) / kThreads;
  if (src_map.layout == WB200_LAYOUT_NCX && dst_map.layout == WB200_LAYOUT_NCX && src_map.rank == 4 && dst_map.rank == 4 &&
      dst_map.element_count < (1ll << 32))
  {
    const int grid = static_cast<int>(blocks < 1 ? 1 : blocks);
#define WB200_RED_LAUNCH(COMBINE, FORMAT) formal_reduce_nhwc_kernel<COMBINE, FORMAT><<<grid, kThreads, 0, stream>>>(src, dst, src_map, dst_map, reduced_mask, flags_word)
#define WB200_RED_FORMATS(COMBINE)                                              \
    if (format == WB200_F32) WB200_RED_LAUNCH(COMBINE, WB200_F32);              \
    else if (format == WB200_BF16) WB200_RED_LAUNCH(COMBINE, WB200_BF16);       \
    else WB200_RED_LAUNCH(COMBINE, WB200_F16)
    if (op == WB200_RED_SUM) { WB200_RED_FORMATS(WB200_EW_ADD); }
    else if (op == WB200_RED_MAX) { WB200_RED_FORMATS(WB200_EW_MAX); }
    else { WB200_RED_FORMATS(WB200_EW_MIN); }
#undef WB200_RED_FORMATS
#undef WB200_RED_LAUNCH
  }
  else
    formal_reduce_kernel<<<static_cast<int>(blocks < 1 ? 1 : blocks), kThreads, 0, stream>>>(op, format, src, dst, src_map, dst_map, reduced_mask, flags_word);
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

wb200_status launch_pool_formal(int combine, int format, const uint8_t *src, uint8_t *dst, const LayoutMap &src_map,
                                const LayoutMap &dst_map, PoolWindow window, uint32_t *flags_word, cudaStream_t stream) {
  if (dst_map.element_count >= (1ll << 32)) return fail(WB200_ERR_LIMIT, "pooling output has more than 2^32 - 1 elements");
  // Four channels per thread need every channel run, block and slice to start on a multiple of four elements.
  auto by_four = [](const LayoutMap &m) {
    return m.shape[3] % 4 == 0 && m.c_block % 4 == 0 && m.c0 % 4 == 0 && m.outer_slice_stride % 4 == 0;
  };
  const bool vec4 = by_four(src_map) && by_four(dst_map) && all_aligned16(src, dst);
  const int grid = grid_for(dst_map.element_count / (vec4 ? 4 : 1));
#define WB200_POOL_LAUNCH(COMBINE, FORMAT)                                                                                      \
  do {                                                                                                                          \
    if (vec4) formal_pool_kernel<COMBINE, FORMAT, 4><<<grid, kThreads, 0, stream>>>(src, dst, src_map, dst_map, window, flags_word); \
    else formal_pool_kernel<COMBINE, FORMAT, 1><<<grid, kThreads, 0, stream>>>(src, dst, src_map, dst_map, window, flags_word);     \
  } while (0)
#define WB200_POOL_FORMATS(COMBINE)                                             \
  if (format == WB200_F32) WB200_POOL_LAUNCH(COMBINE, WB200_F32);               \
  else if (format == WB200_BF16) WB200_POOL_LAUNCH(COMBINE, WB200_BF16);        \
  else WB200_POOL_LAUNCH(COMBINE, WB200_F16)
  if (combine == WB200_EW_ADD) { WB200_POOL_FORMATS(WB200_EW_ADD); }
  else if (combine == WB200_EW_MAX) { WB200_POOL_FORMATS(WB200_EW_MAX); }
  else { WB200_POOL_FORMATS(WB200_EW_MIN); }
#undef WB200_POOL_FORMATS
#undef WB200_POOL_LAUNCH
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

wb200_status launch_convert(int src_format, int dst_format, const uint8_t *src, uint8_t *dst,
                            const LayoutMap &src_map, const LayoutMap &dst_map, int *nan_flag, cudaStream_t stream) {
  auto linear_layout = [](const LayoutMap &m) { return m.layout == WB200_LAYOUT_TENSOR || m.layout == WB200_LAYOUT_NTENSOR; };
  const bool linear = linear_layout(src_map) && linear_layout(dst_map) && all_aligned16(src, dst);
  int64_t blocks = (src_map.element_count / 8 + kThreads - 1) / kThreads;
  const int grid = static_cast<int>(blocks < 1 ? 1 : blocks > 148 * 32 ? 148 * 32 : blocks);
#define WB200_MCV(SRC, DST) convert_linear_kernel<SRC, DST><<<grid, kThreads, 0, stream>>>(src, dst, src_map.element_count, nan_flag)
#define WB200_MCV_TO(SRC)                                        \
  if (dst_format == WB200_F32) WB200_MCV(SRC, WB200_F32);        \
  else if (dst_format == WB200_BF16) WB200_MCV(SRC, WB200_BF16); \
  else WB200_MCV(SRC, WB200_F16)
  if (linear && is_float_format(src_format) && is_float_format(dst_format)) {
    if (src_format == WB200_F32) { WB200_MCV_TO(WB200_F32); }
    else if (src_format == WB200_BF16) { WB200_MCV_TO(WB200_BF16); }
    else { WB200_MCV_TO(WB200_F16); }
  } else {
    convert_kernel<<<grid_for(src_map.element_count), kThreads, 0, stream>>>(src_format, dst_format, src, dst, src_map, dst_map, nan_flag);
  }
#undef WB200_MCV_TO
#undef WB200_MCV
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

wb200_status launch_reduce(int op, int format, const uint8_t *src, uint8_t *dst, const LayoutMap &src_map,
                           const LayoutMap &dst_map, uint32_t reduced_mask, int *nan_flag, cudaStream_t stream) {
  const int64_t blocks = (dst_map.element_count + kThreads - 1) / kThreads;
  const int grid = static_cast<int>(blocks < 1 ? 1 : blocks);
  if (src_map.layout == WB200_LAYOUT_NCX && dst_map.layout == WB200_LAYOUT_NCX && src_map.rank == 4 && dst_map.rank == 4 &&
      dst_map.element_count < (1ll << 32)) {
#define WB200_MRED(OP, FORMAT) reduce_nhwc_kernel<OP, FORMAT><<<grid, kThreads, 0, stream>>>(src, dst, src_map, dst_map, reduced_mask, nan_flag)
#define WB200_MRED_FORMATS(OP)                                   \
    if (format == WB200_F32) WB200_MRED(OP, WB200_F32);          \
    else if (format == WB200_BF16) WB200_MRED(OP, WB200_BF16);   \
    else WB200_MRED(OP, WB200_F16)
    if (op == WB200_RED_SUM) { WB200_MRED_FORMATS(WB200_RED_SUM); }
    else if (op == WB200_RED_MAX) { WB200_MRED_FORMATS(WB200_RED_MAX); }
    else { WB200_MRED_FORMATS(WB200_RED_MIN); }
#undef WB200_MRED_FORMATS
#undef WB200_MRED
  } else {
    reduce_kernel<<<grid, kThreads, 0, stream>>>(op, format, src, dst, src_map, dst_map, reduced_mask, nan_flag);
  }
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
