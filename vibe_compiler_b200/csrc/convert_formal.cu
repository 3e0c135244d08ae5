// Formal scalar conversion routes on the device: the integer <-> floating and floating <-> floating conversions of
// lib/Wafer/Target/PhysicalTensor/TargetScalarConversion.cpp:166-361 with its four deterministic rounding modes, IEEE
// flags (tininess after rounding at unbounded exponent range, lib/Wafer/Target/PhysicalTensor/TargetFloatArithmetic.cpp:
// 82-158; the directed-overflow completion of TargetScalarConversion.cpp:60-76, 128-136) and its refusals. Every value
// is handled as an exact dyadic sign * significand * 2^exponent in integer arithmetic, so no rounding depends on the
// device's floating-point unit. HBM-bound: source bytes in, destination bytes out.
#include "backend.h"

using namespace wb200;

namespace {

constexpr int kThreads = 256;
enum { MODE_NEAREST_EVEN = 0, MODE_TOWARD_ZERO = 1, MODE_TOWARD_POSITIVE = 2, MODE_TOWARD_NEGATIVE = 3 };
enum { FLAG_INVALID = 1, FLAG_OVERFLOW = 4, FLAG_UNDERFLOW = 8, FLAG_INEXACT = 16 };
enum { ERR_NON_FINITE = 1, ERR_OUT_OF_RANGE = 2, ERR_SOURCE_ENCODING = 3 };

// precision (significand bits with the hidden one), exponent bits, unused low storage bits (TF32 keeps its 19
// semantic bits in storage [31:13]).
struct FloatSpec {
  int precision, exponent_bits, shift;
};
__host__ __device__ inline bool float_spec(int format, FloatSpec *spec) {
  switch (format) {
    case WB200_F16: *spec = {11, 5, 0}; return true;
    case WB200_BF16: *spec = {8, 8, 0}; return true;
    case WB200_F32: *spec = {24, 8, 0}; return true;
    case WB200_TF32: *spec = {11, 8, 13}; return true;
    default: return false;
  }
}
__host__ __device__ inline int integer_width(int format) {
  return format == WB200_I8 ? 8 : format == WB200_I16 ? 16 : format == WB200_I32 ? 32 : 0;
}

// Every significand of these routes fits 32 bits (|i32| <= 2^31, float significands < 2^24).
__device__ __forceinline__ int top_bit(uint32_t value) { return 31 - __clz(static_cast<int>(value)); }

__device__ __forceinline__ bool round_up(int mode, bool negative, uint32_t kept, uint32_t lost, int shift) {
  if (lost == 0) return false;
  switch (mode) {
    case MODE_NEAREST_EVEN: {
      const uint32_t half = 1u << (shift - 1);
      return lost > half || (lost == half && (kept & 1));
    }
    case MODE_TOWARD_POSITIVE: return !negative;
    case MODE_TOWARD_NEGATIVE: return negative;
    default: return false;
  }
}

// Drops `shift` low bits of `significand` under `mode`. A shift past the whole significand leaves a value below half
// a unit, which only a directed mode rounds away from zero.
__device__ __forceinline__ uint32_t shift_right_rounded(uint32_t significand, int shift, int mode, bool negative, bool *inexact) {
  if (shift <= 0) return significand << -shift;   // callers only widen into fewer than 32 bits
  if (shift > 31) {                               // the whole significand lies below half a unit (it has at most 32 bits)
    *inexact = significand != 0;
    const bool above_half = shift == 32 && significand > 0x80000000u;   // only a full-width significand can pass one half
    const bool tie = shift == 32 && significand == 0x80000000u;
    const bool away = significand != 0 && ((mode == MODE_TOWARD_POSITIVE && !negative) || (mode == MODE_TOWARD_NEGATIVE && negative) ||
                                           (mode == MODE_NEAREST_EVEN && above_half && !tie));
    return away ? 1u : 0u;
  }
  const uint32_t kept = significand >> shift, lost = significand & ((1u << shift) - 1u);
  *inexact = lost != 0;
  return kept + (round_up(mode, negative, kept, lost, shift) ? 1u : 0u);
}

// sign * significand * 2^exponent -> destination float bits.
__device__ __forceinline__ uint32_t round_to_float(bool negative, uint32_t significand, int exponent, const FloatSpec &spec, int mode,
                                   bool float_source, uint32_t *flags) {
  const int fraction_bits = spec.precision - 1;
  const uint32_t sign = negative ? 1u << (fraction_bits + spec.exponent_bits) : 0u;
  if (significand == 0) return sign << spec.shift;
  const int bias = (1 << (spec.exponent_bits - 1)) - 1, minimum = 1 - bias, maximum = bias;
  const int top = top_bit(significand) + exponent;
  // Tininess is judged after rounding to `precision` bits with an unbounded exponent range.
  bool tiny_inexact = false;
  uint32_t unbounded = shift_right_rounded(significand, top_bit(significand) + 1 - spec.precision, mode, negative, &tiny_inexact);
  int unbounded_top = top;
  if (unbounded >> spec.precision) unbounded_top += 1;
  const bool tiny = unbounded_top < minimum;
  const bool exceeds_maximum = top > maximum || (top == maximum && unbounded_top > maximum) ||
                               (top == maximum && [&] {   // magnitude above the largest finite value
                                 const int width = top_bit(significand) + 1;
                                 if (width <= spec.precision) return false;
                                 const uint32_t ones = ((1u << spec.precision) - 1u) << (width - spec.precision);
                                 return significand > ones;
                               }());
  const int quantum = (top > minimum ? top : minimum) - fraction_bits;
  bool inexact = false;
  uint32_t rounded = shift_right_rounded(significand, quantum - exponent, mode, negative, &inexact);
  int biased;
  if (rounded >> spec.precision) {   // carried into the next binade
    rounded >>= 1;
    biased = quantum + fraction_bits + 1 + bias;
  } else if (rounded >> fraction_bits) {
    biased = quantum + fraction_bits + bias;
  } else {
    biased = 0;                      // subnormal or zero
  }
  const uint32_t all_ones = (1u << spec.exponent_bits) - 1;
  const bool returns_finite = mode == MODE_TOWARD_ZERO || (mode == MODE_TOWARD_POSITIVE && negative) || (mode == MODE_TOWARD_NEGATIVE && !negative);
  uint32_t semantic;
  if (biased >= static_cast<int>(all_ones)) {
    if (returns_finite) semantic = ((all_ones - 1) << fraction_bits) | ((1u << fraction_bits) - 1);
    else semantic = all_ones << fraction_bits;
    *flags |= FLAG_OVERFLOW | FLAG_INEXACT;
  } else {
    semantic = (static_cast<uint32_t>(biased) << fraction_bits) | (rounded & ((1u << fraction_bits) - 1));
    if (inexact) *flags |= FLAG_INEXACT;
    if (exceeds_maximum && returns_finite) *flags |= FLAG_OVERFLOW | FLAG_INEXACT;
    if (float_source && inexact && tiny) *flags |= FLAG_UNDERFLOW;
  }
  return (sign | semantic) << spec.shift;
}

// One element. Returns false (with *error set) when the reference refuses the value.
__device__ __forceinline__ bool convert_scalar(int src_format, int dst_format, int mode, uint32_t bits, uint32_t *result, uint32_t *flags, int *error) {
  FloatSpec src_spec{}, dst_spec{};
  const bool src_float = float_spec(src_format, &src_spec), dst_float = float_spec(dst_format, &dst_spec);
  bool negative;
  uint32_t significand;
  int exponent = 0;
  if (!src_float) {
    const int width = integer_width(src_format);
    const long long value = width == 32 ? static_cast<int>(bits) : static_cast<short>(bits & 0xffffu);
    negative = value < 0;
    significand = static_cast<uint32_t>(negative ? -value : value);
  } else {
    if (src_spec.shift && (bits & ((1u << src_spec.shift) - 1))) { *error = ERR_SOURCE_ENCODING; return false; }
    const uint32_t semantic = bits >> src_spec.shift;
    const int fraction_bits = src_spec.precision - 1;
    const uint32_t fraction = semantic & ((1u << fraction_bits) - 1);
    const uint32_t field = (semantic >> fraction_bits) & ((1u << src_spec.exponent_bits) - 1);
    negative = (semantic >> (fraction_bits + src_spec.exponent_bits)) & 1u;
    const int bias = (1 << (src_spec.exponent_bits - 1)) - 1;
    if (field == (1u << src_spec.exponent_bits) - 1) {
      if (!dst_float) { *error = ERR_NON_FINITE; return false; }
      const int dst_fraction = dst_spec.precision - 1;
      const uint32_t all_ones = (1u << dst_spec.exponent_bits) - 1;
      if (fraction == 0) {
        *result = (((negative ? 1u : 0u) << (dst_fraction + dst_spec.exponent_bits)) | (all_ones << dst_fraction)) << dst_spec.shift;
      } else {
        if (!(fraction >> (fraction_bits - 1))) *flags |= FLAG_INVALID;   // signalling NaN
        *result = ((all_ones << dst_fraction) | (1u << (dst_fraction - 1))) << dst_spec.shift;
      }
      return true;
    }
    if (dst_float && dst_format != WB200_TF32) {
      // Hardware path for finite values that stay clear of the destination's subnormal range: every source value is
      // an f32 value, the f32 -> f16 / bf16 conversion instructions implement all four IEEE roundings, and the flags
      // follow from the result (tininess is impossible once |x| is at least the smallest normal number).
      const float x = src_format == WB200_F16 ? __half2float(__ushort_as_half(static_cast<unsigned short>(bits)))
                                              : __uint_as_float(src_format == WB200_BF16 ? bits << 16 : bits);
      if (dst_format == WB200_F32) {   // every route into f32 widens exactly
        *result = __float_as_uint(x);
        return true;
      }
      const float magnitude = fabsf(x);
      const float smallest_normal = dst_format == WB200_F16 ? 6.103515625e-05f : 1.17549435e-38f;
      if (magnitude >= smallest_normal) {
        const float largest = dst_format == WB200_F16 ? 65504.0f : 3.38953139e38f;
        uint32_t narrow;
        if (dst_format == WB200_F16) {
          const __half h = mode == MODE_NEAREST_EVEN ? __float2half_rn(x) : mode == MODE_TOWARD_ZERO ? __float2half_rz(x)
                         : mode == MODE_TOWARD_POSITIVE ? __float2half_ru(x) : __float2half_rd(x);
          narrow = __half_as_ushort(h);
        } else {
          const __nv_bfloat16 h = mode == MODE_NEAREST_EVEN ? __float2bfloat16_rn(x) : mode == MODE_TOWARD_ZERO ? __float2bfloat16_rz(x)
                                : mode == MODE_TOWARD_POSITIVE ? __float2bfloat16_ru(x) : __float2bfloat16_rd(x);
          narrow = __bfloat16_as_ushort(h);
        }
        const uint32_t exponent_mask = dst_format == WB200_F16 ? 0x7c00u : 0x7f80u;
        const bool became_infinite = (narrow & 0x7fffu) == exponent_mask;
        const float back = dst_format == WB200_F16 ? __half2float(__ushort_as_half(static_cast<unsigned short>(narrow))) : __uint_as_float(narrow << 16);
        const bool returns_finite = mode == MODE_TOWARD_ZERO || (mode == MODE_TOWARD_POSITIVE && negative) || (mode == MODE_TOWARD_NEGATIVE && !negative);
        if (became_infinite || (magnitude > largest && returns_finite)) *flags |= FLAG_OVERFLOW | FLAG_INEXACT;
        else if (back != x) *flags |= FLAG_INEXACT;
        *result = narrow;
        return true;
      }
    }
    significand = field ? (fraction | (1u << fraction_bits)) : fraction;
    exponent = (field ? static_cast<int>(field) : 1) - bias - fraction_bits;
  }
  if (dst_float) {
    *result = round_to_float(negative, significand, exponent, dst_spec, mode, src_float, flags);
    return true;
  }
  // floating -> integer: round to an integer under `mode`, then the value must fit the signed destination width.
  const int width = integer_width(dst_format);
  if (significand == 0) { *result = 0; return true; }
  if (top_bit(significand) + exponent >= 32) { *error = ERR_OUT_OF_RANGE; return false; }   // |value| >= 2^32 fits no route
  bool inexact = false;
  const uint32_t magnitude = shift_right_rounded(significand, -exponent, mode, negative, &inexact);
  const uint32_t limit = 1u << (width - 1);
  if (negative ? magnitude > limit : magnitude > limit - 1u) { *error = ERR_OUT_OF_RANGE; return false; }
  if (inexact) *flags |= FLAG_INEXACT;
  const uint32_t value = negative ? 0u - magnitude : magnitude;   // two's complement
  *result = width == 32 ? value : value & ((1u << width) - 1u);
  return true;
}

__device__ __forceinline__ uint32_t load_bits(const uint8_t *base, int64_t index, int bytes) {
  return bytes == 4 ? reinterpret_cast<const uint32_t *>(base)[index] : bytes == 2 ? reinterpret_cast<const uint16_t *>(base)[index] : base[index];
}
__device__ __forceinline__ void store_bits(uint8_t *base, int64_t index, int bytes, uint32_t bits) {
  if (bytes == 4) reinterpret_cast<uint32_t *>(base)[index] = bits;
  else if (bytes == 2) reinterpret_cast<uint16_t *>(base)[index] = static_cast<uint16_t>(bits);
  else base[index] = static_cast<uint8_t>(bits);
}

// `first_error`: the smallest (element << 8 | error code) over all refused elements; `store` = 0 only validates.
// One thread per 8 consecutive elements. kLinear: both tensors in Tensor / NTensor layout; with `vector` set (16-byte
// aligned pointers) full groups move with 128-bit accesses.
// kSrc >= 0 fixes both formats at compile time (every route in linear layout), which folds the generic scalar routine.
template <bool kLinear, int kSrc, int kDst>
__global__ void __launch_bounds__(kThreads)
formal_convert_kernel(int runtime_src, int runtime_dst, int mode, const uint8_t *src, uint8_t *dst, const LayoutMap src_map,
                      const LayoutMap dst_map, int store, int vector, uint32_t *flags_word, unsigned long long *first_error) {
  const int src_format = kSrc >= 0 ? kSrc : runtime_src, dst_format = kSrc >= 0 ? kDst : runtime_dst;
  const int src_bytes = format_bits(src_format) / 8, dst_bytes = format_bits(dst_format) / 8;
  const int64_t total = src_map.element_count, groups = (total + 7) / 8;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  uint32_t flags = 0;
  unsigned long long error_key = ~0ull;
  for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < groups; g += stride) {
    const int64_t first = g * 8;
    const int count = total - first < 8 ? static_cast<int>(total - first) : 8;
    const bool wide = kLinear && vector && count == 8;
    uint32_t in[8], out[8];
    if (wide) load_group8(src, g, src_bytes, in);
    bool refused = false;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (e >= count) break;
      const int64_t i = first + e;
      if (!wide) in[e] = load_bits(src, kLinear ? i : physical_index(src_map, i), src_bytes);
      uint32_t element_flags = 0;
      int error = 0;
      out[e] = 0;
      if (convert_scalar(src_format, dst_format, mode, in[e], &out[e], &element_flags, &error)) {
        flags |= element_flags;
      } else {
        refused = true;
        const unsigned long long key = (static_cast<unsigned long long>(i) << 8) | static_cast<unsigned>(error);
        error_key = key < error_key ? key : error_key;
      }
    }
    if (!store) continue;
    if (wide && !refused) {
      store_group8(dst, g, dst_bytes, out);
    } else {
      // a group with a refused element keeps that element's destination as it was (the host fails the command anyway)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (e >= count) break;
        uint32_t unused_result, unused_flags = 0;
        int error = 0;
        if (refused && !convert_scalar(src_format, dst_format, mode, in[e], &unused_result, &unused_flags, &error)) continue;
        store_bits(dst, kLinear ? first + e : physical_index(dst_map, first + e), dst_bytes, out[e]);
      }
    }
  }
  merge_block_flags(flags_word, store ? flags : 0u);
  if (error_key != ~0ull) atomicMin(first_error, error_key);
}

// Picks the linear, format-specialised instantiation when both layouts allow it.
void launch_formal_convert(cudaStream_t stream, int src_format, int dst_format, int mode, const uint8_t *src, uint8_t *dst, const LayoutMap &src_map,
                           const LayoutMap &dst_map, int store, uint32_t *flags_word, unsigned long long *first_error) {
  auto linear_layout = [](const LayoutMap &m) { return m.layout == WB200_LAYOUT_TENSOR || m.layout == WB200_LAYOUT_NTENSOR; };
  int64_t blocks = ((src_map.element_count + 7) / 8 + kThreads - 1) / kThreads;
  blocks = blocks < 1 ? 1 : blocks > 148 * 32 ? 148 * 32 : blocks;
  const int grid = static_cast<int>(blocks);
  const int vector = all_aligned16(src, dst);
#define WB200_CV_LAUNCH(LINEAR, SRC, DST, VECTOR)                                                                                      \
  formal_convert_kernel<LINEAR, SRC, DST><<<grid, kThreads, 0, stream>>>(src_format, dst_format, mode, src, dst, src_map, dst_map, store, VECTOR, \
                                                                         flags_word, first_error)
#define WB200_CV_TO(SRC)                                                                \
  switch (dst_format) {                                                                 \
    case WB200_F16: WB200_CV_LAUNCH(true, SRC, WB200_F16, vector); return;              \
    case WB200_BF16: WB200_CV_LAUNCH(true, SRC, WB200_BF16, vector); return;            \
    case WB200_F32: WB200_CV_LAUNCH(true, SRC, WB200_F32, vector); return;              \
    case WB200_TF32: WB200_CV_LAUNCH(true, SRC, WB200_TF32, vector); return;            \
    case WB200_I8: WB200_CV_LAUNCH(true, SRC, WB200_I8, vector); return;                \
    case WB200_I16: WB200_CV_LAUNCH(true, SRC, WB200_I16, vector); return;              \
    case WB200_I32: WB200_CV_LAUNCH(true, SRC, WB200_I32, vector); return;              \
    default: break;                                                                     \
  }
  if (linear_layout(src_map) && linear_layout(dst_map)) {
    switch (src_format) {
      case WB200_I16: WB200_CV_TO(WB200_I16) break;
      case WB200_I32: WB200_CV_TO(WB200_I32) break;
      case WB200_F16: WB200_CV_TO(WB200_F16) break;
      case WB200_BF16: WB200_CV_TO(WB200_BF16) break;
      case WB200_F32: WB200_CV_TO(WB200_F32) break;
      case WB200_TF32: WB200_CV_TO(WB200_TF32) break;
      default: break;
    }
    WB200_CV_LAUNCH(true, -1, 0, vector);
    return;
  }
  WB200_CV_LAUNCH(false, -1, 0, 0);
#undef WB200_CV_TO
#undef WB200_CV_LAUNCH
}

struct Route {
  int source, destination, parameter;   // parameter: 0 none, 1 rounding mode, 2 zero point
};
// lib/Wafer/Target/TargetFormat.cpp:163-200.
bool find_route(uint32_t opcode, Route *route) {
  static const Route table[36] = {
      {WB200_I8, WB200_F16, 2},   {WB200_I8, WB200_BF16, 2},  {WB200_I8, WB200_F32, 2},    {WB200_I8, WB200_TF32, 2},
      {WB200_I16, WB200_F16, 0},  {WB200_I16, WB200_BF16, 1}, {WB200_I16, WB200_F32, 1},   {WB200_I16, WB200_TF32, 1},
      {WB200_I32, WB200_F16, 1},  {WB200_I32, WB200_BF16, 1}, {WB200_I32, WB200_F32, 1},   {WB200_I32, WB200_TF32, 1},
      {WB200_BF16, WB200_I8, 0},  {WB200_BF16, WB200_I16, 1}, {WB200_BF16, WB200_I32, 1},  {WB200_BF16, WB200_F16, 0},
      {WB200_BF16, WB200_F32, 0}, {WB200_BF16, WB200_TF32, 0}, {WB200_F16, WB200_I8, 1},   {WB200_F16, WB200_I16, 1},
      {WB200_F16, WB200_I32, 1},  {WB200_F16, WB200_BF16, 1}, {WB200_F16, WB200_F32, 0},   {WB200_F16, WB200_TF32, 0},
      {WB200_F32, WB200_I8, 1},   {WB200_F32, WB200_I16, 1},  {WB200_F32, WB200_I32, 1},   {WB200_F32, WB200_F16, 1},
      {WB200_F32, WB200_BF16, 1}, {WB200_F32, WB200_TF32, 1}, {WB200_TF32, WB200_I8, 1},   {WB200_TF32, WB200_I16, 1},
      {WB200_TF32, WB200_I32, 1}, {WB200_TF32, WB200_F16, 0}, {WB200_TF32, WB200_BF16, 1}, {WB200_TF32, WB200_F32, 0}};
  if (opcode < 139 || opcode > 174) return false;
  *route = table[opcode - 139];
  return true;
}

wb200_status check_route(uint32_t opcode, uint32_t rounding_mode, Route *route, int *mode) {
  if (!find_route(opcode, route)) return fail(WB200_ERR_INVALID_ARGUMENT, "convert opcode is not a target route");
  if (route->parameter == 2)
    return fail(WB200_ERR_UNSUPPORTED, "unsupported-operation: parameterless scalar conversion has inconsistent parameters (zero-point routes have no formal evaluation)");
  if (rounding_mode > 4) return fail(WB200_ERR_INVALID_ARGUMENT, "convert rounding mode is out of range");
  if (route->parameter == 1 && rounding_mode == 4)
    return fail(WB200_ERR_UNSUPPORTED, "unsupported-operation: scalar conversion accepts only deterministic rounding modes");
  *mode = route->parameter == 1 ? static_cast<int>(rounding_mode) : MODE_NEAREST_EVEN;
  return WB200_OK;
}

wb200_status refusal(unsigned long long key) {
  const std::string where = " at element " + std::to_string(key >> 8);
  switch (key & 0xff) {
    case ERR_NON_FINITE: return fail(WB200_ERR_NAN_DOMAIN, "float-to-integer-non-finite: NaN and infinity do not produce a floating-to-integer result" + where);
    case ERR_OUT_OF_RANGE: return fail(WB200_ERR_NAN_DOMAIN, "float-to-integer-out-of-range: finite input is outside the destination integer range after rounding" + where);
    default: return fail(WB200_ERR_INVALID_ARGUMENT, "invalid-source-encoding: non-canonical TF32 storage bits" + where);
  }
}

// Validates every element first where the route can refuse one, so that a refused command writes nothing.
wb200_status run_convert(wb200_backend *backend, const Route &route, int mode, const uint8_t *src, uint8_t *dst, const LayoutMap &src_map,
                         const LayoutMap &dst_map, cudaStream_t stream, uint32_t *flags) {
  void *scratch;
  wb200_status st = backend->buffer(3, 16, &scratch);
  if (st != WB200_OK) return st;
  uint32_t *d_flags = static_cast<uint32_t *>(scratch);
  unsigned long long *d_error = reinterpret_cast<unsigned long long *>(static_cast<uint8_t *>(scratch) + 8);
  WB200_CUDA_CHECK(cudaMemsetAsync(d_flags, 0, 8, stream));
  WB200_CUDA_CHECK(cudaMemsetAsync(d_error, 0xff, 8, stream));
  const bool can_refuse = integer_width(route.destination) != 0 || route.source == WB200_TF32;
  unsigned long long error = ~0ull;
  if (can_refuse) {
    launch_formal_convert(stream, route.source, route.destination, mode, src, dst, src_map, dst_map, 0, d_flags, d_error);
    WB200_CUDA_CHECK(cudaGetLastError());
    backend->launches += 1;
    WB200_CUDA_CHECK(cudaMemcpyAsync(&error, d_error, sizeof(error), cudaMemcpyDeviceToHost, stream));
    WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
    if (error != ~0ull) return refusal(error);
  }
  launch_formal_convert(stream, route.source, route.destination, mode, src, dst, src_map, dst_map, 1, d_flags, d_error);
  WB200_CUDA_CHECK(cudaGetLastError());
  backend->launches += 1;
  uint32_t host_flags = 0;
  WB200_CUDA_CHECK(cudaMemcpyAsync(&host_flags, d_flags, sizeof(host_flags), cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  if (flags) *flags = host_flags;
  return WB200_OK;
}


struct ImageConvert {
  Route route;
  int mode;
  LayoutMap src_map, dst_map;
  const uint8_t *src;
  uint8_t *dst;
};

// Route, mode and 1-D Tensor placement of one wafer_tx81_convert_<route> call on a scratch-pad image.
wb200_status plan_image_convert(wb200_spm_image *image, uint32_t opcode, uint64_t source, uint64_t destination, uint32_t count,
                                uint32_t rounding_mode, ImageConvert *plan) {
  if (!image) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  wb200_status st = check_route(opcode, rounding_mode, &plan->route, &plan->mode);
  if (st != WB200_OK) return st;
  if (count == 0) return fail(WB200_ERR_INVALID_ARGUMENT, "convert element count must be positive");
  auto vector = [&](int format) {
    wb200_tensor_desc d{};
    d.format = static_cast<uint8_t>(format);
    d.layout = WB200_LAYOUT_TENSOR;
    d.rank = 1;
    d.shape[0] = count;
    return d;
  };
  wb200_geometry src_geo, dst_geo;
  if ((st = make_layout_map(vector(plan->route.source), &plan->src_map, &src_geo)) != WB200_OK) return st;
  if ((st = make_layout_map(vector(plan->route.destination), &plan->dst_map, &dst_geo)) != WB200_OK) return st;
  if ((st = image_range(image, source, src_geo.physical_bytes, "convert source")) != WB200_OK) return st;
  if ((st = image_range(image, destination, dst_geo.physical_bytes, "convert destination")) != WB200_OK) return st;
  plan->src = image->device ? image->device + (source - image->base) : nullptr;
  plan->dst = image->device ? image->device + (destination - image->base) : nullptr;
  return WB200_OK;
}

}  // namespace

namespace wb200 {

// The same call without a host round trip, for command streams that are captured into a graph: elements the reference
// refuses are reported through `d_error` (smallest element << 8 | code) for the caller to read after the stream.
wb200_status enqueue_image_convert(wb200_spm_image *image, uint32_t opcode, uint64_t source, uint64_t destination, uint32_t count,
                                   uint32_t rounding_mode, bool execute, uint32_t *d_flags, unsigned long long *d_error) {
  ImageConvert plan;
  wb200_status st = plan_image_convert(image, opcode, source, destination, count, rounding_mode, &plan);
  if (st != WB200_OK || !execute) return st;
  launch_formal_convert(image->work_stream(), plan.route.source, plan.route.destination, plan.mode, plan.src, plan.dst, plan.src_map, plan.dst_map, 1, d_flags, d_error);
  WB200_CUDA_CHECK(cudaGetLastError());
  image->backend->launches += 1;
  return WB200_OK;
}

wb200_status convert_refusal(unsigned long long key) { return refusal(key); }

}  // namespace wb200

extern "C" {

wb200_status wb200_convert_formal(wb200_backend *backend, const wb200_convert_request *r, wb200_evidence *evidence) {
  if (!backend || !r) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  Route route;
  int mode;
  wb200_status st = check_route(r->opcode, r->rounding_mode, &route, &mode);
  if (st != WB200_OK) return st;
  const wb200_tensor_desc &src = r->source, &dst = r->destination;
  if (src.format != route.source || dst.format != route.destination)
    return fail(WB200_ERR_INVALID_ARGUMENT, "source-format-mismatch: convert descriptors do not have the route's formats");
  if (!same_shape(src, dst)) return fail(WB200_ERR_INVALID_ARGUMENT, "convert tensors do not have one same-shape domain");
  LayoutMap src_map, dst_map;
  wb200_geometry src_geo, dst_geo;
  if ((st = check_storage(src, r->source_bytes, r->source_storage, "source", &src_map, &src_geo)) != WB200_OK) return st;
  if ((st = check_storage(dst, r->destination_bytes, r->destination_template, "destination template", &dst_map, &dst_geo)) != WB200_OK) return st;
  if (!r->destination_out) return fail(WB200_ERR_INVALID_ARGUMENT, "destination_out is null");
  if ((st = check_budget(backend, dst_map.element_count, r->max_scalar_evaluations, r->source_bytes + r->destination_bytes,
                         2 * static_cast<uint64_t>(dst_map.element_count))) != WB200_OK) return st;
  DeviceGuard guard(backend->device);
  cudaStream_t stream = backend->stream;
  void *d_src, *d_dst;
  if ((st = backend->buffer(0, r->source_bytes, &d_src)) != WB200_OK) return st;
  if ((st = backend->buffer(2, r->destination_bytes, &d_dst)) != WB200_OK) return st;
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_src, r->source_storage, r->source_bytes, cudaMemcpyHostToDevice, stream));
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_dst, r->destination_template, r->destination_bytes, cudaMemcpyHostToDevice, stream));
  uint32_t flags = 0;
  const uint64_t before = backend->launches;
  if ((st = backend->timing_begin(stream)) != WB200_OK) return st;
  if ((st = run_convert(backend, route, mode, static_cast<const uint8_t *>(d_src), static_cast<uint8_t *>(d_dst), src_map, dst_map, stream, &flags)) != WB200_OK) return st;
  if ((st = backend->timing_end(stream)) != WB200_OK) return st;
  WB200_CUDA_CHECK(cudaMemcpyAsync(r->destination_out, d_dst, r->destination_bytes, cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  fill_evidence(backend, evidence, "sm100a-formal-convert");
  if (evidence) {
    evidence->device_us = backend->timing_microseconds();
    evidence->scalar_evaluations = dst_map.element_count;
    evidence->gpu_launches = static_cast<uint32_t>(backend->launches - before);
    evidence->flags = flags;
  }
  return WB200_OK;
}

wb200_status wb200_target_call_convert(wb200_spm_image *image, uint32_t opcode, uint64_t source, uint64_t destination, uint32_t count,
                                       uint32_t zero_point, uint32_t rounding_mode, uint32_t *flags) {
  (void)zero_point;   // only the zero-point routes read it, and those are declined
  ImageConvert plan;
  wb200_status st = plan_image_convert(image, opcode, source, destination, count, rounding_mode, &plan);
  if (st != WB200_OK) return st;
  DeviceGuard guard(image->backend->device);
  return run_convert(image->backend, plan.route, plan.mode, plan.src, plan.dst, plan.src_map, plan.dst_map, image->work_stream(), flags);
}

}  // extern "C"
