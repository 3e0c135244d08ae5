// Expected-output gate on the device: the element decode, absolute error, tolerance, ULP distance, counts, maxima
// and nearest-rank quantiles of lib/Wafer/Simulator/Invocation/ProgramTensorComparison.cpp:276-503, evaluated by one
// statistics pass plus an exact most-significant-digit-first radix select over the two tensors. HBM-bound: every
// pass streams both tensors once (2 * count * element bytes) and keeps its histogram in shared memory.
#include <algorithm>
#include <cmath>
#include <limits>

#include "backend.h"

using namespace wb200;

namespace {

constexpr int kDigitBits = 11;
constexpr int kBins = 1 << kDigitBits;
constexpr int kQueries = 4;
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr unsigned long long kNone = ~0ull;

// A value kept as an unevaluated sum hi + lo of two doubles.
struct DD {
  double hi, lo;
};

__host__ __device__ inline void dd_add(DD &s, double x) {
#ifdef __CUDA_ARCH__
  const double t = __dadd_rn(s.hi, x);
  const double v = __dsub_rn(t, s.hi);
  const double err = __dadd_rn(__dsub_rn(s.hi, __dsub_rn(t, v)), __dsub_rn(x, v));
  s.hi = t;
  s.lo = __dadd_rn(s.lo, err);
#else
  volatile double t = s.hi + x;
  volatile double v = t - s.hi;
  volatile double w = t - v;
  volatile double err = (s.hi - w) + (x - v);
  s.hi = t;
  s.lo = s.lo + err;
#endif
}
__host__ __device__ inline void dd_merge(DD &s, const DD &o) {
  dd_add(s, o.hi);
  s.lo += o.lo;
}

struct Partial {
  unsigned long long exact, mismatch, ulp_sum, max_ulp;
  unsigned long long first_actual_nonfinite, first_expected_nonfinite, first_bad_tolerance, first_mismatch;
  double max_abs;
  double mismatch_max_abs;
  unsigned long long mismatch_max_abs_element;
  double mismatch_max_ratio;  // -1: no mismatch yet
  unsigned long long mismatch_max_ratio_element;
  DD dot, actual_squared, expected_squared, error_squared, abs_sum;
};

__host__ __device__ inline void partial_clear(Partial &p) {
  p.exact = p.mismatch = p.ulp_sum = p.max_ulp = 0;
  p.first_actual_nonfinite = p.first_expected_nonfinite = p.first_bad_tolerance = p.first_mismatch = kNone;
  p.max_abs = 0.0;
  p.mismatch_max_abs = -1.0;
  p.mismatch_max_abs_element = kNone;
  p.mismatch_max_ratio = -1.0;
  p.mismatch_max_ratio_element = kNone;
  p.dot = p.actual_squared = p.expected_squared = p.error_squared = p.abs_sum = DD{0.0, 0.0};
}

// "The first element attaining the largest value": a larger value wins, an equal one only with a smaller index.
__host__ __device__ inline void keep_largest(double &value, unsigned long long &element, double other,
                                             unsigned long long other_element) {
  if (other > value || (other == value && other_element < element)) {
    value = other;
    element = other_element;
  }
}

__host__ __device__ inline void partial_merge(Partial &p, const Partial &o) {
  p.exact += o.exact;
  p.mismatch += o.mismatch;
  p.ulp_sum += o.ulp_sum;
  p.max_ulp = o.max_ulp > p.max_ulp ? o.max_ulp : p.max_ulp;
  p.first_actual_nonfinite = o.first_actual_nonfinite < p.first_actual_nonfinite ? o.first_actual_nonfinite : p.first_actual_nonfinite;
  p.first_expected_nonfinite = o.first_expected_nonfinite < p.first_expected_nonfinite ? o.first_expected_nonfinite : p.first_expected_nonfinite;
  p.first_bad_tolerance = o.first_bad_tolerance < p.first_bad_tolerance ? o.first_bad_tolerance : p.first_bad_tolerance;
  p.first_mismatch = o.first_mismatch < p.first_mismatch ? o.first_mismatch : p.first_mismatch;
  p.max_abs = o.max_abs > p.max_abs ? o.max_abs : p.max_abs;
  keep_largest(p.mismatch_max_abs, p.mismatch_max_abs_element, o.mismatch_max_abs, o.mismatch_max_abs_element);
  keep_largest(p.mismatch_max_ratio, p.mismatch_max_ratio_element, o.mismatch_max_ratio, o.mismatch_max_ratio_element);
  dd_merge(p.dot, o.dot);
  dd_merge(p.actual_squared, o.actual_squared);
  dd_merge(p.expected_squared, o.expected_squared);
  dd_merge(p.error_squared, o.error_squared);
  dd_merge(p.abs_sum, o.abs_sum);
}

// One radix-select question: among the elements whose key agrees with `prefix` above bit shift + kDigitBits, count
// the digit at `shift`. kind 0: the absolute error's f64 bits (monotonic for non-negative values); 1: the ULP distance.
struct Query {
  int kind, shift, active, reserved;
  unsigned long long prefix;
};
struct SelectParams {
  Query query[kQueries];
};

struct Element {
  double abs_error;
  unsigned long long ulp;
};

__device__ __forceinline__ bool finite_bits(uint32_t bits, int format) {
  if (format == WB200_F32) return (bits & 0x7f800000u) != 0x7f800000u;
  if (format == WB200_BF16) return (bits & 0x7f80u) != 0x7f80u;
  return (bits & 0x7c00u) != 0x7c00u;
}

// Sign-magnitude order key of ProgramTensorComparison.cpp:147-152.
__device__ __forceinline__ unsigned long long ulp_order_key(uint32_t bits, int width) {
  const unsigned long long sign = 1ull << (width - 1);
  const unsigned long long magnitude = bits & (sign - 1);
  return (bits & sign) ? sign - magnitude : sign + magnitude;
}

template <bool kStats>
__device__ __forceinline__ Element visit(uint32_t actual_bits, uint32_t expected_bits, unsigned long long element,
                                         int format, double atol, double rtol, Partial &part) {
  const double actual = static_cast<double>(widen_bits(actual_bits, format));
  const double expected = static_cast<double>(widen_bits(expected_bits, format));
  const double difference = __dsub_rn(actual, expected);
  Element e;
  e.abs_error = fabs(difference);
  if (actual == expected) {
    e.ulp = 0;
  } else {
    const int width = format == WB200_F32 ? 32 : 16;
    const unsigned long long ka = ulp_order_key(actual_bits, width), ke = ulp_order_key(expected_bits, width);
    e.ulp = ka >= ke ? ka - ke : ke - ka;
  }
  if (kStats) {
    if (!finite_bits(actual_bits, format) && element < part.first_actual_nonfinite) part.first_actual_nonfinite = element;
    if (!finite_bits(expected_bits, format) && element < part.first_expected_nonfinite) part.first_expected_nonfinite = element;
    const double tolerance = __dadd_rn(atol, __dmul_rn(rtol, fabs(expected)));
    if (!isfinite(tolerance) && element < part.first_bad_tolerance) part.first_bad_tolerance = element;
    part.exact += e.abs_error == 0.0;
    part.ulp_sum += e.ulp;
    part.max_ulp = e.ulp > part.max_ulp ? e.ulp : part.max_ulp;
    part.max_abs = e.abs_error > part.max_abs ? e.abs_error : part.max_abs;
    if (e.abs_error > tolerance) {
      part.mismatch += 1;
      if (element < part.first_mismatch) part.first_mismatch = element;
      keep_largest(part.mismatch_max_abs, part.mismatch_max_abs_element, e.abs_error, element);
      const double ratio = tolerance == 0.0 ? INFINITY : __ddiv_rn(e.abs_error, tolerance);
      keep_largest(part.mismatch_max_ratio, part.mismatch_max_ratio_element, ratio, element);
    }
    // Products of two values of at most 24 significant bits are exact in f64.
    dd_add(part.dot, __dmul_rn(actual, expected));
    dd_add(part.actual_squared, __dmul_rn(actual, actual));
    dd_add(part.expected_squared, __dmul_rn(expected, expected));
    // (actual - expected)^2 from the exact difference d + r: d^2 split by an FMA, plus 2 d r.
    const double v = __dsub_rn(difference, actual);
    const double r = __dadd_rn(__dsub_rn(actual, __dsub_rn(difference, v)), __dsub_rn(-expected, v));
    const double square = __dmul_rn(difference, difference);
    const double square_low = __fma_rn(difference, difference, -square);
    dd_add(part.error_squared, square);
    dd_add(part.error_squared, __dadd_rn(square_low, __dmul_rn(2.0 * difference, r)));
    dd_add(part.abs_sum, e.abs_error);
  }
  return e;
}

__device__ __forceinline__ void count_digits(const Element &e, const SelectParams &params, uint32_t (*histogram)[kBins]) {
#pragma unroll
  for (int q = 0; q < kQueries; ++q) {
    const Query &query = params.query[q];
    if (!query.active) continue;
    const unsigned long long key = query.kind == 0 ? static_cast<unsigned long long>(__double_as_longlong(e.abs_error)) : e.ulp;
    const int above = query.shift + kDigitBits;
    if (above < 64 && (key >> above) != query.prefix) continue;
    atomicAdd(&histogram[q][(key >> query.shift) & (kBins - 1)], 1u);
  }
}

__device__ __forceinline__ double shuffle_down(double v, int delta) { return __shfl_down_sync(0xffffffffu, v, delta); }
__device__ __forceinline__ unsigned long long shuffle_down(unsigned long long v, int delta) {
  return __shfl_down_sync(0xffffffffu, v, delta);
}
__device__ __forceinline__ DD shuffle_down(const DD &v, int delta) {
  return DD{shuffle_down(v.hi, delta), shuffle_down(v.lo, delta)};
}
__device__ __forceinline__ Partial shuffle_down(const Partial &p, int delta) {
  Partial o;
  o.exact = shuffle_down(p.exact, delta);
  o.mismatch = shuffle_down(p.mismatch, delta);
  o.ulp_sum = shuffle_down(p.ulp_sum, delta);
  o.max_ulp = shuffle_down(p.max_ulp, delta);
  o.first_actual_nonfinite = shuffle_down(p.first_actual_nonfinite, delta);
  o.first_expected_nonfinite = shuffle_down(p.first_expected_nonfinite, delta);
  o.first_bad_tolerance = shuffle_down(p.first_bad_tolerance, delta);
  o.first_mismatch = shuffle_down(p.first_mismatch, delta);
  o.max_abs = shuffle_down(p.max_abs, delta);
  o.mismatch_max_abs = shuffle_down(p.mismatch_max_abs, delta);
  o.mismatch_max_abs_element = shuffle_down(p.mismatch_max_abs_element, delta);
  o.mismatch_max_ratio = shuffle_down(p.mismatch_max_ratio, delta);
  o.mismatch_max_ratio_element = shuffle_down(p.mismatch_max_ratio_element, delta);
  o.dot = shuffle_down(p.dot, delta);
  o.actual_squared = shuffle_down(p.actual_squared, delta);
  o.expected_squared = shuffle_down(p.expected_squared, delta);
  o.error_squared = shuffle_down(p.error_squared, delta);
  o.abs_sum = shuffle_down(p.abs_sum, delta);
  return o;
}

// kVec elements per thread and step (16-byte loads when the pointers allow it, else 1).
template <bool kStats, int kBytes, int kVec>
__global__ void __launch_bounds__(kThreads) compare_pass_kernel(const uint8_t *__restrict__ actual,
                                                                 const uint8_t *__restrict__ expected,
                                                                 unsigned long long count, int format, double atol,
                                                                 double rtol, SelectParams params,
                                                                 unsigned long long *__restrict__ histogram_out,
                                                                 Partial *__restrict__ partial_out) {
  __shared__ uint32_t histogram[kQueries][kBins];
  __shared__ Partial warp_partial[kStats ? kWarps : 1];
  for (int i = threadIdx.x; i < kQueries * kBins; i += kThreads) (&histogram[0][0])[i] = 0;
  __syncthreads();

  Partial part;
  partial_clear(part);
  const unsigned long long groups = count / kVec;
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * kThreads;
  for (unsigned long long g = static_cast<unsigned long long>(blockIdx.x) * kThreads + threadIdx.x; g < groups; g += stride) {
    uint32_t a_bits[kVec], e_bits[kVec];
    if (kVec == 1) {
      a_bits[0] = load_element_bits(actual, static_cast<int64_t>(g), format);
      e_bits[0] = load_element_bits(expected, static_cast<int64_t>(g), format);
    } else {
      const uint4 a = reinterpret_cast<const uint4 *>(actual)[g];
      const uint4 e = reinterpret_cast<const uint4 *>(expected)[g];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, ew[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        if (kBytes == 4) {
          a_bits[i] = aw[i];
          e_bits[i] = ew[i];
        } else {
          a_bits[i] = (aw[i / 2] >> ((i & 1) * 16)) & 0xffffu;
          e_bits[i] = (ew[i / 2] >> ((i & 1) * 16)) & 0xffffu;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const Element e = visit<kStats>(a_bits[i], e_bits[i], g * kVec + i, format, atol, rtol, part);
      count_digits(e, params, histogram);
    }
  }
  // Ragged tail (fewer than kVec elements): the last thread of the grid takes it.
  if (kVec > 1 && blockIdx.x == gridDim.x - 1 && threadIdx.x == kThreads - 1) {
    for (unsigned long long element = groups * kVec; element < count; ++element) {
      const Element e = visit<kStats>(load_element_bits(actual, static_cast<int64_t>(element), format),
                                      load_element_bits(expected, static_cast<int64_t>(element), format), element, format,
                                      atol, rtol, part);
      count_digits(e, params, histogram);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kQueries * kBins; i += kThreads) {
    const uint32_t n = (&histogram[0][0])[i];
    if (n) atomicAdd(&histogram_out[i], static_cast<unsigned long long>(n));
  }
  if (kStats) {
    for (int delta = 16; delta > 0; delta >>= 1) {
      const Partial other = shuffle_down(part, delta);
      partial_merge(part, other);
    }
    if ((threadIdx.x & 31) == 0) warp_partial[threadIdx.x >> 5] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
      Partial total = warp_partial[0];
      for (int w = 1; w < kWarps; ++w) partial_merge(total, warp_partial[w]);
      partial_out[blockIdx.x] = total;
    }
  }
}

__global__ void __launch_bounds__(kThreads) compare_raw_kernel(const uint8_t *__restrict__ actual,
                                                                const uint8_t *__restrict__ expected,
                                                                unsigned long long bytes, int wide,
                                                                unsigned long long *__restrict__ first) {
  unsigned long long found = kNone;
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * kThreads;
  const unsigned long long start = static_cast<unsigned long long>(blockIdx.x) * kThreads + threadIdx.x;
  if (wide) {
    const unsigned long long groups = bytes / 16;
    for (unsigned long long g = start; g < groups && found == kNone; g += stride) {
      const uint4 a = reinterpret_cast<const uint4 *>(actual)[g];
      const uint4 e = reinterpret_cast<const uint4 *>(expected)[g];
      if (a.x != e.x || a.y != e.y || a.z != e.z || a.w != e.w) {
        for (int i = 0; i < 16; ++i)
          if (actual[g * 16 + i] != expected[g * 16 + i]) {
            found = g * 16 + i;
            break;
          }
      }
    }
    if (start == 0)
      for (unsigned long long i = groups * 16; i < bytes; ++i)
        if (actual[i] != expected[i]) {
          found = i < found ? i : found;
          break;
        }
  } else {
    for (unsigned long long i = start; i < bytes && found == kNone; i += stride)
      if (actual[i] != expected[i]) found = i;
  }
  if (found != kNone) atomicMin(first, found);
}

template <bool kStats>
wb200_status launch_pass(const uint8_t *actual, const uint8_t *expected, uint64_t count, int format, double atol,
                         double rtol, const SelectParams &params, unsigned long long *histogram, Partial *partials,
                         int blocks, cudaStream_t stream) {
  const bool aligned = ((reinterpret_cast<uintptr_t>(actual) | reinterpret_cast<uintptr_t>(expected)) & 15) == 0;
  if (format == WB200_F32) {
    if (aligned)
      compare_pass_kernel<kStats, 4, 4><<<blocks, kThreads, 0, stream>>>(actual, expected, count, format, atol, rtol, params, histogram, partials);
    else
      compare_pass_kernel<kStats, 4, 1><<<blocks, kThreads, 0, stream>>>(actual, expected, count, format, atol, rtol, params, histogram, partials);
  } else {
    if (aligned)
      compare_pass_kernel<kStats, 2, 8><<<blocks, kThreads, 0, stream>>>(actual, expected, count, format, atol, rtol, params, histogram, partials);
    else
      compare_pass_kernel<kStats, 2, 1><<<blocks, kThreads, 0, stream>>>(actual, expected, count, format, atol, rtol, params, histogram, partials);
  }
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

double decode_host(uint32_t bits, int format) {
  uint32_t word;
  if (format == WB200_F32) {
    word = bits;
  } else if (format == WB200_BF16) {
    word = bits << 16;
  } else {
    const uint32_t sign = (bits >> 15) & 1, exponent = (bits >> 10) & 0x1f, fraction = bits & 0x3ff;
    double value = exponent == 0 ? std::ldexp(static_cast<double>(fraction), -24)
                                 : std::ldexp(static_cast<double>(0x400 | fraction), static_cast<int>(exponent) - 25);
    return sign ? -value : value;
  }
  float f;
  memcpy(&f, &word, sizeof(f));
  return static_cast<double>(f);
}

wb200_status fetch_value(const uint8_t *device, uint64_t element, int format, cudaStream_t stream, double *out) {
  const size_t width = format == WB200_F32 ? 4 : 2;
  uint32_t bits = 0;
  WB200_CUDA_CHECK(cudaMemcpyAsync(&bits, device + element * width, width, cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  *out = decode_host(bits, format);
  return WB200_OK;
}

// raw_ostream << double: "%e", with "nan", "INF" and "-INF" spelled out (llvm/lib/Support/NativeFormatting.cpp write_double).
std::string format_e(double value) {
  if (std::isnan(value)) return "nan";
  if (std::isinf(value)) return value < 0 ? "-INF" : "INF";
  char buffer[48];
  snprintf(buffer, sizeof(buffer), "%e", value);
  return buffer;
}

// "element=<i> actual=<a> expected=<e> abs_error=<d> tolerance=<t>" (ProgramTensorComparison.cpp:167-176); the
// reference streams doubles through raw_ostream, which prints them as "%e".
wb200_status mismatch_sample(const uint8_t *actual, const uint8_t *expected, uint64_t element, int format, double atol,
                             double rtol, cudaStream_t stream, std::string *text, double *abs_error, double *tolerance) {
  double a, e;
  wb200_status st;
  if ((st = fetch_value(actual, element, format, stream, &a)) != WB200_OK) return st;
  if ((st = fetch_value(expected, element, format, stream, &e)) != WB200_OK) return st;
  volatile double product = rtol * std::fabs(e);
  *tolerance = atol + product;
  *abs_error = std::fabs(a - e);
  *text = "element=" + std::to_string(element) + " actual=" + format_e(a) + " expected=" + format_e(e) +
          " abs_error=" + format_e(*abs_error) + " tolerance=" + format_e(*tolerance);
  return WB200_OK;
}

void set_detail(wb200_comparison *out, const std::string &text) {
  strncpy(out->detail, text.c_str(), sizeof(out->detail) - 1);
  out->detail[sizeof(out->detail) - 1] = 0;
}

uint64_t nearest_rank_index(double quantile, uint64_t count) {
  uint64_t rank = static_cast<uint64_t>(std::ceil(quantile * static_cast<double>(count)));
  rank = std::max<uint64_t>(1, std::min<uint64_t>(rank, count));
  return rank - 1;
}

}  // namespace

extern "C" wb200_status wb200_compare(wb200_backend *backend, uint32_t format, uint64_t count, const void *actual,
                                      const void *expected, uint32_t memory, double atol, double rtol,
                                      uint32_t use_similarity, double minimum_cosine, double maximum_relative_l2,
                                      wb200_comparison *out) {
  if (!backend || !out) return fail(WB200_ERR_INVALID_ARGUMENT, "wb200_compare: backend and out must not be null");
  memset(out, 0, sizeof(*out));
  if (format != WB200_F16 && format != WB200_BF16 && format != WB200_F32)
    return fail(WB200_ERR_UNSUPPORTED, "wb200_compare: the tolerant comparison covers f16, bf16 and f32 only");
  if (count && (!actual || !expected)) return fail(WB200_ERR_INVALID_ARGUMENT, "wb200_compare: null tensor pointer");
  if (memory != WB200_MEM_HOST && memory != WB200_MEM_DEVICE) return fail(WB200_ERR_INVALID_ARGUMENT, "wb200_compare: bad memory kind");
  out->element = kNone;
  out->first_mismatch = out->max_abs_mismatch = out->max_ratio_mismatch = kNone;
  out->cosine = 1.0;
  // validateProgramTensorComparisonPolicy (ProgramTensorComparison.cpp:505-524).
  if (!std::isfinite(atol) || !std::isfinite(rtol) || atol < 0.0 || rtol < 0.0) {
    out->outcome = WB200_CMP_INVALID_TOLERANCE;
    set_detail(out, "absolute and relative tolerances must be finite and nonnegative");
    return WB200_OK;
  }
  if (use_similarity && (!std::isfinite(minimum_cosine) || minimum_cosine < 0.0 || minimum_cosine > 1.0 ||
                         !std::isfinite(maximum_relative_l2) || maximum_relative_l2 < 0.0)) {
    out->outcome = WB200_CMP_INVALID_TOLERANCE;
    set_detail(out, "similarity requires finite minimum cosine in [0,1] and nonnegative relative L2");
    return WB200_OK;
  }
  if (count == 0) {
    if (use_similarity) {
      out->outcome = WB200_CMP_EMPTY;
      set_detail(out, "similarity requires a non-empty tensor");
    }
    return WB200_OK;
  }

  DeviceGuard guard(backend->device);
  cudaStream_t stream = backend->stream;
  const size_t width = format == WB200_F32 ? 4 : 2;
  const uint8_t *d_actual = static_cast<const uint8_t *>(actual), *d_expected = static_cast<const uint8_t *>(expected);
  wb200_status st;
  if (memory == WB200_MEM_HOST) {
    void *slot_a, *slot_e;
    if ((st = backend->buffer(0, count * width, &slot_a)) != WB200_OK) return st;
    if ((st = backend->buffer(1, count * width, &slot_e)) != WB200_OK) return st;
    WB200_CUDA_CHECK(cudaMemcpyAsync(slot_a, actual, count * width, cudaMemcpyHostToDevice, stream));
    WB200_CUDA_CHECK(cudaMemcpyAsync(slot_e, expected, count * width, cudaMemcpyHostToDevice, stream));
    d_actual = static_cast<const uint8_t *>(slot_a);
    d_expected = static_cast<const uint8_t *>(slot_e);
  }
  const uint64_t per_block = static_cast<uint64_t>(kThreads) * 8;
  const int blocks = static_cast<int>(std::max<uint64_t>(1, std::min<uint64_t>((count + per_block - 1) / per_block,
                                                                                 static_cast<uint64_t>(backend->sm_count) * 4)));
  const size_t histogram_bytes = sizeof(unsigned long long) * kQueries * kBins;
  void *scratch;
  if ((st = backend->buffer(3, histogram_bytes + sizeof(Partial) * blocks, &scratch)) != WB200_OK) return st;
  unsigned long long *d_histogram = static_cast<unsigned long long *>(scratch);
  Partial *d_partials = reinterpret_cast<Partial *>(static_cast<uint8_t *>(scratch) + histogram_bytes);

  // Queries 0, 1: p99 / p99.9 of the absolute error (63 key bits, six digits); 2, 3: of the ULP distance (at most
  // 33 key bits, three digits, answered in the first three passes).
  const uint64_t rank[kQueries] = {nearest_rank_index(0.99, count), nearest_rank_index(0.999, count),
                                   nearest_rank_index(0.99, count), nearest_rank_index(0.999, count)};
  uint64_t remaining[kQueries] = {rank[0], rank[1], rank[2], rank[3]};
  uint64_t prefix[kQueries] = {0, 0, 0, 0};
  std::vector<unsigned long long> histogram(kQueries * kBins);
  std::vector<Partial> partials(blocks);
  Partial total;
  partial_clear(total);
  const int abs_shift[6] = {55, 44, 33, 22, 11, 0};
  const int ulp_shift[3] = {22, 11, 0};
  for (int pass = 0; pass < 6; ++pass) {
    SelectParams params{};
    for (int q = 0; q < kQueries; ++q) {
      Query &query = params.query[q];
      query.kind = q / 2;
      query.active = query.kind == 0 || pass < 3;
      query.shift = query.kind == 0 ? abs_shift[pass] : ulp_shift[pass < 3 ? pass : 2];
      query.prefix = prefix[q];
    }
    // p99 and p99.9 ask the same question until their prefixes part: count it once and share the histogram
    int source_of[kQueries];
    for (int q = 0; q < kQueries; ++q) {
      source_of[q] = q;
      for (int earlier = 0; earlier < q; ++earlier)
        if (params.query[q].active && params.query[earlier].active && params.query[q].kind == params.query[earlier].kind &&
            params.query[q].shift == params.query[earlier].shift && params.query[q].prefix == params.query[earlier].prefix) {
          source_of[q] = earlier;
          break;
        }
    }
    bool wanted[kQueries];
    for (int q = 0; q < kQueries; ++q) {
      wanted[q] = params.query[q].active != 0;
      if (source_of[q] != q) params.query[q].active = 0;
    }
    WB200_CUDA_CHECK(cudaMemsetAsync(d_histogram, 0, histogram_bytes, stream));
    if (pass == 0)
      st = launch_pass<true>(d_actual, d_expected, count, static_cast<int>(format), atol, rtol, params, d_histogram, d_partials, blocks, stream);
    else
      st = launch_pass<false>(d_actual, d_expected, count, static_cast<int>(format), atol, rtol, params, d_histogram, d_partials, blocks, stream);
    if (st != WB200_OK) return st;
    backend->launches += 1;
    WB200_CUDA_CHECK(cudaMemcpyAsync(histogram.data(), d_histogram, histogram_bytes, cudaMemcpyDeviceToHost, stream));
    if (pass == 0)
      WB200_CUDA_CHECK(cudaMemcpyAsync(partials.data(), d_partials, sizeof(Partial) * blocks, cudaMemcpyDeviceToHost, stream));
    WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
    if (pass == 0) {
      for (const Partial &p : partials) partial_merge(total, p);
      // The reference stops at the first offending element, checking actual, expected, then the tolerance.
      const uint64_t first = std::min({total.first_actual_nonfinite, total.first_expected_nonfinite, total.first_bad_tolerance});
      if (first != kNone) {
        out->element = first;
        if (total.first_actual_nonfinite == first) {
          out->outcome = WB200_CMP_ACTUAL_NONFINITE;
          set_detail(out, "element=" + std::to_string(first));
        } else if (total.first_expected_nonfinite == first) {
          out->outcome = WB200_CMP_EXPECTED_NONFINITE;
          set_detail(out, "element=" + std::to_string(first));
        } else {
          out->outcome = WB200_CMP_INVALID_TOLERANCE;
          set_detail(out, "computed tolerance is not finite at element=" + std::to_string(first));
        }
        return WB200_OK;
      }
    }
    for (int q = 0; q < kQueries; ++q) {
      if (!wanted[q]) continue;
      const unsigned long long *bins = histogram.data() + static_cast<size_t>(source_of[q]) * kBins;
      int bin = 0;
      while (bin < kBins - 1 && remaining[q] >= bins[bin]) remaining[q] -= bins[bin++];
      prefix[q] = (prefix[q] << kDigitBits) | static_cast<uint64_t>(bin);
    }
  }

  out->element_count = count;
  out->exact_count = total.exact;
  out->mismatch_count = total.mismatch;
  out->exact_fraction = static_cast<double>(total.exact) / static_cast<double>(count);
  const long double n = static_cast<long double>(count);
  auto wide = [](const DD &v) { return static_cast<long double>(v.hi) + static_cast<long double>(v.lo); };
  out->mean_abs = static_cast<double>(wide(total.abs_sum) / n);
  out->mean_ulp = static_cast<double>(static_cast<long double>(total.ulp_sum) / n);
  memcpy(&out->p99_abs, &prefix[0], sizeof(double));
  memcpy(&out->p999_abs, &prefix[1], sizeof(double));
  out->max_abs = total.max_abs;
  out->p99_ulp = prefix[2];
  out->p999_ulp = prefix[3];
  out->max_ulp = total.max_ulp;
  const long double dot = wide(total.dot), aa = wide(total.actual_squared), bb = wide(total.expected_squared),
                    ee = wide(total.error_squared);
  // TensorSimilarity::cosine / relativeL2 (ProgramTensorComparison.cpp:38-52): zero vectors have an explicit contract.
  if (aa == 0.0L || bb == 0.0L)
    out->cosine = aa == bb ? 1.0 : 0.0;
  else
    out->cosine = static_cast<double>(std::min(1.0L, std::max(-1.0L, dot / std::sqrt(aa) / std::sqrt(bb))));
  if (bb == 0.0L)
    out->relative_l2 = ee == 0.0L ? 0.0 : std::numeric_limits<double>::infinity();
  else
    out->relative_l2 = static_cast<double>(std::sqrt(ee / bb));
  out->first_mismatch = total.first_mismatch;
  out->max_abs_mismatch = total.mismatch_max_abs_element;
  out->max_ratio_mismatch = total.mismatch_max_ratio_element;

  if (use_similarity) {
    if (out->cosine >= minimum_cosine && out->relative_l2 <= maximum_relative_l2) return WB200_OK;
    out->outcome = WB200_CMP_NUMERIC_MISMATCH;
    set_detail(out, "cosine=" + format_e(out->cosine) + " minimum_cosine=" + format_e(minimum_cosine) + " relative_l2=" +
                        format_e(out->relative_l2) + " maximum_relative_l2=" + format_e(maximum_relative_l2) +
                        " elementwise_mismatches=" + std::to_string(total.mismatch) + "/" + std::to_string(count));
    return WB200_OK;
  }
  if (total.mismatch == 0) return WB200_OK;
  out->outcome = WB200_CMP_NUMERIC_MISMATCH;
  out->element = total.first_mismatch;
  std::string first_text, max_abs_text, ratio_text;
  double abs_error, tolerance;
  if ((st = mismatch_sample(d_actual, d_expected, total.first_mismatch, format, atol, rtol, stream, &first_text, &abs_error, &tolerance)) != WB200_OK) return st;
  if ((st = mismatch_sample(d_actual, d_expected, total.mismatch_max_abs_element, format, atol, rtol, stream, &max_abs_text, &abs_error, &tolerance)) != WB200_OK) return st;
  if ((st = mismatch_sample(d_actual, d_expected, total.mismatch_max_ratio_element, format, atol, rtol, stream, &ratio_text, &abs_error, &tolerance)) != WB200_OK) return st;
  const double ratio = tolerance == 0.0 ? std::numeric_limits<double>::infinity() : abs_error / tolerance;
  set_detail(out, "mismatches=" + std::to_string(total.mismatch) + "/" + std::to_string(count) + " first={" + first_text +
                      "} max_abs={" + max_abs_text + "} max_tolerance_ratio=" + format_e(ratio) +
                      " at_element=" + std::to_string(total.mismatch_max_ratio_element));
  return WB200_OK;
}

extern "C" wb200_status wb200_compare_raw(wb200_backend *backend, uint64_t bytes, const void *actual, const void *expected,
                                          uint32_t memory, wb200_comparison *out) {
  if (!backend || !out) return fail(WB200_ERR_INVALID_ARGUMENT, "wb200_compare_raw: backend and out must not be null");
  memset(out, 0, sizeof(*out));
  out->element = kNone;
  out->first_mismatch = out->max_abs_mismatch = out->max_ratio_mismatch = kNone;
  out->cosine = 1.0;
  if (bytes && (!actual || !expected)) return fail(WB200_ERR_INVALID_ARGUMENT, "wb200_compare_raw: null tensor pointer");
  if (memory != WB200_MEM_HOST && memory != WB200_MEM_DEVICE) return fail(WB200_ERR_INVALID_ARGUMENT, "wb200_compare_raw: bad memory kind");
  if (bytes == 0) return WB200_OK;
  DeviceGuard guard(backend->device);
  cudaStream_t stream = backend->stream;
  const uint8_t *d_actual = static_cast<const uint8_t *>(actual), *d_expected = static_cast<const uint8_t *>(expected);
  wb200_status st;
  if (memory == WB200_MEM_HOST) {
    void *slot_a, *slot_e;
    if ((st = backend->buffer(0, bytes, &slot_a)) != WB200_OK) return st;
    if ((st = backend->buffer(1, bytes, &slot_e)) != WB200_OK) return st;
    WB200_CUDA_CHECK(cudaMemcpyAsync(slot_a, actual, bytes, cudaMemcpyHostToDevice, stream));
    WB200_CUDA_CHECK(cudaMemcpyAsync(slot_e, expected, bytes, cudaMemcpyHostToDevice, stream));
    d_actual = static_cast<const uint8_t *>(slot_a);
    d_expected = static_cast<const uint8_t *>(slot_e);
  }
  void *scratch;
  if ((st = backend->buffer(3, sizeof(unsigned long long), &scratch)) != WB200_OK) return st;
  unsigned long long *d_first = static_cast<unsigned long long *>(scratch);
  WB200_CUDA_CHECK(cudaMemsetAsync(d_first, 0xff, sizeof(unsigned long long), stream));
  const int wide = ((reinterpret_cast<uintptr_t>(d_actual) | reinterpret_cast<uintptr_t>(d_expected)) & 15) == 0;
  const uint64_t per_block = static_cast<uint64_t>(kThreads) * (wide ? 64 : 4);
  const int blocks = static_cast<int>(std::max<uint64_t>(1, std::min<uint64_t>((bytes + per_block - 1) / per_block,
                                                                                 static_cast<uint64_t>(backend->sm_count) * 8)));
  compare_raw_kernel<<<blocks, kThreads, 0, stream>>>(d_actual, d_expected, bytes, wide, d_first);
  WB200_CUDA_CHECK(cudaGetLastError());
  backend->launches += 1;
  unsigned long long first = kNone;
  WB200_CUDA_CHECK(cudaMemcpyAsync(&first, d_first, sizeof(first), cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  if (first == kNone) return WB200_OK;
  uint8_t a = 0, e = 0;
  WB200_CUDA_CHECK(cudaMemcpyAsync(&a, d_actual + first, 1, cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaMemcpyAsync(&e, d_expected + first, 1, cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  out->outcome = WB200_CMP_RAW_MISMATCH;
  out->element = first;
  set_detail(out, "byte=" + std::to_string(first) + " actual=" + std::to_string(static_cast<unsigned>(a)) +
                      " expected=" + std::to_string(static_cast<unsigned>(e)));
  return WB200_OK;
}
