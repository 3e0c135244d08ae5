// oracle.cpp - CPU restatement of the reference's numeric path. TEST INFRASTRUCTURE ONLY (see
// oracle.h). Build with -ffp-contract=off: every rounding below is meant to happen where written.
//
// Each function names the reference file:line whose behaviour it restates (paths inside the
// reference project).
#include "oracle.h"

#include <math.h>
#include <string.h>

#include <algorithm>
#include <limits>
#include <thread>
#include <vector>

namespace {

enum Format { I8 = 0, I16, F16, BF16, I32, F32, TF32, BOOL, U8, U16, U32, I64, U64 };
enum Layout { TENSOR = 0, NTENSOR, CX, NCX };

int format_bits(int f) {
  switch (f) {
    case I8: case U8: return 8;
    case I16: case U16: case F16: case BF16: return 16;
    case I32: case U32: case F32: case TF32: return 32;
    case I64: case U64: return 64;
    case BOOL: return 1;
    default: return 0;
  }
}
bool is_float(int f) { return f == F16 || f == BF16 || f == F32; }

float bits_to_float(uint32_t b) { float v; memcpy(&v, &b, 4); return v; }
uint32_t float_to_bits(float v) { uint32_t b; memcpy(&b, &v, 4); return b; }

// f16 -> f32, exact. lib/Wafer/Simulator/Reference/ManagedReferenceTargetModel.cpp:60-86 and
// lib/Wafer/Simulator/OneDNN/OneDNNGemmAdapter.cpp:60-79 perform this same widening.
uint32_t widen_f16(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  const uint32_t exponent = (h >> 10) & 0x1fu;
  uint32_t fraction = h & 0x3ffu;
  if (exponent == 0) {
    if (fraction == 0) return sign;
    int e = -14;
    while (!(fraction & 0x400u)) { fraction <<= 1; --e; }
    return sign | (static_cast<uint32_t>(e + 127) << 23) | ((fraction & 0x3ffu) << 13);
  }
  if (exponent == 31) return sign | 0x7f800000u | (fraction << 13);
  return sign | ((exponent + 112u) << 23) | (fraction << 13);
}

uint32_t widen(int format, uint32_t bits) {
  if (format == F32) return bits;
  if (format == BF16) return bits << 16;
  return widen_f16(static_cast<uint16_t>(bits));
}

// f32 -> f16 round-to-nearest-even (ManagedReferenceTargetModel.cpp:88-135); NaN -> 0x7e00
// (canonical quiet NaN, lib/Wafer/Simulator/Reference/Formal/FormalNumericGemm.cpp:131-139).
uint16_t narrow_f16(uint32_t f) {
  const uint16_t sign = static_cast<uint16_t>((f >> 16) & 0x8000u);
  const uint32_t exponent_bits = (f >> 23) & 0xffu;
  const uint32_t fraction = f & 0x7fffffu;
  if (exponent_bits == 0xff) return fraction ? 0x7e00 : static_cast<uint16_t>(sign | 0x7c00);
  const int e = static_cast<int>(exponent_bits) - 127;
  if (e > 15) return static_cast<uint16_t>(sign | 0x7c00);
  if (e >= -14) {
    uint32_t out_e = static_cast<uint32_t>(e + 15), out_f = fraction >> 13;
    const uint32_t rest = fraction & 0x1fffu;
    if (rest > 0x1000u || (rest == 0x1000u && (out_f & 1u))) {
      if (++out_f == 0x400u) { out_f = 0; if (++out_e >= 0x1fu) return static_cast<uint16_t>(sign | 0x7c00); }
    }
    return static_cast<uint16_t>(sign | (out_e << 10) | out_f);
  }
  if (e < -25) return sign;
  const uint32_t significand = fraction | 0x800000u;
  const uint32_t shift = static_cast<uint32_t>(-e - 1);
  uint32_t out_f = significand >> shift;
  const uint32_t rest = significand & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rest > half || (rest == half && (out_f & 1u))) ++out_f;
  return static_cast<uint16_t>(sign | out_f);  // out_f == 0x400 lands exactly on the smallest normal
}

// f32 -> bf16 round-to-nearest-even (target convert route fp32_bf16,
// lib/Wafer/Target/PhysicalTensor/TargetScalarConversion.cpp:279-322); NaN -> 0x7fc0.
uint16_t narrow_bf16(uint32_t f) {
  if ((f & 0x7f800000u) == 0x7f800000u && (f & 0x7fffffu)) return 0x7fc0;
  const uint32_t lsb = (f >> 16) & 1u;
  return static_cast<uint16_t>((f + 0x7fffu + lsb) >> 16);
}

uint32_t narrow(int format, uint32_t f32_bits) {
  if (format == F32) {
    if ((f32_bits & 0x7f800000u) == 0x7f800000u && (f32_bits & 0x7fffffu)) return 0x7fc00000u;
    return f32_bits;
  }
  if (format == BF16) return narrow_bf16(f32_bits);
  return narrow_f16(f32_bits);
}

uint32_t load_bits(const void *base, int64_t i, int format) {
  if (format == F32) return static_cast<const uint32_t *>(base)[i];
  return static_cast<const uint16_t *>(base)[i];
}
void store_bits(void *base, int64_t i, int format, uint32_t bits) {
  if (format == F32) static_cast<uint32_t *>(base)[i] = bits;
  else static_cast<uint16_t *>(base)[i] = static_cast<uint16_t>(bits);
}
float load_value(const void *base, int64_t i, int format) { return bits_to_float(widen(format, load_bits(base, i, format))); }
void store_value(void *base, int64_t i, int format, float v) { store_bits(base, i, format, narrow(format, float_to_bits(v))); }

// ---------------------------------------------------------------- physical layout
// lib/Wafer/Target/PhysicalTensor/PhysicalLayout.cpp:51-85 (tail decision), :111-200 (geometry),
// :249-310 (offsets).
struct Geometry {
  int layout = 0, rank = 0, bits = 0;
  int64_t shape[8] = {0};
  int64_t count = 1;
  oracle_geometry g{};
};

int64_t align_tail(int64_t t) { return t <= 4 ? 4 : t <= 8 ? 8 : t <= 16 ? 16 : t <= 32 ? 32 : 64; }

bool make_geometry(int format, int layout, int rank, const uint64_t *shape, Geometry *out) {
  const int bits = format_bits(format);
  if (!bits || rank < 1 || rank > 8 || layout < 0 || layout > NCX) return false;
  Geometry G;
  G.layout = layout; G.rank = rank; G.bits = bits;
  for (int d = 0; d < rank; ++d) { G.shape[d] = static_cast<int64_t>(shape[d]); G.count *= G.shape[d]; }
  G.g.element_bytes = (bits + 7) / 8;
  G.g.compact_bytes = (G.count * bits + 7) / 8;
  if (layout == TENSOR || layout == NTENSOR) {
    G.g.physical_elements = G.count;
    G.g.physical_bytes = (G.count * bits + 7) / 8;
  } else {
    const bool int8 = format == I8 || format == U8;
    const int64_t block = int8 ? 128 : 64, keep = int8 ? 64 : 32;
    const int64_t channels = G.shape[rank - 1], q = channels / block, r = channels % block;
    if (r == 0) { G.g.cx_blocks = q; G.g.c0 = 0; G.g.aligned_c = q * block; }
    else if (r <= keep) { G.g.cx_blocks = q; G.g.c0 = align_tail(r); G.g.aligned_c = q * block + G.g.c0; }
    else { G.g.cx_blocks = q + 1; G.g.c0 = 0; G.g.aligned_c = (q + 1) * block; }
    if (2048 % bits) return false;
    G.g.c_block = block;
    G.g.bank_align_elements = 2048 / bits;
    int64_t slices = 1, block_outer = 1;
    if (layout == NCX) {
      slices = rank > 1 ? G.shape[0] : 1;
      for (int d = 1; d + 1 < rank; ++d) block_outer *= G.shape[d];
    } else {
      for (int d = 0; d + 1 < rank; ++d) block_outer *= G.shape[d];
    }
    const int64_t unpadded = block_outer * G.g.aligned_c;
    const int64_t stride = (unpadded + G.g.bank_align_elements - 1) / G.g.bank_align_elements * G.g.bank_align_elements;
    G.g.block_outer_elements = block_outer;
    G.g.outer_elements = slices * block_outer;
    G.g.outer_slice_stride_elements = stride;
    G.g.physical_elements = slices * stride;
    G.g.physical_bytes = (G.g.physical_elements * bits + 7) / 8;
  }
  *out = G;
  return true;
}

// Physical element index of a logical coordinate.
int64_t physical_element(const Geometry &G, const int64_t *index) {
  if (G.layout == TENSOR || G.layout == NTENSOR) {
    int64_t linear = 0;
    for (int d = 0; d < G.rank; ++d) linear = linear * G.shape[d] + index[d];
    return linear;
  }
  const int64_t c = index[G.rank - 1];
  const int first_outer = G.layout == NCX ? 1 : 0;
  int64_t outer = 0;
  for (int d = first_outer; d + 1 < G.rank; ++d) outer = outer * G.shape[d] + index[d];
  int64_t base = 0;
  if (G.layout == NCX && G.rank > 1) base = index[0] * G.g.outer_slice_stride_elements;
  const int64_t full_c = G.g.cx_blocks * G.g.c_block;
  if (c < full_c)
    return base + (c / G.g.c_block) * (G.g.block_outer_elements * G.g.c_block) + outer * G.g.c_block + c % G.g.c_block;
  return base + G.g.cx_blocks * G.g.block_outer_elements * G.g.c_block + outer * G.g.c0 + (c - full_c);
}

template <typename Fn>
void for_each_coordinate(const Geometry &G, Fn fn) {
  if (G.count == 0) return;
  int64_t index[8] = {0};
  int64_t linear = 0;
  while (true) {
    fn(linear++, index);
    int d = G.rank - 1;
    for (; d >= 0; --d) {
      if (++index[d] < G.shape[d]) break;
      index[d] = 0;
    }
    if (d < 0) return;
  }
}

template <typename Fn>
void parallel_for(int64_t count, int threads, Fn fn) {
  if (threads <= 1 || count < 2) { for (int64_t i = 0; i < count; ++i) fn(i); return; }
  if (threads > count) threads = static_cast<int>(count);
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t)
    pool.emplace_back([=] { for (int64_t i = t; i < count; i += threads) fn(i); });
  for (auto &th : pool) th.join();
}

}  // namespace

extern "C" {

int oracle_physical_geometry(int format, int layout, int rank, const uint64_t *shape, oracle_geometry *out) {
  Geometry G;
  if (!make_geometry(format, layout, rank, shape, &G)) return 1;
  *out = G.g;
  return 0;
}

int64_t oracle_physical_bit_offset(int format, int layout, int rank, const uint64_t *shape, const int64_t *index) {
  Geometry G;
  if (!make_geometry(format, layout, rank, shape, &G)) return -1;
  for (int d = 0; d < rank; ++d) if (index[d] < 0 || index[d] >= G.shape[d]) return -1;
  return physical_element(G, index) * G.bits;
}

// lib/Wafer/Target/PhysicalTensor/PhysicalTensorCodec.h:57-73: logical values are written into a copy
// of the template; every byte no logical value maps to keeps the template's value.
int oracle_pack(int format, int layout, int rank, const uint64_t *shape, const uint8_t *compact,
                const uint8_t *storage_template, uint8_t *storage_out) {
  Geometry G;
  if (!make_geometry(format, layout, rank, shape, &G) || G.bits < 8) return 1;
  if (storage_out != storage_template) memcpy(storage_out, storage_template, static_cast<size_t>(G.g.physical_bytes));
  const int64_t eb = G.g.element_bytes;
  for_each_coordinate(G, [&](int64_t linear, const int64_t *index) {
    memcpy(storage_out + physical_element(G, index) * eb, compact + linear * eb, static_cast<size_t>(eb));
  });
  return 0;
}

int oracle_unpack(int format, int layout, int rank, const uint64_t *shape, const uint8_t *storage, uint8_t *compact_out) {
  Geometry G;
  if (!make_geometry(format, layout, rank, shape, &G) || G.bits < 8) return 1;
  const int64_t eb = G.g.element_bytes;
  for_each_coordinate(G, [&](int64_t linear, const int64_t *index) {
    memcpy(compact_out + linear * eb, storage + physical_element(G, index) * eb, static_cast<size_t>(eb));
  });
  return 0;
}

uint32_t oracle_widen_to_f32_bits(int format, uint32_t bits) { return widen(format, bits); }
uint32_t oracle_narrow_from_f32_bits(int format, uint32_t f32_bits) { return narrow(format, f32_bits); }

// lib/Wafer/Simulator/Reference/Numeric/FormalTensorNumeric.cpp:271-361: per output, accumulator
// +0f, k ascending, one correctly rounded f32 FMA per step
// (lib/Wafer/Simulator/Reference/Formal/FormalNumericGemm.cpp:81-85), then `acc + psum` as an f32
// add (:319-327), then one RNE conversion to the destination format (:115-157). A NaN accumulator is
// replaced by the canonical quiet NaN after every step (:102-107), which the final narrowing
// reproduces because any NaN narrows to the canonical NaN.
int oracle_formal_gemm(int in_format, int out_format, int batch, int m, int k, int n, int lhs_transposed,
                       int rhs_transposed, const void *lhs, const void *rhs, const float *psum, void *out, int threads) {
  if (!is_float(in_format) || !is_float(out_format)) return 2;
  const int64_t outputs = static_cast<int64_t>(batch) * m * n;
  parallel_for(outputs, threads, [&](int64_t index) {
    const int64_t col = index % n, row = (index / n) % m, b = index / (static_cast<int64_t>(m) * n);
    const int64_t lhs_base = b * m * k, rhs_base = b * k * n;
    float acc = 0.0f;
    for (int64_t kk = 0; kk < k; ++kk) {
      const float a = load_value(lhs, lhs_base + (lhs_transposed ? kk * m + row : row * k + kk), in_format);
      const float w = load_value(rhs, rhs_base + (rhs_transposed ? col * k + kk : kk * n + col), in_format);
      acc = fmaf(a, w, acc);
    }
    if (psum) acc = acc + psum[index];
    store_value(out, index, out_format, acc);
  });
  return 0;
}

}  // extern "C"

// ---------------------------------------------------------------- managed-reference commands
namespace {

// lib/Wafer/Simulator/Reference/ManagedReferenceTargetModel.cpp:265-270: multiply by log2(e) in f32,
// then exp2 in f32.
float exp_lp(float x) { return exp2f(x * 0x1.715476p+0F); }

// One f32 operation per element (ManagedReferenceTargetModel.cpp:230-299). Ordinals are the
// reference's TargetElementwiseOperation (include/Wafer/Target/TargetOperation.h:58-93).
bool evaluate_elementwise(int op, float x, float y, float *out) {
  switch (op) {
    case 0: *out = fabsf(x); return true;                       // abs
    case 1: *out = 1.0F / x; return true;                       // recip
    case 2: *out = x * x; return true;                          // square
    case 3: *out = sqrtf(x); return true;                       // sqrt
    case 4: *out = 1.0F / sqrtf(x); return true;                // rsqrt
    case 5: *out = -x; return true;                             // neg
    case 6: *out = fmaxf(x, y); return true;                    // max
    case 7: *out = fminf(x, y); return true;                    // min
    case 8: *out = x + y; return true;                          // add
    case 9: *out = x - y; return true;                          // sub
    case 10: *out = x * y; return true;                         // mul
    case 22: *out = log2f(x); return true;
    case 23: *out = logf(x); return true;
    case 24: *out = exp2f(x); return true;
    case 25: *out = expf(x); return true;
    case 26: *out = exp_lp(x); return true;
    case 27: *out = sinf(x); return true;
    case 28: *out = cosf(x); return true;
    case 29: *out = tanhf(x); return true;
    case 30: *out = x >= 0.0F ? 1.0F / (1.0F + expf(-x)) : expf(x) / (1.0F + expf(x)); return true;
    case 31: *out = x < 0.0F ? 0.0F : x; return true;           // relu
    case 34: *out = fmaxf(x, 0.0F) + log1pf(expf(-fabsf(x))); return true;  // softplus
    default: return false;
  }
}

int elementwise_arity(int op) { return (op >= 6 && op <= 10) ? 2 : 1; }

}  // namespace

extern "C" {

int oracle_elementwise(int op, int format, int64_t count, const void *in0, const void *in1, void *out) {
  if (!is_float(format)) return 2;
  const int arity = elementwise_arity(op);
  for (int64_t i = 0; i < count; ++i) {
    const float x = load_value(in0, i, format);
    const float y = arity == 2 ? load_value(in1, i, format) : 0.0F;
    if (x != x || y != y) return 3;  // decodeNonNaN, :137-155
    float r;
    if (!evaluate_elementwise(op, x, y, &r)) return 2;
    if (r != r) return 3;            // encodeNonNaN, :157-160
    store_value(out, i, format, r);
  }
  return 0;
}

// ManagedReferenceTargetModel.cpp:344-379: decode to f32 (exact), encode RNE.
int oracle_convert(int src_format, int dst_format, int64_t count, const void *src, void *dst) {
  if (!is_float(src_format) || !is_float(dst_format)) return 2;
  for (int64_t i = 0; i < count; ++i) {
    const float x = load_value(src, i, src_format);
    if (x != x) return 3;
    store_value(dst, i, dst_format, x);
  }
  return 0;
}

// ManagedReferenceTargetModel.cpp:381-458: running f32 accumulator per output, inputs visited in
// row-major order; signed-zero rule for max/min (:435-439); identities -inf / +inf / 0 (:403-407).
int oracle_reduce(int op, int format, int rank, const uint64_t *shape, uint32_t reduced_mask, const void *src, void *dst) {
  if (!is_float(format) || op < 0 || op > 2 || (op == 0 && format != F32) || rank < 1 || rank > 8) return 2;
  int64_t total = 1, outputs = 1;
  for (int d = 0; d < rank; ++d) {
    total *= static_cast<int64_t>(shape[d]);
    if (!(reduced_mask & (1u << d))) outputs *= static_cast<int64_t>(shape[d]);
  }
  const float identity = op == 1 ? -INFINITY : op == 2 ? INFINITY : 0.0F;
  std::vector<float> acc(static_cast<size_t>(outputs), identity);
  for (int64_t i = 0; i < total; ++i) {
    int64_t remaining = i, coord[8];
    for (int d = rank - 1; d >= 0; --d) { coord[d] = remaining % static_cast<int64_t>(shape[d]); remaining /= static_cast<int64_t>(shape[d]); }
    int64_t o = 0;
    for (int d = 0; d < rank; ++d) if (!(reduced_mask & (1u << d))) o = o * static_cast<int64_t>(shape[d]) + coord[d];
    const float v = load_value(src, i, format);
    if (v != v) return 3;
    float &a = acc[static_cast<size_t>(o)];
    if (op == 0) a += v;
    else if (a == 0.0F && v == 0.0F) {
      const bool negative = op == 1 ? (signbit(a) && signbit(v)) : (signbit(a) || signbit(v));
      a = negative ? -0.0F : 0.0F;
    } else a = op == 1 ? fmaxf(a, v) : fminf(a, v);
    if (a != a) return 3;
  }
  for (int64_t o = 0; o < outputs; ++o) store_value(dst, o, format, acc[static_cast<size_t>(o)]);
  return 0;
}

}  // extern "C"

// ---------------------------------------------------------------- attention
namespace {

struct RowState {
  float m = -INFINITY, l = 0.0F;
  std::vector<float> acc;
};

// One online update over keys [key_begin, key_end) of one query row, in steps of tile_n keys.
// Steps 1-11 of lib/Wafer/Transforms/Linalg/OnlineAttentionDecomposition.cpp:568-594. The two
// contractions are evaluated the way the lowered GEMM commands evaluate them: a k-ascending f32 FMA
// chain from +0, then added to the scaled old accumulator through the psum port
// (FormalTensorNumeric.cpp:301-327); exp is ExpLp. `visible_end` already folds the causal and
// valid-length masks of the row (OnlineAttentionDecomposition.cpp:319-331): keys >= visible_end
// score -inf.
void online_update(const oracle_attention &p, const float *q_row, const void *k, const void *v, int64_t kv_base,
                   int64_t key_begin, int64_t key_end, int64_t visible_end, RowState &st, std::vector<float> &scores) {
  const int D = p.head_dim;
  const int tile = p.tile_n > 0 ? p.tile_n : 128;
  for (int64_t t0 = key_begin; t0 < key_end; t0 += tile) {
    const int64_t t1 = std::min<int64_t>(t0 + tile, key_end);
    const int count = static_cast<int>(t1 - t0);
    float tile_max = -INFINITY;
    for (int j = 0; j < count; ++j) {
      const int64_t key = t0 + j;
      float s;
      if (key >= visible_end) s = -INFINITY;                    // additive 0 / -inf mask template
      else {
        float dot = 0.0F;
        const int64_t row = kv_base + key * D;
        for (int d = 0; d < D; ++d) dot = fmaf(q_row[d], load_value(k, row + d, p.format), dot);
        s = dot * p.scale;                                       // step 2
      }
      scores[j] = s;
      tile_max = fmaxf(tile_max, s);
    }
    const float m_new = fmaxf(tile_max, st.m);                   // step 3
    const float m_exp = m_new == -INFINITY ? 0.0F : m_new;       // step 4
    const float alpha = exp_lp(st.m - m_exp);                    // step 5
    float l = st.l * alpha;                                      // step 6
    for (int j = 0; j < count; ++j) {
      scores[j] = exp_lp(scores[j] - m_exp);                     // step 7
      l += scores[j];                                            // step 8 (un-rounded P)
    }
    st.l = l;
    st.m = m_new;
    for (int j = 0; j < count; ++j)                              // step 10: P rounded to V's storage type
      scores[j] = bits_to_float(widen(p.format, narrow(p.format, float_to_bits(scores[j]))));
    for (int d = 0; d < D; ++d) {
      float pv = 0.0F;
      for (int j = 0; j < count; ++j)
        pv = fmaf(scores[j], load_value(v, kv_base + (t0 + j) * D + d, p.format), pv);
      st.acc[d] = pv + st.acc[d] * alpha;                        // steps 9 and 11
    }
  }
}

int64_t visible_end_for(const oracle_attention &p, int64_t row) {
  int64_t end = p.key_end > 0 ? p.key_end - p.key_start : p.kv_len;
  if (end > p.kv_len) end = p.kv_len;
  if (p.causal) end = std::min<int64_t>(end, (p.query_start - p.key_start) + row + 1);
  return std::max<int64_t>(end, 0);
}

// lib/Wafer/Transforms/Linalg/OnlineAttentionMaterialization.cpp:264-373
void merge_states(RowState &left, const RowState &right) {
  const float m = fmaxf(left.m, right.m);
  const float m_exp = m == -INFINITY ? 0.0F : m;
  const float sl = exp_lp(left.m - m_exp), sr = exp_lp(right.m - m_exp);
  left.l = left.l * sl + right.l * sr;
  for (size_t d = 0; d < left.acc.size(); ++d) left.acc[d] = left.acc[d] * sl + right.acc[d] * sr;
  left.m = m;
}

// OnlineAttentionMaterialization.cpp:196-262
void finalize_row(const RowState &st, int format, int zero_fully_masked, void *out, int64_t out_base, float *lse,
                  float *row_max, float *row_sum, int64_t stat_index) {
  float c = 1.0F / st.l;
  if (zero_fully_masked && st.l == 0.0F) c = 0.0F;
  for (size_t d = 0; d < st.acc.size(); ++d) store_value(out, out_base + static_cast<int64_t>(d), format, st.acc[d] * c);
  if (lse) lse[stat_index] = st.l == 0.0F ? -INFINITY : st.m + logf(st.l);
  if (row_max) row_max[stat_index] = st.m;
  if (row_sum) row_sum[stat_index] = st.l;
}

// Runs rows of (batch*heads*q_len); `splits` independent online passes per row, left-folded.
int run_attention(const oracle_attention &p, int splits, float *state_out) {
  if (!is_float(p.format) || p.kv_heads <= 0 || p.q_heads % p.kv_heads || splits < 1) return 2;
  const int D = p.head_dim, group = p.q_heads / p.kv_heads;
  const int64_t rows = static_cast<int64_t>(p.batch) * p.q_heads * p.q_len;
  parallel_for(rows, p.threads, [&](int64_t r) {
    const int64_t qi = r % p.q_len, bh = r / p.q_len;
    const int64_t b = bh / p.q_heads, h = bh % p.q_heads;
    const int64_t kv_base = (b * p.kv_heads + h / group) * static_cast<int64_t>(p.kv_len) * D;
    std::vector<float> q_row(D), scores(p.tile_n > 0 ? p.tile_n : 128);
    for (int d = 0; d < D; ++d) q_row[d] = load_value(p.q, r * D + d, p.format);
    const int64_t visible = visible_end_for(p, qi);
    RowState total;
    total.acc.assign(D, 0.0F);
    if (splits == 1) {
      online_update(p, q_row.data(), p.k, p.v, kv_base, 0, visible, visible, total, scores);
    } else {
      // K2 split into `splits` contiguous intervals of the visible range (rounded up to 64 keys like
      // the device kernel's granule so both fold the same partition).
      int64_t per = (visible + splits - 1) / splits;
      per = (per + 63) / 64 * 64;
      if (per == 0) per = 64;
      for (int s = 0; s < splits; ++s) {
        RowState part;
        part.acc.assign(D, 0.0F);
        const int64_t begin = std::min<int64_t>(s * per, visible), end = std::min<int64_t>(begin + per, visible);
        online_update(p, q_row.data(), p.k, p.v, kv_base, begin, end, visible, part, scores);
        if (s == 0) total = part;
        else merge_states(total, part);
      }
    }
    if (state_out) {
      float *dst = state_out + r * (D + 2);
      for (int d = 0; d < D; ++d) dst[d] = total.acc[d];
      dst[D] = total.m;
      dst[D + 1] = total.l;
    } else {
      finalize_row(total, p.format, p.zero_fully_masked, p.out, r * D, p.lse, p.row_max, p.row_sum, r);
    }
  });
  return 0;
}

}  // namespace

extern "C" {

int oracle_attention_fa(const oracle_attention *p) { return run_attention(*p, 1, nullptr); }
int oracle_attention_fd(const oracle_attention *p, int splits) { return run_attention(*p, splits, nullptr); }
int oracle_attention_fd_state(const oracle_attention *p, int splits, float *state) { return run_attention(*p, splits, state); }

int oracle_attention_fd_merge(int rows, int head_dim, int format, int zero_fully_masked, int shards, const float *states,
                              void *out, float *lse) {
  if (!is_float(format) || shards < 1) return 2;
  const int rec = head_dim + 2;
  for (int r = 0; r < rows; ++r) {
    RowState total;
    for (int s = 0; s < shards; ++s) {
      const float *src = states + (static_cast<int64_t>(s) * rows + r) * rec;
      RowState part;
      part.acc.assign(src, src + head_dim);
      part.m = src[head_dim];
      part.l = src[head_dim + 1];
      if (s == 0) total = part;
      else merge_states(total, part);
    }
    finalize_row(total, format, zero_fully_masked, out, static_cast<int64_t>(r) * head_dim, lse, nullptr, nullptr, r);
  }
  return 0;
}

// dot_general -> (+bias) -> (GELU by erf) -> single narrowing. Accumulation is the formal GEMM's
// k-ascending f32 FMA chain; the f32 elementwise chain is applied before the only rounding
// (lib/Wafer/Transforms/Linalg/ContractionAccumulation.cpp:147-218).
int oracle_gemm_epilogue(int in_format, int out_format, int m, int n, int k, int lhs_transposed, int rhs_transposed,
                         int epilogue, const void *a, const void *b, const float *bias, void *out, int threads) {
  if (!is_float(in_format) || !is_float(out_format)) return 2;
  // Widen once so the inner loop is a plain f32 FMA chain.
  std::vector<float> A(static_cast<size_t>(m) * k), B(static_cast<size_t>(k) * n);
  for (int64_t i = 0; i < static_cast<int64_t>(m) * k; ++i) {
    const int64_t row = i / k, kk = i % k;
    A[i] = load_value(a, lhs_transposed ? kk * m + row : i, in_format);
  }
  for (int64_t i = 0; i < static_cast<int64_t>(k) * n; ++i) {  // stored [n][k] for unit-stride reads
    const int64_t col = i / k, kk = i % k;
    B[i] = load_value(b, rhs_transposed ? col * k + kk : kk * n + col, in_format);
  }
  parallel_for(m, threads, [&](int64_t row) {
    for (int col = 0; col < n; ++col) {
      float acc = 0.0F;
      const float *ar = &A[static_cast<size_t>(row) * k], *bc = &B[static_cast<size_t>(col) * k];
      for (int kk = 0; kk < k; ++kk) acc = fmaf(ar[kk], bc[kk], acc);
      if (epilogue >= 1) acc = acc + bias[col];
      if (epilogue == 2) acc = 0.5F * acc * (1.0F + erff(acc * 0.70710678118654752440F));
      store_value(out, row * n + col, out_format, acc);
    }
  });
  return 0;
}

// lib/Wafer/Simulator/Invocation/ProgramTensorComparison.cpp:20-52 (similarity in long double),
// :149-176 (ULP order key, nearest-rank quantiles), :341-352 (tolerance atol + rtol*|expected|).
int oracle_compare(int format, int64_t count, const void *actual, const void *expected, double atol, double rtol,
                   oracle_comparison *out) {
  if (!is_float(format)) return 2;
  memset(out, 0, sizeof(*out));
  out->element_count = static_cast<uint64_t>(count);
  out->finite = 1;
  out->cosine = 1.0;
  if (count == 0) return 0;
  const unsigned width = format == F32 ? 32 : 16;
  auto key = [&](uint32_t bits) -> uint64_t {
    const uint64_t sign = 1ull << (width - 1), mag = bits & (sign - 1);
    return (bits & sign) ? sign - mag : sign + mag;
  };
  std::vector<double> abs_err(static_cast<size_t>(count));
  std::vector<uint64_t> ulp(static_cast<size_t>(count));
  long double dot = 0, aa = 0, ee = 0, err2 = 0, abs_sum = 0, ulp_sum = 0;
  for (int64_t i = 0; i < count; ++i) {
    const uint32_t ab = load_bits(actual, i, format), eb = load_bits(expected, i, format);
    const double a = bits_to_float(widen(format, ab)), e = bits_to_float(widen(format, eb));
    if (!std::isfinite(a) || !std::isfinite(e)) { out->finite = 0; return 0; }
    const double d = fabs(a - e);
    abs_err[i] = d;
    abs_sum += d;
    out->exact_count += (d == 0.0);  // +0 against -0 counts as exact (:477-478)
    const uint64_t u = a == e ? 0 : (key(ab) >= key(eb) ? key(ab) - key(eb) : key(eb) - key(ab));
    ulp[i] = u;
    ulp_sum += u;
    if (d > atol + rtol * fabs(e)) out->mismatch_count++;
    dot += static_cast<long double>(a) * e; aa += static_cast<long double>(a) * a; ee += static_cast<long double>(e) * e;
    err2 += static_cast<long double>(a - e) * (a - e);
  }
  std::sort(abs_err.begin(), abs_err.end());
  std::sort(ulp.begin(), ulp.end());
  auto rank = [&](double q) { size_t r = static_cast<size_t>(ceil(q * count)); r = std::max<size_t>(1, std::min<size_t>(r, count)); return r - 1; };
  out->mean_abs = static_cast<double>(abs_sum / count);
  out->p99_abs = abs_err[rank(0.99)]; out->p999_abs = abs_err[rank(0.999)]; out->max_abs = abs_err.back();
  out->mean_ulp = static_cast<double>(ulp_sum / count);
  out->p99_ulp = ulp[rank(0.99)]; out->p999_ulp = ulp[rank(0.999)]; out->max_ulp = ulp.back();
  if (aa == 0 || ee == 0) out->cosine = aa == ee ? 1.0 : 0.0;
  else out->cosine = static_cast<double>(std::min<long double>(1.0L, std::max<long double>(-1.0L, dot / sqrtl(aa) / sqrtl(ee))));
  out->relative_l2 = ee == 0 ? (err2 == 0 ? 0.0 : std::numeric_limits<double>::infinity()) : static_cast<double>(sqrtl(err2 / ee));
  return 0;
}

}  // extern "C"
