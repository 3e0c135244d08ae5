// Correctly rounded unary functions for binary32 operands (and, with 11 bits of precision, TF32): the reference's MPFR
// family (lib/Wafer/Simulator/Reference/Numeric/MPFRNumeric.cpp:439-520, 553-682) evaluates the exact function and rounds
// it once to nearest-even; this file reaches the same bits without multi-precision arithmetic.
//
// Every function is first evaluated in binary64 (error a few units in the last place of binary64). If the value minus
// and plus 2^-47 of itself round to the same result, that result is the correctly rounded one (Ziv's rounding test).
// Otherwise - about one operand in four million - the function is evaluated again in double-double arithmetic (two
// binary64 numbers, about 100 significant bits: argument reduction with multi-word constants or exact integer arithmetic,
// Taylor series, Newton corrections) and rounded once from there. The hardest binary32 cases of these functions need
// fewer than 70 bits. The code compiles for the host too: the generator of the golden vectors scans the complete
// binary32 operand space with it to find the operands that take the second step.
#pragma once

#include <math.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define WB200_HD __host__ __device__ __forceinline__
#else
#define WB200_HD inline
#endif

namespace wb200 {
namespace ff32 {

struct dd {
  double hi, lo;
};

WB200_HD dd two_sum(double a, double b) {
  const double s = a + b, bb = s - a;
  return {s, (a - (s - bb)) + (b - bb)};
}
WB200_HD dd quick_two_sum(double a, double b) {   // |a| >= |b|
  const double s = a + b;
  return {s, b - (s - a)};
}
WB200_HD dd two_prod(double a, double b) {
  const double p = a * b;
  return {p, fma(a, b, -p)};
}
WB200_HD dd dd_add(dd a, dd b) {
  dd s = two_sum(a.hi, b.hi);
  const dd t = two_sum(a.lo, b.lo);
  s.lo += t.hi;
  s = quick_two_sum(s.hi, s.lo);
  s.lo += t.lo;
  return quick_two_sum(s.hi, s.lo);
}
WB200_HD dd dd_add_d(dd a, double b) {
  dd s = two_sum(a.hi, b);
  s.lo += a.lo;
  return quick_two_sum(s.hi, s.lo);
}
WB200_HD dd dd_neg(dd a) { return {-a.hi, -a.lo}; }
WB200_HD dd dd_sub(dd a, dd b) { return dd_add(a, dd_neg(b)); }
WB200_HD dd dd_mul(dd a, dd b) {
  dd p = two_prod(a.hi, b.hi);
  p.lo += a.hi * b.lo + a.lo * b.hi;
  return quick_two_sum(p.hi, p.lo);
}
WB200_HD dd dd_mul_d(dd a, double b) {
  dd p = two_prod(a.hi, b);
  p.lo += a.lo * b;
  return quick_two_sum(p.hi, p.lo);
}
WB200_HD dd dd_div(dd a, dd b) {
  const double q1 = a.hi / b.hi;
  dd r = dd_sub(a, dd_mul_d(b, q1));
  const double q2 = r.hi / b.hi;
  r = dd_sub(r, dd_mul_d(b, q2));
  const double q3 = r.hi / b.hi;
  dd q = quick_two_sum(q1, q2);
  return dd_add_d(q, q3);
}
WB200_HD dd dd_ldexp(dd a, int e) { return {ldexp(a.hi, e), ldexp(a.lo, e)}; }

// ---------------------------------------------------------------- e^r - 1 for |r| <= 0.36 (double-double in and out)
// Argument scaled by 2^-10, a degree-10 Taylor series, then ten applications of E(2s) = E(s) (E(s) + 2).
WB200_HD dd expm1_reduced(dd r) {
  const dd s = dd_ldexp(r, -10);
  // Horner on s: E = s (1 + s/2 (1 + s/3 (1 + ... (1 + s/10))))
  dd e = {1.0, 0.0};
  for (int n = 10; n >= 2; --n) {
    e = dd_mul(e, s);
    e = dd_div(e, dd{static_cast<double>(n), 0.0});
    e = dd_add_d(e, 1.0);
  }
  e = dd_mul(e, s);
  for (int i = 0; i < 10; ++i) e = dd_mul(e, dd_add_d(e, 2.0));
  return e;
}

// ln 2 in three pieces, the first with 32 significant bits so that k * kLn2A is exact for |k| < 2^20.
constexpr double kLn2A = 0x1.62e42fee00000p-1, kLn2B = 0x1.a39ef35793c76p-33, kLn2C = 0x1.cc01f97b57a08p-87;
constexpr dd kLn2 = {0x1.62e42fefa39efp-1, 0x1.abc9e3b39803fp-56};
constexpr dd kInvLn2 = {0x1.71547652b82fep+0, 0x1.777d0ffda0d24p-56};
constexpr dd kPio2 = {0x1.921fb54442d18p+0, 0x1.1a62633145c07p-54};

// e^x = (1 + E) 2^k for a binary64 x with |x| < 2^12: returns E (|E| <= 0.42) and k.
WB200_HD dd exp_parts(double x, int *k_out) {
  const double kd = rint(x * 0x1.71547652b82fep+0);
  dd r = two_sum(x, -kd * kLn2A);              // exact product, exact sum
  r = dd_add(r, dd_neg(two_prod(kd, kLn2B)));
  r = dd_add_d(r, -kd * kLn2C);
  *k_out = static_cast<int>(kd);
  return expm1_reduced(r);
}
// The same for a double-double argument (used with r = f ln 2).
WB200_HD dd exp_parts_dd(dd x, int *k_out) {
  const double kd = rint(x.hi * 0x1.71547652b82fep+0);
  dd r = two_sum(x.hi, -kd * kLn2A);
  r = dd_add_d(r, x.lo);
  r = dd_add(r, dd_neg(two_prod(kd, kLn2B)));
  r = dd_add_d(r, -kd * kLn2C);
  *k_out = static_cast<int>(kd);
  return expm1_reduced(r);
}
// e^x - 1 for a binary64 x, |x| < 2^10.
WB200_HD dd expm1_dd(double x) {
  int k;
  const dd e = exp_parts(x, &k);
  if (k == 0) return e;
  // (1 + E) 2^k - 1: no cancellation worth speaking of, since |x| > 0.34 here
  return dd_add_d(dd_ldexp(dd_add_d(e, 1.0), k), -1.0);
}

// ln(x) for a binary64 x > 0: one Newton step on y -> e^y from the binary64 logarithm doubles its accuracy.
WB200_HD dd log_dd(double x) {
  const double y0 = log(x);
  int k;
  const dd e = exp_parts(-y0, &k);
  // p = x e^(-y0) = x 2^k (1 + E) = 1 + delta
  const double xs = ldexp(x, k);
  dd p = dd_add_d(dd_mul_d(e, xs), xs);     // xs E + xs
  const dd delta = dd_add_d(p, -1.0);
  // ln(1 + delta) = delta - delta^2 / 2 + ..., |delta| < 2^-50
  dd correction = dd_add_d(delta, -0.5 * delta.hi * delta.hi);
  return dd_add(dd{y0, 0.0}, correction);
}

// ln(1 + u) for a double-double u in (0, 1]: Newton from the binary64 log1p, without forming 1 + u.
WB200_HD dd log1p_dd(dd u) {
  const double y0 = log1p(u.hi);
  const dd e = expm1_dd(-y0);                               // e^(-y0) - 1
  // (1 + u)(1 + E) - 1 = E + u + u E: E is about -y0 and u about +y0, the sum is tiny and exact to the last bits
  dd delta = dd_add(dd_add(e, u), dd_mul(u, e));
  delta = dd_add_d(delta, -0.5 * delta.hi * delta.hi);
  return dd_add(dd{y0, 0.0}, delta);
}

// ---------------------------------------------------------------- sine and cosine
// x = r + q pi/2 with |r| <= pi/4 for a binary32 x (given as binary64): q mod 4 and r in double-double. The product of
// the 24-bit significand with a 224-bit window of 2/pi is formed in integer arithmetic, so the reduction is exact up to
// the window's last bits (more than 150 bits below the binary point).
WB200_HD dd reduce_pio2(double x, int *quadrant) {
  // 2 / pi, 512 bits after the binary point, most significant word first.
  constexpr uint32_t kTwoOverPi[16] = {0xa2f9836eu, 0x4e441529u, 0xfc2757d1u, 0xf534ddc0u, 0xdb629599u, 0x3c439041u, 0xfe5163abu, 0xdebbc561u,
                                       0xb7246e3au, 0x424dd2e0u, 0x06492eeau, 0x09d1921cu, 0xfe1deb1cu, 0xb129a73eu, 0xe88235f5u, 0x2ebb4484u};
  const double ax = fabs(x);
  if (ax <= 0.75) {
    *quadrant = 0;
    return {x, 0.0};
  }
  int e;
  const double mantissa = frexp(ax, &e);                         // ax = mantissa 2^e, mantissa in [0.5, 1)
  const uint64_t m = static_cast<uint64_t>(ldexp(mantissa, 24));  // 24-bit integer, ax = m 2^(e - 24)
  // ax 2/pi = m 2^(e-24) sum_i b_i 2^-i. Bits of 2/pi with i < e - 24 - 1 only add multiples of 4 to the quotient. The
  // window starts at bit position `first` (1-based), 224 bits long.
  int first = e - 24 - 1;
  if (first < 1) first = 1;
  uint32_t window[7];
  for (int w = 0; w < 7; ++w) {
    const int bit = first - 1 + 32 * w;                           // 0-based bit offset into the table
    const int word = bit >> 5, shift = bit & 31;
    const uint32_t hi_word = word < 16 ? kTwoOverPi[word] : 0u, lo_word = word + 1 < 16 ? kTwoOverPi[word + 1] : 0u;
    window[w] = shift ? (hi_word << shift) | (lo_word >> (32 - shift)) : hi_word;
  }
  // product = m * window: 24 + 224 bits in eight 32-bit limbs (limb 0 most significant)
  uint32_t product[8];
  uint64_t carry = 0;
  for (int w = 6; w >= 0; --w) {
    const uint64_t t = m * window[w] + carry;
    product[w + 1] = static_cast<uint32_t>(t);
    carry = t >> 32;
  }
  product[0] = static_cast<uint32_t>(carry);
  // The window's first bit has weight 2^-first, so the product, read as an integer of 256 bits, has its unit at weight
  // 2^(e - 24 - first - 223). The binary point of ax 2/pi therefore sits `point` bits from the product's least significant end.
  const int point = first + 223 - (e - 24);                      // >= 223 + 2 - ... always within the 256 bits
  // Extract the two integer bits just above the binary point and 160 fraction bits below it.
  auto bit_at = [&](int position_from_lsb) -> uint32_t {          // position 0 = least significant bit of product[7]
    if (position_from_lsb < 0 || position_from_lsb > 255) return 0u;
    const int limb = 7 - (position_from_lsb >> 5);
    return (product[limb] >> (position_from_lsb & 31)) & 1u;
  };
  int q = static_cast<int>(bit_at(point) | (bit_at(point + 1) << 1));
  // fraction as three 53-bit-safe pieces: take 3 x 48 bits below the point
  double fraction_hi = 0.0, fraction_mid = 0.0, fraction_lo = 0.0;
  {
    uint64_t piece[3] = {0, 0, 0};
    for (int i = 0; i < 144; ++i) {
      const uint32_t b = bit_at(point - 1 - i);
      piece[i / 48] = (piece[i / 48] << 1) | b;
    }
    fraction_hi = ldexp(static_cast<double>(piece[0]), -48);
    fraction_mid = ldexp(static_cast<double>(piece[1]), -96);
    fraction_lo = ldexp(static_cast<double>(piece[2]), -144);
  }
  dd fraction = quick_two_sum(fraction_hi, fraction_mid);
  fraction = dd_add_d(fraction, fraction_lo);
  if (fraction.hi >= 0.5) {                                       // nearest multiple: fraction in [-0.5, 0.5)
    fraction = dd_add_d(fraction, -1.0);
    q += 1;
  }
  dd r = dd_mul(fraction, kPio2);
  // third piece of pi/2 for the product's tail
  r = dd_add_d(r, fraction.hi * -0x1.f1976b7ed8fbcp-110);
  if (x < 0.0) {
    r = dd_neg(r);
    q = -q;
  }
  *quadrant = q & 3;
  return r;
}
// sin r and cos r for |r| <= pi/4 + a little, by Taylor series in double-double.
WB200_HD void sincos_reduced(dd r, dd *sine, dd *cosine) {
  const dd r2 = dd_mul(r, r);
  // sin r = r (1 - r2/6 (1 - r2/20 (1 - ... ))) with terms up to r^31; cos r likewise up to r^30
  dd s = {1.0, 0.0}, c = {1.0, 0.0};
  for (int n = 15; n >= 1; --n) {
    s = dd_div(dd_mul(s, r2), dd{static_cast<double>((2 * n) * (2 * n + 1)), 0.0});
    s = dd_sub(dd{1.0, 0.0}, s);
    c = dd_div(dd_mul(c, r2), dd{static_cast<double>((2 * n - 1) * (2 * n)), 0.0});
    c = dd_sub(dd{1.0, 0.0}, c);
  }
  *sine = dd_mul(s, r);
  *cosine = c;
}

// ---------------------------------------------------------------- rounding to the result format
enum { kInvalid = 1, kDivByZero = 2, kOverflow = 4, kUnderflow = 8, kInexact = 16 };

WB200_HD float float_toward_zero(double v) {
  float f = static_cast<float>(v);
  if (fabs(static_cast<double>(f)) > fabs(v)) f = nextafterf(f, 0.0f);
  return f;
}
// Round-to-odd binary32 of the exact sum hi + lo (|lo| far below an ulp of hi): the 24-bit truncation with its last bit
// forced to one whenever anything was cut off. A later rounding to fewer bits from this value is correct.
WB200_HD uint32_t round_to_odd_bits(dd v) {
  const float t = float_toward_zero(v.hi);
  uint32_t bits;
  {
    union { float f; uint32_t u; } pun;
    pun.f = t;
    bits = pun.u;
  }
  const double back = static_cast<double>(t);
  if (back != v.hi) return bits | 1u;
  if (v.lo == 0.0 || isinf(t)) return bits;
  const bool away = (v.lo > 0.0) == (v.hi > 0.0);                  // the tail points away from zero
  if (v.hi == 0.0) return bits;
  if (away) return bits | 1u;
  // the exact value lies just inside of t: between t's predecessor (toward zero) and t
  return (bits & 1u) ? bits : ((bits - 1u) | 1u);
}
// Nearest-even binary32 of hi + lo.
WB200_HD uint32_t round_nearest_f32(dd v) {
  const float nearest = static_cast<float>(v.hi);
  union { float f; uint32_t u; } pun;
  pun.f = nearest;
  // A representable hi is the answer (the tail is far below half an ulp); so is the nearest value of any hi that is not
  // exactly half way between two neighbours: such midpoints are binary64 numbers, so a different hi lies at least one
  // binary64 ulp away from them, more than the tail.
  if (v.lo == 0.0 || isinf(nearest) || static_cast<double>(nearest) == v.hi) return pun.u;
  // hi is not representable: is it exactly half way between its two neighbours?
  const float down = static_cast<double>(nearest) <= v.hi ? nearest : nextafterf(nearest, -INFINITY);
  const float up = nextafterf(down, INFINITY);
  const double below = v.hi - static_cast<double>(down), above = static_cast<double>(up) - v.hi;   // both exact
  if (below != above) return pun.u;
  pun.f = v.lo > 0.0 ? up : down;                                  // the tail breaks the tie
  return pun.u;
}
// Nearest-even to TF32 (8 exponent bits, 10 fraction bits in storage bits 31..13) from hi + lo.
WB200_HD uint32_t round_nearest_tf32(dd v) {
  const uint32_t odd = round_to_odd_bits(v);
  if ((odd & 0x7f800000u) == 0x7f800000u) return odd & 0xff800000u;          // infinite after the first step
  const uint32_t rounded = odd + 0x0fffu + ((odd >> 13) & 1u);
  return rounded & 0xffffe000u;
}

WB200_HD bool tiny_after_rounding_dd(double value, int precision, double min_normal) {
  if (value == 0.0) return false;
  int exponent;
  const double mantissa = frexp(fabs(value), &exponent);
  const double rounded = ldexp(rint(ldexp(mantissa, precision)), exponent - precision);
  return rounded < min_normal;
}

enum Function { kSqrt, kRsqrt, kLog2, kLn, kPow2, kExp, kSin, kCos, kTanh, kSigmoid, kSoftplus };

// The accurate step: the function of a finite, non-special binary32 operand x (as binary64) in double-double.
WB200_HD dd evaluate_dd(int function, double x) {
  switch (function) {
    case kSqrt: {
      const double y = sqrt(x);
      // y + (x - y^2) / (2 y)
      const dd square = two_prod(y, y);
      const dd residual = dd_add_d(dd_neg(square), x);
      return dd_add_d(dd{y, 0.0}, residual.hi / (2.0 * y));
    }
    case kRsqrt: {
      const double y = 1.0 / sqrt(x);
      // y + y (1 - x y^2) / 2
      const dd y2 = two_prod(y, y);
      const dd t = dd_add_d(dd_neg(dd_mul_d(y2, x)), 1.0);
      return dd_add(dd{y, 0.0}, dd_mul_d(t, 0.5 * y));
    }
    case kLn:
      return log_dd(x);
    case kLog2: {
      int e;
      const double mantissa = frexp(x, &e);                    // [0.5, 1)
      // log2 x = e + ln(mantissa) / ln 2, with mantissa moved to [0.75, 1.5) so that the two terms do not cancel
      double m = mantissa;
      if (m < 0.75) { m *= 2.0; e -= 1; }
      return dd_add_d(dd_mul(log_dd(m), kInvLn2), static_cast<double>(e));
    }
    case kPow2: {
      const double n = rint(x), f = x - n;                     // exact
      int k;
      const dd e = exp_parts_dd(dd_mul_d(kLn2, f), &k);
      return dd_ldexp(dd_add_d(e, 1.0), k + static_cast<int>(n));
    }
    case kExp: {
      int k;
      const dd e = exp_parts(x, &k);
      return dd_ldexp(dd_add_d(e, 1.0), k);
    }
    case kSin:
    case kCos: {
      int q;
      const dd r = reduce_pio2(x, &q);
      dd s, c;
      sincos_reduced(r, &s, &c);
      if (function == kCos) q += 1;                           // cos x = sin(x + pi/2)
      switch (q & 3) {
        case 0: return s;
        case 1: return c;
        case 2: return dd_neg(s);
        default: return dd_neg(c);
      }
    }
    case kTanh: {
      const dd e = expm1_dd(2.0 * x);                           // |x| < 20
      return dd_div(e, dd_add_d(e, 2.0));
    }
    case kSigmoid: {
      int k;
      if (x >= 0.0) {                                         // 1 / (1 + e^-x)
        const dd e = exp_parts(-x, &k);
        return dd_div(dd{1.0, 0.0}, dd_add_d(dd_ldexp(dd_add_d(e, 1.0), k), 1.0));
      }
      const dd e = exp_parts(x, &k);                           // e^x / (1 + e^x), e^x <= 1
      const dd ex = dd_add_d(e, 1.0);                           // mantissa of e^x
      return dd_ldexp(dd_div(ex, dd_add_d(dd_ldexp(ex, k), 1.0)), k);
    }
    default: {                                                // softplus = ln(1 + e^x)
      int k;
      if (x > 0.0) {                                          // x + ln(1 + e^-x)
        const dd e = exp_parts(-x, &k);
        return dd_add_d(log1p_dd(dd_ldexp(dd_add_d(e, 1.0), k)), x);
      }
      const dd e = exp_parts(x, &k);
      const dd ex = dd_ldexp(dd_add_d(e, 1.0), k);               // e^x in (0, 1]
      if (k < -60) {                                          // ln(1 + u) = u - u^2 / 2 to double-double accuracy
        return dd_add_d(ex, -0.5 * ex.hi * ex.hi);
      }
      return log1p_dd(ex);
    }
  }
}

// Binary64 evaluation (the first step). Accurate to a few ulp of binary64.
WB200_HD double evaluate_f64(int function, double x) {
  switch (function) {
    case kSqrt: return sqrt(x);
    case kRsqrt: return 1.0 / sqrt(x);
    case kLog2: return log2(x);
    case kLn: return log(x);
    case kPow2: return exp2(x);
    case kExp: return exp(x);
    case kSin: return sin(x);
    case kCos: return cos(x);
    case kTanh: return tanh(x);
    case kSigmoid: return x >= 0.0 ? 1.0 / (1.0 + exp(-x)) : exp(x) / (1.0 + exp(x));
    default: return x > 0.0 ? x + log1p(exp(-x)) : log1p(exp(x));
  }
}

// Result bits and IEEE flags of `function` for the operand encoding `a` of binary32 (tf32 == false) or TF32 (the 19
// significant bits in 31..13; the low 13 bits must be zero). `*second_step` reports whether the double-double step ran.
WB200_HD uint32_t correctly_rounded(int function, bool tf32, uint32_t a, uint32_t *flags_out, bool *second_step) {
  const uint32_t sign = 0x80000000u, exp_mask = 0x7f800000u, mant_mask = tf32 ? 0x007fe000u : 0x007fffffu;
  const uint32_t canonical_nan = 0x7fc00000u, one = 0x3f800000u, pos_inf = exp_mask, neg_inf = exp_mask | sign;
  const int precision = tf32 ? 11 : 24;
  const double min_normal = 0x1p-126;
  if (second_step) *second_step = false;
  auto finish = [&](uint32_t bits, uint32_t flags) { *flags_out = flags; return bits; };
  if ((a & exp_mask) == exp_mask && (a & 0x007fffffu) != 0) return finish(canonical_nan, (a & 0x00400000u) ? 0u : kInvalid);
  (void)mant_mask;
  const bool negative = (a & sign) != 0, zero = (a & ~sign) == 0, inf = (a & ~sign) == exp_mask;
  union { uint32_t u; float f; } pun;
  pun.u = a;
  const double x = static_cast<double>(pun.f);
  bool exact = false;
  switch (function) {
    case kSqrt:
      if (zero) return finish(a, 0);
      if (negative) return finish(canonical_nan, kInvalid);
      if (inf) return finish(pos_inf, 0);
      break;
    case kRsqrt:
      if (zero) return finish(negative ? neg_inf : pos_inf, kDivByZero);
      if (negative) return finish(canonical_nan, kInvalid);
      if (inf) return finish(0u, 0);
      { int e; exact = frexp(x, &e) == 0.5 && ((e - 1) & 1) == 0; }
      break;
    case kLog2:
    case kLn:
      if (zero) return finish(neg_inf, kDivByZero);
      if (negative) return finish(canonical_nan, kInvalid);
      if (inf) return finish(pos_inf, 0);
      if (function == kLog2) { int e; exact = frexp(x, &e) == 0.5; }
      else exact = x == 1.0;
      break;
    case kPow2:
    case kExp:
      if (inf) return finish(negative ? 0u : pos_inf, 0);
      exact = function == kPow2 ? (x == rint(x)) : zero;
      // far outside the result range: the rounding is decided (and the evaluations below stay in their domain)
      if (x >= 200.0) return finish(pos_inf, kOverflow | kInexact);
      if (x <= -200.0) return finish(0u, kUnderflow | kInexact);
      break;
    case kSin:
    case kCos:
      if (inf) return finish(canonical_nan, kInvalid);
      if (zero) return finish(function == kSin ? a : one, 0);
      break;
    case kTanh:
      if (zero) return finish(a, 0);
      if (inf) return finish(negative ? (one | sign) : one, 0);
      if (fabs(x) >= 20.0) return finish(negative ? (one | sign) : one, kInexact);   // 1 - |tanh| < 2^-56
      break;
    case kSigmoid:
      if (inf) return finish(negative ? 0u : one, 0);
      if (zero) return finish(0x3f000000u, 0);
      if (x >= 32.0) return finish(one, kInexact);
      if (x <= -200.0) return finish(0u, kUnderflow | kInexact);
      break;
    default:
      if (inf) return finish(negative ? 0u : pos_inf, 0);
      if (x >= 32.0) return finish(a, kInexact);                   // softplus(x) - x < e^-32, below 2^-50 of x
      if (x <= -200.0) return finish(0u, kUnderflow | kInexact);
      break;
  }
  // first step
  const double value = evaluate_f64(function, x);
  uint32_t bits;
  {
    const double slack = fabs(value) * 0x1p-47;
    const dd low = {value - slack, 0.0}, high = {value + slack, 0.0};
    const uint32_t bits_low = tf32 ? round_nearest_tf32(low) : round_nearest_f32(low);
    const uint32_t bits_high = tf32 ? round_nearest_tf32(high) : round_nearest_f32(high);
    if (bits_low == bits_high && !exact) {
      bits = bits_low;
    } else {
      if (second_step) *second_step = true;
      const dd accurate = evaluate_dd(function, x);
      bits = tf32 ? round_nearest_tf32(accurate) : round_nearest_f32(accurate);
    }
  }
  uint32_t flags = 0;
  const bool never_zero = function == kPow2 || function == kExp || function == kSigmoid || function == kSoftplus;
  pun.u = bits;
  if ((bits & ~sign) == exp_mask) flags |= kOverflow | kInexact;
  else if ((bits & ~sign) == 0 && never_zero) flags |= kUnderflow | kInexact;
  else if (!exact) {
    // The mathematically exact cases (log2 of a power of two, 2^n, rsqrt of 4^k, ln 1, e^0) have representable results
    // here - the unrepresentable ones were caught above as overflow or as an underflow to zero - and raise nothing,
    // whatever the last bit of the binary64 evaluation says. Everything else is inexact, except perfect squares.
    bool inexact = true;
    if (function == kSqrt) inexact = static_cast<double>(pun.f) * static_cast<double>(pun.f) != x;   // 48-bit product: exact in binary64
    if (inexact) {
      flags |= kInexact;
      if (tiny_after_rounding_dd(value, precision, min_normal)) flags |= kUnderflow;
    }
  }
  return finish(bits, flags);
}

}  // namespace ff32
}  // namespace wb200
