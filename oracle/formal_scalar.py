"""TEST INFRASTRUCTURE ONLY - exact-rational restatement of the reference's formal elementwise family.

Follows lib/Wafer/Simulator/Reference/Formal/FormalNumericElementwise.cpp:23-248: operands are decoded to exact
rationals, the operation is carried out exactly, the result is rounded once to the operand format (round to nearest,
ties to even, gradual underflow) and the IEEE flags are derived from the definitions LLVM's APFloat uses (underflow =
the rounded result is subnormal or zero and inexact) plus the reference's own addition for mul / square (:228-238:
also underflow when the exact product, rounded with an unbounded exponent, is below the smallest normal number).
Pinned by the reference's vectors (unittests FormalTensorNumericTest.cpp:189-249, in tests/golden/reference_kats.json
and tests/test_formal_elementwise.py). Pure Python on purpose: small cases only. Only tests may import this module.
"""
from fractions import Fraction

FORMATS = {"f16": (5, 10), "bf16": (8, 7), "f32": (8, 23), "tf32": (8, 10)}   # exponent bits, stored mantissa bits (tf32: the 19-bit encoding, storage bits 31..13)
INVALID, DIV_BY_ZERO, OVERFLOW, UNDERFLOW, INEXACT = 1, 2, 4, 8, 16
RELATIONS = {"eq", "ne", "ge", "gt", "le", "lt"}
LOGIC = {"logic_not", "logic_and", "logic_or", "logic_xor"}
UNARY = {"abs", "neg", "recip", "square", "relu", "logic_not"}


def _layout(fmt):
    e, m = FORMATS[fmt]
    return e, m, (1 << (e - 1)) - 1   # bias


def decode(fmt, bits):
    """-> (kind, negative, value) with kind in nan / snan / inf / zero / finite; value is a Fraction for zero / finite."""
    e, m, bias = _layout(fmt)
    negative = bool(bits >> (e + m))
    exponent = (bits >> m) & ((1 << e) - 1)
    mantissa = bits & ((1 << m) - 1)
    if exponent == (1 << e) - 1:
        if mantissa == 0:
            return "inf", negative, None
        return ("nan" if mantissa >> (m - 1) else "snan"), negative, None
    if exponent == 0:
        value = Fraction(mantissa, 1 << m) * Fraction(2) ** (1 - bias)
    else:
        value = (1 + Fraction(mantissa, 1 << m)) * Fraction(2) ** (exponent - bias)
    if value == 0:
        return "zero", negative, Fraction(0)
    return "finite", negative, -value if negative else value


def canonical_nan(fmt):
    e, m, _ = _layout(fmt)
    return (((1 << e) - 1) << m) | (1 << (m - 1))


def _rne(numerator: Fraction) -> int:
    floor = numerator.numerator // numerator.denominator
    rest = numerator - floor
    if rest > Fraction(1, 2) or (rest == Fraction(1, 2) and floor & 1):
        return floor + 1
    return floor


def round_to_format(fmt, value: Fraction, negative_zero=False):
    """Exact value -> (bits, flags) with one RNE rounding."""
    e, m, bias = _layout(fmt)
    sign = (1 << (e + m)) if (value < 0 or (value == 0 and negative_zero)) else 0
    magnitude = abs(value)
    if magnitude == 0:
        return sign, 0
    exponent = magnitude.numerator.bit_length() - magnitude.denominator.bit_length()
    if Fraction(2) ** exponent > magnitude:
        exponent -= 1                                     # 2^exponent <= magnitude < 2^(exponent + 1)
    emin = 1 - bias
    quantum_exponent = max(exponent, emin) - m            # weight of the last kept bit
    scaled = magnitude / Fraction(2) ** quantum_exponent
    kept = _rne(scaled)
    inexact = Fraction(kept) != scaled
    rounded = Fraction(kept) * Fraction(2) ** quantum_exponent
    flags = INEXACT if inexact else 0
    if rounded >= Fraction(2) ** (bias + 1):              # beyond the largest finite number after rounding
        return sign | (((1 << e) - 1) << m), OVERFLOW | INEXACT
    if rounded < Fraction(2) ** emin:                     # subnormal or zero after rounding
        if inexact:
            flags |= UNDERFLOW
        return sign | kept, flags
    result_exponent = rounded.numerator.bit_length() - rounded.denominator.bit_length()
    if Fraction(2) ** result_exponent > rounded:
        result_exponent -= 1
    mantissa = int(rounded / Fraction(2) ** (result_exponent - m)) - (1 << m)
    return sign | ((result_exponent + bias) << m) | mantissa, flags


def _tiny_after_unbounded_rounding(fmt, value: Fraction) -> bool:
    e, m, bias = _layout(fmt)
    magnitude = abs(value)
    if magnitude == 0:
        return False
    exponent = magnitude.numerator.bit_length() - magnitude.denominator.bit_length()
    if Fraction(2) ** exponent > magnitude:
        exponent -= 1
    quantum = Fraction(2) ** (exponent - m)
    return Fraction(_rne(magnitude / quantum)) * quantum < Fraction(2) ** (1 - bias)


def evaluate(op, fmt, out_fmt, a_bits, b_bits=0):
    """-> (result bits in out_fmt ('bool' gives 0 / 1), flags)."""
    if op in LOGIC:
        lhs, rhs = a_bits != 0, b_bits != 0
        return int({"logic_not": not lhs, "logic_and": lhs and rhs, "logic_or": lhs or rhs, "logic_xor": lhs != rhs}[op]), 0
    binary = op not in UNARY
    ka, na, va = decode(fmt, a_bits)
    kb, nb, vb = decode(fmt, b_bits) if binary else ("zero", False, Fraction(0))
    flags = INVALID if "snan" in (ka, kb) else 0
    has_nan = ka in ("nan", "snan") or kb in ("nan", "snan")
    e, m, _ = _layout(fmt)
    sign_bit = 1 << (e + m)

    def order(kind, negative, value):          # total order key for non-NaN values, zeros equal
        if kind == "inf":
            return (-1 if negative else 1, Fraction(0))
        return (0, value)
    if op in RELATIONS:
        if has_nan:
            truth = op == "ne"
        else:
            x, y = order(ka, na, va), order(kb, nb, vb)
            truth = {"eq": x == y, "ne": x != y, "ge": x >= y, "gt": x > y, "le": x <= y, "lt": x < y}[op]
        if out_fmt == "bool":
            return int(truth), flags
        eo, mo, biaso = _layout(out_fmt)
        return (biaso << mo) if truth else 0, flags
    if has_nan and op in ("abs", "neg", "max", "min", "relu"):
        return canonical_nan(fmt), flags
    if op == "abs":
        return a_bits & ~sign_bit, flags
    if op == "neg":
        return a_bits ^ sign_bit, flags
    if op == "relu":
        return (0 if (na and ka != "zero") else a_bits), flags
    if op in ("max", "min"):
        if ka == "zero" and kb == "zero":
            negative = (na and nb) if op == "max" else (na or nb)
            return (sign_bit if negative else 0), flags
        x, y = order(ka, na, va), order(kb, nb, vb)
        choose_rhs = x < y if op == "max" else x > y
        return (b_bits if choose_rhs else a_bits), flags
    if has_nan:
        return canonical_nan(fmt), flags
    inf_bits = ((1 << e) - 1) << m
    if op == "recip":
        if ka == "zero":
            return (sign_bit if na else 0) | inf_bits, flags | DIV_BY_ZERO
        if ka == "inf":
            return (sign_bit if na else 0), flags
        bits, more = round_to_format(fmt, 1 / va)
        return bits, flags | more
    if op in ("mul", "square"):
        if op == "square":
            kb, nb, vb = ka, na, va
        negative = na != nb
        if "inf" in (ka, kb):
            if "zero" in (ka, kb):
                return canonical_nan(fmt), flags | INVALID
            return (sign_bit if negative else 0) | inf_bits, flags
        product = va * vb
        bits, more = round_to_format(fmt, product, negative_zero=negative)
        if product == 0:
            bits = sign_bit if negative else 0
        if (more & INEXACT) and _tiny_after_unbounded_rounding(fmt, product):
            more |= UNDERFLOW
        return bits, flags | more
    # add / sub
    if op == "sub":
        nb = not nb
        vb = -vb if vb is not None else None
    if "inf" in (ka, kb):
        if ka == "inf" and kb == "inf" and na != nb:
            return canonical_nan(fmt), flags | INVALID
        negative = na if ka == "inf" else nb
        return (sign_bit if negative else 0) | inf_bits, flags
    total = va + vb
    if total == 0:
        negative = na and nb if (ka == "zero" and kb == "zero") else False   # x + (-x) = +0 under round-to-nearest
        return (sign_bit if negative else 0), flags
    bits, more = round_to_format(fmt, total)
    return bits, flags | more


# ------------------------------------------------------------------------------------------------ function family
FUNCTIONS = ("sqrt", "rsqrt", "log2", "ln", "pow2", "exp", "sin", "cos", "tanh", "sigmoid", "softplus")


def evaluate_function(op, fmt, bits):
    """Correctly rounded unary function of the reference's MPFR family
    (lib/Wafer/Simulator/Reference/Numeric/MPFRNumeric.cpp:372-470, 560-682): -> (result bits, flags). The function is
    evaluated with 200 bits (mpmath), converted to an exact rational and rounded once; exactly representable results
    are decided by the mathematics (powers of two, zero, one), not by the 200-bit value."""
    import mpmath
    kind, negative, value = decode(fmt, bits)
    e, m, bias = _layout(fmt)
    sign_bit, inf_bits, one = 1 << (e + m), ((1 << e) - 1) << m, bias << m
    if kind in ("nan", "snan"):
        return canonical_nan(fmt), (INVALID if kind == "snan" else 0)
    zero, inf = kind == "zero", kind == "inf"
    if op == "sqrt":
        if zero:
            return bits, 0
        if negative:
            return canonical_nan(fmt), INVALID
        if inf:
            return inf_bits, 0
    elif op == "rsqrt":
        if zero:
            return (sign_bit if negative else 0) | inf_bits, DIV_BY_ZERO
        if negative:
            return canonical_nan(fmt), INVALID
        if inf:
            return 0, 0
    elif op in ("log2", "ln"):
        if zero:
            return sign_bit | inf_bits, DIV_BY_ZERO
        if negative:
            return canonical_nan(fmt), INVALID
        if inf:
            return inf_bits, 0
    elif op in ("pow2", "exp"):
        if inf:
            return (0 if negative else inf_bits), 0
    elif op in ("sin", "cos"):
        if inf:
            return canonical_nan(fmt), INVALID
        if zero:
            return (bits if op == "sin" else one), 0
    elif op == "tanh":
        if zero:
            return bits, 0
        if inf:
            return (sign_bit if negative else 0) | one, 0
    elif op == "sigmoid":
        if inf:
            return (0 if negative else one), 0
        if zero:
            return (bias - 1) << m, 0
    elif op == "softplus":
        if inf:
            return (0 if negative else inf_bits), 0
    mpmath.mp.prec = 800
    x = mpmath.mpf(value.numerator) / mpmath.mpf(value.denominator)   # exact: operands have at most 24 significant bits
    exact = None
    if op == "log2" and value.numerator == 1 or (op == "log2" and value.denominator == 1 and value.numerator & (value.numerator - 1) == 0):
        # a power of two: log2 is the exponent, exactly
        exact = Fraction(value.numerator.bit_length() - value.denominator.bit_length())
    elif op == "pow2" and value.denominator == 1 and abs(value) < 4096:
        exact = Fraction(2) ** int(value)
    # Arguments whose result is far outside every format's range, or indistinguishable from its limit at any
    # supported precision, get a representative with the same rounding fate; the multiprecision evaluation of
    # 2^(10^38) does not terminate in practice.
    tiny, huge = Fraction(1, 2 ** 4096), Fraction(2 ** 4096)
    if exact is None:
        if op in ("pow2", "exp") and abs(value) >= 4096:
            exact = huge if value > 0 else tiny
        elif op == "tanh" and abs(value) >= 64:
            exact = (1 - Fraction(1, 2 ** 200)) * (1 if value > 0 else -1)
        elif op == "sigmoid" and (value >= 128 or value <= -4096):      # 1 - e^-128 needs 185 bits: the last one 200 resolve
            exact = 1 - Fraction(1, 2 ** 200) if value > 0 else tiny
        elif op == "softplus" and (value >= 128 or value <= -4096):
            exact = value + Fraction(1, 2 ** 300) if value > 0 else tiny
    if exact is None:
        # sin x = x - x^3/6..., cos x = 1 - x^2/2...: for the smallest bf16 operands (2^-133) the second term sits 266
        # bits below the first, so tiny operands are evaluated with 700 bits; 200 bits resolve everything else.
        with mpmath.workprec(700 if abs(value) < Fraction(1, 2 ** 40) else 200):
            y = {"sqrt": mpmath.sqrt, "rsqrt": lambda t: 1 / mpmath.sqrt(t), "log2": lambda t: mpmath.log(t, 2), "ln": mpmath.log,
                 "pow2": lambda t: mpmath.power(2, t), "exp": mpmath.exp, "sin": mpmath.sin, "cos": mpmath.cos, "tanh": mpmath.tanh,
                 "sigmoid": lambda t: 1 / (1 + mpmath.exp(-t)), "softplus": lambda t: mpmath.log1p(mpmath.exp(t))}[op](x)
            mantissa, exponent = int(y.man) * (-1 if y._mpf_[0] else 1), int(y.exp)
            # Magnitudes far outside every format's range (2^x of a large bf16 operand) are replaced by a representative
            # beyond the range with the same fate: an exact rational with a 10^38-bit exponent cannot be built.
            magnitude_exponent = exponent + mantissa.bit_length()
            if magnitude_exponent > 4096:
                mantissa, exponent = (1 if mantissa > 0 else -1), 4096
            elif magnitude_exponent < -4096:
                mantissa, exponent = (1 if mantissa > 0 else -1), -4096
            exact = Fraction(mantissa) * Fraction(2) ** exponent
    result, flags = round_to_format(fmt, exact)
    flags &= ~UNDERFLOW
    if (flags & INEXACT) and not (flags & OVERFLOW) and _tiny_after_unbounded_rounding(fmt, exact):
        flags |= UNDERFLOW
    return result, flags
