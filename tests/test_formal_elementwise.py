"""Formal (bit-exact) elementwise family: the exact-rational oracle against the reference's vectors (CPU), and the
GPU entry point wb200_elementwise_formal against the oracle bit for bit, IEEE flags included (GPU).
Reference vectors: unittests/Simulator/Reference/FormalTensorNumericTest.cpp:189-249."""
import numpy as np
import pytest

from oracle import formal_scalar as F
from vibe_compiler_b200 import _abi as abi
from vibe_compiler_b200.backend import NumericTensor, PhysicalTensorDescriptor

FMT = {"f16": abi.F16, "bf16": abi.BF16, "f32": abi.F32, "tf32": abi.TF32}
DTYPE = {"f16": np.uint16, "bf16": np.uint16, "f32": np.uint32, "tf32": np.uint32}
ARITHMETIC = ["abs", "neg", "recip", "square", "max", "min", "add", "sub", "mul", "relu"]
RELATIONS = ["eq", "ne", "ge", "gt", "le", "lt"]
BOOL = 7


def test_reference_vectors():
    assert F.evaluate("add", "f32", "f32", 0x3f800000, 0x40400000) == (0x40800000, 0)
    assert F.evaluate("add", "f32", "f32", 0x40000000, 0x40800000) == (0x40c00000, 0)
    assert F.evaluate("ne", "f16", "bool", 0x7e00, 0x3c00) == (1, 0)          # a NaN operand: only `ne` holds
    assert F.evaluate("ne", "f16", "bool", 0x3c00, 0x3c00) == (0, 0)
    assert [F.evaluate("logic_xor", "bool", "bool", a, b)[0] for a, b in ((0, 0), (1, 0), (1, 1))] == [0, 1, 0]


def test_flag_definitions():
    assert F.evaluate("recip", "f32", "f32", 0x40400000)[1] == F.INEXACT                       # 1 / 3
    assert F.evaluate("recip", "f32", "f32", 0x40000000) == (0x3f000000, 0)                    # 1 / 2 exact
    assert F.evaluate("recip", "f16", "f16", 0x8000) == (0xfc00, F.DIV_BY_ZERO)                # 1 / -0 = -inf
    assert F.evaluate("add", "f16", "f16", 0x7bff, 0x7bff) == (0x7c00, F.OVERFLOW | F.INEXACT)
    assert F.evaluate("mul", "f16", "f16", 0x0001, 0x0001) == (0x0000, F.UNDERFLOW | F.INEXACT)
    assert F.evaluate("sub", "f32", "f32", 0x7f800000, 0x7f800000) == (0x7fc00000, F.INVALID)  # inf - inf
    assert F.evaluate("mul", "bf16", "bf16", 0x0000, 0x7f80) == (0x7fc0, F.INVALID)            # 0 * inf
    assert F.evaluate("abs", "bf16", "bf16", 0xff81) == (0x7fc0, F.INVALID)                    # signalling NaN
    assert F.evaluate("max", "f32", "f32", 0x80000000, 0x00000000) == (0x00000000, 0)          # max(-0, +0) = +0
    assert F.evaluate("min", "f32", "f32", 0x80000000, 0x00000000) == (0x80000000, 0)
    assert F.evaluate("relu", "f16", "f16", 0x8000) == (0x8000, 0)                             # -0 is kept
    assert F.evaluate("add", "f16", "f16", 0x3c00, 0xbc00) == (0x0000, 0)                      # x + (-x) = +0, exact
    # subnormal result that is exact raises nothing; the same magnitude reached inexactly raises underflow
    assert F.evaluate("mul", "f16", "f16", 0x0400, 0x3800) == (0x0200, 0)
    assert F.evaluate("mul", "f16", "f16", 0x0401, 0x3800)[1] == F.UNDERFLOW | F.INEXACT


def _patterns(fmt, count, rng):
    bits = 32 if fmt == "f32" else 16
    values = rng.integers(0, 2 ** bits, count, dtype=np.uint64)
    exp_mask = {"f16": 0x7c00, "bf16": 0x7f80, "f32": 0x7f800000}[fmt]
    special = [0, 1 << (bits - 1), exp_mask, exp_mask | (1 << (bits - 1)), exp_mask | 1, F.canonical_nan(fmt), 1, exp_mask - 1,
               {"f16": 0x3c00, "bf16": 0x3f80, "f32": 0x3f800000}[fmt], {"f16": 0x0400, "bf16": 0x0080, "f32": 0x00800000}[fmt]]
    values[:len(special)] = special
    rng.shuffle(values)
    return values.astype(DTYPE[fmt])


def _run(backend, op, fmt, out_fmt, a, b=None):
    key = PhysicalTensorDescriptor(FMT[fmt], abi.LAYOUT_TENSOR, [len(a)])
    out_key = PhysicalTensorDescriptor(BOOL if out_fmt == "bool" else FMT[out_fmt], abi.LAYOUT_TENSOR, [len(a)])
    out_bytes = (len(a) + 7) // 8 if out_fmt == "bool" else len(a) * np.dtype(DTYPE[out_fmt]).itemsize
    template = np.full(out_bytes, 0xFF, dtype=np.uint8)
    inputs = [NumericTensor(key, a)] + ([NumericTensor(key, b)] if b is not None else [])
    result = backend.execute_elementwise(op, inputs, NumericTensor(out_key, template), formal=True)
    return result.destination.storage, result.evidence


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["f16", "bf16", "f32"])
def test_formal_arithmetic_matches_the_exact_oracle(backend, fmt):
    rng = np.random.default_rng(20260803)
    n = 1501                                    # not a multiple of 8
    a, b = _patterns(fmt, n, rng), _patterns(fmt, n, rng)
    for op in ARITHMETIC:
        unary = op in F.UNARY
        storage, evidence = _run(backend, op, fmt, fmt, a, None if unary else b)
        got = storage.view(DTYPE[fmt])
        want, flags = [], 0
        for x, y in zip(a, b):
            bits, f = F.evaluate(op, fmt, fmt, int(x), int(y))
            want.append(bits)
            flags |= f
        assert np.array_equal(got, np.array(want, dtype=DTYPE[fmt])), op
        assert evidence.flags == flags, (op, evidence.flags, flags)
        assert evidence.scalar_evaluations == n


@pytest.mark.gpu
def test_flags_per_element(backend):
    # one element per request, so the flags of that element are seen in isolation
    rng = np.random.default_rng(5)
    for fmt in ("f16", "bf16", "f32"):
        a, b = _patterns(fmt, 60, rng), _patterns(fmt, 60, rng)
        for op in ("recip", "square", "add", "sub", "mul"):
            for x, y in zip(a, b):
                one = np.array([x], dtype=DTYPE[fmt])
                other = None if op in F.UNARY else np.array([y], dtype=DTYPE[fmt])
                storage, evidence = _run(backend, op, fmt, fmt, one, other)
                assert (int(storage.view(DTYPE[fmt])[0]), evidence.flags) == F.evaluate(op, fmt, fmt, int(x), int(y)), (fmt, op, hex(x), hex(y))


@pytest.mark.gpu
def test_f32_products_around_the_residual_and_underflow_thresholds(backend):
    # one element per request. The kernel takes the product's rounding error from one f32 fused multiply-add when
    # |product| >= 2^-100 and from f64 arithmetic below; cases sit on both sides of that threshold, around the smallest
    # normal number, in the subnormal range and at overflow, with full-width and few-bit (exact product) significands.
    rng = np.random.default_rng(99)
    cases = []
    for total in list(range(-153, -143)) + list(range(-130, -122)) + list(range(-104, -96)) + [-60, 0, 60, 125, 126, 127, 128]:
        for width in (24, 12, 3):
            e1 = int(rng.integers(max(-126, total - 127), min(127, total + 126) + 1))
            e2 = total - e1
            m1 = (int(rng.integers(1 << (width - 1), 1 << width)) | 1) << (24 - width)
            m2 = (int(rng.integers(1 << (width - 1), 1 << width)) | 1) << (24 - width)
            x = np.float32(np.ldexp(float(m1), e1 - 23)) * np.float32(rng.choice([-1.0, 1.0]))
            y = np.float32(np.ldexp(float(m2), e2 - 23))
            cases.append((int(np.array(x, np.float32).view(np.uint32)), int(np.array(y, np.float32).view(np.uint32))))
    for x, y in cases:
        for op in ("mul", "square"):
            one = np.array([x], dtype=np.uint32)
            other = None if op == "square" else np.array([y], dtype=np.uint32)
            storage, evidence = _run(backend, op, "f32", "f32", one, other)
            assert (int(storage.view(np.uint32)[0]), evidence.flags) == F.evaluate(op, "f32", "f32", x, y), (op, hex(x), hex(y))


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["f16", "bf16"])
def test_16_bit_arithmetic_values_and_flag_classes(backend, fmt):
    # values element by element on 6000 operand pairs (random bit patterns and moderate magnitudes); flags class by
    # class: all pairs the oracle gives one flag set run as one request, whose OR must be exactly that set
    rng = np.random.default_rng(314)
    n = 6000
    def moderate():
        values = (rng.standard_normal(n // 2) * np.exp(rng.uniform(-6, 6, n // 2))).astype(np.float32)
        if fmt == "bf16":
            return (values.view(np.uint32) >> 16).astype(np.uint16)
        return values.astype(np.float16).view(np.uint16)
    a = np.concatenate([_patterns(fmt, n // 2, rng), moderate()])
    b = np.concatenate([_patterns(fmt, n // 2, rng), moderate()])
    b[n // 2:n // 2 + 500] = a[n // 2:n // 2 + 500] ^ 0x8000            # exact cancellations
    for op in ("add", "sub", "mul", "square"):
        unary = op in F.UNARY
        expected = [F.evaluate(op, fmt, fmt, int(x), int(y)) for x, y in zip(a, b)]
        storage, _ = _run(backend, op, fmt, fmt, a, None if unary else b)
        assert np.array_equal(storage.view(np.uint16), np.array([bits for bits, _ in expected], dtype=np.uint16)), op
        classes = {}
        for index, (_, flags) in enumerate(expected):
            classes.setdefault(flags, []).append(index)
        for flags, members in classes.items():
            _, evidence = _run(backend, op, fmt, fmt, a[members], None if unary else b[members])
            assert evidence.flags == flags, (op, flags, evidence.flags, len(members))


@pytest.mark.gpu
def test_16_bit_products_that_round_up_to_the_smallest_normal_number(backend):
    # A product of two 16-bit operands is exact in f32; it becomes inexact only when it is narrowed. Just below the
    # smallest normal number such a product can round up to it and is then still tiny after rounding with an unbounded
    # exponent: underflow and inexact, with a normal result (f16 0x1fff * 0x2000 = 2^-14 - 2^-25 -> 0x0400).
    assert F.evaluate("mul", "f16", "f16", 0x1fff, 0x2000) == (0x0400, F.UNDERFLOW | F.INEXACT)
    assert F.evaluate("mul", "bf16", "bf16", 0x3fff, 0x0040) == (0x0080, F.UNDERFLOW | F.INEXACT)
    sweeps = {"f16": (range(0x1ff0, 0x2010), (0x2000, 0x1fff, 0x2001, 0x1c00)), "bf16": (range(0x3ff0, 0x4010), (0x0040, 0x0041, 0x003f, 0x0080))}
    for fmt, (lhs, rhs) in sweeps.items():
        for x in lhs:
            for y in rhs:
                storage, evidence = _run(backend, "mul", fmt, fmt, np.array([x], dtype=np.uint16), np.array([y], dtype=np.uint16))
                assert (int(storage.view(np.uint16)[0]), evidence.flags) == F.evaluate("mul", fmt, fmt, x, y), (fmt, hex(x), hex(y))


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["f16", "bf16", "f32"])
def test_relations_to_bool_and_to_numbers(backend, fmt):
    rng = np.random.default_rng(9)
    n = 203
    a = _patterns(fmt, n, rng)
    b = a.copy()
    b[::3] = _patterns(fmt, len(b[::3]), rng)          # a mix of equal and unequal pairs
    for op in RELATIONS:
        want = [F.evaluate(op, fmt, "bool", int(x), int(y))[0] for x, y in zip(a, b)]
        storage, evidence = _run(backend, op, fmt, "bool", a, b)
        unpacked = np.unpackbits(storage, bitorder="little")
        assert list(unpacked[:n]) == want, op
        assert all(unpacked[n:] == 1)                   # bits past the tensor keep the template's value
        numeric, _ = _run(backend, op, fmt, "bf16", a, b)
        assert list(numeric.view(np.uint16)) == [0x3f80 if t else 0 for t in want]


@pytest.mark.gpu
def test_logic_on_packed_bool(backend):
    rng = np.random.default_rng(3)
    n = 77
    bits_a, bits_b = rng.integers(0, 2, n), rng.integers(0, 2, n)
    a, b = np.packbits(bits_a.astype(np.uint8), bitorder="little"), np.packbits(bits_b.astype(np.uint8), bitorder="little")
    key = PhysicalTensorDescriptor(BOOL, abi.LAYOUT_TENSOR, [n])
    template = np.zeros(len(a), dtype=np.uint8)
    for op, fn in (("logic_not", lambda x, y: 1 - x), ("logic_and", lambda x, y: x & y), ("logic_or", lambda x, y: x | y), ("logic_xor", lambda x, y: x ^ y)):
        inputs = [NumericTensor(key, a)] + ([] if op == "logic_not" else [NumericTensor(key, b)])
        result = backend.execute_elementwise(op, inputs, NumericTensor(key, template), formal=True)
        got = np.unpackbits(result.destination.storage, bitorder="little")[:n]
        assert list(got) == list(fn(bits_a, bits_b)), op
        assert result.evidence.flags == 0


@pytest.mark.gpu
def test_formal_entry_rejects_what_it_does_not_cover(backend):
    from vibe_compiler_b200.backend import WB200Error
    a = np.zeros(8, dtype=np.uint16)
    with pytest.raises(WB200Error, match="outside the formal"):
        _run(backend, "exp_lp", "f16", "f16", a)
    with pytest.raises(WB200Error, match="TF32 for the function family"):
        _run(backend, "add", "tf32", "tf32", np.zeros(8, dtype=np.uint32), np.zeros(8, dtype=np.uint32))
    with pytest.raises(WB200Error, match="arity"):
        _run(backend, "add", "f16", "f16", a)
    with pytest.raises(WB200Error, match="result format"):
        _run(backend, "add", "f16", "f32", a, a)


# ------------------------------------------------------------------------------------------------ function family
def _function_expected():
    import json
    from pathlib import Path
    return json.loads((Path(__file__).resolve().parent / "golden" / "formal_function_expected.json").read_text())


def test_function_oracle_reference_vectors():
    # unittests/Simulator/Reference/FormalTensorNumericTest.cpp:236-248: bf16 exp(0) = 1.0, signalling NaN -> canonical NaN + invalid
    assert F.evaluate_function("exp", "bf16", 0x0000) == (0x3f80, 0)
    assert F.evaluate_function("exp", "bf16", 0x7f81) == (0x7fc0, F.INVALID)
    assert F.evaluate_function("sqrt", "f16", 0x4400) == (0x4000, 0)                              # sqrt(4) = 2, exact
    assert F.evaluate_function("log2", "f16", 0x4800) == (0x4200, 0)                              # log2(8) = 3, exact
    assert F.evaluate_function("rsqrt", "f16", 0x8000) == (0xfc00, F.DIV_BY_ZERO)                 # the reference's own -0 rule
    assert F.evaluate_function("ln", "bf16", 0xbf80) == (0x7fc0, F.INVALID)
    assert F.evaluate_function("exp", "f16", 0x4d00) == (0x7c00, F.OVERFLOW | F.INEXACT)          # e^20 > 65504
    assert F.evaluate_function("exp", "f16", 0xcd00)[1] == F.UNDERFLOW | F.INEXACT
    assert F.evaluate_function("sigmoid", "bf16", 0x0000) == (0x3f00, 0)
    assert F.evaluate_function("tanh", "bf16", 0xff80) == (0xbf80, 0)
    expected = _function_expected()
    for key, entry in list(expected.items())[::5]:                                                # the fixture is what the oracle says
        fmt, op = key.split(":")
        for bits, (result, flags) in list(entry["samples"].items())[::16]:
            assert F.evaluate_function(op, fmt, int(bits)) == (result, flags), (key, bits)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["f16", "bf16"])
def test_function_family_over_the_complete_operand_space(backend, fmt):
    import hashlib
    expected = _function_expected()
    everything = np.arange(65536, dtype=np.uint16)
    for op in F.FUNCTIONS:
        entry = expected[f"{fmt}:{op}"]
        storage, evidence = _run(backend, op, fmt, fmt, everything)
        got = storage.view(np.uint16)
        if hashlib.sha256(got.tobytes()).hexdigest() != entry["sha256"]:
            wrong = [(bits, int(got[int(bits)]), want[0]) for bits, want in entry["samples"].items() if int(got[int(bits)]) != want[0]]
            raise AssertionError(f"{fmt} {op}: result table differs from the 200-bit evaluation; sampled mismatches {wrong[:8]}")
        assert evidence.flags == entry["flags_or"], (op, evidence.flags, entry["flags_or"])


@pytest.mark.gpu
def test_function_family_flags_per_element(backend):
    expected = _function_expected()
    for key, entry in expected.items():
        fmt, op = key.split(":")
        for bits, (result, flags) in list(entry["samples"].items())[::3]:
            storage, evidence = _run(backend, op, fmt, fmt, np.array([int(bits)], dtype=np.uint16))
            assert (int(storage.view(np.uint16)[0]), evidence.flags) == (result, flags), (key, hex(int(bits)))


# ------------------------------------------------------------------------------------------------ binary32 / TF32 operands
def _f32_expected():
    from pathlib import Path
    return np.load(Path(__file__).resolve().parent / "golden" / "formal_function_f32_expected.npz")


def _f32_generator():
    import importlib.util
    from pathlib import Path
    spec = importlib.util.spec_from_file_location("make_f32", Path(__file__).resolve().parent / "golden" / "make_formal_function_f32_expected.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_f32_function_oracle_and_host_evaluator_agree_with_the_vectors():
    """CPU: the 200-bit oracle reproduces a sample of the committed vectors, and the library's evaluator compiled for the host
    reproduces all of them (listed hard cases and specials element by element, 2^20 random operands and the complete TF32
    space by hash)."""
    import hashlib
    data, gen = _f32_expected(), _f32_generator()
    assert F.evaluate_function("exp", "f32", 0x00000000) == (0x3f800000, 0)
    assert F.evaluate_function("log2", "f32", 0x41000000) == (0x40400000, 0)                   # log2(8) = 3
    assert F.evaluate_function("sqrt", "f32", 0x40800000) == (0x40000000, 0)
    assert F.evaluate_function("exp", "f32", 0x42b20000) == (0x7f800000, F.OVERFLOW | F.INEXACT)   # e^89
    assert F.evaluate_function("pow2", "f32", 0xc3160000) == (0x00000000, F.UNDERFLOW | F.INEXACT) # 2^-150: ties to zero
    assert F.evaluate_function("pow2", "tf32", 0x3f800000 >> 13) == (0x40000000 >> 13, 0)
    tool = gen.build_tool()
    for function, op in enumerate(F.FUNCTIONS):
        listed, want, flags = data[f"f32_{op}_operands"], data[f"f32_{op}_results"], data[f"f32_{op}_flags"]
        for i in range(0, len(listed), 97):
            assert F.evaluate_function(op, "f32", int(listed[i])) == (int(want[i]), int(flags[i])), (op, hex(int(listed[i])))
        got, got_flags = gen.host_eval(tool, function, False, listed)
        assert np.array_equal(got, want) and np.array_equal(got_flags.astype(np.uint8), flags), op
        got, got_flags = gen.host_eval(tool, function, False, gen.random_operands(function))
        assert hashlib.sha256(got.astype("<u4").tobytes()).hexdigest() == str(data[f"f32_{op}_random_sha256"]), op
        assert int(np.bitwise_or.reduce(got_flags)) == int(data[f"f32_{op}_random_flags_or"]), op
        got, got_flags = gen.host_eval(tool, function, True, np.arange(1 << 19, dtype=np.uint32) << 13)
        assert hashlib.sha256(got.astype("<u4").tobytes()).hexdigest() == str(data[f"tf32_{op}_sha256"]), op
        assert int(np.bitwise_or.reduce(got_flags)) == int(data[f"tf32_{op}_flags_or"]), op


@pytest.mark.gpu
def test_function_family_f32_hard_cases_specials_and_random_operands(backend):
    """binary32 operands: every operand of the complete space that needs more than binary64 to round (found by a host scan
    with the same evaluator), the special operands, and 2^20 seeded random operands, against the 200-bit evaluation."""
    import hashlib
    data, gen = _f32_expected(), _f32_generator()
    for function, op in enumerate(F.FUNCTIONS):
        listed, want, flags = data[f"f32_{op}_operands"], data[f"f32_{op}_results"], data[f"f32_{op}_flags"]
        for value in np.unique(flags):                      # operands with equal expected flags share a call: OR of the call == that value
            pick = flags == value
            storage, evidence = _run(backend, op, "f32", "f32", listed[pick])
            got = storage.view(np.uint32)
            wrong = np.nonzero(got != want[pick])[0]
            assert len(wrong) == 0, (op, [(hex(int(listed[pick][i])), hex(int(got[i])), hex(int(want[pick][i]))) for i in wrong[:6]])
            assert evidence.flags == int(value), (op, evidence.flags, int(value))
        for i in range(0, len(listed), 61):                 # and a sample one by one, so a missing flag cannot hide in an OR
            storage, evidence = _run(backend, op, "f32", "f32", listed[i:i + 1])
            assert (int(storage.view(np.uint32)[0]), evidence.flags) == (int(want[i]), int(flags[i])), (op, hex(int(listed[i])))
        storage, evidence = _run(backend, op, "f32", "f32", gen.random_operands(function))
        assert hashlib.sha256(storage.view(np.uint32).astype("<u4").tobytes()).hexdigest() == str(data[f"f32_{op}_random_sha256"]), op
        assert evidence.flags == int(data[f"f32_{op}_random_flags_or"]), op


@pytest.mark.gpu
def test_function_family_tf32_over_the_complete_operand_space(backend):
    import hashlib
    data = _f32_expected()
    everything = np.arange(1 << 19, dtype=np.uint32) << 13
    for op in F.FUNCTIONS:
        storage, evidence = _run(backend, op, "tf32", "tf32", everything)
        assert hashlib.sha256(storage.view(np.uint32).astype("<u4").tobytes()).hexdigest() == str(data[f"tf32_{op}_sha256"]), op
        assert evidence.flags == int(data[f"tf32_{op}_flags_or"]), op
