"""Acceptance gate: ProgramTensor `.npy` I/O, the comparison policy and the device comparator.

The GPU cases restate the reference's own vectors for this path
(unittests/Simulator/Invocation/ProgramTensorComparisonTest.cpp:45-99, 101-177, 179-255, 257-267, 327-368, 370-402) through
the product API, then check the device statistics against the long-double CPU restatement on seeded random tensors:
counts, maxima, ULP and absolute-error quantiles bit for bit; the four extended-precision figures to 1e-14 relative."""
import json
import lzma
import math
from pathlib import Path

import numpy as np
import pytest

from vibe_compiler_b200 import gate
from vibe_compiler_b200.gate import ComparisonPolicy, ProgramTensor, ProgramTensorComparisonError

ROOT = Path(__file__).resolve().parent.parent


def tensor(dtype, shape, values):
    return ProgramTensor(dtype, shape, np.asarray(values, dtype=np.uint8))


def words(dtype, shape, bits):
    width = np.uint32 if dtype == "f32" else np.uint16
    return ProgramTensor(dtype, shape, np.asarray(bits, dtype=width))


# ------------------------------------------------------------------------------------------------ CPU: files and policy
def test_npy_round_trip_and_numpy_interoperability(tmp_path):
    rng = np.random.default_rng(20260803)
    for dtype, numpy_dtype in (("f32", np.float32), ("f16", np.float16), ("i32", np.int32), ("i8", np.int8), ("bool", np.bool_), ("i64", np.int64)):
        array = rng.integers(0, 2, size=(3, 5, 7)).astype(numpy_dtype)
        np.save(tmp_path / "a.npy", array)
        loaded = gate.load_npy(tmp_path / "a.npy")
        assert (loaded.dtype, loaded.shape) == (dtype, (3, 5, 7)) and loaded.data.tobytes() == array.tobytes()
        gate.save_npy(tmp_path / "b.npy", loaded)
        assert np.array_equal(np.load(tmp_path / "b.npy"), array)
    bf16 = words("bf16", (4,), [0x3f80, 0x4000, 0xbf80, 0x0001])
    gate.save_npy(tmp_path / "c.npy", bf16)
    assert np.load(tmp_path / "c.npy").dtype == np.dtype("V2")
    again = gate.load_npy(tmp_path / "c.npy")
    assert again.dtype == "bf16" and again.data.tobytes() == bf16.data.tobytes()
    scalar = ProgramTensor("f32", (), np.zeros(4, np.uint8))
    gate.save_npy(tmp_path / "d.npy", scalar)
    assert gate.load_npy(tmp_path / "d.npy").shape == () and np.load(tmp_path / "d.npy").shape == ()
    one_d = ProgramTensor("f32", (3,), np.zeros(12, np.uint8))
    gate.save_npy(tmp_path / "e.npy", one_d)
    assert gate.load_npy(tmp_path / "e.npy").shape == (3,) and np.load(tmp_path / "e.npy").shape == (3,)


def test_npy_version_two_header(tmp_path):
    header = b"{'descr': '<f4', 'fortran_order': False, 'shape': (2, 2), }\n"
    payload = np.arange(4, dtype=np.float32).tobytes()
    (tmp_path / "v2.npy").write_bytes(b"\x93NUMPY\x02\x00" + len(header).to_bytes(4, "little") + header + payload)
    loaded = gate.load_npy(tmp_path / "v2.npy")
    assert loaded.shape == (2, 2) and loaded.data.tobytes() == payload


@pytest.mark.parametrize("content, fragment", [
    (b"NOTNUMPY" * 4, "missing magic"),
    (b"\x93NUMPY\x03\x00\x10\x00" + b" " * 16, "unsupported npy payload version"),
    (b"\x93NUMPY\x01\x00\xff\x00{'descr'", "truncated npy payload header"),
    (b"\x93NUMPY\x01\x00\x10\x00{'shape': (2,)}  \n", "invalid npy payload header"),
])
def test_npy_rejections(tmp_path, content, fragment):
    (tmp_path / "bad.npy").write_bytes(content)
    with pytest.raises(ValueError, match=fragment):
        gate.load_npy(tmp_path / "bad.npy")


def test_npy_rejects_fortran_order_unknown_dtypes_and_short_payloads(tmp_path):
    np.save(tmp_path / "f.npy", np.asfortranarray(np.ones((2, 3), np.float32)))
    with pytest.raises(ValueError, match="must be row-major"):
        gate.load_npy(tmp_path / "f.npy")
    np.save(tmp_path / "u.npy", np.ones(3, np.uint16))
    with pytest.raises(ValueError, match="unsupported dtype"):
        gate.load_npy(tmp_path / "u.npy")
    np.save(tmp_path / "big.npy", np.ones(3, ">f4"))
    with pytest.raises(ValueError, match="unsupported dtype"):
        gate.load_npy(tmp_path / "big.npy")
    np.save(tmp_path / "t.npy", np.ones(16, np.float32))
    whole = (tmp_path / "t.npy").read_bytes()
    (tmp_path / "t.npy").write_bytes(whole[:-4])
    with pytest.raises(ValueError, match="payload is truncated"):
        gate.load_npy(tmp_path / "t.npy")


def test_pair_and_policy_checks_need_no_device():
    f16 = tensor("f16", (1,), [0x00, 0x3c])
    two = tensor("f16", (2,), [0x00, 0x3c, 0x00, 0x40])
    integer = tensor("i16", (1,), [0, 0])
    with pytest.raises(ProgramTensorComparisonError) as error:
        gate.compare_expected_output(None, integer, f16)
    assert error.value.code == "dtype-mismatch" and error.value.detail == "actual=i16 expected=f16"
    with pytest.raises(ProgramTensorComparisonError) as error:
        gate.compare_expected_output(None, two, f16)
    assert error.value.code == "shape-mismatch" and error.value.detail == "actual=[2] expected=[1]"
    f64 = ProgramTensor("f64", (1,), np.zeros(8, np.uint8))
    with pytest.raises(ProgramTensorComparisonError) as error:
        gate.compare_expected_output(None, f64, f64)
    assert error.value.code == "unsupported-floating-dtype"
    with pytest.raises(ProgramTensorComparisonError) as error:
        gate.compute_statistics(None, integer, integer)
    assert error.value.code == "unsupported-statistics-dtype"
    empty = ProgramTensor("f16", (0,), np.zeros(0, np.uint8))
    with pytest.raises(ProgramTensorComparisonError, match="require a non-empty tensor"):
        gate.compute_statistics(None, empty, empty)
    for bad in (-1.0, 1.1, float("nan"), float("inf")):
        with pytest.raises(ProgramTensorComparisonError) as error:
            gate.compare_expected_output(None, f16, f16, ComparisonPolicy(0.004, 0.002, (bad, 0.01)))
        assert error.value.code == "invalid-tolerance"
    for bad in (-1.0, float("nan"), float("inf")):
        with pytest.raises(ProgramTensorComparisonError):
            gate.compare_expected_output(None, f16, f16, ComparisonPolicy(0.004, 0.002, (0.9999, bad)))
        with pytest.raises(ProgramTensorComparisonError):
            gate.compare_expected_output(None, f16, f16, ComparisonPolicy(bad, 0.0))
    with pytest.raises(ValueError, match="byte size"):
        ProgramTensor("f32", (2,), np.zeros(4, np.uint8))


def test_statistics_line_and_option_parsing():
    s = gate.ComparisonStatistics(1000, 989, 0.989, 12.0 / 1024.0 / 1000.0, 1 / 1024, 1 / 1024, 2 / 1024, 11, 0.5, 0.25, 0.012, 1, 1, 2)
    line = gate.format_statistics(0, 3, "f16", s, ComparisonPolicy(0.004, 0.002, (0.9999, 0.01)))
    assert line == ("target model numeric statistics index=0 launch_slot=3 dtype=f16 elements=1000 exact=989 "
                    "exact_fraction=0.98899999999999999 mean_abs=1.171875e-05 p99_abs=0.0009765625 p999_abs=0.0009765625 "
                    "max_abs=0.001953125 mean_ulp=0.012 p99_ulp=1 p999_ulp=1 max_ulp=2 elementwise_mismatches=11 "
                    "atol=4.000000e-03 rtol=2.000000e-03 cosine=0.5 relative_l2=0.25 comparison=similarity "
                    "minimum_cosine=9.999000e-01 maximum_relative_l2=1.000000e-02")
    assert gate.format_statistics(1, 0, "f32", s, ComparisonPolicy()).endswith("atol=0.000000e+00 rtol=0.000000e+00 cosine=0.5 relative_l2=0.25 comparison=elementwise")
    assert gate._indexed_paths(["0=a.npy", "12=dir/b=c.npy"], "--model-input") == {0: "a.npy", 12: "dir/b=c.npy"}
    for bad in (["a.npy"], ["-1=a.npy"], ["x=a.npy"], ["1="], ["0=a.npy", "0=b.npy"]):
        with pytest.raises(SystemExit):
            gate._indexed_paths(bad, "--model-input")
    assert gate.main(["--target-model", "nowhere", "--model-input", "0=a.npy"]) == 1
    assert gate.main(["--target-model", "nowhere", "--model-input", "0=a.npy", "--model-expected", "0=b.npy", "--model-min-cosine", "0.9"]) == 1


# ------------------------------------------------------------------------------------------------ GPU: reference vectors
SIMILARITY = ComparisonPolicy(0.004, 0.002, (0.9999, 0.01))


def code_of(call):
    try:
        call()
    except ProgramTensorComparisonError as error:
        return error.code
    return None


@pytest.mark.gpu
@pytest.mark.parametrize("dtype, one, perturbed, two", [("f16", 0x3c00, 0x3c80, 0x4000), ("bf16", 0x3f80, 0x3f90, 0x4000),
                                                      ("f32", 0x3f800000, 0x3f900000, 0x40000000)])
@pytest.mark.parametrize("extent", [1024, 1025, 1031])
def test_similarity_uses_all_elements_and_keeps_the_diagnostics(backend, dtype, one, perturbed, two, extent):
    count = 4 * extent
    make = lambda fill, last: words(dtype, (2, 2, extent), [fill] * (count - 1) + [last])
    expected, actual = make(one, one), make(one, perturbed)
    assert code_of(lambda: gate.compare_expected_output(backend, actual, expected, ComparisonPolicy(0.004, 0.002))) == "numeric-mismatch"
    gate.compare_expected_output(backend, actual, expected, SIMILARITY)
    stats = gate.compute_statistics(backend, actual, expected, SIMILARITY)
    assert stats.mismatch_count == 1 and stats.max_abs == 0.125
    assert abs(stats.relative_l2 - 0.125 / math.sqrt(count)) <= 1e-15
    assert abs(stats.cosine - (count + 0.125) / math.sqrt(count) / math.sqrt(count + 0.265625)) <= 1e-14
    scaled = gate.compute_statistics(backend, make(two, two), expected, SIMILARITY)
    assert scaled.cosine == 1.0 and scaled.relative_l2 == 1.0
    assert code_of(lambda: gate.compare_expected_output(backend, make(two, two), expected, SIMILARITY)) == "numeric-mismatch"


@pytest.mark.gpu
def test_similarity_zero_and_failure_contracts(backend):
    zero, one, negative = tensor("f16", (1,), [0, 0]), tensor("f16", (1,), [0, 0x3c]), tensor("f16", (1,), [0, 0xbc])
    infinity, nan = tensor("f16", (1,), [0, 0x7c]), tensor("f16", (1,), [1, 0x7c])
    empty = ProgramTensor("f16", (0,), np.zeros(0, np.uint8))
    ordered, permuted = tensor("f16", (2,), [0, 0x3c, 0, 0x40]), tensor("f16", (2,), [0, 0x40, 0, 0x3c])
    stats = gate.compute_statistics(backend, permuted, ordered, SIMILARITY)
    assert stats.cosine == 0.8 and stats.relative_l2 == math.sqrt(0.4)
    assert code_of(lambda: gate.compare_expected_output(backend, permuted, ordered, SIMILARITY)) == "numeric-mismatch"
    gate.compare_expected_output(backend, zero, zero, SIMILARITY)
    zeros = gate.compute_statistics(backend, zero, zero, SIMILARITY)
    assert zeros.cosine == 1.0 and zeros.relative_l2 == 0.0
    for actual in (zero, negative):
        assert code_of(lambda: gate.compare_expected_output(backend, actual, one, SIMILARITY)) == "numeric-mismatch"
    assert math.isinf(gate.compute_statistics(backend, one, zero, SIMILARITY).relative_l2)
    assert code_of(lambda: gate.compare_expected_output(backend, one, zero, SIMILARITY)) == "numeric-mismatch"
    for bad in (infinity, nan):
        assert code_of(lambda: gate.compare_expected_output(backend, bad, one, SIMILARITY)) == "actual-nonfinite"
        assert code_of(lambda: gate.compare_expected_output(backend, one, bad, SIMILARITY)) == "expected-nonfinite"
        assert code_of(lambda: gate.compute_statistics(backend, bad, one)) == "actual-nonfinite"
    assert code_of(lambda: gate.compare_expected_output(backend, empty, empty, SIMILARITY)) == "unsupported-statistics-dtype"
    gate.compare_expected_output(backend, empty, empty, ComparisonPolicy())
    integer, wrong = tensor("i16", (1,), [0, 0]), tensor("i16", (1,), [1, 0])
    assert code_of(lambda: gate.compare_expected_output(backend, integer, wrong, SIMILARITY)) == "raw-mismatch"


@pytest.mark.gpu
def test_tolerances_per_format_signed_zero_and_subnormals(backend):
    ok = lambda a, e, atol, rtol: code_of(lambda: gate.compare_expected_output(backend, a, e, ComparisonPolicy(atol, rtol)))
    assert ok(tensor("f16", (1,), [0x01, 0x3c]), tensor("f16", (1,), [0x00, 0x3c]), 0.00048828125, 0.00048828125) is None
    assert ok(tensor("f16", (1,), [0x01, 0x3c]), tensor("f16", (1,), [0x00, 0x3c]), 0.0004, 0.0005) == "numeric-mismatch"
    assert ok(tensor("bf16", (1,), [0x01, 0x3f]), tensor("bf16", (1,), [0x00, 0x3f]), 0.0, 0.008) is None
    assert ok(tensor("bf16", (1,), [0x01, 0x3f]), tensor("bf16", (1,), [0x00, 0x3f]), 0.0, 0.007) == "numeric-mismatch"
    assert ok(tensor("f32", (1,), [1, 0, 0x80, 0x3f]), tensor("f32", (1,), [0, 0, 0x80, 0x3f]), 1.2e-7, 0.0) is None
    assert ok(tensor("f32", (1,), [1, 0, 0x80, 0x3f]), tensor("f32", (1,), [0, 0, 0x80, 0x3f]), 1.0e-7, 0.0) == "numeric-mismatch"
    assert ok(tensor("f16", (1,), [0, 0x80]), tensor("f16", (1,), [0, 0]), 0.0, 0.0) is None
    assert ok(tensor("f16", (1,), [1, 0]), tensor("f16", (1,), [0, 0]), 2.0 ** -24, 0.0) is None
    assert ok(tensor("f16", (1,), [1, 0]), tensor("f16", (1,), [0, 0]), 2.0 ** -25, 0.0) == "numeric-mismatch"
    assert ok(tensor("f16", (1,), [0, 0x7c]), tensor("f16", (1,), [0, 0x3c]), 100.0, 100.0) == "actual-nonfinite"
    assert ok(tensor("bf16", (1,), [0x80, 0x3f]), tensor("bf16", (1,), [0xc1, 0x7f]), 100.0, 100.0) == "expected-nonfinite"
    # rtol * |expected| overflows: the reference reports the tolerance, not the values.
    assert ok(tensor("f32", (1,), [0, 0, 0x80, 0x7f - 1]), tensor("f32", (1,), [0, 0, 0x80, 0x7f - 1]), 0.0, 1e300) == "invalid-tolerance"


@pytest.mark.gpu
def test_mismatch_summary_and_raw_comparison(backend):
    expected = tensor("f16", (3,), [0x00, 0x3c, 0x00, 0x3c, 0x00, 0x3c])
    actual = tensor("f16", (3,), [0x00, 0x3c, 0x00, 0x40, 0x00, 0x42])
    with pytest.raises(ProgramTensorComparisonError) as error:
        gate.compare_expected_output(backend, actual, expected)
    assert error.value.detail == ("mismatches=2/3 first={element=1 actual=2.000000e+00 expected=1.000000e+00 abs_error=1.000000e+00 "
                                  "tolerance=0.000000e+00} max_abs={element=2 actual=3.000000e+00 expected=1.000000e+00 "
                                  "abs_error=2.000000e+00 tolerance=0.000000e+00} max_tolerance_ratio=INF at_element=1")
    same = tensor("i16", (2,), [0x00, 0x01, 0x00, 0x02])
    gate.compare_expected_output(backend, same, tensor("i16", (2,), [0x00, 0x01, 0x00, 0x02]), ComparisonPolicy(100.0, 100.0))
    with pytest.raises(ProgramTensorComparisonError) as error:
        gate.compare_expected_output(backend, tensor("i16", (2,), [0x00, 0x01, 0x01, 0x02]), same, ComparisonPolicy(100.0, 100.0))
    assert error.value.code == "raw-mismatch" and error.value.detail == "byte=2 actual=1 expected=0"
    rng = np.random.default_rng(5)
    big = rng.integers(0, 256, size=3_000_017, dtype=np.uint8)
    other = big.copy()
    other[[2_999_999, 1_234_567, 2_000_000]] ^= 0x10
    with pytest.raises(ProgramTensorComparisonError) as error:
        gate.compare_expected_output(backend, ProgramTensor("i8", (big.size,), other), ProgramTensor("i8", (big.size,), big))
    assert error.value.detail.startswith("byte=1234567 ")
    gate.compare_expected_output(backend, ProgramTensor("i8", (big.size,), big.copy()), ProgramTensor("i8", (big.size,), big))


@pytest.mark.gpu
def test_statistics_use_nearest_rank_and_sign_aware_ulp_distance(backend):
    bits = np.full(1000, 0x3c00, dtype=np.uint16)
    actual = bits.copy()
    actual[989:] += 1
    actual[999] += 1
    s = gate.compute_statistics(backend, words("f16", (1000,), actual), words("f16", (1000,), bits))
    assert (s.element_count, s.exact_count, s.exact_fraction) == (1000, 989, 0.989)
    assert s.mean_abs == 12.0 / 1024.0 / 1000.0 and s.p99_abs == s.p999_abs == 1.0 / 1024.0 and s.max_abs == 2.0 / 1024.0
    assert s.mean_ulp == 12.0 / 1000.0 and (s.p99_ulp, s.p999_ulp, s.max_ulp) == (1, 1, 2)
    zero = gate.compute_statistics(backend, tensor("f16", (1,), [0, 0x80]), tensor("f16", (1,), [0, 0]))
    assert zero.exact_count == 1 and zero.max_ulp == 0
    bf16 = gate.compute_statistics(backend, tensor("bf16", (1,), [1, 0x3f]), tensor("bf16", (1,), [0, 0x3f]))
    assert bf16.max_abs == 1.0 / 256.0 and bf16.max_ulp == 1
    f32 = gate.compute_statistics(backend, tensor("f32", (1,), [1, 0, 0x80, 0x3f]), tensor("f32", (1,), [0, 0, 0x80, 0x3f]))
    assert f32.max_abs == 2.0 ** -23 and f32.max_ulp == 1
    # Opposite signs: the order key counts through zero (0x0001 against 0x8001 is two steps apart).
    crossing = gate.compute_statistics(backend, tensor("f16", (1,), [1, 0x80]), tensor("f16", (1,), [1, 0]))
    assert crossing.max_ulp == 2


# ------------------------------------------------------------------------------------------------ GPU: against the oracle
def _random_pair(rng, dtype, count):
    if dtype == "f32":
        expected = rng.standard_normal(count).astype(np.float32)
        noise = (rng.standard_normal(count) * 1e-4).astype(np.float32)
        noise[rng.random(count) < 0.3] = 0
        actual = (expected + noise).astype(np.float32)
        # a few wide-range and sign-crossing elements
        special = min(4, count)
        expected[:special] = [1e30, -1e-30, 3.0e38, 0.0][:special]
        actual[:special] = [1.0001e30, 1e-30, -3.0e38, -0.0][:special]
        return actual.view(np.uint32), expected.view(np.uint32)
    import torch
    torch_dtype = torch.bfloat16 if dtype == "bf16" else torch.float16
    generator = torch.Generator().manual_seed(int(rng.integers(1 << 30)))
    e = torch.randn(count, generator=generator)
    a = e + torch.randn(count, generator=generator) * (2e-3 if dtype == "bf16" else 3e-4)
    to_bits = lambda t: t.to(torch_dtype).view(torch.int16).numpy().view(np.uint16).copy()
    return to_bits(a), to_bits(e)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("count", [1, 7, 1000, 65_537, 2_000_003])
def test_device_statistics_agree_with_the_cpu_restatement(backend, oracle, dtype, count):
    rng = np.random.default_rng(20260803 + count)
    actual, expected = _random_pair(rng, dtype, count)
    atol, rtol = 1e-4, 1e-3
    want = oracle.compare(dtype, actual, expected, atol, rtol)
    got = gate.compute_statistics(backend, words(dtype, (count,), actual), words(dtype, (count,), expected), ComparisonPolicy(atol, rtol))
    assert got.element_count == want["element_count"] and got.exact_count == want["exact_count"]
    assert got.mismatch_count == want["mismatch_count"]
    for name in ("p99_abs", "p999_abs", "max_abs"):
        assert getattr(got, name) == want[name], name
    assert (got.p99_ulp, got.p999_ulp, got.max_ulp) == (want["p99_ulp"], want["p999_ulp"], want["max_ulp"])
    for name in ("mean_abs", "mean_ulp", "cosine", "relative_l2"):
        assert getattr(got, name) == pytest.approx(want[name], rel=1e-14, abs=0.0), name


@pytest.mark.gpu
def test_first_offending_element_follows_the_scan_order(backend):
    rng = np.random.default_rng(11)
    count = 500_003
    actual, expected = _random_pair(rng, "f32", count)
    actual, expected = actual.copy(), expected.copy()
    actual[[400_000, 77_777]] = 0x7f800000
    expected[[77_777, 60_001]] = 0x7fc00000
    with pytest.raises(ProgramTensorComparisonError) as error:
        gate.compare_expected_output(backend, words("f32", (count,), actual), words("f32", (count,), expected), ComparisonPolicy(1.0, 1.0))
    assert (error.value.code, error.value.detail) == ("expected-nonfinite", "element=60001")
    expected[60_001] = 0x3f800000
    with pytest.raises(ProgramTensorComparisonError) as error:
        gate.compare_expected_output(backend, words("f32", (count,), actual), words("f32", (count,), expected), ComparisonPolicy(1.0, 1.0))
    assert (error.value.code, error.value.detail) == ("actual-nonfinite", "element=77777")


@pytest.mark.gpu
def test_device_pointers_and_unaligned_views(backend):
    """The C entry takes device pointers too; a view that starts 2 bytes into an allocation takes the scalar loads."""
    import ctypes as C
    import torch
    from vibe_compiler_b200 import _abi as abi
    count = 300_001
    generator = torch.Generator().manual_seed(3)
    e = torch.randn(count + 1, generator=generator).to(torch.bfloat16)
    a = (e.float() + torch.randn(count + 1, generator=generator) * 1e-2).to(torch.bfloat16)
    host = gate.compute_statistics(backend, ProgramTensor("bf16", (count,), a[1:].view(torch.int16).numpy().view(np.uint16)),
                                   ProgramTensor("bf16", (count,), e[1:].view(torch.int16).numpy().view(np.uint16)))
    da, de = a.cuda(), e.cuda()
    out = abi.Comparison()
    torch.cuda.synchronize()
    status = abi.load().wb200_compare(backend._handle, abi.BF16, count, da.data_ptr() + 2, de.data_ptr() + 2, abi.MEM_DEVICE,
                                      0.0, 0.0, 0, 0.0, 0.0, C.byref(out))
    assert status == abi.OK and out.outcome == abi.CMP_NUMERIC_MISMATCH
    assert (out.exact_count, out.p99_abs, out.p999_ulp, out.max_ulp, out.cosine) == (host.exact_count, host.p99_abs, host.p999_ulp, host.max_ulp, host.cosine)


@pytest.mark.gpu
def test_gate_runs_a_shipped_plan_from_npy_files(backend, tmp_path, capsys):
    import torch
    fixture = json.loads(lzma.decompress((ROOT / "tests" / "golden" / "gemm_tile_modules.json.xz").read_bytes()))
    plan = "tensor-candidate-39"
    modules = tmp_path / "modules"
    modules.mkdir()
    for index, text in enumerate(fixture["plans"][plan]):
        (modules / f"tile_{index:02d}.ll").write_text(text)
    generator = torch.Generator().manual_seed(20260803)
    arg0 = (torch.randn(1, 1024, 4096, generator=generator) * 0.25).to(torch.bfloat16)
    arg1 = (torch.randn(1, 4096, 1024, generator=generator) * 0.25).to(torch.bfloat16)
    product = (arg1[0].float().cuda() @ arg0[0].float().cuda()).cpu().to(torch.bfloat16)
    bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)
    gate.save_npy(tmp_path / "arg0.npy", ProgramTensor("bf16", (1, 1024, 4096), bits(arg0)))
    gate.save_npy(tmp_path / "arg1.npy", ProgramTensor("bf16", (1, 4096, 1024), bits(arg1)))
    gate.save_npy(tmp_path / "out.npy", ProgramTensor("bf16", (1, 4096, 4096), bits(product)))
    arguments = ["--target-model", str(modules), "--model-input", f"0={tmp_path / 'arg0.npy'}", "--model-input", f"1={tmp_path / 'arg1.npy'}",
                 "--model-expected", f"0={tmp_path / 'out.npy'}"]
    assert gate.main(arguments + ["--model-min-cosine", "0.9999", "--model-max-relative-l2", "0.01", "--model-report-numeric-statistics"]) == 0
    printed = capsys.readouterr().out.splitlines()
    assert printed[0].startswith("wb200-gate: target model numeric statistics index=0 launch_slot=0 dtype=bf16 elements=16777216 exact=")
    assert " comparison=similarity minimum_cosine=9.999000e-01 maximum_relative_l2=1.000000e-02" in printed[0]
    assert printed[-1].startswith("wb200-gate: target model outputs matched; tiles=16 commands=")
    # Elementwise with zero tolerance: bf16 roundings of a differently ordered sum cannot all agree.
    assert gate.main(arguments) == 1
    assert "target model output differs at index 0: program tensor comparison numeric-mismatch: mismatches=" in capsys.readouterr().err
