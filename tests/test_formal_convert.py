"""Formal scalar conversion routes: the exact-rational oracle against the reference's own vectors (CPU), and the device
entries wb200_convert_formal / wb200_target_call_convert against the oracle bit for bit, IEEE flags and refusals included.
Reference vectors: unittests/Simulator/Reference/FormalNumericTest.cpp:203-600."""
import numpy as np
import pytest

from oracle import formal_convert as K
from vibe_compiler_b200 import _abi as abi
from vibe_compiler_b200.backend import NumericTensor, PhysicalTensorDescriptor, WB200Error
from vibe_compiler_b200.target_calls import ScratchPad

FORMAT = {"i8": abi.I8, "i16": abi.I16, "i32": abi.I32, "f16": abi.F16, "bf16": abi.BF16, "f32": abi.F32, "tf32": abi.TF32}
DTYPE = {"i8": np.uint8, "i16": np.uint16, "i32": np.uint32, "f16": np.uint16, "bf16": np.uint16, "f32": np.uint32, "tf32": np.uint32}
NE, TZ, TP, TN = K.NEAREST_EVEN, K.TOWARD_ZERO, K.TOWARD_POSITIVE, K.TOWARD_NEGATIVE


def test_route_table():
    assert len(K.ROUTES) == 36 and K.ROUTES[139][0] == "int8_fp16" and K.ROUTES[174] == ("tf32_fp32", "tf32", "f32", K.NONE)
    assert K.ROUTES[157] == ("fp16_int8", "f16", "i8", K.ROUNDING) and K.ROUTES[143][3] == K.NONE and K.ROUTES[151][3] == K.NONE
    for opcode in range(139, 143):                       # zero-point routes have no formal evaluation
        with pytest.raises(K.ConversionError, match="unsupported-operation"):
            K.convert(opcode, NE, 0)
    with pytest.raises(K.ConversionError, match="unsupported-operation"):
        K.convert(149, K.STOCHASTIC, 0)


def test_zero_and_boundary_smoke_for_every_route():
    largest = {"f16": 0x7bff, "bf16": 0x7f7f, "f32": 0x7f7fffff, "tf32": 0x7f7fe000}
    for opcode, (_, source, destination, kind) in K.ROUTES.items():
        if kind == K.ZERO_POINT:
            continue
        for mode in ((NE, TZ, TP, TN) if kind == K.ROUNDING else (NE,)):
            assert K.convert(opcode, mode, 0) == (0, 0)
            boundaries = [largest[source]] if source in K.FLOATS else [(1 << (K.INTEGERS[source] - 1)) - 1, 1 << (K.INTEGERS[source] - 1)]
            for bits in boundaries:
                try:
                    result, _ = K.convert(opcode, mode, bits)
                except K.ConversionError as error:
                    assert error.code == "float-to-integer-out-of-range" and destination in K.INTEGERS
                    continue
                if destination == "tf32":
                    assert result & 0x1fff == 0


def test_reference_vectors():
    for mode, positive, negative in ((NE, 0x02, 0xfe), (TZ, 0x01, 0xff), (TP, 0x02, 0xff), (TN, 0x01, 0xfe)):
        assert K.convert(157, mode, 0x3e00) == (positive, K.INEXACT) and K.convert(157, mode, 0xbe00) == (negative, K.INEXACT)
    for mode, positive, negative in ((NE, 0x6800, 0xe800), (TZ, 0x6800, 0xe800), (TP, 0x6801, 0xe800), (TN, 0x6800, 0xe801)):
        assert K.convert(147, mode, 0x00000801) == (positive, K.INEXACT) and K.convert(147, mode, 0xfffff7ff) == (negative, K.INEXACT)
    assert K.convert(156, NE, 0x3fc0) == (0x3fc00000, 0) and K.convert(173, NE, 0x3fc00000) == (0x3fc0, 0)
    for mode, positive, negative in ((NE, 0x3f800000, 0xbf800000), (TZ, 0x3f800000, 0xbf800000), (TP, 0x3f802000, 0xbf800000), (TN, 0x3f800000, 0xbf802000)):
        assert K.convert(168, mode, 0x3f801000) == (positive, K.INEXACT) and K.convert(168, mode, 0xbf801000) == (negative, K.INEXACT)
    assert K.convert(166, TP, 0x80000000) == (0x8000, 0) and K.convert(156, NE, 0x8000) == (0x80000000, 0)
    assert K.convert(171, TN, 0x80000000) == (0, 0)                                   # -0 to an integer is 0
    assert K.convert(166, NE, 0xffc12345) == (0x7e00, 0) and K.convert(166, NE, 0xff812345) == (0x7e00, K.INVALID)
    assert K.convert(174, NE, 0xff802000) == (0x7fc00000, K.INVALID) and K.convert(174, NE, 0xffc02000) == (0x7fc00000, 0)
    assert K.convert(166, NE, 0x33800000) == (0x0001, 0)                              # exact subnormal
    assert K.convert(166, NE, 0x33000000) == (0x0000, K.UNDERFLOW | K.INEXACT)        # tiny tie
    assert K.convert(166, NE, 0x387fe000) == (0x0400, K.UNDERFLOW | K.INEXACT)        # tiny before, normal after
    assert K.convert(166, NE, 0x387ff000) == (0x0400, K.INEXACT)
    for opcode, positive_source, negative_source in ((147, 0x7fffffff, 0x80000000), (166, 0x7f7fffff, 0xff7fffff)):
        for mode, positive, negative in ((NE, 0x7c00, 0xfc00), (TZ, 0x7bff, 0xfbff), (TP, 0x7c00, 0xfbff), (TN, 0x7bff, 0xfc00)):
            assert K.convert(opcode, mode, positive_source) == (positive, K.OVERFLOW | K.INEXACT)
            assert K.convert(opcode, mode, negative_source) == (negative, K.OVERFLOW | K.INEXACT)
    assert K.convert(145, TP, 0xffff) == (0xbf800000, 0) and K.convert(149, NE, 0x80000000) == (0xcf000000, 0)
    assert K.convert(159, NE, 0x7bff) == (0x0000ffe0, 0)
    for bits in (0x7f800000, 0xff800000, 0x7fc01234, 0x7f801234):
        with pytest.raises(K.ConversionError, match="float-to-integer-non-finite"):
            K.convert(163, NE, bits)
    for bits in (0x43000000, 0x42ff0000):                                             # 128, and 127.5 under nearest-even
        with pytest.raises(K.ConversionError, match="float-to-integer-out-of-range"):
            K.convert(163, NE, bits)
    assert K.convert(163, TZ, 0x42ff0000) == (0x7f, K.INEXACT)
    with pytest.raises(K.ConversionError, match="invalid-source-encoding"):
        K.convert(174, NE, 0x3f800001)


# ------------------------------------------------------------------------------------------------------------ GPU
def _sources(source, destination, rng, count):
    """Bit patterns of `source`; for an integer destination only finite values near its range."""
    if source in K.INTEGERS:
        width = K.INTEGERS[source]
        values = rng.integers(0, 1 << width, count, dtype=np.uint64)
        values[:6] = [0, 1, (1 << width) - 1, (1 << (width - 1)) - 1, 1 << (width - 1), 0x801 & ((1 << width) - 1)]
        return values.astype(DTYPE[source])
    p, ebits, shift = K.FLOATS[source]
    semantic_bits = p + ebits
    if destination in K.INTEGERS:
        import torch
        limit = float(1 << (K.INTEGERS[destination] - 1))
        if source == "f16":
            limit = min(limit, 60000.0)                                       # stay inside the half range
        generator = torch.Generator().manual_seed(int(rng.integers(1 << 30)))
        values = (torch.rand(count, generator=generator, dtype=torch.float64) * 2 - 1) * limit * 1.02
        values[::5] = torch.round(values[::5] * 2) / 2                       # ties
        values[:4] = torch.tensor([0.0, -0.0, 0.5, -0.5], dtype=torch.float64)
        f32 = values.to(torch.float32).view(torch.int32).numpy().view(np.uint32).astype(np.uint64)
        drop = 32 - semantic_bits                                            # truncate f32 to the source's semantic bits
        if source == "f16":
            return values.to(torch.float16).view(torch.int16).numpy().view(np.uint16).copy()
        return (((f32 >> drop) << shift) if source != "f32" else f32).astype(DTYPE[source])
    values = rng.integers(0, 1 << semantic_bits, count, dtype=np.uint64)
    exponent_mask = ((1 << ebits) - 1) << (p - 1)
    special = [0, 1 << (semantic_bits - 1), exponent_mask, exponent_mask | 1, exponent_mask | (1 << (p - 2)), 1, exponent_mask - 1,
               (1 << (p - 1)), (1 << (p - 1)) - 1]
    values[:len(special)] = special
    return (values << shift).astype(DTYPE[source])


def _oracle(opcode, mode, sources):
    keep, want, flags = [], [], 0
    for index, bits in enumerate(sources):
        try:
            result, f = K.convert(opcode, mode, int(bits))
        except K.ConversionError:
            continue
        keep.append(index)
        want.append(result)
        flags |= f
    return keep, want, flags


def _run(backend, opcode, mode, sources):
    _, source, destination, _ = K.ROUTES[opcode]
    key = PhysicalTensorDescriptor(FORMAT[source], abi.LAYOUT_TENSOR, [len(sources)])
    out_key = PhysicalTensorDescriptor(FORMAT[destination], abi.LAYOUT_TENSOR, [len(sources)])
    template = np.full(len(sources) * np.dtype(DTYPE[destination]).itemsize, 0xa5, dtype=np.uint8)
    result = backend.execute_convert(opcode, NumericTensor(key, sources), NumericTensor(out_key, template), rounding_mode=mode, formal=True)
    return result.destination.storage.view(DTYPE[destination]), result.evidence


@pytest.mark.gpu
@pytest.mark.parametrize("opcode", [op for op, route in K.ROUTES.items() if route[3] != K.ZERO_POINT])
def test_every_route_and_mode_matches_the_oracle(backend, opcode):
    _, source, destination, kind = K.ROUTES[opcode]
    rng = np.random.default_rng(20260803 + opcode)
    for mode in ((NE, TZ, TP, TN) if kind == K.ROUNDING else (NE,)):
        candidates = _sources(source, destination, rng, 1500)
        keep, want, flags = _oracle(opcode, mode, candidates)
        assert len(keep) > 700, (opcode, mode, len(keep))
        sources = candidates[keep]
        got, evidence = _run(backend, opcode, mode, sources)
        assert np.array_equal(got, np.array(want, dtype=DTYPE[destination])), (opcode, mode)
        assert evidence.flags == flags and evidence.scalar_evaluations == len(sources)


@pytest.mark.gpu
@pytest.mark.parametrize("opcode, modes", [(160, (NE, TZ, TP, TN)), (154, (NE,)), (144, (NE, TP)), (143, (NE,))])
def test_complete_sixteen_bit_operand_space(backend, opcode, modes):
    sources = np.arange(65536, dtype=np.uint16)
    _, _, destination, _ = K.ROUTES[opcode]
    for mode in modes:
        keep, want, flags = _oracle(opcode, mode, sources)
        assert len(keep) == 65536
        got, evidence = _run(backend, opcode, mode, sources)
        assert np.array_equal(got, np.array(want, dtype=DTYPE[destination])), (opcode, mode)
        assert evidence.flags == flags


@pytest.mark.gpu
def test_flags_of_single_elements(backend):
    cases = [(166, NE, 0x33800000), (166, NE, 0x33000000), (166, NE, 0x387fe000), (166, NE, 0x387ff000), (166, TZ, 0x7f7fffff),
             (166, TP, 0xff7fffff), (147, TN, 0x7fffffff), (168, TP, 0x3f801000), (166, NE, 0xff812345), (174, NE, 0xff802000),
             (167, TN, 0x00000001), (167, TP, 0x00000001), (163, TZ, 0x42ff0000), (171, TN, 0x80000000), (149, NE, 0x80000000)]
    for opcode, mode, bits in cases:
        source = K.ROUTES[opcode][1]
        got, evidence = _run(backend, opcode, mode, np.array([bits], dtype=DTYPE[source]))
        assert (int(got[0]), evidence.flags) == K.convert(opcode, mode, bits), (opcode, mode, hex(bits))


@pytest.mark.gpu
def test_refused_elements_fail_the_command_and_write_nothing(backend):
    sources = np.array([0x3f800000, 0x42fe0000, 0x7f800000, 0x43000000], dtype=np.uint32)         # 1, 127, +inf, 128
    with pytest.raises(WB200Error, match="float-to-integer-non-finite.* at element 2"):
        _run(backend, 163, NE, sources)
    with pytest.raises(WB200Error, match="float-to-integer-out-of-range.* at element 3"):
        _run(backend, 163, NE, sources[[0, 1, 1, 3]])
    with pytest.raises(WB200Error, match="invalid-source-encoding.* at element 1"):
        _run(backend, 174, NE, np.array([0x3f800000, 0x3f800001], dtype=np.uint32))
    with pytest.raises(WB200Error, match="zero-point routes"):
        _run(backend, 141, NE, np.zeros(4, dtype=np.uint8))
    with pytest.raises(WB200Error, match="deterministic rounding modes"):
        _run(backend, 163, K.STOCHASTIC, sources)
    pad = ScratchPad(backend, 1 << 16)
    pad.write(0, sources)
    pad.write(0x1000, np.full(4, 0xa5, np.uint8))
    with pytest.raises(WB200Error, match="float-to-integer-non-finite"):
        pad.convert(163, 0, 0x1000, 4)
    assert list(pad.read(0x1000, 4)) == [0xa5] * 4
    assert pad.convert(163, 0, 0x1000, 2) == 0 and list(pad.read(0x1000, 4)) == [1, 127, 0xa5, 0xa5]
    pad.write(0, np.array([0x3fc00000, 0xbfc00000], dtype=np.uint32))                               # +-1.5
    assert pad.convert(165, 0, 0x2000, 2, rounding_mode=TP) == K.INEXACT
    assert list(pad.read(0x2000, 8).view(np.uint32)) == [2, 0xffffffff]
