"""TargetCall-level elementwise forms and pooling on a device-resident scratch-pad image, bit for bit against the
exact-rational oracle applied the way the reference expands the operands
(lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:296-372 for the second-operand forms, :466-583 for pooling)."""
import numpy as np
import pytest

from oracle import formal_scalar as F
from vibe_compiler_b200 import _abi as abi
from vibe_compiler_b200.backend import NumericTensor, PhysicalTensorDescriptor, WB200Error
from vibe_compiler_b200.target_calls import ScratchPad

FMT = {"f16": abi.F16, "bf16": abi.BF16, "f32": abi.F32}
DTYPE = {"f16": np.uint16, "bf16": np.uint16, "f32": np.uint32}
ONE = {"f16": 0x3c00, "bf16": 0x3f80, "f32": 0x3f800000}


def _patterns(fmt, count, rng, finite=False):
    bits = 32 if fmt == "f32" else 16
    values = rng.integers(0, 2 ** bits, count, dtype=np.uint64)
    exp_mask = {"f16": 0x7c00, "bf16": 0x7f80, "f32": 0x7f800000}[fmt]
    if finite:
        values = np.where((values & exp_mask) == exp_mask, ONE[fmt], values)
    else:
        special = [0, 1 << (bits - 1), exp_mask, exp_mask | 1, 1, exp_mask - 1, ONE[fmt]]
        values[:min(len(special), count)] = special[:count]
        rng.shuffle(values)
    return values.astype(DTYPE[fmt])


def _expected(op, fmt, out_fmt, a, b_of):
    want, flags = [], 0
    for i, x in enumerate(a):
        bits, f = F.evaluate(op, fmt, out_fmt, int(x), int(b_of(i)))
        want.append(bits)
        flags |= f
    return want, flags


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["f16", "bf16", "f32"])
def test_second_operand_forms(backend, fmt):
    rng = np.random.default_rng(20260803)
    pad = ScratchPad(backend, 1 << 20)
    width = np.dtype(DTYPE[fmt]).itemsize
    lhs_at, rhs_at, dst_at = 0x1000, 0x9000, 0x12000
    # (count, unit, group): a repeated unit of 5 elements; one 64-element row per 128-element group; full vector
    for op in ("add", "mul", "max", "sub"):
        count = 203
        a, unit = _patterns(fmt, count, rng), _patterns(fmt, 5, rng)
        pad.write(lhs_at, a)
        pad.write(rhs_at, unit)
        flags = pad.elementwise(op, lhs_at, dst_at, count, FMT[fmt], rhs=rhs_at, rhs_unit_elements=5)
        want, want_flags = _expected(op, fmt, fmt, a, lambda i: unit[i % 5])
        assert list(pad.read(dst_at, count * width).view(DTYPE[fmt])) == want, (op, "unit")
        assert flags == want_flags

        count = 512
        a, rows = _patterns(fmt, count, rng), _patterns(fmt, count // 128 * 64, rng)
        pad.write(lhs_at, a)
        pad.write(rhs_at, np.concatenate([rows, np.zeros(count - rows.size, DTYPE[fmt])]))
        flags = pad.elementwise(op, lhs_at, dst_at, count, FMT[fmt], rhs=rhs_at, rhs_group_elements=128)
        want, want_flags = _expected(op, fmt, fmt, a, lambda i: rows[i // 128 * 64 + i % 64])
        assert list(pad.read(dst_at, count * width).view(DTYPE[fmt])) == want, (op, "group")
        assert flags == want_flags

        count = 77
        a = _patterns(fmt, count, rng)
        scalar = int(_patterns(fmt, 1, rng, finite=True)[0])
        pad.write(lhs_at, a)
        flags = pad.elementwise(op, lhs_at, dst_at, count, FMT[fmt], scalar_bits=scalar)
        want, want_flags = _expected(op, fmt, fmt, a, lambda i: scalar)
        assert list(pad.read(dst_at, count * width).view(DTYPE[fmt])) == want, (op, "scalar")
        assert flags == want_flags

        b = _patterns(fmt, count, rng)
        pad.write(rhs_at, b)
        flags = pad.elementwise(op, lhs_at, dst_at, count, FMT[fmt], rhs=rhs_at)
        want, want_flags = _expected(op, fmt, fmt, a, lambda i: b[i])
        assert list(pad.read(dst_at, count * width).view(DTYPE[fmt])) == want, (op, "vector")
        assert flags == want_flags


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["f16", "bf16", "f32"])
def test_relations_against_an_immediate_and_unary_calls(backend, fmt):
    rng = np.random.default_rng(4)
    pad = ScratchPad(backend, 1 << 20)
    width = np.dtype(DTYPE[fmt]).itemsize
    count = 93
    a = _patterns(fmt, count, rng)
    a[::4] = ONE[fmt]
    pad.write(0, a)
    for op in ("eq", "ne", "ge", "lt"):
        want, want_flags = _expected(op, fmt, "bool", a, lambda i: ONE[fmt])      # a signalling NaN operand raises invalid
        pad.write(0x4000, np.full(16, 0xff, np.uint8))
        assert pad.elementwise(op, 0, 0x4000, count, FMT[fmt], scalar_bits=ONE[fmt]) == want_flags
        packed = np.unpackbits(pad.read(0x4000, 12), bitorder="little")
        assert list(packed[:count]) == want and all(packed[count:] == 1), op      # the three spare bits keep their value
        pad.elementwise(op, 0, 0x5000, count, FMT[fmt], scalar_bits=ONE[fmt], numeric_result=True)
        assert list(pad.read(0x5000, count * width).view(DTYPE[fmt])) == [ONE[fmt] if t else 0 for t in want], op
    for op in ("abs", "neg", "relu", "square", "recip"):
        flags = pad.elementwise(op, 0, 0x6000, count, FMT[fmt])
        want, want_flags = _expected(op, fmt, fmt, a, lambda i: 0)
        assert list(pad.read(0x6000, count * width).view(DTYPE[fmt])) == want and flags == want_flags, op
    # logic on the packed relation result: not(x >= 1) == (x < 1) wherever x is not NaN
    pad.elementwise("ge", 0, 0x4000, count, FMT[fmt], scalar_bits=ONE[fmt])
    pad.elementwise("logic_not", 0x4000, 0x4100, count, abi.BOOL)
    inverted = np.unpackbits(pad.read(0x4100, 12), bitorder="little")[:count]
    assert list(inverted) == [1 - F.evaluate("ge", fmt, "bool", int(x), ONE[fmt])[0] for x in a]
    if fmt != "f32":
        flags = pad.elementwise("exp", 0, 0x6000, count, FMT[fmt])
        want = [F.evaluate_function("exp", fmt, int(x)) for x in a]
        assert list(pad.read(0x6000, count * width).view(DTYPE[fmt])) == [w[0] for w in want]
        assert flags == int(np.bitwise_or.reduce([w[1] for w in want]))


@pytest.mark.gpu
def test_malformed_elementwise_calls_are_rejected(backend):
    pad = ScratchPad(backend, 1 << 16)
    with pytest.raises(WB200Error, match="multiples of 64"):
        pad.elementwise("add", 0, 0x2000, 256, abi.F32, rhs=0x1000, rhs_group_elements=96)
    with pytest.raises(WB200Error, match="outside the memory image"):
        pad.elementwise("add", 0, 0x2000, 1 << 15, abi.F32, rhs=0x1000)
    with pytest.raises(WB200Error, match="no formal evaluation"):
        pad.elementwise("exp_lp", 0, 0x2000, 16, abi.F32)
    with pytest.raises(WB200Error, match="TF32 for the function family"):
        pad.elementwise("add", 0, 0x2000, 16, abi.TF32, rhs=0x1000)
    lib = abi.load()
    assert lib.wb200_target_call_elementwise(pad._handle, abi.ELEMENTWISE_OPS["add"], 0, 0, 0x2000, 16, abi.F32, 0, 2, 0, None) == abi.ERR_INVALID_ARGUMENT
    assert lib.wb200_target_call_elementwise(pad._handle, abi.ELEMENTWISE_OPS["eq"], 0, 0, 0x2000, 16, abi.F32, 0, 0, 2, None) == abi.ERR_INVALID_ARGUMENT
    assert lib.wb200_target_call_elementwise(pad._handle, abi.ELEMENTWISE_OPS["add"], 0, 1 << 32, 0x2000, 16, abi.F32, 0, 1, 0, None) == abi.ERR_INVALID_ARGUMENT


def _pool_oracle(kind, fmt, compact, source_shape, destination_shape, kernel_strides):
    kw_, kh_, sw, sh = kernel_strides
    n_, oh, ow, c_ = destination_shape
    _, ih, iw, _ = source_shape
    op = {"max": "max", "min": "min", "sum": "add"}[kind]
    out, flags = np.zeros(n_ * oh * ow * c_, dtype=DTYPE[fmt]), 0
    for n in range(n_):
        for h in range(oh):
            for w in range(ow):
                for c in range(c_):
                    result = 0
                    for kh in range(kh_):
                        for kw in range(kw_):
                            tap = int(compact[((n * ih + h * sh + kh) * iw + w * sw + kw) * c_ + c])
                            if kh == 0 and kw == 0 and kind != "sum":
                                result = tap
                            else:
                                result, f = F.evaluate(op, fmt, fmt, result, tap)
                                flags |= f
                    out[((n * oh + h) * ow + w) * c_ + c] = result
    return out, flags


@pytest.mark.gpu
@pytest.mark.parametrize("kind, fmt, channels", [("max", "f16", 70), ("min", "bf16", 70), ("max", "f32", 70), ("sum", "f32", 70),
                                                 ("max", "bf16", 72), ("sum", "f32", 72), ("min", "f16", 128)])
def test_pooling_folds_each_window_in_the_reference_order(backend, kind, fmt, channels):
    rng = np.random.default_rng(17)
    # 70 channels: one full block of 64 and a ragged tail (one channel per thread); 72 and 128: four channels per thread
    source_shape, kernel_strides = (2, 7, 9, channels), (3, 2, 2, 1)
    destination_shape = (2, (7 - 2) // 1 + 1, (9 - 3) // 2 + 1, channels)
    compact = _patterns(fmt, int(np.prod(source_shape)), rng, finite=(kind == "sum"))
    if kind == "sum":
        compact[:3] = [0x7f7fffff, 0x7f7fffff, 0x00000001]           # an overflow and a subnormal among the taps
    source_key = PhysicalTensorDescriptor(FMT[fmt], abi.LAYOUT_NCX, list(source_shape))
    destination_key = PhysicalTensorDescriptor(FMT[fmt], abi.LAYOUT_NCX, list(destination_shape))
    source_bytes, destination_bytes = backend.physical_bytes(source_key), backend.physical_bytes(destination_key)
    storage = backend.pack(source_key, compact, np.zeros(source_bytes, np.uint8))
    pad = ScratchPad(backend, 1 << 20)
    dst_at = (source_bytes + 0xfff) & ~0xfff
    pad.write(0, storage)
    pad.write(dst_at, np.full(destination_bytes, 0xa5, np.uint8))
    flags = pad.pool(kind, 0, dst_at, source_shape, destination_shape, kernel_strides, FMT[fmt])
    produced = pad.read(dst_at, destination_bytes)
    got = backend.unpack(NumericTensor(destination_key, produced)).view(DTYPE[fmt]).reshape(-1)
    want, want_flags = _pool_oracle(kind, fmt, compact, source_shape, destination_shape, kernel_strides)
    assert np.array_equal(got, want)
    assert flags == want_flags
    # padding bytes of the physical destination are left as they were
    repacked = backend.pack(destination_key, got, np.full(destination_bytes, 0xa5, np.uint8))
    assert np.array_equal(repacked, produced)


@pytest.mark.gpu
def test_pooling_outside_the_plain_domain_is_declined(backend):
    pad = ScratchPad(backend, 1 << 20)
    shape, out = (1, 4, 4, 64), (1, 2, 2, 64)
    with pytest.raises(WB200Error, match="no qualified plain numeric implementation"):
        pad.pool(115, 0, 0x8000, shape, out, (2, 2, 2, 2), abi.F32)
    with pytest.raises(WB200Error, match="F32 accumulation only"):
        pad.pool("sum", 0, 0x8000, shape, out, (2, 2, 2, 2), abi.BF16)
    with pytest.raises(WB200Error, match="explicit input padding"):
        pad.pool("max", 0, 0x8000, shape, out, (2, 2, 2, 2), abi.F32, pads=(1, 0, 0, 0))
    with pytest.raises(WB200Error, match="window geometry"):
        pad.pool("max", 0, 0x8000, shape, (1, 3, 2, 64), (2, 2, 2, 2), abi.F32)
    with pytest.raises(WB200Error, match="batch and channel"):
        pad.pool("max", 0, 0x8000, shape, (1, 2, 2, 32), (2, 2, 2, 2), abi.F32)


def _reduce_oracle(operation, fmt, compact, shape, reduced):
    """Fold of lib/Wafer/Simulator/Reference/Numeric/FormalTensorNumeric.cpp:363-425 with the exact-rational step."""
    out_shape = [1 if d in reduced else extent for d, extent in enumerate(shape)]
    infinity = {"f16": 0x7c00, "bf16": 0x7f80, "f32": 0x7f800000}[fmt]
    sign = 0x80000000 if fmt == "f32" else 0x8000
    identity = {"sum": 0, "max": infinity | sign, "min": infinity}[operation]
    op = {"sum": "add", "max": "max", "min": "min"}[operation]
    out = np.full(int(np.prod(out_shape)), identity, dtype=np.uint64)
    flags = 0
    for index, bits in enumerate(compact):
        coordinates = np.unravel_index(index, shape)
        kept = [c for d, c in enumerate(coordinates) if d not in reduced]
        kept_shape = [e for d, e in enumerate(shape) if d not in reduced]
        destination = int(np.ravel_multi_index(kept, kept_shape)) if kept else 0
        out[destination], f = F.evaluate(op, fmt, fmt, int(out[destination]), int(bits))
        flags |= f
    return out.astype(DTYPE[fmt]), out_shape, flags


@pytest.mark.gpu
@pytest.mark.parametrize("operation, fmt, dimension, reduced", [
    ("sum", "f32", "trailing0", (3,)), ("sum", "f32", "trailing2and1", (1, 2)), ("max", "bf16", "trailing1", (2,)),
    ("min", "f16", "trailing2and1and0", (1, 2, 3)), ("max", "f32", "trailing3", (0,)), ("min", "bf16", "trailing2", (1,))])
def test_formal_reduce_folds_in_row_major_order(backend, operation, fmt, dimension, reduced):
    rng = np.random.default_rng(23)
    shape = (2, 3, 5, 70)
    compact = _patterns(fmt, int(np.prod(shape)), rng, finite=(operation == "sum"))
    if operation == "sum":
        compact[:3] = [0x7f7fffff, 0x7f7fffff, 0x00000001]          # an overflowing pair and a subnormal
    want, out_shape, want_flags = _reduce_oracle(operation, fmt, compact, shape, reduced)
    source_key = PhysicalTensorDescriptor(FMT[fmt], abi.LAYOUT_NCX, list(shape))
    destination_key = PhysicalTensorDescriptor(FMT[fmt], abi.LAYOUT_NCX, out_shape)
    storage = backend.pack(source_key, compact, np.zeros(backend.physical_bytes(source_key), np.uint8))
    template = np.full(backend.physical_bytes(destination_key), 0xa5, np.uint8)
    result = backend.execute_reduce(operation, dimension, NumericTensor(source_key, storage), NumericTensor(destination_key, template), formal=True)
    got = backend.unpack(result.destination).view(DTYPE[fmt]).reshape(-1)
    assert np.array_equal(got, want) and result.evidence.flags == want_flags
    assert result.evidence.scalar_evaluations == compact.size
    pad = ScratchPad(backend, 1 << 20)
    dst_at = (storage.size + 0xfff) & ~0xfff
    pad.write(0, storage)
    pad.write(dst_at, template)
    assert pad.reduce(operation, 0, dst_at, dimension, shape, FMT[fmt]) == want_flags
    assert np.array_equal(pad.read(dst_at, template.size), result.destination.storage)


@pytest.mark.gpu
def test_formal_reduce_domain(backend):
    pad = ScratchPad(backend, 1 << 20)
    with pytest.raises(WB200Error, match="F32 sum"):
        pad.reduce("sum", 0, 0x8000, "trailing0", (1, 2, 2, 64), abi.BF16)
    with pytest.raises(WB200Error, match="F32 sum"):
        pad.reduce("avg", 0, 0x8000, "trailing0", (1, 2, 2, 64), abi.F32)
    with pytest.raises(WB200Error, match="outside the memory image"):
        pad.reduce("max", 0, 0x8000, "trailing0", (64, 64, 64, 64), abi.F32)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["f16", "bf16", "f32"])
def test_bit2fp_and_mask_move(backend, fmt):
    """lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:198-286."""
    rng = np.random.default_rng(31)
    pad = ScratchPad(backend, 1 << 16)
    count, width = 203, np.dtype(DTYPE[fmt]).itemsize
    bits = rng.integers(0, 2, count).astype(np.uint8)
    pad.write(0, np.packbits(bits, bitorder="little"))
    pad.bit2fp(0, 0x1000, count, FMT[fmt])
    mask = pad.read(0x1000, count * width).view(DTYPE[fmt])
    assert list(mask) == [ONE[fmt] if b else 0 for b in bits]
    source, destination = _patterns(fmt, count, rng), _patterns(fmt, count, rng)
    pad.write(0x2000, source)
    pad.write(0x3000, destination)
    pad.mask_move(0x2000, 0x1000, 0x3000, count, FMT[fmt])
    assert list(pad.read(0x3000, count * width).view(DTYPE[fmt])) == [int(s) if b else int(d) for s, b, d in zip(source, bits, destination)]
    # a mask value that is neither 0 nor 1.0 (here -0 at element 5 and 2.0 at element 9) refuses the command; nothing moves
    bad = mask.copy()
    bad[5] = 0x80000000 if fmt == "f32" else 0x8000
    bad[9] = {"f16": 0x4000, "bf16": 0x4000, "f32": 0x40000000}[fmt]
    pad.write(0x1000, bad)
    pad.write(0x3000, destination)
    with pytest.raises(WB200Error, match="canonical zero/one mask values at element 5"):
        pad.mask_move(0x2000, 0x1000, 0x3000, count, FMT[fmt])
    assert list(pad.read(0x3000, count * width).view(DTYPE[fmt])) == [int(d) for d in destination]
    with pytest.raises(WB200Error, match="F16, BF16 or F32"):
        pad.bit2fp(0, 0x1000, count, abi.I32)
    with pytest.raises(WB200Error, match="outside the memory image"):
        pad.mask_move(0x2000, 0x1000, 0xfff0, count, FMT[fmt])
