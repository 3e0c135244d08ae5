"""Command-level parity on the GPU, through the C ABI, on physical storage bytes: formal GEMM,
elementwise, convert, reduce and the codec against the CPU oracle and the reference's KATs.
Bit-exact for everything except the libm transcendentals (tolerance stated per test)."""
import numpy as np
import pytest
import torch

from tests import helpers
from vibe_compiler_b200 import _abi as abi
from vibe_compiler_b200.backend import FormalGemmOperation, NumericTensor, PhysicalTensorDescriptor, WB200Error

pytestmark = pytest.mark.gpu
DT = {"f16": np.uint16, "bf16": np.uint16, "f32": np.uint32}
CONVERT_OPCODE = {("bf16", "f16"): 154, ("bf16", "f32"): 155, ("f16", "bf16"): 160, ("f16", "f32"): 161,
                  ("f32", "f16"): 166, ("f32", "bf16"): 167}


def hexes(values, fmt):
    return np.array([int(v, 16) for v in values], dtype=DT[fmt])


def key(oracle, fmt, layout, shape):
    return PhysicalTensorDescriptor(oracle.FORMATS[fmt], oracle.LAYOUTS[layout], list(shape))


def storage(oracle, fmt, layout, shape, compact, fill=0xA5):
    size = oracle.geometry(fmt, layout, shape)["physical_bytes"]
    return oracle.pack(fmt, layout, shape, np.asarray(compact, dtype=DT[fmt]), np.full(size, fill, np.uint8))


def template(oracle, fmt, layout, shape, fill=0xA5):
    return np.full(oracle.geometry(fmt, layout, shape)["physical_bytes"], fill, np.uint8)


def run_gemm(backend, oracle, fmt, out_fmt, layout, batch, m, k, n, lhs, rhs, psum, lt, rt, policy=abi.GEMM_FORMAL):
    def shape(rows, cols):
        return [rows, cols] if layout == "cx" else [batch, rows, cols]
    ls, rs, ds = shape(k, m) if lt else shape(m, k), shape(n, k) if rt else shape(k, n), shape(m, n)
    op = FormalGemmOperation(key(oracle, fmt, layout, ls), key(oracle, fmt, layout, rs), key(oracle, out_fmt, layout, ds),
                             m, k, n, batch, int(lt), int(rt), key(oracle, "f32", layout, ds) if psum is not None else None)
    result = backend.try_execute(
        op, NumericTensor(op.lhs, storage(oracle, fmt, layout, ls, lhs)), NumericTensor(op.rhs, storage(oracle, fmt, layout, rs, rhs)),
        NumericTensor(op.destination, template(oracle, out_fmt, layout, ds)),
        NumericTensor(op.psum, storage(oracle, "f32", layout, ds, psum)) if psum is not None else None, policy=policy)
    return result, (out_fmt, layout, ds)


def test_gemm_kats_bit_exact(backend, oracle, kats):
    for case in kats["gemm"]:
        psum = hexes(case["psum"], "f32") if case["psum"] else None
        result, (out_fmt, layout, ds) = run_gemm(backend, oracle, case["format"], case["out_format"], case["layout"], case["batch"],
                                                 case["m"], case["k"], case["n"], hexes(case["lhs"], case["format"]),
                                                 hexes(case["rhs"], case["format"]), psum, case["lhs_transposed"], case["rhs_transposed"])
        assert result is not None
        want = storage(oracle, out_fmt, layout, ds, hexes(case["out"], out_fmt))
        assert np.array_equal(result.destination.storage, want), case["source"]  # includes the 0xA5 padding bytes
        assert result.evidence.formal_fused_multiply_adds == case["batch"] * case["m"] * case["n"] * case["k"]


@pytest.mark.parametrize("fmt", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("n", [1024, 1025, 1031])
@pytest.mark.parametrize("orientations", [0, 1, 2, 3])
@pytest.mark.parametrize("with_partial", [False, True])
def test_formal_gemm_equals_oracle(backend, oracle, fmt, n, orientations, with_partial):
    # Inputs of the reference's parallel-vs-serial test (FormalTensorNumericTest.cpp:251-348), including the
    # signalling NaN in the last rhs element: every NaN result must be the canonical quiet NaN.
    one, sign = {"f16": (0x3c00, 0x8000), "bf16": (0x3f80, 0x8000), "f32": (0x3f800000, 0x80000000)}[fmt]
    batches, m, k = 2, 2, 17
    lt, rt = bool(orientations & 1), bool(orientations & 2)
    lhs = np.array([(one + i % 13) | (sign if i % 7 == 0 else 0) for i in range(batches * m * k)], dtype=DT[fmt])
    rhs = np.array([(one + i % 29) | (sign if i % 11 == 0 else 0) for i in range(batches * k * n)], dtype=DT[fmt])
    rhs[-1] = {"f16": 0x7d01, "bf16": 0x7f81, "f32": 0x7f800001}[fmt]
    psum = np.full(batches * m * n, 0xbf000001, dtype=np.uint32) if with_partial else None
    want = oracle.formal_gemm(fmt, fmt, batches, m, k, n, lhs, rhs, psum, lt, rt)
    result, (out_fmt, layout, ds) = run_gemm(backend, oracle, fmt, fmt, "ncx", batches, m, k, n, lhs, rhs, psum, lt, rt)
    got = oracle.unpack(out_fmt, layout, ds, result.destination.storage)
    assert np.array_equal(got, want)
    assert np.array_equal(result.destination.storage, storage(oracle, out_fmt, layout, ds, want))


@pytest.mark.parametrize("shape", [(1, 64, 64, 64), (1, 100, 77, 130), (3, 33, 129, 65), (1, 1, 16384, 3)])
@pytest.mark.parametrize("fmt,out_fmt", [("f32", "f32"), ("bf16", "bf16"), ("bf16", "f32"), ("f16", "f16")])
def test_formal_gemm_random(backend, oracle, shape, fmt, out_fmt):
    batch, m, k, n = shape
    rng = np.random.default_rng(20260803)
    a = rng.standard_normal(batch * m * k).astype(np.float32)
    b = rng.standard_normal(batch * k * n).astype(np.float32)
    rc, lhs = oracle.convert("f32", fmt, a.view(np.uint32))
    rc, rhs = oracle.convert("f32", fmt, b.view(np.uint32))
    layout = "cx" if batch == 1 else "ncx"
    want = oracle.formal_gemm(fmt, out_fmt, batch, m, k, n, lhs, rhs, threads=8)
    result, (_, _, ds) = run_gemm(backend, oracle, fmt, out_fmt, layout, batch, m, k, n, lhs, rhs, None, False, False)
    assert np.array_equal(oracle.unpack(out_fmt, layout, ds, result.destination.storage), want)


def test_gemm_rejects_bad_requests(backend, oracle):
    lhs = np.zeros(4, np.uint32)
    with pytest.raises(WB200Error) as err:
        op = FormalGemmOperation(key(oracle, "f32", "cx", [2, 2]), key(oracle, "f32", "cx", [2, 2]), key(oracle, "f32", "cx", [2, 3]), 2, 2, 2)
        backend.try_execute(op, NumericTensor(op.lhs, storage(oracle, "f32", "cx", [2, 2], lhs)),
                            NumericTensor(op.rhs, storage(oracle, "f32", "cx", [2, 2], lhs)),
                            NumericTensor(op.destination, template(oracle, "f32", "cx", [2, 3])), policy=abi.GEMM_FORMAL)
    assert err.value.status == abi.ERR_INVALID_ARGUMENT
    with pytest.raises(WB200Error) as err:  # short storage
        op = FormalGemmOperation(key(oracle, "f32", "cx", [2, 2]), key(oracle, "f32", "cx", [2, 2]), key(oracle, "f32", "cx", [2, 2]), 2, 2, 2)
        backend.try_execute(op, NumericTensor(op.lhs, storage(oracle, "f32", "cx", [2, 2], lhs)[:-1]),
                            NumericTensor(op.rhs, storage(oracle, "f32", "cx", [2, 2], lhs)),
                            NumericTensor(op.destination, template(oracle, "f32", "cx", [2, 2])), policy=abi.GEMM_FORMAL)
    assert err.value.status == abi.ERR_INVALID_ARGUMENT
    # tensor policy declines what the reference's tensor backend declines: psum, transposed operands
    result, _ = run_gemm(backend, oracle, "bf16", "bf16", "cx", 1, 8, 8, 8, np.zeros(64, np.uint16), np.zeros(64, np.uint16), None, True, False,
                         policy=abi.GEMM_TENSOR)
    assert result is None


EXACT_OPS = ["abs", "neg", "recip", "square", "sqrt", "rsqrt", "relu", "add", "sub", "mul", "max", "min"]
LIBM_OPS = ["log2", "ln", "pow2", "exp", "exp_lp", "sin", "cos", "tanh", "sigmoid", "softplus"]


def elementwise_inputs(oracle, fmt, op, count):
    rng = np.random.default_rng(7 + len(op))
    x = rng.standard_normal(count).astype(np.float32) * 3
    y = rng.standard_normal(count).astype(np.float32) * 3
    if op in ("sqrt", "rsqrt", "log2", "ln"):
        x = np.abs(x) + 1e-3
    if op in ("exp", "pow2", "exp_lp", "softplus"):
        x = np.clip(x, -10.0, 10.0)   # keeps f16 results finite
    x[:8] = [0.0, -0.0, 1.0, -1.0, 0.5, 65504.0 if op not in ("exp", "pow2", "exp_lp") else 10.0, 1e-8, -1e-8] if op not in ("sqrt", "rsqrt", "log2", "ln") else x[:8]
    y[:4] = [-0.0, 0.0, 1.0, -1.0]
    return oracle.convert("f32", fmt, x.view(np.uint32))[1], oracle.convert("f32", fmt, y.view(np.uint32))[1]


@pytest.mark.parametrize("fmt", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("op", EXACT_OPS)
@pytest.mark.parametrize("layout,shape", [("tensor", [2, 1025, 1]), ("cx", [3, 97]), ("ncx", [2, 5, 1031])])
def test_elementwise_bit_exact(backend, oracle, fmt, op, layout, shape):
    count = int(np.prod(shape))
    x, y = elementwise_inputs(oracle, fmt, op, count)
    binary = op in ("add", "sub", "mul", "max", "min")
    rc, want = oracle.elementwise(op, fmt, x, y if binary else None)
    assert rc == 0
    k = key(oracle, fmt, layout, shape)
    inputs = [NumericTensor(k, storage(oracle, fmt, layout, shape, x))]
    if binary:
        inputs.append(NumericTensor(k, storage(oracle, fmt, layout, shape, y)))
    result = backend.execute_elementwise(op, inputs, NumericTensor(k, template(oracle, fmt, layout, shape)))
    got = oracle.unpack(fmt, layout, shape, result.destination.storage)
    if op in ("max", "min"):
        # fmax/fmin may return either zero for (+0, -0): compare values, not zero signs
        assert np.array_equal(helpers.values(got, fmt), helpers.values(want, fmt))
    else:
        assert np.array_equal(got, want)
        assert np.array_equal(result.destination.storage, storage(oracle, fmt, layout, shape, want))
    assert result.evidence.scalar_evaluations == count and result.evidence.implementation


@pytest.mark.parametrize("fmt", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("op", LIBM_OPS)
def test_elementwise_libm_within_ulps(backend, oracle, fmt, op):
    # The reference evaluates these with the host libm (no bit-level pin, its own test allows 5e-6 relative);
    # CUDA's f32 functions are within a few f32 ulps, which the narrowing to f16/bf16 mostly hides.
    shape = [2, 1031, 3]
    x, _ = elementwise_inputs(oracle, fmt, op, int(np.prod(shape)))
    rc, want = oracle.elementwise(op, fmt, x)
    assert rc == 0
    k = key(oracle, fmt, "tensor", shape)
    result = backend.execute_elementwise(op, [NumericTensor(k, storage(oracle, fmt, "tensor", shape, x))],
                                         NumericTensor(k, template(oracle, fmt, "tensor", shape)))
    got = oracle.unpack(fmt, "tensor", shape, result.destination.storage)
    stats = oracle.compare(fmt, got, want)
    assert stats["finite"] == 1 and stats["max_ulp"] <= (8 if fmt == "f32" else 1), stats
    a, e = helpers.values(got, fmt), helpers.values(want, fmt)
    assert np.all(np.abs(a - e) <= 5e-6 * np.abs(e) + (0 if fmt == "f32" else np.abs(e) * 2 ** -7) + 1e-30)


def test_elementwise_kats_and_nan_rejection(backend, oracle, kats):
    for case in kats["elementwise"]:
        fmt = case["format"]
        x = hexes(case["in0"], fmt)
        k = key(oracle, fmt, "tensor", [len(x)])
        inputs = [NumericTensor(k, x.view(np.uint8))]
        if case["in1"]:
            inputs.append(NumericTensor(k, hexes(case["in1"], fmt).view(np.uint8)))
        result = backend.execute_elementwise(case["op"], inputs, NumericTensor(k, template(oracle, fmt, "tensor", [len(x)])))
        assert result.destination.storage.view(DT[fmt]).tolist() == hexes(case["out"], fmt).tolist(), case["source"]
    for case in kats["nan_rejected"]:
        fmt = case["format"]
        x = hexes(case["in0"], fmt)
        k = key(oracle, fmt, "tensor", [len(x)])
        with pytest.raises(WB200Error) as err:
            backend.execute_elementwise(case["op"], [NumericTensor(k, x.view(np.uint8))], NumericTensor(k, template(oracle, fmt, "tensor", [len(x)])))
        assert err.value.status == abi.ERR_NAN_DOMAIN and "non-NaN domain" in err.value.message
    # scalar budget (ManagedReferenceTargetModelTest.cpp:374-380)
    k = key(oracle, "f32", "tensor", [1])
    with pytest.raises(WB200Error) as err:
        backend.execute_elementwise("exp", [NumericTensor(k, np.array([0x3f800000], np.uint32).view(np.uint8))],
                                    NumericTensor(k, template(oracle, "f32", "tensor", [1])), max_scalar_evaluations=0)
    assert err.value.status == abi.ERR_BUDGET and "scalar evaluation budget exceeded" in err.value.message
    with pytest.raises(WB200Error) as err:
        backend.execute_elementwise("eq", [NumericTensor(k, np.zeros(4, np.uint8))] * 2, NumericTensor(k, template(oracle, "f32", "tensor", [1])))
    assert err.value.status == abi.ERR_UNSUPPORTED


@pytest.mark.parametrize("src,dst", list(CONVERT_OPCODE))
@pytest.mark.parametrize("extent", [1024, 1025, 1031])
def test_convert_bit_exact(backend, oracle, src, dst, extent):
    # Sample set of ManagedReferenceTargetModelTest.cpp:67-88 plus random values.
    samples = np.array([0, 0x80000000, 0x00010000, 0x80010000, 0x3f808000, 0x3f818000, 0x3f808001, 0xbf807fff, 0x7f7f0000,
                        0xff7f0000, 0x33800000, 0x477ff000, 0xc77ff000, 0x7f800000, 0xff800000], dtype=np.uint32)
    rng = np.random.default_rng(extent)
    f32 = np.concatenate([np.resize(samples, extent), rng.standard_normal(extent).astype(np.float32).view(np.uint32)])
    x = f32 if src == "f32" else oracle.convert("f32", src, f32)[1]
    shape = [2, extent, 1]
    rc, want = oracle.convert(src, dst, x)
    assert rc == 0
    for layout in ("tensor", "ncx"):
        result = backend.execute_convert(CONVERT_OPCODE[(src, dst)], NumericTensor(key(oracle, src, layout, shape), storage(oracle, src, layout, shape, x)),
                                         NumericTensor(key(oracle, dst, layout, shape), template(oracle, dst, layout, shape)))
        assert np.array_equal(result.destination.storage, storage(oracle, dst, layout, shape, want))
    with pytest.raises(WB200Error):
        backend.execute_convert(CONVERT_OPCODE[(src, dst)], NumericTensor(key(oracle, src, "tensor", shape), storage(oracle, src, "tensor", shape, x)),
                                NumericTensor(key(oracle, dst, "tensor", shape), template(oracle, dst, "tensor", shape)), rounding_mode=1)


def test_convert_kats(backend, oracle, kats):
    case = kats["convert"][1]  # through Cx storage, TargetModelKernelTest.cpp:1321-1349
    src = hexes(case["in"], "f32")
    result = backend.execute_convert(166, NumericTensor(key(oracle, "f32", "cx", [2]), storage(oracle, "f32", "cx", [2], src)),
                                     NumericTensor(key(oracle, "f16", "cx", [2]), template(oracle, "f16", "cx", [2], 0)))
    assert oracle.unpack("f16", "cx", [2], result.destination.storage).tolist() == hexes(case["out"], "f16").tolist()
    nan_case = kats["convert"][0]
    with pytest.raises(WB200Error) as err:
        backend.execute_convert(166, NumericTensor(key(oracle, "f32", "tensor", [3]), hexes(nan_case["in"], "f32").view(np.uint8)),
                                NumericTensor(key(oracle, "f16", "tensor", [3]), template(oracle, "f16", "tensor", [3])))
    assert err.value.status == abi.ERR_NAN_DOMAIN


@pytest.mark.parametrize("fmt", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("extent", [1024, 1025, 1031])
def test_extrema_reduce_kat(backend, oracle, fmt, extent):
    single, half = fmt == "f32", fmt == "f16"
    sign = 0x80000000 if single else 0x8000
    one = 0x3f800000 if single else (0x3c00 if half else 0x3f80)
    inf = 0x7f800000 if single else (0x7c00 if half else 0x7f80)
    values = np.full(3 * extent, sign | one, dtype=DT[fmt])
    values[extent:2 * extent] = one
    values[2 * extent:] = [sign if i % 2 else 0 for i in range(extent)]
    values[extent - 1] = sign | inf
    values[2 * extent - 1] = inf
    shape, out_shape = [1, 1, 3, extent], [1, 1, 3, 1]
    src = NumericTensor(key(oracle, fmt, "ncx", shape), storage(oracle, fmt, "ncx", shape, values))
    for op, expected in (("max", [sign | one, inf, 0]), ("min", [sign | inf, one, sign])):
        result = backend.execute_reduce(op, "trailing0", src, NumericTensor(key(oracle, fmt, "ncx", out_shape), template(oracle, fmt, "ncx", out_shape)))
        assert np.array_equal(result.destination.storage, storage(oracle, fmt, "ncx", out_shape, np.array(expected, dtype=DT[fmt])))
        assert result.evidence.scalar_evaluations == 3 * extent
        with pytest.raises(WB200Error) as err:
            backend.execute_reduce(op, "trailing0", src, NumericTensor(key(oracle, fmt, "ncx", out_shape), template(oracle, fmt, "ncx", out_shape)),
                                   max_scalar_evaluations=3 * extent - 1)
        assert err.value.status == abi.ERR_BUDGET
    values[-1] = inf | 1
    with pytest.raises(WB200Error) as err:
        backend.execute_reduce("max", "trailing0", NumericTensor(key(oracle, fmt, "ncx", shape), storage(oracle, fmt, "ncx", shape, values)),
                               NumericTensor(key(oracle, fmt, "ncx", out_shape), template(oracle, fmt, "ncx", out_shape)))
    assert err.value.status == abi.ERR_NAN_DOMAIN


@pytest.mark.parametrize("channels", [4, 5, 64, 70])
@pytest.mark.parametrize("dimension,dims", [("trailing0", [3]), ("trailing1", [2]), ("trailing2", [1]), ("trailing2and1", [1, 2]),
                                            ("trailing2and1and0", [1, 2, 3])])
def test_sum_reduce_over_ncx(backend, oracle, channels, dimension, dims):
    # Value pattern of TargetModelKernelTest.cpp:1255-1318.
    shape = [1, 2, 3, channels]
    values = np.array([1 + h * 3 + w + c % 5 for h in range(2) for w in range(3) for c in range(channels)], dtype=np.float32)
    out_shape = [1 if d in dims else e for d, e in enumerate(shape)]
    rc, want = oracle.reduce("sum", "f32", shape, dims, values.view(np.uint32))
    result = backend.execute_reduce("sum", dimension, NumericTensor(key(oracle, "f32", "ncx", shape), storage(oracle, "f32", "ncx", shape, values.view(np.uint32))),
                                    NumericTensor(key(oracle, "f32", "ncx", out_shape), template(oracle, "f32", "ncx", out_shape, 0)))
    assert np.array_equal(oracle.unpack("f32", "ncx", out_shape, result.destination.storage), want)
    if dimension == "trailing0":
        second = result.destination.storage[16:20].view(np.uint32)[0]  # C0 = 4 f32: second scalar sits at byte 16
        assert second == want[1] and not result.destination.storage[4:8].any()


def test_f32_sum_is_sequential(backend, oracle):
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(4 * 4099) * 1e3).astype(np.float32)
    shape = [1, 1, 4, 4099]
    rc, want = oracle.reduce("sum", "f32", shape, [3], x.view(np.uint32))
    result = backend.execute_reduce("sum", "trailing0", NumericTensor(key(oracle, "f32", "ncx", shape), storage(oracle, "f32", "ncx", shape, x.view(np.uint32))),
                                    NumericTensor(key(oracle, "f32", "ncx", [1, 1, 4, 1]), template(oracle, "f32", "ncx", [1, 1, 4, 1])))
    assert np.array_equal(oracle.unpack("f32", "ncx", [1, 1, 4, 1], result.destination.storage), want)


@pytest.mark.parametrize("fmt,layout,shape", [("f16", "cx", [2, 3]), ("f32", "cx", [2, 128]), ("f32", "ncx", [2, 3, 128]), ("f16", "cx", [2, 65]),
                                              ("bf16", "ncx", [3, 5, 1031]), ("f32", "tensor", [7, 9])])
def test_device_codec_equals_oracle(backend, oracle, fmt, layout, shape):
    count = int(np.prod(shape))
    compact = (np.arange(count) * 2654435761 % (2 ** (16 if fmt != "f32" else 32))).astype(DT[fmt])
    k = key(oracle, fmt, layout, shape)
    tmpl = template(oracle, fmt, layout, shape)
    packed = backend.pack(k, compact, tmpl)
    assert np.array_equal(packed, oracle.pack(fmt, layout, shape, compact, tmpl))
    assert np.array_equal(backend.unpack(NumericTensor(k, packed)).view(DT[fmt]), compact)


def test_bounded_wait_runs_out_and_the_backend_stays_usable(backend):
    """A device-side wait that nothing satisfies gives up at its limit, the status word carries the timeout to the host, and
    the context is intact afterwards (no trap, no hang)."""
    from vibe_compiler_b200 import _abi as abi
    from vibe_compiler_b200.backend import WB200Error
    waited = backend.selftest_bounded_wait(200_000)
    assert 200_000 <= waited < 20_000_000
    with pytest.raises(WB200Error) as err:
        backend.poll()
    assert err.value.status == abi.ERR_DEVICE_TIMEOUT
    backend.poll()                                   # the status was cleared
    a = torch.ones(64, 64, dtype=torch.bfloat16, device="cuda")
    out = backend.gemm_epilogue(a, a)
    torch.cuda.synchronize()
    backend.poll()
    assert torch.equal(out.float().cpu(), torch.full((64, 64), 64.0))


def test_two_backends_on_two_devices_in_one_process(oracle):
    """Kernel attributes (the opt-in to large dynamic shared memory) belong to a device: a second backend on another GPU of
    the same process must launch the tcgen05 GEMM, the prefill and the decode kernels too. Needs two visible devices."""
    if torch.cuda.device_count() < 2:
        pytest.skip("one visible device")
    from vibe_compiler_b200.backend import B200TargetModelBackend
    g = torch.Generator(device="cpu").manual_seed(11)
    a = (torch.rand(256, 128, generator=g) * 2 - 1).bfloat16()
    q = torch.randn(1, 4, 300, 128, generator=g).bfloat16()
    k = torch.randn(1, 2, 300, 128, generator=g).bfloat16()
    q1 = torch.randn(1, 8, 1, 128, generator=g).bfloat16()
    results = []
    for index in (0, 1):
        be = B200TargetModelBackend(index)
        device = torch.device("cuda", index)
        with torch.cuda.device(device):
            c = be.gemm_epilogue(a.to(device), a.t().contiguous().to(device))
            o = be.attention_fa(q.to(device), k.to(device), k.to(device), 128 ** -0.5, True)
            d = be.attention_fd(q1.to(device), k.to(device), k.to(device), 128 ** -0.5)
            torch.cuda.synchronize(device)
            be.poll()
        results.append((c.cpu(), o.cpu(), d.cpu()))
        be.close()
    for first, second in zip(*results):
        assert torch.equal(first.view(torch.int16), second.view(torch.int16))
