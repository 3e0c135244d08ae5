"""tcgen05 GEMM parity on the GPU through the C ABI: against the CPU oracle (k-ascending f32 FMA
chain) within the bf16/f16 bound of 1e-2 max relative error, bit-exact where every product and sum is
exactly representable, and against the committed PyTorch golden outputs."""
import numpy as np
import pytest
import torch

from tests import helpers
from tests.helpers import fixtures
from vibe_compiler_b200 import _abi as abi
from vibe_compiler_b200.backend import FormalGemmOperation, NumericTensor, PhysicalTensorDescriptor

pytestmark = pytest.mark.gpu
BOUND_16BIT = 1e-2  # max |a - e| / max |e| for bf16 / f16 storage, fp32 accumulation


def make_inputs(m, k, n, dtype, lt, rt, seed=20260803):
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = (torch.rand((k, m) if lt else (m, k), generator=g) * 2 - 1).to(dtype)   # ~U[-1, 1]
    b = (torch.rand((n, k) if rt else (k, n), generator=g) * 2 - 1).to(dtype)
    bias = torch.randn(n, generator=g) * 0.02
    return a, b, bias


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 320), (200, 264, 72), (8, 8, 8), (1000, 136, 1032)])
@pytest.mark.parametrize("lt,rt", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_umma_gemm_orientations_and_tails(backend, oracle, m, n, k, lt, rt, dtype):
    fmt = helpers.FMT_OF[dtype]
    a, b, _ = make_inputs(m, k, n, dtype, lt, rt)
    got = backend.gemm_epilogue(a, b, lhs_transposed=lt, rhs_transposed=rt)   # host buffers: staged by the library
    want = oracle.gemm_epilogue(fmt, fmt, m, n, k, helpers.bits(a), helpers.bits(b), lhs_transposed=lt, rhs_transposed=rt, threads=8)
    assert helpers.max_rel_err(helpers.values(helpers.bits(got), fmt), helpers.values(want, fmt)) <= BOUND_16BIT
    helpers.reference_gate(oracle, fmt, helpers.bits(got), want)


@pytest.mark.parametrize("epilogue", [abi.EPI_NONE, abi.EPI_BIAS, abi.EPI_BIAS_GELU])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_umma_gemm_epilogues(backend, oracle, epilogue, out_dtype):
    m, n, k = 384, 520, 264
    a, b, bias = make_inputs(m, k, n, torch.bfloat16, False, False)
    out_fmt = helpers.FMT_OF[out_dtype]
    got = backend.gemm_epilogue(a.cuda(), b.cuda(), bias.cuda(), epilogue=epilogue, out_dtype=out_dtype)   # device buffers
    torch.cuda.synchronize()
    backend.poll()
    want = oracle.gemm_epilogue("bf16", out_fmt, m, n, k, helpers.bits(a), helpers.bits(b), bias.numpy(), epilogue, threads=8)
    bound = BOUND_16BIT if out_fmt != "f32" else 1e-5 * 50  # f32 output still carries tensor-core summation order
    assert helpers.max_rel_err(helpers.values(helpers.bits(got), out_fmt), helpers.values(want, out_fmt)) <= bound


def test_umma_gemm_is_exact_on_exactly_representable_sums(backend, oracle):
    # Signed sixteenths (the reference's exact-input long-K case): every f32 product and partial sum is exact,
    # so any summation order gives the same bits and the tensor path must equal the formal chain bit for bit.
    name = "gemm_f16_exact_long_k"
    a, b = fixtures.gemm_inputs(name)
    got = backend.gemm_epilogue(a, b)
    assert np.array_equal(helpers.bits(got), helpers.golden()[name])
    m, k = a.shape
    want = oracle.formal_gemm("f16", "f16", 1, m, k, b.shape[1], helpers.bits(a).reshape(-1), helpers.bits(b).reshape(-1), threads=8)
    assert np.array_equal(helpers.bits(got).reshape(-1), want)
    got32 = backend.gemm_epilogue(a, b, out_dtype=torch.float32)
    want32 = oracle.formal_gemm("f16", "f32", 1, m, k, b.shape[1], helpers.bits(a).reshape(-1), helpers.bits(b).reshape(-1), threads=8)
    assert np.array_equal(helpers.bits(got32).reshape(-1), want32)


def test_umma_gemm_golden_bf16(backend, oracle):
    a, b = fixtures.gemm_inputs("gemm_bf16")
    got = backend.gemm_epilogue(a, b)
    expected = helpers.golden()["gemm_bf16"]
    assert helpers.max_rel_err(helpers.values(helpers.bits(got), "bf16"), helpers.values(expected, "bf16")) <= BOUND_16BIT
    helpers.reference_gate(oracle, "bf16", helpers.bits(got), expected)


def test_subulp_partial_survives_in_f32_output(backend, oracle):
    # TargetModelKernelTest.cpp:1424-1459 scaled up to a tensor-core tile: 1*1 + eps*1 must keep eps in f32.
    m = n = 128
    k = 64
    a = torch.zeros(m, k, dtype=torch.bfloat16)
    a[:, 0] = 1.0
    a[:, 1] = 2.0 ** -10
    b = torch.zeros(k, n, dtype=torch.bfloat16)
    b[0, :] = 1.0
    b[1, :] = 1.0
    got = backend.gemm_epilogue(a, b, out_dtype=torch.float32)
    assert torch.all(got == 1.0 + 2.0 ** -10)


@pytest.mark.parametrize("batch,m,k,n", [(1, 128, 64, 256), (1, 136, 72, 264), (2, 64, 128, 128)])
def test_tensor_policy_through_physical_storage(backend, oracle, batch, m, k, n):
    # wb200_gemm with the tensor policy: Cx / NCx bytes in, Cx / NCx bytes out, padding preserved.
    rng = np.random.default_rng(5)
    lhs = oracle.convert("f32", "bf16", (rng.random(batch * m * k, dtype=np.float32) * 2 - 1).view(np.uint32))[1]
    rhs = oracle.convert("f32", "bf16", (rng.random(batch * k * n, dtype=np.float32) * 2 - 1).view(np.uint32))[1]
    layout = "cx" if batch == 1 else "ncx"
    shape = (lambda r, c: [r, c] if batch == 1 else [batch, r, c])

    def key(fmt, s):
        return PhysicalTensorDescriptor(oracle.FORMATS[fmt], oracle.LAYOUTS[layout], s)

    def store(fmt, s, compact):
        return oracle.pack(fmt, layout, s, compact, np.full(oracle.geometry(fmt, layout, s)["physical_bytes"], 0xA5, np.uint8))

    op = FormalGemmOperation(key("bf16", shape(m, k)), key("bf16", shape(k, n)), key("bf16", shape(m, n)), m, k, n, batch)
    tmpl = np.full(oracle.geometry("bf16", layout, shape(m, n))["physical_bytes"], 0xA5, np.uint8)
    result = backend.try_execute(op, NumericTensor(op.lhs, store("bf16", shape(m, k), lhs)), NumericTensor(op.rhs, store("bf16", shape(k, n), rhs)),
                                 NumericTensor(op.destination, tmpl), policy=abi.GEMM_TENSOR)
    assert result is not None
    assert result.evidence.matmul_invocations == 1 and result.evidence.formal_fused_multiply_adds == 0
    assert result.evidence.reorder_invocations <= 1 and result.evidence.digest and result.evidence.implementation
    got = oracle.unpack("bf16", layout, shape(m, n), result.destination.storage)
    want = oracle.formal_gemm("bf16", "bf16", batch, m, k, n, lhs, rhs, threads=8)
    assert helpers.max_rel_err(helpers.values(got, "bf16"), helpers.values(want, "bf16")) <= BOUND_16BIT
    # padding bytes of the template survive
    repacked = oracle.pack("bf16", layout, shape(m, n), got, tmpl)
    assert np.array_equal(repacked, result.destination.storage)


def test_full_size_gemm_properties(backend):
    # Config M = N = K = 8192 is too large for the CPU oracle; check size-independent properties instead:
    # linearity in A (exact for power-of-two scaling) and agreement of a sampled block with an f64 reference.
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(20260803)
    a = (torch.rand(n, n, device="cuda", generator=g) * 2 - 1).bfloat16()
    b = (torch.rand(n, n, device="cuda", generator=g) * 2 - 1).bfloat16()
    bias = (torch.randn(n, device="cuda", generator=g) * 0.02)
    plain = backend.gemm_epilogue(a, b, out_dtype=torch.float32)
    scaled = backend.gemm_epilogue(a * 4, b, out_dtype=torch.float32)
    torch.cuda.synchronize()
    backend.poll()
    assert torch.equal(scaled, plain * 4)
    rows = torch.arange(0, n, 613, device="cuda")
    ref = a[rows].double() @ b.double()
    assert ((plain[rows].double() - ref).abs().max() / ref.abs().max()).item() <= 1e-4
    fused = backend.gemm_epilogue(a, b, bias, epilogue=abi.EPI_BIAS_GELU)
    torch.cuda.synchronize()
    backend.poll()
    ref = torch.nn.functional.gelu(ref + bias.double())
    assert ((fused[rows].double() - ref).abs().max() / ref.abs().max()).item() <= BOUND_16BIT
