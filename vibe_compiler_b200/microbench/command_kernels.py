"""Throughput of the HBM-bound command kernels against the copy roofline.

    python -m vibe_compiler_b200.microbench.command_kernels [--elements N] [--repeats R]

Times, through the C ABI on device-resident operands, the formal elementwise forms, the formal convert routes, the formal
reduce, pooling and the comparison gate, and prints one JSON line per kernel: algorithmic bytes (operand bytes read +
result bytes written per call; for the gate 2 x count x element bytes x 6 passes), the median wall time of a call and
the achieved GB/s beside the measured copy peak. Every call ends with a stream synchronisation inside the library (the
flag word is read back), so the wall clock around a call of tens of milliseconds is the kernel time plus ~20 us.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import statistics
import time
from pathlib import Path

import numpy as np
import torch

from .. import _abi as abi
from ..backend import B200TargetModelBackend
from ..target_calls import ScratchPad


def _peak_gbs() -> float:
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"])
    except Exception:
        return 6650.0


def _time(call, repeats: int) -> float:
    call()
    samples = []
    for _ in range(repeats):
        torch.cuda.synchronize()
        start = time.perf_counter()
        call()
        samples.append(time.perf_counter() - start)
    return statistics.median(samples)


def main(argv=None) -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--elements", type=int, default=1 << 27, help="elements per operand (f32: 512 MiB each)")
    parser.add_argument("--repeats", type=int, default=7)
    parser.add_argument("--only", default="", help="run only the kernels whose name contains this text")
    args = parser.parse_args(argv)
    n = args.elements
    backend = B200TargetModelBackend(0)
    peak = _peak_gbs()
    pad = ScratchPad(backend, 4 * n * 3 + (1 << 20))
    a_at, b_at, c_at = 0, 4 * n, 8 * n
    # operands: pseudo-random finite f32 written once through the image
    rng = np.random.default_rng(1)
    block = rng.standard_normal(1 << 22).astype(np.float32)
    for base in (a_at, b_at):
        for offset in range(0, 4 * n, block.nbytes):
            pad.write(base + offset, block[: min(block.size, (4 * n - offset) // 4)])
    results = []

    def report(name, bytes_per_call, call):
        if args.only not in name:
            return
        seconds = _time(call, args.repeats)
        line = {"kernel": name, "elements": n, "bytes": bytes_per_call, "ms": round(seconds * 1e3, 3),
                "gbs": round(bytes_per_call / seconds / 1e9, 1), "peak_gbs": peak, "frac": round(bytes_per_call / seconds / 1e9 / peak, 3)}
        results.append(line)
        print(json.dumps(line), flush=True)

    report("formal_elementwise add f32 (vector rhs)", 12 * n, (lambda: pad.elementwise("add", a_at, c_at, n, abi.F32, rhs=b_at)))
    report("formal_elementwise mul f32 (immediate rhs)", 8 * n, (lambda: pad.elementwise("mul", a_at, c_at, n, abi.F32, scalar_bits=0x3fc00000)))
    report("formal_elementwise ge f32 -> packed bool", 8 * n + n // 8, (lambda: pad.elementwise("ge", a_at, c_at, n, abi.F32, rhs=b_at)))
    report("formal_convert fp32_bf16 nearest-even", 6 * n, (lambda: pad.convert(167, a_at, c_at, n)))
    report("formal_convert fp32_int32 toward-zero (validate + store)", 12 * n, (lambda: pad.convert(165, a_at, c_at, n, rounding_mode=1)))
    shape = (n // (64 * 64 * 64), 64, 64, 64)
    count = int(np.prod(shape))
    report("formal_reduce max f32 over w", 4 * count + 4 * count // 64, (lambda: pad.reduce("max", a_at, c_at, "trailing1", shape, abi.F32)))
    report("formal_reduce sum f32 over w", 4 * count + 4 * count // 64, (lambda: pad.reduce("sum", a_at, c_at, "trailing1", shape, abi.F32)))
    out_shape = (shape[0], 32, 32, 64)
    report("formal_pool sum f32 2x2 stride 2", 4 * count + 4 * count // 4,
           (lambda: pad.pool("sum", a_at, c_at, shape, out_shape, (2, 2, 2, 2), abi.F32)))
    report("formal_pool max f32 2x2 stride 2", 4 * count + 4 * count // 4,
           (lambda: pad.pool("max", a_at, c_at, shape, out_shape, (2, 2, 2, 2), abi.F32)))
    # one bit-exact GEMM command of the shipped Tile programs: Cx operands in place, bf16 -> f32 with an f32 partial sum
    gm, gk, gn = 256, 256, 1024
    from ..backend import PhysicalTensorDescriptor as _Desc
    sizes = [backend.physical_bytes(_Desc(abi.BF16, abi.LAYOUT_CX, [gm, gk])), backend.physical_bytes(_Desc(abi.BF16, abi.LAYOUT_CX, [gk, gn])),
             backend.physical_bytes(_Desc(abi.F32, abi.LAYOUT_CX, [gm, gn]))]
    lhs_at, rhs_at = 0, (sizes[0] + 0xfff) & ~0xfff
    dst_at = rhs_at + ((sizes[1] + 0xfff) & ~0xfff)
    psum_at = dst_at + ((sizes[2] + 0xfff) & ~0xfff)
    report(f"formal GEMM command {gm}x{gk}x{gn} bf16 -> f32 + psum (FMAs as bytes: 2 flop each)", 2 * gm * gk * gn,
           (lambda: pad.gemm(lhs_at, rhs_at, dst_at, gm, gk, gn, in_format=abi.BF16, out_format=abi.F32, psum=psum_at, psum_format=abi.F32)))
    if "bf16 (vector rhs)" in args.only or not args.only:
        # bf16 operands: the top halves of the same pseudo-random f32 values, 2 n elements per operand over the a / b regions
        block16 = (block.view(np.uint32) >> 16).astype(np.uint16)
        for base in (a_at, b_at):
            for offset in range(0, 4 * n, block16.nbytes):
                pad.write(base + offset, block16[: min(block16.size, (4 * n - offset) // 2)])
        report("formal_elementwise add bf16 (vector rhs)", 6 * 2 * n, (lambda: pad.elementwise("add", a_at, c_at, 2 * n, abi.BF16, rhs=b_at)))
        report("formal_elementwise mul bf16 (vector rhs)", 6 * 2 * n, (lambda: pad.elementwise("mul", a_at, c_at, 2 * n, abi.BF16, rhs=b_at)))
    # seam-1 commands take host storage (the reference passes std::vector bytes): the kernel time comes from the
    # evidence's device_us, the call time is dominated by the two host <-> device copies
    from ..backend import NumericTensor, PhysicalTensorDescriptor
    m = min(n, 1 << 26)
    host_a = rng.standard_normal(m).astype(np.float32)
    host_b = rng.standard_normal(m).astype(np.float32)

    def boundary(name, bytes_per_call, call):
        if args.only not in name:
            return
        call()
        samples = sorted(call().evidence.device_us for _ in range(max(3, args.repeats // 2)))
        seconds = samples[len(samples) // 2] * 1e-6
        line = {"kernel": name, "elements": m, "bytes": bytes_per_call, "ms": round(seconds * 1e3, 3),
                "gbs": round(bytes_per_call / seconds / 1e9, 1), "peak_gbs": peak, "frac": round(bytes_per_call / seconds / 1e9 / peak, 3),
                "timing": "device_us of the evidence (CUDA events around the kernel)"}
        print(json.dumps(line), flush=True)

    vec = PhysicalTensorDescriptor(abi.F32, abi.LAYOUT_TENSOR, [m])
    half = PhysicalTensorDescriptor(abi.BF16, abi.LAYOUT_TENSOR, [m])
    tmpl32, tmpl16 = np.zeros(4 * m, np.uint8), np.zeros(2 * m, np.uint8)
    boundary("managed elementwise add f32 (wb200_elementwise)", 12 * m,
             lambda: backend.execute_elementwise("add", [NumericTensor(vec, host_a), NumericTensor(vec, host_b)], NumericTensor(vec, tmpl32)))
    boundary("managed elementwise exp f32 (wb200_elementwise)", 8 * m,
             lambda: backend.execute_elementwise("exp", [NumericTensor(vec, host_a)], NumericTensor(vec, tmpl32)))
    boundary("managed convert fp32_bf16 (wb200_convert)", 6 * m, lambda: backend.execute_convert(167, NumericTensor(vec, host_a), NumericTensor(half, tmpl16)))
    cx = PhysicalTensorDescriptor(abi.F32, abi.LAYOUT_NCX, [m // (64 * 64 * 64), 64, 64, 64])
    cx_out = PhysicalTensorDescriptor(abi.F32, abi.LAYOUT_NCX, [m // (64 * 64 * 64), 64, 1, 64])
    out_bytes = backend.physical_bytes(cx_out)
    boundary("managed reduce sum f32 over w, NCx (wb200_reduce)", 4 * m + out_bytes,
             lambda: backend.execute_reduce("sum", "trailing1", NumericTensor(cx, host_a), NumericTensor(cx_out, np.zeros(out_bytes, np.uint8))))
    boundary("formal elementwise add f32, host storage (wb200_elementwise_formal)", 12 * m,
             lambda: backend.execute_elementwise("add", [NumericTensor(vec, host_a), NumericTensor(vec, host_b)], NumericTensor(vec, tmpl32), formal=True))
    # the gate on device pointers
    lib = abi.load()
    x = torch.randn(n, device="cuda")
    y = x + 1e-4 * torch.randn(n, device="cuda")
    out = abi.Comparison()
    torch.cuda.synchronize()

    def gate():
        status = lib.wb200_compare(backend._handle, abi.F32, n, x.data_ptr(), y.data_ptr(), abi.MEM_DEVICE, 1e-3, 1e-3, 1, 0.9999, 0.01, C.byref(out))
        assert status == abi.OK

    report("compare gate f32 (statistics + 4 quantiles, 6 passes)", 6 * 8 * n, gate)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
