"""Target-model acceptance gate: ProgramTensor `.npy` files in, the reference's comparison verdict and statistics out.

Host-side mirror of the reference's gate for one invocation (tools/wafer-compile/TargetModelGate.cpp:21-252): load the
`--model-input` / `--model-expected` tensors, run the Tile program, compare every output against its expected tensor
under the `--model-atol/--model-rtol[/--model-min-cosine/--model-max-relative-l2]` policy and print the reference's
one-line numeric statistics. The comparison itself runs on the device (`wb200_compare`, `wb200_compare_raw`).

    python -m vibe_compiler_b200.gate --target-model <dir with one .ll per Tile> \\
        --model-input 0=a.npy --model-input 1=b.npy --model-expected 0=out.npy \\
        --model-min-cosine 0.9999 --model-max-relative-l2 0.01 --model-report-numeric-statistics
"""
from __future__ import annotations

import argparse
import ast
import ctypes as C
import math
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import Optional, Sequence, Tuple

import numpy as np

from . import _abi as abi
from .backend import B200TargetModelBackend, WB200Error

# `descr` strings the reference admits (lib/Wafer/Frontend/NpyPayload.cpp:177-204) -> (element type, bytes).
_DESCR = {"<f4": ("f32", 4), "=f4": ("f32", 4), "<f8": ("f64", 8), "=f8": ("f64", 8), "<f2": ("f16", 2), "=f2": ("f16", 2),
          "|V2": ("bf16", 2), "|b1": ("bool", 1), "|i1": ("i8", 1), "<i2": ("i16", 2), "=i2": ("i16", 2),
          "<i4": ("i32", 4), "=i4": ("i32", 4), "<i8": ("i64", 8), "=i8": ("i64", 8)}
_CANONICAL_DESCR = {"f32": "<f4", "f64": "<f8", "f16": "<f2", "bf16": "|V2", "bool": "|b1", "i8": "|i1", "i16": "<i2",
                    "i32": "<i4", "i64": "<i8"}
_ELEMENT_BYTES = {name: size for name, size in _DESCR.values()}
_FLOATING = ("f16", "bf16", "f32", "f64")
_TOLERANT = {"f16": abi.F16, "bf16": abi.BF16, "f32": abi.F32}
_FORMAT_NAME = {abi.F16: "f16", abi.BF16: "bf16", abi.F32: "f32", abi.I8: "i8", abi.I16: "i16", abi.I32: "i32",
                abi.I64: "i64", abi.BOOL: "bool"}
_OUTCOME_CODE = {abi.CMP_INVALID_TOLERANCE: "invalid-tolerance", abi.CMP_ACTUAL_NONFINITE: "actual-nonfinite",
                 abi.CMP_EXPECTED_NONFINITE: "expected-nonfinite", abi.CMP_NUMERIC_MISMATCH: "numeric-mismatch",
                 abi.CMP_EMPTY: "unsupported-statistics-dtype", abi.CMP_RAW_MISMATCH: "raw-mismatch"}


@dataclass
class ProgramTensor:
    """Compact row-major little-endian tensor (include/Wafer/Simulator/Invocation/ProgramInvocation.h `ProgramTensor`)."""
    dtype: str
    shape: Tuple[int, ...]
    data: np.ndarray   # uint8, C-contiguous, exactly prod(shape) * element bytes

    def __post_init__(self):
        if self.dtype not in _ELEMENT_BYTES:
            raise ValueError(f"unknown program element type: {self.dtype}")
        self.shape = tuple(int(d) for d in self.shape)
        self.data = np.ascontiguousarray(self.data).view(np.uint8).reshape(-1)
        if any(d < 0 for d in self.shape) or self.data.size != math.prod(self.shape) * _ELEMENT_BYTES[self.dtype]:
            raise ValueError("program tensor byte size does not match its dtype and shape")

    @property
    def element_count(self) -> int:
        return math.prod(self.shape)


def load_npy(path) -> ProgramTensor:
    """ProgramTensor::loadNpy (lib/Wafer/Simulator/Invocation/ProgramInvocation.cpp:175-180) with the header rules of
    lib/Wafer/Frontend/NpyPayload.cpp:109-175, 383-432: format version 1 or 2, row-major only, the dtype set above."""
    path = str(path)
    raw = Path(path).read_bytes()
    if len(raw) < 10 or raw[:6] != b"\x93NUMPY":
        raise ValueError(f"npy payload is missing magic: {path}")
    major = raw[6]
    if major == 1:
        offset, length = 10, int.from_bytes(raw[8:10], "little")
    elif major == 2:
        if len(raw) < 12:
            raise ValueError(f"truncated npy v2 header: {path}")
        offset, length = 12, int.from_bytes(raw[8:12], "little")
    else:
        raise ValueError(f"unsupported npy payload version: {path}")
    if len(raw) < offset + length:
        raise ValueError(f"truncated npy payload header: {path}")
    try:
        header = ast.literal_eval(raw[offset:offset + length].decode("latin-1").strip())
        descr, fortran, shape = header["descr"], header["fortran_order"], header["shape"]
        if not isinstance(descr, str) or not isinstance(fortran, bool) or not isinstance(shape, tuple) or \
                not all(isinstance(d, int) and not isinstance(d, bool) and d >= 0 for d in shape):
            raise ValueError
    except Exception:
        raise ValueError(f"invalid npy payload header: {path}") from None
    if fortran:
        raise ValueError(f"npy payload must be row-major: {path}")
    if descr not in _DESCR or (descr[0] == "=" and sys.byteorder != "little"):
        raise ValueError(f"npy payload has unsupported dtype: {path}")
    dtype, width = _DESCR[descr]
    size = width * math.prod(shape)
    if size >= 1 << 64:
        raise ValueError(f"npy payload byte count is not representable: {path}")
    start = offset + length
    if size > len(raw) - start:
        raise ValueError(f"npy tensor payload is truncated: {path}")
    return ProgramTensor(dtype, shape, np.frombuffer(raw, dtype=np.uint8, count=size, offset=start).copy())


def save_npy(path, tensor: ProgramTensor) -> None:
    """Writes a version-1 `.npy` file load_npy() and the reference's loader both accept (bf16 as `|V2`)."""
    shape = "(" + ", ".join(str(d) for d in tensor.shape) + ("," if len(tensor.shape) == 1 else "") + ")"
    header = f"{{'descr': '{_CANONICAL_DESCR[tensor.dtype]}', 'fortran_order': False, 'shape': {shape}, }}"
    header += " " * ((-(10 + len(header) + 1)) % 64) + "\n"
    with open(path, "wb") as handle:
        handle.write(b"\x93NUMPY\x01\x00" + len(header).to_bytes(2, "little") + header.encode("latin-1"))
        handle.write(tensor.data.tobytes())


@dataclass
class ComparisonPolicy:
    """ProgramTensorComparisonPolicy (include/Wafer/Simulator/Invocation/ProgramTensorComparison.h:38-44): without
    `similarity` the comparison is elementwise; with it atol / rtol only feed the diagnostics."""
    atol: float = 0.0
    rtol: float = 0.0
    similarity: Optional[Tuple[float, float]] = None   # (minimum cosine, maximum relative L2)


class ProgramTensorComparisonError(Exception):
    """`code` is one of the reference's error-code strings (ProgramTensorComparison.cpp:236-262)."""

    def __init__(self, code: str, detail: str):
        super().__init__(f"program tensor comparison {code}: {detail}")
        self.code, self.detail = code, detail


@dataclass
class ComparisonStatistics:
    element_count: int
    exact_count: int
    exact_fraction: float
    mean_abs: float
    p99_abs: float
    p999_abs: float
    max_abs: float
    mismatch_count: int
    cosine: float
    relative_l2: float
    mean_ulp: float
    p99_ulp: int
    p999_ulp: int
    max_ulp: int


def _format_shape(shape) -> str:
    return "[" + ",".join(str(d) for d in shape) + "]"


def _check_pair(actual: ProgramTensor, expected: ProgramTensor) -> None:
    if actual.dtype != expected.dtype:
        raise ProgramTensorComparisonError("dtype-mismatch", f"actual={actual.dtype} expected={expected.dtype}")
    if actual.shape != expected.shape:
        raise ProgramTensorComparisonError("shape-mismatch", f"actual={_format_shape(actual.shape)} expected={_format_shape(expected.shape)}")
    if actual.data.size != expected.data.size:
        raise ProgramTensorComparisonError("byte-size-mismatch", f"actual={actual.data.size} expected={expected.data.size}")


def _device_compare(backend: B200TargetModelBackend, actual: ProgramTensor, expected: ProgramTensor,
                    policy: ComparisonPolicy) -> abi.Comparison:
    lib = abi.load()
    out = abi.Comparison()
    similarity = policy.similarity is not None
    minimum_cosine, maximum_l2 = policy.similarity if similarity else (0.0, 0.0)
    status = lib.wb200_compare(backend._handle, _TOLERANT[actual.dtype], actual.element_count, actual.data.ctypes.data,
                               expected.data.ctypes.data, abi.MEM_HOST, policy.atol, policy.rtol, int(similarity),
                               minimum_cosine, maximum_l2, C.byref(out))
    if status != abi.OK:
        raise WB200Error(status, lib.wb200_last_error().decode())
    return out


def compare_expected_output(backend: B200TargetModelBackend, actual: ProgramTensor, expected: ProgramTensor,
                            policy: ComparisonPolicy = ComparisonPolicy()) -> None:
    """compareProgramTensorExpectedOutput (ProgramTensorComparison.cpp:276-403): returns on a match, raises
    ProgramTensorComparisonError otherwise. Non-floating tensors are compared byte for byte."""
    _check_policy(policy)
    _check_pair(actual, expected)
    if actual.dtype in _FLOATING and actual.dtype not in _TOLERANT:
        raise ProgramTensorComparisonError("unsupported-floating-dtype", f"dtype={actual.dtype} has no expected-output policy")
    if actual.dtype not in _TOLERANT:
        lib = abi.load()
        out = abi.Comparison()
        status = lib.wb200_compare_raw(backend._handle, actual.data.size, actual.data.ctypes.data, expected.data.ctypes.data,
                                       abi.MEM_HOST, C.byref(out))
        if status != abi.OK:
            raise WB200Error(status, lib.wb200_last_error().decode())
    else:
        out = _device_compare(backend, actual, expected, policy)
    if out.outcome != abi.CMP_MATCH:
        raise ProgramTensorComparisonError(_OUTCOME_CODE[out.outcome], out.detail.decode())


def compute_statistics(backend: B200TargetModelBackend, actual: ProgramTensor, expected: ProgramTensor,
                       policy: ComparisonPolicy = ComparisonPolicy()) -> ComparisonStatistics:
    """computeProgramTensorComparisonStatistics (ProgramTensorComparison.cpp:405-503)."""
    _check_policy(policy)
    _check_pair(actual, expected)
    if actual.dtype not in _TOLERANT:
        raise ProgramTensorComparisonError("unsupported-statistics-dtype", f"dtype={actual.dtype} has no source/model numeric statistics policy")
    if actual.element_count == 0:
        raise ProgramTensorComparisonError("unsupported-statistics-dtype", "numeric statistics require a non-empty tensor")
    out = _device_compare(backend, actual, expected, ComparisonPolicy(policy.atol, policy.rtol, None))
    if out.outcome in (abi.CMP_INVALID_TOLERANCE, abi.CMP_ACTUAL_NONFINITE, abi.CMP_EXPECTED_NONFINITE):
        raise ProgramTensorComparisonError(_OUTCOME_CODE[out.outcome], out.detail.decode())
    return ComparisonStatistics(out.element_count, out.exact_count, out.exact_fraction, out.mean_abs, out.p99_abs, out.p999_abs,
                                out.max_abs, out.mismatch_count, out.cosine, out.relative_l2, out.mean_ulp, out.p99_ulp,
                                out.p999_ulp, out.max_ulp)


def _check_policy(policy: ComparisonPolicy) -> None:
    """validateProgramTensorComparisonPolicy (ProgramTensorComparison.cpp:505-524)."""
    if not (math.isfinite(policy.atol) and math.isfinite(policy.rtol)) or policy.atol < 0 or policy.rtol < 0:
        raise ProgramTensorComparisonError("invalid-tolerance", "absolute and relative tolerances must be finite and nonnegative")
    if policy.similarity is not None:
        cosine, l2 = policy.similarity
        if not math.isfinite(cosine) or cosine < 0 or cosine > 1 or not math.isfinite(l2) or l2 < 0:
            raise ProgramTensorComparisonError("invalid-tolerance", "similarity requires finite minimum cosine in [0,1] and nonnegative relative L2")


def _e(value: float) -> str:
    """The reference streams these doubles through raw_ostream, which prints "%e" (and spells out nan / INF)."""
    if math.isnan(value):
        return "nan"
    if math.isinf(value):
        return "-INF" if value < 0 else "INF"
    return "%e" % value


def format_statistics(index: int, launch_slot: int, dtype: str, s: ComparisonStatistics, policy: ComparisonPolicy) -> str:
    """The one-line report of tools/wafer-compile/TargetModelGate.cpp:175-204, field for field."""
    g = lambda v: "%.17g" % v
    line = (f"target model numeric statistics index={index} launch_slot={launch_slot} dtype={dtype} elements={s.element_count}"
            f" exact={s.exact_count} exact_fraction={g(s.exact_fraction)} mean_abs={g(s.mean_abs)} p99_abs={g(s.p99_abs)}"
            f" p999_abs={g(s.p999_abs)} max_abs={g(s.max_abs)} mean_ulp={g(s.mean_ulp)} p99_ulp={s.p99_ulp}"
            f" p999_ulp={s.p999_ulp} max_ulp={s.max_ulp} elementwise_mismatches={s.mismatch_count}"
            f" atol={_e(policy.atol)} rtol={_e(policy.rtol)} cosine={g(s.cosine)} relative_l2={g(s.relative_l2)}"
            f" comparison={'similarity' if policy.similarity is not None else 'elementwise'}")
    if policy.similarity is not None:
        line += f" minimum_cosine={_e(policy.similarity[0])} maximum_relative_l2={_e(policy.similarity[1])}"
    return line


def _indexed_paths(values: Sequence[str], option: str):
    """`<index>=<path>` lists with the checks of tools/wafer-compile/DriverOptions.cpp:538-560."""
    parsed = {}
    for value in values:
        index_text, _, path = value.partition("=")
        if not path or not index_text.isdigit():
            raise SystemExit(f"wb200-gate: invalid {option} value: {value}")
        if int(index_text) in parsed:
            raise SystemExit(f"wb200-gate: duplicate {option} index: {int(index_text)}")
        parsed[int(index_text)] = path
    return parsed


def run_gate(modules: Sequence[str], inputs: dict, expected: dict, policy: ComparisonPolicy, report_statistics: bool = False,
             gemm_policy: int = abi.GEMM_FORMAL, backend: Optional[B200TargetModelBackend] = None, out=None) -> bool:
    """Runs one invocation and gates every output. Returns True when all outputs matched (the reference's
    runTargetModelGate returns false for success; this returns the plain meaning)."""
    from .tile_program import TileProgram
    out = out or sys.stdout
    backend = backend or B200TargetModelBackend()
    program = TileProgram(modules, backend)
    arrays = []
    for index, info in enumerate(program.inputs):
        if index not in inputs:
            print(f"wb200-gate: missing target model input {index}", file=sys.stderr)
            return False
        tensor = inputs[index]
        if tensor.dtype != _FORMAT_NAME.get(info.format) or tensor.data.size != info.compact_bytes:
            print(f"wb200-gate: target model input {index} does not have the program's dtype and size", file=sys.stderr)
            return False
        arrays.append(tensor.data)
    outputs, stats = program.run(arrays, gemm_policy)
    for index, (bits, info) in enumerate(zip(outputs, program.outputs)):
        if index not in expected:
            print(f"wb200-gate: missing target model expected output {index}", file=sys.stderr)
            return False
        actual = ProgramTensor(_FORMAT_NAME[info.format], info.shape, bits)
        want = expected[index]
        try:
            if report_statistics or (policy.similarity is not None and actual.dtype in _TOLERANT):
                statistics = compute_statistics(backend, actual, want, policy)
                print("wb200-gate: " + format_statistics(index, 0, actual.dtype, statistics, policy), file=out)
            compare_expected_output(backend, actual, want, policy)
        except ProgramTensorComparisonError as error:
            print(f"wb200-gate: target model output differs at index {index}: {error}", file=sys.stderr)
            return False
    print(f"wb200-gate: target model outputs matched; tiles={len(modules)} commands={stats['commands']}"
          f" gemm_commands={stats['gemm_commands']} movement_commands={stats['movement_commands']}"
          f" gpu_launches={stats['gpu_launches']} device_ms={stats['device_ms']:.3f}", file=out)
    return True


def main(argv: Optional[Sequence[str]] = None) -> int:
    parser = argparse.ArgumentParser(prog="python -m vibe_compiler_b200.gate", description=__doc__.split("\n\n")[0])
    parser.add_argument("--target-model", required=True, metavar="DIR", help="directory holding one target LLVM module (*.ll) per Tile")
    parser.add_argument("--model-input", action="append", default=[], metavar="INDEX=NPY")
    parser.add_argument("--model-expected", action="append", default=[], metavar="INDEX=NPY")
    parser.add_argument("--model-atol", type=float, default=0.0)
    parser.add_argument("--model-rtol", type=float, default=0.0)
    parser.add_argument("--model-min-cosine", type=float)
    parser.add_argument("--model-max-relative-l2", type=float)
    parser.add_argument("--model-report-numeric-statistics", action="store_true")
    parser.add_argument("--gemm-policy", choices=("formal", "tensor"), default="formal")
    args = parser.parse_args(argv)
    if not args.model_input or not args.model_expected:
        print("wb200-gate: target model execution requires both --model-input and --model-expected", file=sys.stderr)
        return 1
    if (args.model_min_cosine is None) != (args.model_max_relative_l2 is None):
        print("wb200-gate: --model-min-cosine and --model-max-relative-l2 must be supplied together", file=sys.stderr)
        return 1
    if args.model_min_cosine is not None and args.model_min_cosine > 1.0:
        print("wb200-gate: --model-min-cosine must be in [0,1]", file=sys.stderr)
        return 1
    similarity = None if args.model_min_cosine is None else (args.model_min_cosine, args.model_max_relative_l2)
    policy = ComparisonPolicy(args.model_atol, args.model_rtol, similarity)
    try:
        _check_policy(policy)
        inputs = {i: load_npy(p) for i, p in _indexed_paths(args.model_input, "--model-input").items()}
        expected = {i: load_npy(p) for i, p in _indexed_paths(args.model_expected, "--model-expected").items()}
    except (ValueError, OSError, ProgramTensorComparisonError) as error:
        print(f"wb200-gate: {error}", file=sys.stderr)
        return 1
    modules = [p.read_text() for p in sorted(Path(args.target_model).glob("*.ll"))]
    if not modules:
        print(f"wb200-gate: no target LLVM modules (*.ll) under {args.target_model}", file=sys.stderr)
        return 1
    try:
        matched = run_gate(modules, inputs, expected, policy, args.model_report_numeric_statistics,
                           abi.GEMM_TENSOR if args.gemm_policy == "tensor" else abi.GEMM_FORMAL)
    except WB200Error as error:
        print(f"wb200-gate: {error}", file=sys.stderr)
        return 1
    return 0 if matched else 1


if __name__ == "__main__":
    raise SystemExit(main())
