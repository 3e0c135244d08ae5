"""The C-ABI library loads without a GPU, exports every symbol include/wb200.h declares, refuses to
run without a device, and its host-side layout arithmetic equals the oracle's. CPU only."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

from vibe_compiler_b200 import _abi as abi

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    header = (ROOT / "include" / "wb200.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return sorted(set(re.findall(r"\b(wb200_[a-z0-9_]+)\s*\(", header)))


def test_library_exports_every_declared_symbol():
    lib = abi.load()
    names = declared_symbols()
    assert len(names) >= 25
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/wb200.h but not exported"
        assert name in abi.SIGNATURES, f"{name} has no ctypes signature"
    assert lib.wb200_abi_version() == 4


def test_struct_layouts_match_the_header():
    # sizes follow from the header's field order under the C ABI
    assert C.sizeof(abi.TensorDesc) == 8 + 8 * abi.MAX_RANK
    assert C.sizeof(abi.Geometry) == 12 * 8
    assert C.sizeof(abi.Evidence) == 4 * 8 + 4 * 4 + 96 + 64
    assert C.sizeof(abi.AttentionParams) == 6 * 4 + 4 + 4 + 3 * 8 + 8 * 8 + 8
    assert C.sizeof(abi.GemmEpilogueParams) == 3 * 4 + 8 + 4 + 5 * 8


def test_backend_creation_fails_loudly_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the no-device path is exercised on CPU boxes")
    lib = abi.load()
    handle = C.c_void_p()
    assert lib.wb200_backend_create(0, C.byref(handle)) == abi.ERR_NO_DEVICE
    assert b"no CPU path" in lib.wb200_last_error()
    from vibe_compiler_b200.backend import B200TargetModelBackend, WB200Error
    with pytest.raises(WB200Error):
        B200TargetModelBackend(0)


SHAPES = [[1], [5], [64], [65], [96], [97], [129], [2, 3], [2, 65], [3, 1000], [3, 129], [2, 3, 1000], [2, 1, 2], [2, 2, 1],
          [1, 1, 3, 1031], [4, 7, 33], [2, 3, 5, 70], [1, 2, 3, 4, 200]]


@pytest.mark.parametrize("fmt", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("layout", ["tensor", "cx", "ncx"])
def test_host_geometry_equals_oracle(oracle, fmt, layout):
    from vibe_compiler_b200.backend import B200TargetModelBackend, PhysicalTensorDescriptor
    for shape in SHAPES:
        want = oracle.geometry(fmt, layout, shape)
        got = B200TargetModelBackend.geometry(PhysicalTensorDescriptor(oracle.FORMATS[fmt], oracle.LAYOUTS[layout], shape))
        assert got == want, (fmt, layout, shape)


def test_host_geometry_kats(kats, oracle):
    from vibe_compiler_b200.backend import B200TargetModelBackend, PhysicalTensorDescriptor
    for case in kats["geometry"]:
        got = B200TargetModelBackend.geometry(
            PhysicalTensorDescriptor(oracle.FORMATS[case["format"]], oracle.LAYOUTS[case["layout"]], case["shape"]))
        for key in ("compact_bytes", "physical_bytes", "c_block", "cx_blocks", "aligned_c", "c0", "outer_slice_stride_elements"):
            if key in case:
                assert got[key] == case[key], (case["source"], key)


def test_invalid_descriptors_are_rejected():
    lib = abi.load()
    out = C.c_uint64()
    bad = abi.make_desc(99, abi.LAYOUT_CX, [2, 3])
    assert lib.wb200_physical_bytes(C.byref(bad), C.byref(out)) == abi.ERR_INVALID_ARGUMENT
    bad = abi.make_desc(abi.F32, 7, [2, 3])
    assert lib.wb200_physical_bytes(C.byref(bad), C.byref(out)) == abi.ERR_INVALID_ARGUMENT
    bad = abi.make_desc(abi.F32, abi.LAYOUT_CX, [])
    assert lib.wb200_physical_bytes(C.byref(bad), C.byref(out)) == abi.ERR_INVALID_ARGUMENT
    assert lib.wb200_physical_bytes(None, C.byref(out)) == abi.ERR_INVALID_ARGUMENT


def test_microbenchmarks_import_and_parse_their_arguments():
    """The benchmarking tools that ship in the package import without a device and insist on their inputs."""
    import importlib
    for name in ("replay", "chain_replay", "command_kernels"):
        module = importlib.import_module(f"vibe_compiler_b200.microbench.{name}")
        assert callable(module.main)
    replay = importlib.import_module("vibe_compiler_b200.microbench.replay")
    with pytest.raises(SystemExit):
        replay.main([])            # --fixture is required: no default into the test tree
