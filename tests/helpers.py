"""Shared helpers for the parity tests."""
import importlib.util
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
FMT_OF = {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}

_spec = importlib.util.spec_from_file_location("make_torch_fixtures", ROOT / "tests" / "golden" / "make_torch_fixtures.py")
fixtures = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(fixtures)


def golden():
    return np.load(ROOT / "tests" / "golden" / "torch_expected.npz")


def bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    return t.view(torch.int32).numpy().view(np.uint32) if t.dtype == torch.float32 else t.view(torch.int16).numpy().view(np.uint16)


def values(bits_array: np.ndarray, fmt: str) -> np.ndarray:
    """Raw bits -> float64 values."""
    if fmt == "f32":
        return bits_array.view(np.float32).astype(np.float64)
    if fmt == "f16":
        return bits_array.view(np.float16).astype(np.float64)
    return (bits_array.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def max_rel_err(actual: np.ndarray, expected: np.ndarray) -> float:
    """max |a - e| / max |e|: the bound north_star states for bf16 (1e-2) and f32 (1e-5) paths."""
    return float(np.abs(actual - expected).max() / max(np.abs(expected).max(), 1e-30))


def reference_gate(oracle, fmt, actual_bits, expected_bits, atol=0.008, rtol=0.006):
    """The reference's attention acceptance gate: cosine >= 0.9999 and relative L2 <= 0.01
    (test/Board/PyTorch/wafer_pytorch_board_common.py:60-73)."""
    stats = oracle.compare(fmt, actual_bits, expected_bits, atol, rtol)
    assert stats["finite"] == 1
    assert stats["cosine"] >= 0.9999 and stats["relative_l2"] <= 0.01, stats
    return stats
