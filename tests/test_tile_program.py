"""Replay of the reference compiler's shipped per-Tile target LLVM modules (GEMM optimisation ladder: seven plans x
16 Tiles of out[4096,4096] = arg1[4096,1024] . arg0[1024,4096], bf16).

CPU: the parser / interpreter / scheduler (device-free trace), the IR subset and its error reports, the CPU trace
replay on a tiny hand-written program. GPU: all seven plans bit for bit against the committed CPU-replay hashes, one
plan against the live CPU replay, every plan under the reference's similarity gate against the f32 matrix product."""
import hashlib
import importlib.util
import json
import lzma
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import helpers
from vibe_compiler_b200 import _abi as abi
from vibe_compiler_b200.backend import WB200Error
from vibe_compiler_b200.tile_program import TileProgram

ROOT = Path(__file__).resolve().parent.parent
FIXTURE = json.loads(lzma.decompress((ROOT / "tests" / "golden" / "gemm_tile_modules.json.xz").read_bytes()))
EXPECTED = json.loads((ROOT / "tests" / "golden" / "gemm_tile_program_expected.json").read_text())
_spec = importlib.util.spec_from_file_location("make_tile_program_expected", ROOT / "tests" / "golden" / "make_tile_program_expected.py")
expected_tools = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(expected_tools)

PLANS = sorted(FIXTURE["plans"])


def _module(body: str, arguments: str = "i64 %0, i64 %1", rows=None, tile: int = 0) -> str:
    rows = rows or ['!{i64 0, !"external-input", i64 0, !"", !"f32", !"tensor", i64 1024, i64 256, !"read-only", i64 16, i64 16, i64 0}',
                    '!{i64 1, !"external-output", i64 0, !"", !"f32", !"tensor", i64 1024, i64 256, !"write-only", i64 16, i64 16, i64 0}']
    names = ", ".join(f"!{10 + i}" for i in range(len(rows)))
    meta = "\n".join(f"!{10 + i} = {row}" for i, row in enumerate(rows))
    return (f"define void @entry({arguments}) {{\n{body}\n}}\n!wafer.target.tile_id = !{{!2}}\n!wafer.target.entry_arguments = !{{{names}}}\n"
            f"!2 = !{{i64 {tile}}}\n{meta}\n")


# A 16x16 f32 matrix is read row-reversed, transposed in the scratch-pad and written back.
REVERSE_ROWS = _module("""
  br label %3
3:
  %4 = phi i64 [ 0, %2 ], [ %9, %6 ]
  %5 = icmp ult i64 %4, 16
  br i1 %5, label %6, label %10
6:
  %7 = sub i64 15, %4
  %8 = mul i64 %7, 64
  %src = add i64 %0, %8
  %dstoff = shl i64 %4, 6
  %dst = add i64 4096, %dstoff
  call void @wafer_tx81_rdma(i64 %src, i64 %dst, i32 64, i32 64, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  %9 = add nuw i64 %4, 1
  br label %3
10:
  call void @wafer_tx81_gather_scatter(i64 4096, i64 8192, i32 1024, i32 4, i32 4, i32 64, i32 0, i32 16, i32 16, i32 1, i32 64, i32 4, i32 0, i32 16, i32 16, i32 1, i32 0)
  call void @wafer_tx81_ncc_join(i32 1)
  call void @wafer_tx81_wdma(i64 8192, i64 %1, i32 1024, i32 1024, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  ret void
""")


def test_every_shipped_plan_parses_schedules_and_covers_the_product():
    for plan in PLANS:
        program = TileProgram(FIXTURE["plans"][plan])
        assert [t.shape for t in program.inputs] == [(1, 1024, 4096), (1, 4096, 1024)]
        assert [t.shape for t in program.outputs] == [(1, 4096, 4096)]
        commands, stats = program.trace()
        assert stats["gemm_fused_multiply_adds"] == 4096 * 4096 * 1024       # every (m, n, k) triple exactly once
        assert stats["commands"] == sum(1 for c in commands if c.name != "direct_dte_transfer")
        sends = sum(1 for c in commands if c.name == "wafer_tx81_direct_dte_send_issue")
        assert stats["transfer_commands"] == sends == sum(1 for c in commands if c.name == "direct_dte_transfer")
        out_bytes = sum(c.args[2] for c in commands if c.name == "wafer_tx81_wdma")
        assert out_bytes == 4096 * 4096 * 2                                   # the output is written exactly once


def test_interpreter_runs_a_small_program_and_the_cpu_replay_executes_its_trace():
    from oracle import binding, trace_replay
    binding.build()
    program = TileProgram([REVERSE_ROWS])
    commands, stats = program.trace()
    assert [c.name for c in commands].count("wafer_tx81_rdma") == 16 and stats["movement_commands"] == 18
    place_in, place_out = program.placement(False, 0), program.placement(True, 0)
    ddr = np.zeros(place_in["ddr_bytes"], dtype=np.uint8)
    matrix = np.arange(256, dtype=np.float32).reshape(16, 16)
    at = place_in["address"] - place_in["ddr_base"]
    ddr[at:at + 1024] = matrix.view(np.uint8).reshape(-1)
    trace_replay.replay(commands, ddr, 1, spm_bytes=1 << 16)
    at = place_out["address"] - place_out["ddr_base"]
    got = ddr[at:at + 1024].view(np.float32).reshape(16, 16)
    assert np.array_equal(got, matrix[::-1].T)


# 256 f32 values: y = relu(x + 0.5) * unit[i % 4]; mask = (y >= 1) as numbers; out = bf16(y * mask) rounded toward +inf.
NUMERIC = _module("""
  call void @wafer_tx81_rdma(i64 %0, i64 0, i32 1024, i32 1024, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  call void @wafer_tx81_rdma(i64 %1, i64 4096, i32 16, i32 16, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  call void @wafer_tx81_ncc_join(i32 1)
  call void @wafer_tx81_elementwise_add(i64 0, i64 1056964608, i64 8192, i32 256, i32 5, i32 0, i32 1, i32 0, i32 1)
  call void @wafer_tx81_elementwise_relu(i64 8192, i64 8192, i32 256, i32 5, i32 1)
  call void @wafer_tx81_elementwise_mul(i64 8192, i64 4096, i64 12288, i32 256, i32 5, i32 4, i32 0, i32 0, i32 1)
  call void @wafer_tx81_elementwise_ge(i64 12288, i64 1065353216, i64 16384, i32 256, i32 5, i32 0, i32 1, i32 1, i32 1)
  call void @wafer_tx81_elementwise_ge(i64 12288, i64 1065353216, i64 24576, i32 256, i32 5, i32 0, i32 1, i32 0, i32 1)
  call void @wafer_tx81_elementwise_logic_not(i64 24576, i64 24640, i32 256, i32 7, i32 1)
  call void @wafer_tx81_elementwise_logic_or(i64 24576, i64 24640, i64 24704, i32 256, i32 7, i32 1)
  call void @wafer_tx81_elementwise_mul(i64 12288, i64 16384, i64 12288, i32 256, i32 5, i32 0, i32 0, i32 0, i32 1)
  call void @wafer_tx81_convert_fp32_bf16(i64 12288, i64 20480, i32 256, i32 0, i32 2, i32 1)
  call void @wafer_tx81_reduce_max(i64 8192, i64 28672, i32 4, i32 1, i32 2, i32 2, i32 64, i32 5, i32 1)
  call void @wafer_tx81_elementwise_add(i64 28672, i64 28672, i64 28672, i32 64, i32 5, i32 0, i32 0, i32 0, i32 1)
  call void @wafer_tx81_convert_fp32_bf16(i64 28672, i64 20480, i32 64, i32 0, i32 0, i32 1)
  call void @wafer_tx81_wdma(i64 20480, i64 %2, i32 512, i32 512, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 3, i32 0)
  call void @wafer_tx81_wdma(i64 24704, i64 %3, i32 32, i32 32, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 8, i32 0)
  ret void
""", arguments="i64 %0, i64 %1, i64 %2, i64 %3", rows=[
    '!{i64 0, !"external-input", i64 0, !"", !"f32", !"tensor", i64 1024, i64 256, !"read-only", i64 16, i64 16, i64 0}',
    '!{i64 1, !"external-input", i64 1, !"", !"f32", !"tensor", i64 16, i64 4, !"read-only", i64 4, i64 0}',
    '!{i64 2, !"external-output", i64 0, !"", !"bf16", !"tensor", i64 512, i64 256, !"write-only", i64 16, i64 16, i64 0}',
    '!{i64 3, !"external-output", i64 1, !"", !"u8", !"tensor", i64 32, i64 32, !"write-only", i64 32, i64 0}'])


def _numeric_inputs():
    rng = np.random.default_rng(20260803)
    x = rng.standard_normal(256).astype(np.float32) * 2
    x[:4] = [np.float32(3.0e38), -0.5, np.float32(1e-40), 2.0]
    return x.reshape(16, 16), np.array([1.0, -2.0, 0.333251953125, 3.0e38], dtype=np.float32)


def _numeric_cpu_replay(program):
    from oracle import binding, trace_replay
    binding.build()
    commands, _ = program.trace()
    x, unit = _numeric_inputs()
    places = [program.placement(False, 0), program.placement(False, 1), program.placement(True, 0), program.placement(True, 1)]
    ddr = np.zeros(places[0]["ddr_bytes"], dtype=np.uint8)
    for place, array in zip(places, (x, unit)):
        at = place["address"] - place["ddr_base"]
        ddr[at:at + array.nbytes] = array.view(np.uint8).reshape(-1)
    report = {}
    trace_replay.replay(commands, ddr, 1, spm_bytes=1 << 16, report=report)
    at, mask_at = places[2]["address"] - places[2]["ddr_base"], places[3]["address"] - places[3]["ddr_base"]
    return commands, ddr[at:at + 512].view(np.uint16).copy(), ddr[mask_at:mask_at + 32].copy(), report["numeric_flags"]


def test_elementwise_and_convert_calls_are_traced_and_replayed_on_the_cpu():
    program = TileProgram([NUMERIC], spm_bytes=1 << 16)
    commands, out, mask, flags = _numeric_cpu_replay(program)
    names = [(c.name, c.operation) for c in commands if "elementwise" in c.name or "convert" in c.name or "reduce" in c.name]
    assert names == [("wafer_tx81_elementwise_binary", 8), ("wafer_tx81_elementwise_unary", 31), ("wafer_tx81_elementwise_binary", 10),
                     ("wafer_tx81_elementwise_binary", 14), ("wafer_tx81_elementwise_binary", 14), ("wafer_tx81_elementwise_unary", 18),
                     ("wafer_tx81_elementwise_logic", 20), ("wafer_tx81_elementwise_binary", 10), ("wafer_tx81_convert", 167),
                     ("wafer_tx81_reduce", 1), ("wafer_tx81_elementwise_binary", 8), ("wafer_tx81_convert", 167)]
    x, unit = _numeric_inputs()
    y = np.maximum(x.reshape(-1) + np.float32(0.5), 0) * np.tile(unit, 64)
    want = np.where(y >= 1, y, np.float32(0)).astype(np.float32)
    assert np.all(mask == 0xff)                                     # (y >= 1) or not (y >= 1)
    got = (out.astype(np.uint32) << 16).view(np.float32)
    tail, want_tail = got[64:], want[64:]
    finite = np.isfinite(want_tail)
    assert np.all(tail[finite] >= want_tail[finite]) and np.all(tail[finite] <= want_tail[finite] * np.float32(1.0079) + 1e-30)   # rounded up
    assert flags & 4 and flags & 16                                 # 2.5 * 3e38 overflows; most results are inexact
    relu = np.maximum(x.reshape(-1) + np.float32(0.5), 0).reshape(4, 64)
    doubled = (relu.max(axis=0) * np.float32(2)).astype(np.float32)
    import torch
    assert np.array_equal(got[:64], torch.from_numpy(doubled).to(torch.bfloat16).float().numpy())
    for body, fragment in (("call void @wafer_tx81_elementwise_frobnicate(i64 0, i64 0, i32 4, i32 5, i32 1)\n ret void", "outside the executed command set"),
                           ("call void @wafer_tx81_elementwise_add(i64 0, i64 0, i32 4, i32 5, i32 1)\n ret void", "does not match its descriptor"),
                           ("call void @wafer_tx81_convert_fp32_fp64(i64 0, i64 0, i32 4, i32 0, i32 0, i32 1)\n ret void", "outside the executed command set")):
        with pytest.raises(WB200Error, match=fragment):
            TileProgram([_module(body)])
    with pytest.raises(WB200Error, match="outside the memory image"):
        TileProgram([_module("call void @wafer_tx81_elementwise_abs(i64 0, i64 65536, i32 4096, i32 5, i32 1)\n ret void")], spm_bytes=1 << 16).trace()


# x where x >= 1, else 7: relation to packed Bool, Bool to numbers, fill, masked move.
SELECT = _module("""
  call void @wafer_tx81_rdma(i64 %0, i64 0, i32 1024, i32 1024, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  call void @wafer_tx81_elementwise_ge(i64 0, i64 1065353216, i64 4096, i32 256, i32 5, i32 0, i32 1, i32 0, i32 1)
  call void @wafer_tx81_bit2fp(i64 4096, i64 8192, i32 256, i32 5, i32 1)
  call void @wafer_tx81_memset(i64 12288, i32 1088421888, i32 256, i32 5, i32 0)
  call void @wafer_tx81_mask_move(i64 0, i32 8192, i64 12288, i32 256, i32 5, i32 1)
  call void @wafer_tx81_wdma(i64 12288, i64 %1, i32 1024, i32 1024, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  ret void
""")


def test_bit2fp_and_mask_move_are_traced_and_replayed_on_the_cpu():
    from oracle import binding, trace_replay
    binding.build()
    program = TileProgram([SELECT], spm_bytes=1 << 16)
    commands, stats = program.trace()
    assert [c.name for c in commands if "bit2fp" in c.name or "mask_move" in c.name] == ["wafer_tx81_bit2fp", "wafer_tx81_mask_move"]
    place_in, place_out = program.placement(False, 0), program.placement(True, 0)
    ddr = np.zeros(place_in["ddr_bytes"], dtype=np.uint8)
    x = np.linspace(-3, 3, 256, dtype=np.float32)
    at = place_in["address"] - place_in["ddr_base"]
    ddr[at:at + 1024] = x.view(np.uint8)
    trace_replay.replay(commands, ddr, 1, spm_bytes=1 << 16)
    at = place_out["address"] - place_out["ddr_base"]
    assert np.array_equal(ddr[at:at + 1024].view(np.float32), np.where(x >= 1, x, np.float32(7)))


# bf16, 509 elements: seven elementwise commands, each taking the previous destination as its first operand (vector and
# immediate second operands, an in-place step, a second operand and a destination that revisit an earlier destination),
# then a command of another length. The interpreter issues the seven as one fused launch.
CHAIN = _module("""
  call void @wafer_tx81_rdma(i64 %0, i64 0, i32 1024, i32 1024, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 3, i32 0)
  call void @wafer_tx81_rdma(i64 %1, i64 2048, i32 1024, i32 1024, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 3, i32 0)
  call void @wafer_tx81_memset(i64 4096, i32 0, i32 3072, i32 5, i32 0)
  call void @wafer_tx81_elementwise_add(i64 0, i64 2048, i64 4096, i32 509, i32 3, i32 0, i32 0, i32 0, i32 1)
  call void @wafer_tx81_elementwise_mul(i64 4096, i64 16128, i64 6144, i32 509, i32 3, i32 0, i32 1, i32 0, i32 1)
  call void @wafer_tx81_elementwise_exp(i64 6144, i64 6144, i32 509, i32 3, i32 1)
  call void @wafer_tx81_elementwise_sub(i64 6144, i64 4096, i64 8192, i32 509, i32 3, i32 0, i32 0, i32 0, i32 1)
  call void @wafer_tx81_elementwise_relu(i64 8192, i64 10240, i32 509, i32 3, i32 1)
  call void @wafer_tx81_elementwise_max(i64 10240, i64 2048, i64 4096, i32 509, i32 3, i32 0, i32 0, i32 0, i32 1)
  call void @wafer_tx81_elementwise_sigmoid(i64 4096, i64 12288, i32 509, i32 3, i32 1)
  call void @wafer_tx81_elementwise_neg(i64 12288, i64 14336, i32 256, i32 3, i32 1)
  call void @wafer_tx81_wdma(i64 4096, i64 %2, i32 12288, i32 12288, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 8, i32 0)
  ret void
""", arguments="i64 %0, i64 %1, i64 %2", rows=[
    '!{i64 0, !"external-input", i64 0, !"", !"bf16", !"tensor", i64 1024, i64 512, !"read-only", i64 512, i64 0}',
    '!{i64 1, !"external-input", i64 1, !"", !"bf16", !"tensor", i64 1024, i64 512, !"read-only", i64 512, i64 0}',
    '!{i64 2, !"external-output", i64 0, !"", !"u8", !"tensor", i64 12288, i64 12288, !"write-only", i64 12288, i64 0}'])


# Online attention over two blocks of 64 keys for 64 queries, head dimension 64, all f32, one Tile: the command run the
# reference's decomposition of an online-attention step lowers to (lib/Wafer/Transforms/Linalg/OnlineAttentionDecomposition.cpp:
# 568-594: scores, score region, new maximum, norm, rescaled sum, probabilities, new sum, rescaled accumulator, PV with the
# accumulator as partial sum) in the transposed form (keys x queries: the queries are the 64 channels, so the per-query
# vectors broadcast with the repeated-unit form and the reductions run over w of NCx [1, 1, keys, queries]). exp is the
# formal (correctly rounded) exp: the reference's ExpLp has no formal evaluation (FormalNumericElementwise.cpp:216-224).
# Scratch-pad: Q 0x0000, K 0x4000, V 0x8000, S^T 0xC000, P^T 0x10000, vectors from 0x14000 (m_old, m_tile, m_new, diff,
# norm, l, l_scaled, p_sum, 1/l), acc^T 0x18000, scaled acc^T 0x1C000 (16 KiB matrices, 256-byte vectors).
# The module is a file of its own (tests/golden/attention_step_tile.ll) so that the replay microbenchmark can time it.
ATTENTION = (ROOT / "tests" / "golden" / "attention_step_tile.ll").read_text()


def _attention_inputs():
    rng = np.random.default_rng(20260803)
    q, k, v = (rng.standard_normal(shape).astype(np.float32) for shape in ((64, 64), (128, 64), (128, 64)))
    return q, k, v


def _attention_cpu_replay(program):
    from oracle import binding, trace_replay
    binding.build()
    commands, stats = program.trace()
    ddr = np.zeros(program.placement(False, 0)["ddr_bytes"], dtype=np.uint8)
    for index, array in enumerate(_attention_inputs()):
        place = program.placement(False, index)
        at = place["address"] - place["ddr_base"]
        ddr[at:at + array.nbytes] = array.view(np.uint8).reshape(-1)
    report = {}
    trace_replay.replay(commands, ddr, 1, spm_bytes=1 << 17, report=report)
    outs = []
    for index, nbytes in enumerate((16384, 256, 256)):
        place = program.placement(True, index)
        at = place["address"] - place["ddr_base"]
        outs.append(ddr[at:at + nbytes].copy().view(np.float32))
    return outs, report["numeric_flags"], stats


def test_attention_step_program_is_replayed_on_the_cpu():
    (out_t, m, l), _, stats = _attention_cpu_replay(TileProgram([ATTENTION], spm_bytes=1 << 17))
    assert stats["commands"] == 41 and stats["gemm_commands"] == 4
    q, k, v = (a.astype(np.float64) for a in _attention_inputs())
    scores = q @ k.T * 0.125
    p = np.exp(scores - scores.max(-1, keepdims=True))
    want = (p / p.sum(-1, keepdims=True)) @ v                           # [queries, D]
    assert np.abs(out_t.reshape(64, 64).T - want).max() <= 1e-5           # the program keeps the accumulator transposed
    assert np.allclose(m, scores.max(-1), rtol=1e-6) and np.allclose(l, p.sum(-1), rtol=1e-5)


def _chain_inputs():
    rng = np.random.default_rng(77)
    x = (rng.standard_normal(512).astype(np.float32) * 3).view(np.uint32) >> 16
    y = (rng.standard_normal(512).astype(np.float32) * 3).view(np.uint32) >> 16
    x[:6] = [0x7f80, 0xff80, 0x7fc1, 0x0001, 0x8000, 0x42c8]   # +inf, -inf, a NaN payload, a subnormal, -0, 100
    y[:6] = [0xff80, 0x3f80, 0x3f80, 0x0001, 0x0000, 0x42c8]
    return x.astype(np.uint16), y.astype(np.uint16)


def _chain_cpu_replay(program):
    from oracle import binding, trace_replay
    binding.build()
    commands, _ = program.trace()
    places = [program.placement(False, 0), program.placement(False, 1), program.placement(True, 0)]
    ddr = np.zeros(places[0]["ddr_bytes"], dtype=np.uint8)
    for place, array in zip(places, _chain_inputs()):
        at = place["address"] - place["ddr_base"]
        ddr[at:at + array.nbytes] = array.view(np.uint8)
    report = {}
    trace_replay.replay(commands, ddr, 1, spm_bytes=1 << 16, report=report)
    at = places[2]["address"] - places[2]["ddr_base"]
    return ddr[at:at + 12288].copy(), report["numeric_flags"]


def test_chain_program_is_replayed_on_the_cpu():
    out, flags = _chain_cpu_replay(TileProgram([CHAIN], spm_bytes=1 << 16))
    assert out[:1018].any() and not out[1018:2048].any() and flags & 1   # inf - inf and the NaN operand raise invalid


# NCx f32 [1, 4, 4, 64]: 2x2 / stride-2 max pooling, then 2x2 sum pooling of the result (one 64-channel block, so the
# physical bytes are the row-major ones).
POOL = _module("""
  call void @wafer_tx81_rdma(i64 %0, i64 0, i32 4096, i32 4096, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  call void @wafer_tx81_pool_max(i64 0, i64 4096, i32 117, i32 1, i32 4, i32 4, i32 64, i32 1, i32 2, i32 2, i32 64, i32 0, i32 0, i32 0, i32 0, i32 2, i32 2, i32 2, i32 2, i32 5, i32 1)
  call void @wafer_tx81_pool_sum(i64 4096, i64 8192, i32 116, i32 1, i32 2, i32 2, i32 64, i32 1, i32 1, i32 1, i32 64, i32 0, i32 0, i32 0, i32 0, i32 2, i32 2, i32 2, i32 2, i32 5, i32 1)
  call void @wafer_tx81_wdma(i64 4096, i64 %1, i32 1024, i32 1024, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  call void @wafer_tx81_wdma(i64 8192, i64 %2, i32 256, i32 256, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  ret void
""", arguments="i64 %0, i64 %1, i64 %2", rows=[
    '!{i64 0, !"external-input", i64 0, !"", !"f32", !"tensor", i64 4096, i64 1024, !"read-only", i64 16, i64 64, i64 0}',
    '!{i64 1, !"external-output", i64 0, !"", !"f32", !"tensor", i64 1024, i64 256, !"write-only", i64 4, i64 64, i64 0}',
    '!{i64 2, !"external-output", i64 1, !"", !"f32", !"tensor", i64 256, i64 64, !"write-only", i64 64, i64 0}'])


def _pool_input():
    x = np.random.default_rng(41).standard_normal((4, 4, 64)).astype(np.float32)
    x[0, 0, :3] = [np.float32(3.0e38), np.float32("nan"), -0.0]
    x[2, 2, 0] = np.float32(3.0e38)    # the sum of the pooled maxima of channel 0 overflows
    return x


def test_pool_calls_are_traced_and_replayed_on_the_cpu():
    from oracle import binding, trace_replay
    binding.build()
    program = TileProgram([POOL], spm_bytes=1 << 16)
    commands, _ = program.trace()
    assert [(c.name, c.operation, len(c.args)) for c in commands if "pool" in c.name] == [("wafer_tx81_pool", 117, 20), ("wafer_tx81_pool", 116, 20)]
    places = [program.placement(False, 0), program.placement(True, 0), program.placement(True, 1)]
    ddr = np.zeros(places[0]["ddr_bytes"], dtype=np.uint8)
    x = _pool_input()
    at = places[0]["address"] - places[0]["ddr_base"]
    ddr[at:at + 4096] = x.view(np.uint8).reshape(-1)
    report = {}
    trace_replay.replay(commands, ddr, 1, spm_bytes=1 << 16, report=report)
    at = places[1]["address"] - places[1]["ddr_base"]
    pooled = ddr[at:at + 1024].view(np.float32).reshape(2, 2, 64)
    finite = np.ones(64, dtype=bool)
    finite[1] = False
    assert np.array_equal(pooled[:, :, finite], x.reshape(2, 2, 2, 2, 64).max(axis=(1, 3))[:, :, finite])
    assert pooled[0, 0, 1].view(np.uint32) == 0x7fc00000 and report["numeric_flags"] & 0x4   # canonical NaN; the sum overflows
    with pytest.raises(WB200Error, match="pool_avg"):
        TileProgram([POOL.replace("pool_sum", "pool_avg")], spm_bytes=1 << 16)
    with pytest.raises(WB200Error, match="kind field"):
        TileProgram([POOL.replace("i32 117", "i32 119")], spm_bytes=1 << 16).trace()


def test_integer_subset_semantics():
    body = """
  %a = add i32 4000000000, 100
  %b = zext i32 %a to i64
  %c = sext i32 %a to i64
  %d = icmp slt i64 %c, 0
  %e = select i1 %d, i64 %b, i64 7
  %f = udiv i64 %e, 3
  %g = call i64 @llvm.smin.i64(i64 %c, i64 5)
  %h = ashr i64 %g, 60
  %i = trunc i64 %h to i8
  %j = zext i8 %i to i64
  %k = lshr i64 %f, 0
  switch i64 %j, label %bad [
    i64 255, label %good
  ]
bad:
  ret void
good:
  %len = and i64 %k, 1023
  %m = urem i64 %len, 1000
  %n = xor i64 %m, 1
  %o = or i64 %n, 64
  %q = freeze i64 %o
  call void @wafer_tx81_memset(i64 %q, i32 1, i32 4, i32 5, i32 0)
  ret void
"""
    commands, stats = TileProgram([_module(body)]).trace()
    # 4000000100 is negative as i32: the select keeps the zero-extended value and smin keeps the sign-extended one,
    # whose arithmetic shift gives all ones -> 255 after trunc / zext -> the switch case is taken.
    expected = ((((4000000100 // 3) & 1023) % 1000) ^ 1) | 64
    assert [(c.name, c.args[0]) for c in commands] == [("wafer_tx81_memset", expected)]
    assert stats["fill_commands"] == 1 and stats["instructions"] >= 18


def test_negative_numbers_take_the_signed_paths():
    body = """
  %a = sub i64 0, 9
  %b = sdiv i64 %a, 2
  %c = srem i64 %a, 4
  %d = add i64 %b, %c
  %e = sub i64 0, %d
  %f = call i64 @llvm.umax.i64(i64 %e, i64 2)
  call void @wafer_tx81_memset(i64 %f, i32 0, i32 1, i32 5, i32 0)
  ret void
"""
    commands, _ = TileProgram([_module(body)]).trace()
    assert commands[0].args[0] == 5          # -9 / 2 = -4 (toward zero), -9 % 4 = -1, -(-5) = 5


@pytest.mark.parametrize("body, fragment", [
    ("  %x = fadd float 1.0, 2.0\n  ret void", "outside"),
    ("  %p = inttoptr i64 %0 to ptr\n  ret void", "outside"),
    ("  call void @wafer_tx81_unpool_unpool(i64 0, i64 64, i32 121, i32 0)\n  ret void", "outside the executed command set"),
    ("  call void @wafer_tx81_memset(i64 0, i32 0, i32 4)\n  ret void", "does not match its descriptor"),
    ("  br label %nowhere", "unknown block"),
    ("  %x = add i64 1, 2", "no terminator"),
])
def test_modules_outside_the_subset_are_rejected_at_load(body, fragment):
    with pytest.raises(WB200Error, match=fragment):
        TileProgram([_module(body)])


def test_runtime_faults_are_reported_not_executed():
    with pytest.raises(WB200Error, match="outside the memory image"):
        TileProgram([_module("  call void @wafer_tx81_memset(i64 3145720, i32 0, i32 4, i32 5, i32 0)\n  ret void")]).trace()
    with pytest.raises(WB200Error, match="byte_count differs"):
        TileProgram([_module("  call void @wafer_tx81_rdma(i64 %0, i64 0, i32 100, i32 64, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)\n  ret void")]).trace()
    with pytest.raises(WB200Error, match="division"):
        TileProgram([_module("  %x = udiv i64 %0, 0\n  ret void")]).trace()
    rows = ['!{i64 0, !"transport-status", i64 0, !"direct_dte_status", !"u32", !"tensor", i64 64, i64 64, !"read-write", i64 1, i64 0}']
    waiting = """
  call void @wafer_tx81_direct_dte_begin(i64 %0, i32 2)
  %h = call i64 @wafer_tx81_direct_dte_recv_prepare(i64 0, i32 64, i32 TILE, i32 PEER, i32 0)
  call void @wafer_tx81_direct_dte_wait(i64 %h)
  call void @wafer_tx81_direct_dte_finish()
  ret void
"""
    modules = [_module(waiting.replace("TILE", str(t)).replace("PEER", str(1 - t)), "i64 %0", rows, tile=t) for t in range(2)]
    with pytest.raises(WB200Error, match="deadlock"):
        TileProgram(modules).trace()          # both Tiles wait to receive, nobody sends
    with pytest.raises(WB200Error, match="no-device|without a backend"):
        TileProgram([REVERSE_ROWS]).run([np.zeros((16, 16), np.float32)])


def test_direct_dte_send_blocks_until_the_receiver_is_prepared():
    rows = ['!{i64 0, !"transport-status", i64 0, !"direct_dte_status", !"u32", !"tensor", i64 64, i64 64, !"read-write", i64 1, i64 0}']
    sender = """
  call void @wafer_tx81_direct_dte_begin(i64 %0, i32 2)
  call void @wafer_tx81_memset(i64 128, i32 1065353216, i32 16, i32 5, i32 0)
  call void @wafer_tx81_ncc_join(i32 1)
  %h = call i64 @wafer_tx81_direct_dte_send_prepare(i64 128, i64 256, i32 64, i32 0, i32 1, i32 3, i32 0)
  call void @wafer_tx81_direct_dte_send_issue(i64 %h)
  call void @wafer_tx81_direct_dte_wait(i64 %h)
  call void @wafer_tx81_direct_dte_finish()
  ret void
"""
    receiver = """
  call void @wafer_tx81_direct_dte_begin(i64 %0, i32 2)
  call void @wafer_tx81_memset(i64 0, i32 0, i32 1024, i32 5, i32 0)
  %h = call i64 @wafer_tx81_direct_dte_recv_prepare(i64 256, i32 64, i32 1, i32 0, i32 3)
  call void @wafer_tx81_direct_dte_wait(i64 %h)
  call void @wafer_tx81_direct_dte_finish()
  ret void
"""
    commands, stats = TileProgram([_module(sender, "i64 %0", rows, 0), _module(receiver, "i64 %0", rows, 1)]).trace()
    names = [(c.tile, c.name.replace("wafer_tx81_", "")) for c in commands]
    # Tile 0 runs first and stops inside send_issue; the payload moves when Tile 1 prepares its receive
    assert names.index((0, "direct_dte_send_issue")) < names.index((1, "direct_dte_recv_prepare")) < names.index((0, "direct_dte_transfer"))
    assert names.index((0, "direct_dte_transfer")) < names.index((0, "direct_dte_wait"))
    assert stats["transfer_commands"] == 1 and stats["bytes_moved"] == 64 + 64 + 4096


# ------------------------------------------------------------------------------------------------ GPU
def _as_torch(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


@pytest.mark.gpu
def test_small_program_runs_on_the_device(backend):
    program = TileProgram([REVERSE_ROWS], backend, spm_bytes=1 << 16)
    matrix = np.random.default_rng(3).standard_normal((16, 16)).astype(np.float32)
    (out,), stats = program.run([matrix])
    assert np.array_equal(out.view(np.float32), matrix[::-1].T)
    assert stats["gpu_launches"] == 18 and stats["device_ms"] > 0


@pytest.mark.gpu
def test_select_program_runs_on_the_device(backend):
    program = TileProgram([SELECT], backend, spm_bytes=1 << 16)
    x = np.random.default_rng(8).standard_normal((16, 16)).astype(np.float32) * 2
    for _ in range(2):
        (out,), stats = program.run([x])
        assert np.array_equal(out.view(np.float32), np.where(x >= 1, x, np.float32(7)))
    assert stats["commands"] == 6 and stats["gpu_launches"] == 6


@pytest.mark.gpu
def test_elementwise_chain_is_fused_and_matches_the_unfused_replay_and_the_cpu(backend, monkeypatch):
    expected, expected_flags = _chain_cpu_replay(TileProgram([CHAIN], spm_bytes=1 << 16))
    fused = TileProgram([CHAIN], backend, spm_bytes=1 << 16)
    monkeypatch.setenv("WB200_REPLAY_FUSE", "0")
    unfused = TileProgram([CHAIN], backend, spm_bytes=1 << 16)
    monkeypatch.delenv("WB200_REPLAY_FUSE")
    x, y = _chain_inputs()
    for _ in range(2):   # the first run captures the graph, the second relaunches it
        (out_fused,), stats_fused = fused.run([x, y])
        (out_unfused,), stats_unfused = unfused.run([x, y])
        assert np.array_equal(out_fused.reshape(-1), expected) and np.array_equal(out_unfused.reshape(-1), expected)
        assert stats_fused["numeric_flags"] == stats_unfused["numeric_flags"] == expected_flags
        assert stats_fused["commands"] == stats_unfused["commands"] == 12
        assert stats_unfused["gpu_launches"] == 12 and stats_fused["gpu_launches"] == 6   # seven commands in one launch


@pytest.mark.gpu
def test_attention_step_run_is_one_launch_and_matches_the_unfused_replay_and_the_cpu(backend, monkeypatch):
    (want_out, want_m, want_l), want_flags, _ = _attention_cpu_replay(TileProgram([ATTENTION], spm_bytes=1 << 17))
    monkeypatch.setenv("WB200_REPLAY_RUNS", "1")     # command runs are opt-in: read when the program is loaded
    fused = TileProgram([ATTENTION], backend, spm_bytes=1 << 17)
    monkeypatch.delenv("WB200_REPLAY_RUNS")
    monkeypatch.setenv("WB200_REPLAY_FUSE", "0")
    unfused = TileProgram([ATTENTION], backend, spm_bytes=1 << 17)
    monkeypatch.delenv("WB200_REPLAY_FUSE")
    inputs = list(_attention_inputs())
    for _ in range(2):   # the first run captures the graph, the second relaunches it
        for program, launches in ((fused, 13), (unfused, 41)):
            (out, m, l), stats = program.run(inputs)
            assert np.array_equal(out.reshape(-1).view(np.uint32), want_out.view(np.uint32))
            assert np.array_equal(m.reshape(-1).view(np.uint32), want_m.view(np.uint32))
            assert np.array_equal(l.reshape(-1).view(np.uint32), want_l.view(np.uint32))
            assert stats["numeric_flags"] == want_flags and stats["commands"] == 41
            # fused: the 14 commands of a step between its loads are one launch, and the two closing commands join the last one
            assert stats["gpu_launches"] == launches


@pytest.mark.gpu
def test_pool_program_matches_the_cpu_replay_bit_for_bit(backend):
    from oracle import binding, trace_replay
    binding.build()
    program = TileProgram([POOL], backend, spm_bytes=1 << 16)
    commands, _ = program.trace()
    places = [program.placement(False, 0), program.placement(True, 0), program.placement(True, 1)]
    ddr = np.zeros(places[0]["ddr_bytes"], dtype=np.uint8)
    x = _pool_input()
    at = places[0]["address"] - places[0]["ddr_base"]
    ddr[at:at + 4096] = x.view(np.uint8).reshape(-1)
    report = {}
    trace_replay.replay(commands, ddr, 1, spm_bytes=1 << 16, report=report)
    (pooled, summed), stats = program.run([x.reshape(16, 64)])
    for place, got in zip(places[1:], (pooled, summed)):
        at = place["address"] - place["ddr_base"]
        assert np.array_equal(got.reshape(-1).view(np.uint8), ddr[at:at + got.nbytes])
    assert stats["numeric_flags"] == report["numeric_flags"] and stats["gpu_launches"] == 5


@pytest.mark.gpu
def test_numeric_program_matches_the_cpu_replay_bit_for_bit(backend):
    program = TileProgram([NUMERIC], backend, spm_bytes=1 << 16)
    _, want_out, want_mask, want_flags = _numeric_cpu_replay(program)
    x, unit = _numeric_inputs()
    for _ in range(2):                                              # the second run relaunches the captured graph
        (out, mask), stats = program.run([x, unit])
        assert np.array_equal(out.reshape(-1), want_out) and np.array_equal(mask.reshape(-1), want_mask)
        assert stats["numeric_flags"] == want_flags and stats["commands"] == 17
    refusing = _module("""
  call void @wafer_tx81_rdma(i64 %0, i64 0, i32 1024, i32 1024, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  call void @wafer_tx81_convert_fp32_int32(i64 0, i64 4096, i32 256, i32 0, i32 0, i32 1)
  call void @wafer_tx81_wdma(i64 4096, i64 %1, i32 1024, i32 1024, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 4, i32 0)
  ret void
""", rows=['!{i64 0, !"external-input", i64 0, !"", !"f32", !"tensor", i64 1024, i64 256, !"read-only", i64 16, i64 16, i64 0}',
           '!{i64 1, !"external-output", i64 0, !"", !"i32", !"tensor", i64 1024, i64 256, !"write-only", i64 16, i64 16, i64 0}'])
    program = TileProgram([refusing], backend, spm_bytes=1 << 16)
    values = np.arange(256, dtype=np.float32).reshape(16, 16) - 100.25
    (out,), stats = program.run([values])
    assert np.array_equal(out.view(np.int32).reshape(-1), np.rint(values.reshape(-1)).astype(np.int32)) and stats["numeric_flags"] == 16
    values[7, 3] = np.inf
    with pytest.raises(WB200Error, match="float-to-integer-non-finite.* at element 115"):
        program.run([values])
    values[7, 3] = 1.0
    (out,), _ = program.run([values])                               # the program stays usable after a refused run
    assert out.view(np.int32).reshape(-1)[115] == 1


@pytest.mark.gpu
@pytest.mark.parametrize("plan", PLANS)
def test_shipped_plan_replays_bit_exactly(backend, oracle, plan):
    inputs = expected_tools.program_inputs()
    assert hashlib.sha256(b"".join(a.tobytes() for a in inputs)).hexdigest() == EXPECTED["inputs_sha256"]
    program = TileProgram(FIXTURE["plans"][plan], backend)
    (out,), stats = program.run(inputs, abi.GEMM_FORMAL)
    assert stats["gemm_commands"] in (256, 1024) and stats["gpu_launches"] >= stats["gemm_commands"] + stats["movement_commands"]
    assert hashlib.sha256(out.tobytes()).hexdigest() == EXPECTED["plans"][plan]["sha256"]
    # the reference's acceptance gate against the source program: out = arg1 . arg0
    want = (_as_torch(inputs[1]).float()[0].cuda() @ _as_torch(inputs[0]).float()[0].cuda()).bfloat16().cpu()
    helpers.reference_gate(oracle, "bf16", out.reshape(-1), helpers.bits(want).reshape(-1))
    program.close()


@pytest.mark.gpu
def test_one_plan_against_the_live_cpu_replay(backend):
    plan = "tensor-winner"
    inputs = expected_tools.program_inputs()
    want = expected_tools.cpu_replay(FIXTURE["plans"][plan], inputs, threads=16)
    (out,), _ = TileProgram(FIXTURE["plans"][plan], backend).run(inputs)
    assert np.array_equal(out, want)


@pytest.mark.gpu
def test_graph_replay_is_reused_and_agrees_with_the_single_stream_order(backend):
    # The first run captures the invocation (one stream per Tile, Direct-DTE transfers as event edges) into a CUDA
    # graph; later runs relaunch it. Doubling arg0 doubles every product exactly, so the second run's output must be
    # exactly twice the first one's.
    plan = "tensor-candidate-38"
    inputs = expected_tools.program_inputs()
    program = TileProgram(FIXTURE["plans"][plan], backend)
    (first,), stats1 = program.run(inputs)
    assert hashlib.sha256(first.tobytes()).hexdigest() == EXPECTED["plans"][plan]["sha256"]
    doubled = (_as_torch(inputs[0]).float() * 2).bfloat16()
    (second,), stats2 = program.run([doubled.view(torch.int16).numpy().view(np.uint16), inputs[1]])
    assert torch.equal(_as_torch(second).float(), _as_torch(first).float() * 2)
    assert stats2["commands"] == stats1["commands"] and stats2["gpu_launches"] == stats1["gpu_launches"]
    (again,), _ = program.run(inputs)
    assert np.array_equal(again, first)


@pytest.mark.gpu
def test_tensor_core_policy_replays_concurrently_and_matches_its_single_stream_order(backend, oracle):
    # Under the tensor-core GEMM policy the Tiles run side by side too (one stream per Tile in a captured graph of its
    # own, compact operands staged in areas private to each Tile). Same kernels, same per-Tile order: the bits must equal
    # the single-stream replay's, the relaunch must equal the first run, and the output passes the reference's gate.
    import os, subprocess, sys
    plan = "tensor-winner"
    inputs = expected_tools.program_inputs()
    program = TileProgram(FIXTURE["plans"][plan], backend)
    (first,), stats1 = program.run(inputs, abi.GEMM_TENSOR)
    (second,), stats2 = program.run(inputs, abi.GEMM_TENSOR)
    assert np.array_equal(first, second) and stats1["gpu_launches"] == stats2["gpu_launches"]
    want = (_as_torch(inputs[1]).float()[0].cuda() @ _as_torch(inputs[0]).float()[0].cuda()).bfloat16().cpu()
    helpers.reference_gate(oracle, "bf16", first.reshape(-1), helpers.bits(want).reshape(-1))
    (formal,), _ = program.run(inputs, abi.GEMM_FORMAL)                 # the other policy's graph lives beside it
    assert hashlib.sha256(formal.tobytes()).hexdigest() == EXPECTED["plans"][plan]["sha256"]
    (third,), _ = program.run(inputs, abi.GEMM_TENSOR)
    assert np.array_equal(first, third)
    code = ("import sys, hashlib; sys.path.insert(0, %r);"
            "from tests.test_tile_program import FIXTURE, expected_tools;"
            "from vibe_compiler_b200 import _abi as abi;"
            "from vibe_compiler_b200.backend import B200TargetModelBackend as B;"
            "from vibe_compiler_b200.tile_program import TileProgram;"
            "(out,), stats = TileProgram(FIXTURE['plans']['tensor-winner'], B(0)).run(expected_tools.program_inputs(), abi.GEMM_TENSOR);"
            "print(hashlib.sha256(out.tobytes()).hexdigest())") % str(ROOT)
    result = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, WB200_REPLAY_GRAPH="0"), capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stderr[-2000:]
    assert result.stdout.strip().splitlines()[-1] == hashlib.sha256(first.tobytes()).hexdigest()
    program.close()


# Two Tiles, each one 256 x 256 x 256 bf16 GEMM without a partial sum (the form the tensor-core policy takes to the
# tcgen05 kernel; every GEMM of the shipped plans carries a partial sum and stays on the bit-exact kernel under either
# policy). The operands are copied flat into the scratch-pad, whose Cx reading permutes them: still a matrix product.
def _two_tile_gemm_modules():
    body = """
  call void @wafer_tx81_rdma(i64 %0, i64 0, i32 131072, i32 131072, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 3, i32 0)
  call void @wafer_tx81_rdma(i64 %1, i64 131072, i32 131072, i32 131072, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 3, i32 0)
  call void @wafer_tx81_gemm(i64 0, i64 131072, i64 262144, i64 0, i32 256, i32 256, i32 256, i32 1, i32 3, i32 3, i32 13, i32 0)
  call void @wafer_tx81_wdma(i64 262144, i64 %2, i32 131072, i32 131072, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 3, i32 0)
  ret void
"""
    def rows(first_input, output):
        matrix = '!"", !"bf16", !"tensor", i64 131072, i64 65536'
        return [f'!{{i64 0, !"external-input", i64 {first_input}, {matrix}, !"read-only", i64 256, i64 256, i64 0}}',
                f'!{{i64 1, !"external-input", i64 {first_input + 1}, {matrix}, !"read-only", i64 256, i64 256, i64 0}}',
                f'!{{i64 2, !"external-output", i64 {output}, {matrix}, !"write-only", i64 256, i64 256, i64 0}}']
    return [_module(body, arguments="i64 %0, i64 %1, i64 %2", rows=rows(0, 0), tile=0),
            _module(body, arguments="i64 %0, i64 %1, i64 %2", rows=rows(2, 1), tile=1)]


def _two_tile_gemm_inputs():
    rng = np.random.default_rng(5)
    return [(rng.uniform(-1, 1, (256, 256)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16) for _ in range(4)]


@pytest.mark.gpu
def test_tensor_core_gemms_of_two_tiles_run_side_by_side(backend):
    import os, subprocess, sys
    program = TileProgram(_two_tile_gemm_modules(), backend)
    inputs = _two_tile_gemm_inputs()
    formal, stats_formal = program.run(inputs, abi.GEMM_FORMAL)
    first, stats1 = program.run(inputs, abi.GEMM_TENSOR)        # captures the tensor-policy graph
    second, stats2 = program.run(inputs, abi.GEMM_TENSOR)       # relaunches it
    assert stats_formal["gpu_launches"] == 8 and stats1["gpu_launches"] == stats2["gpu_launches"] == 14   # + 2 unpacks and a pack per GEMM
    for tile in range(2):
        assert np.array_equal(first[tile], second[tile])
        want, got = _as_torch(formal[tile]).float(), _as_torch(first[tile]).float()
        assert float((got - want).abs().max() / want.abs().max()) <= 1e-2        # f32 accumulation, one rounding, another order
    code = ("import sys, hashlib; sys.path.insert(0, %r);"
            "from tests.test_tile_program import _two_tile_gemm_modules, _two_tile_gemm_inputs;"
            "from vibe_compiler_b200 import _abi as abi;"
            "from vibe_compiler_b200.backend import B200TargetModelBackend as B;"
            "from vibe_compiler_b200.tile_program import TileProgram;"
            "outs, stats = TileProgram(_two_tile_gemm_modules(), B(0)).run(_two_tile_gemm_inputs(), abi.GEMM_TENSOR);"
            "print(hashlib.sha256(b''.join(o.tobytes() for o in outs)).hexdigest())") % str(ROOT)
    result = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, WB200_REPLAY_GRAPH="0"), capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stderr[-2000:]
    assert result.stdout.strip().splitlines()[-1] == hashlib.sha256(b"".join(o.tobytes() for o in first)).hexdigest()
    program.close()


@pytest.mark.gpu
def test_single_stream_replay_matches_the_graph_replay():
    import os, subprocess, sys
    code = ("import sys, json, lzma, hashlib; sys.path.insert(0, %r);"
            "from tests.test_tile_program import FIXTURE, expected_tools;"
            "from vibe_compiler_b200.backend import B200TargetModelBackend as B;"
            "from vibe_compiler_b200.tile_program import TileProgram;"
            "(out,), stats = TileProgram(FIXTURE['plans']['tensor-winner'], B(0)).run(expected_tools.program_inputs());"
            "print(hashlib.sha256(out.tobytes()).hexdigest())") % str(ROOT)
    digests = []
    for mode in ("0", "1"):
        result = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, WB200_REPLAY_GRAPH=mode), capture_output=True, text=True, timeout=300)
        assert result.returncode == 0, result.stderr[-2000:]
        digests.append(result.stdout.strip().splitlines()[-1])
    assert digests[0] == digests[1] == EXPECTED["plans"]["tensor-winner"]["sha256"]
