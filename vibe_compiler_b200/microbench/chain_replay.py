"""Device time of a five-command elementwise chain replayed by the Tile-program interpreter, fused and command by command.

    python -m vibe_compiler_b200.microbench.chain_replay [--elements N ...] [--runs R]

One Tile: two f32 vectors come in by RDMA, `max(relu((x + y) * 0.5) - y, x)` runs as add, mul by an immediate, in-place
relu, sub, max (each command's first operand is the previous destination), the result leaves by WDMA. Prints one JSON
line per vector length with the device time of the whole command stream (CUDA events inside wb200_tile_program_run,
graph relaunch, median) for the movement commands alone, for the fused replay (one launch for the five commands) and
for the replay with WB200_REPLAY_FUSE=0 (five launches), and the elementwise time of each as the difference.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import numpy as np

from ..backend import B200TargetModelBackend
from ..tile_program import TileProgram


def _module(elements: int, with_chain: bool) -> str:
    size = elements * 4
    at = [i * size for i in range(6)]
    dma = f"i32 {size}, i32 {size}, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0"
    body = [f"  call void @wafer_tx81_rdma(i64 %0, i64 {at[0]}, {dma})", f"  call void @wafer_tx81_rdma(i64 %1, i64 {at[1]}, {dma})"]
    if with_chain:
        tail = f"i32 {elements}, i32 5"
        body += [f"  call void @wafer_tx81_elementwise_add(i64 {at[0]}, i64 {at[1]}, i64 {at[2]}, {tail}, i32 0, i32 0, i32 0, i32 1)",
                 f"  call void @wafer_tx81_elementwise_mul(i64 {at[2]}, i64 {0x3f000000}, i64 {at[3]}, {tail}, i32 0, i32 1, i32 0, i32 1)",
                 f"  call void @wafer_tx81_elementwise_relu(i64 {at[3]}, i64 {at[3]}, {tail}, i32 1)",
                 f"  call void @wafer_tx81_elementwise_sub(i64 {at[3]}, i64 {at[1]}, i64 {at[4]}, {tail}, i32 0, i32 0, i32 0, i32 1)",
                 f"  call void @wafer_tx81_elementwise_max(i64 {at[4]}, i64 {at[0]}, i64 {at[5]}, {tail}, i32 0, i32 0, i32 0, i32 1)"]
    body += [f"  call void @wafer_tx81_wdma(i64 {at[5] if with_chain else at[1]}, i64 %2, {dma})", "  ret void"]
    row = lambda i, kind, ordinal, access: (f'!{{i64 {i}, !"{kind}", i64 {ordinal}, !"", !"f32", !"tensor", i64 {size}, i64 {elements}, '
                                            f'!"{access}", i64 {elements}, i64 0}}')
    rows = [row(0, "external-input", 0, "read-only"), row(1, "external-input", 1, "read-only"), row(2, "external-output", 0, "write-only")]
    names = ", ".join(f"!{10 + i}" for i in range(3))
    meta = "\n".join(f"!{10 + i} = {r}" for i, r in enumerate(rows))
    return ("define void @entry(i64 %0, i64 %1, i64 %2) {\n" + "\n".join(body) + "\n}\n!wafer.target.tile_id = !{!2}\n"
            f"!wafer.target.entry_arguments = !{{{names}}}\n!2 = !{{i64 0}}\n{meta}\n")


def _median_ms(program, inputs, runs):
    times = []
    for _ in range(runs + 2):
        (out,), stats = program.run(inputs)
        times.append(stats["device_ms"])
    return statistics.median(times[2:]), stats["gpu_launches"], out


def main(argv=None) -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--elements", type=int, nargs="+", default=[1 << 17, 1 << 24])
    parser.add_argument("--runs", type=int, default=9)
    args = parser.parse_args(argv)
    backend = B200TargetModelBackend(0)
    rng = np.random.default_rng(5)
    for elements in args.elements:
        inputs = [rng.standard_normal(elements).astype(np.float32), rng.standard_normal(elements).astype(np.float32)]
        spm_bytes = 6 * elements * 4
        line = {"elements": elements, "format": "f32"}
        outputs = {}
        for label, chain, fuse in (("movement_only", False, "1"), ("fused", True, "1"), ("unfused", True, "0")):
            os.environ["WB200_REPLAY_FUSE"] = fuse   # read when the program is loaded
            program = TileProgram([_module(elements, chain)], backend, spm_bytes=spm_bytes)
            ms, launches, outputs[label] = _median_ms(program, inputs, args.runs)
            line[label + "_ms"], line[label + "_launches"] = round(ms, 4), launches
            program.close()
        os.environ.pop("WB200_REPLAY_FUSE", None)
        if not np.array_equal(outputs["fused"].view(np.uint32), outputs["unfused"].view(np.uint32)):
            raise SystemExit("fused and unfused replays differ")
        line["fused_elementwise_ms"] = round(line["fused_ms"] - line["movement_only_ms"], 4)
        line["unfused_elementwise_ms"] = round(line["unfused_ms"] - line["movement_only_ms"], 4)
        line["fused_bytes"], line["unfused_bytes"] = 9 * elements * 4, 13 * elements * 4
        print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
