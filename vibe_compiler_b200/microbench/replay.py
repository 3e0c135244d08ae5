"""Replay time of the shipped GEMM Tile programs (16 Tiles x 7 plans, out[4096,4096] = arg1[4096,1024] . arg0[1024,4096], bf16).

    python -m vibe_compiler_b200.microbench.replay --fixture tests/golden/gemm_tile_modules.json.xz [--plan NAME] [--runs N]
    python -m vibe_compiler_b200.microbench.replay --module tests/golden/attention_step_tile.ll --spm-bytes 131072

The second form times one hand-written one-Tile module (f32 inputs drawn from a standard normal distribution): with
WB200_REPLAY_FUSE=0 every command is a launch of its own, by default runs of formal commands are one launch each.

Prints one JSON line per plan: commands, kernel launches and the device time of the command stream (CUDA events inside
wb200_tile_program_run; host <-> device tensor copies excluded). WB200_REPLAY_GRAPH=0 in the environment replays the
commands one by one on a single stream (the form a per-kernel launch list is taken from); the default relaunches the
captured CUDA graph.
"""
from __future__ import annotations

import argparse
import json
import lzma
import statistics
from pathlib import Path

import numpy as np

from .. import _abi as abi
from ..backend import B200TargetModelBackend
from ..tile_program import TileProgram


def main(argv=None) -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--plan", default="", help="only the plans whose name contains this text")
    parser.add_argument("--runs", type=int, default=5)
    parser.add_argument("--gemm-policy", choices=["formal", "tensor"], default="formal",
                        help="bit-exact k-ascending FMA chains, or the tcgen05 kernel on unpacked operands (f32 accumulation, one rounding)")
    parser.add_argument("--module", default="", help="one Tile's .ll module instead of a fixture of plans")
    parser.add_argument("--spm-bytes", type=int, default=0, help="scratch-pad size for --module (default: the library's)")
    parser.add_argument("--fixture", default="",
                        help="packed per-Tile modules (JSON, xz): {plan: {tile name: .ll text}}; the reference's seven GEMM plans are "
                             "packed in tests/golden/gemm_tile_modules.json.xz of the source tree")
    args = parser.parse_args(argv)
    if not args.fixture and not args.module:
        parser.error("give --fixture or --module")
    backend = B200TargetModelBackend(0)
    rng = np.random.default_rng(20260803)
    policy = abi.GEMM_TENSOR if args.gemm_policy == "tensor" else abi.GEMM_FORMAL
    if args.module:
        text = Path(args.module).read_text()
        program = TileProgram([text], backend, **({"spm_bytes": args.spm_bytes} if args.spm_bytes else {}))
        inputs = [rng.standard_normal(t.shape).astype(np.float32) for t in program.inputs]
        times, stats = [], None
        for _ in range(max(2, args.runs)):
            _, stats = program.run(inputs)
            times.append(stats["device_ms"])
        print(json.dumps({"module": Path(args.module).name, "commands": stats["commands"], "gemm_commands": stats["gemm_commands"],
                          "gpu_launches": stats["gpu_launches"], "device_ms_first": round(times[0], 3),
                          "device_ms": round(statistics.median(times[1:]), 4)}), flush=True)
        program.close()
        return 0
    fixture = json.loads(lzma.decompress(Path(args.fixture).read_bytes()))
    for plan in sorted(fixture["plans"]):
        if args.plan not in plan:
            continue
        program = TileProgram(fixture["plans"][plan], backend)
        inputs = [rng.integers(0x3c00, 0x4000, size=t.shape, dtype=np.uint16) for t in program.inputs]   # bf16 values in [0.0078, 2)
        times, stats = [], None
        for _ in range(max(2, args.runs)):
            _, stats = program.run(inputs, policy)
            times.append(stats["device_ms"])
        print(json.dumps({"plan": plan, "gemm_policy": args.gemm_policy, "commands": stats["commands"], "gemm_commands": stats["gemm_commands"],
                          "movement_commands": stats["movement_commands"], "gpu_launches": stats["gpu_launches"],
                          "device_ms_first": round(times[0], 3), "device_ms": round(statistics.median(times[1:]), 3)}), flush=True)
        program.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
