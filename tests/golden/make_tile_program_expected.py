"""Expected outputs of the seven shipped GEMM Tile programs, from the CPU trace replay (oracle/trace_replay.py).

For every plan in gemm_tile_modules.json.xz: the library's device-free trace is executed on the CPU with the
restated command semantics, and the SHA-256 of the output bits (compact row-major bf16) is stored together with the
hash of the seeded inputs. The GPU tests compare the device replay with these hashes bit for bit.

    python tests/golden/make_tile_program_expected.py
"""
import hashlib
import json
import lzma
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import binding, trace_replay  # noqa: E402
from vibe_compiler_b200.tile_program import TileProgram  # noqa: E402

SEED = 20260803
LAYOUT_NAMES = {0: "tensor", 1: "ntensor", 2: "cx", 3: "ncx"}


def program_inputs():
    g = torch.Generator(device="cpu").manual_seed(SEED)
    arg0 = torch.randn(1, 1024, 4096, generator=g).bfloat16()
    arg1 = torch.randn(1, 4096, 1024, generator=g).bfloat16()
    return [t.view(torch.int16).numpy().view(np.uint16) for t in (arg0, arg1)]


def cpu_replay(modules, inputs, threads):
    program = TileProgram(modules)
    commands, _ = program.trace()
    first = program.placement(False, 0)
    ddr = np.zeros(first["ddr_bytes"], dtype=np.uint8)
    for index, (bits, info) in enumerate(zip(inputs, program.inputs)):
        place = program.placement(False, index)
        at = place["address"] - place["ddr_base"]
        ddr[at:at + place["physical_bytes"]] = binding.pack("bf16", LAYOUT_NAMES[info.layout], list(info.shape), bits,
                                                            np.zeros(place["physical_bytes"], np.uint8))
    trace_replay.replay(commands, ddr, len(modules), threads=threads)
    place, info = program.placement(True, 0), program.outputs[0]
    at = place["address"] - place["ddr_base"]
    return binding.unpack("bf16", LAYOUT_NAMES[info.layout], list(info.shape), ddr[at:at + place["physical_bytes"]]).reshape(info.shape)


def main():
    binding.build()
    fixture = json.loads(lzma.decompress((ROOT / "tests" / "golden" / "gemm_tile_modules.json.xz").read_bytes()))
    inputs = program_inputs()
    expected = {"seed": SEED, "inputs_sha256": hashlib.sha256(b"".join(a.tobytes() for a in inputs)).hexdigest(), "plans": {}}
    for plan, modules in fixture["plans"].items():
        out = cpu_replay(modules, inputs, threads=8)
        expected["plans"][plan] = {"sha256": hashlib.sha256(out.tobytes()).hexdigest(), "first_bits": [int(v) for v in out.reshape(-1)[:8]]}
        print(plan, expected["plans"][plan]["sha256"][:16], flush=True)
    (ROOT / "tests" / "golden" / "gemm_tile_program_expected.json").write_text(json.dumps(expected, indent=1) + "\n")


if __name__ == "__main__":
    main()
