"""Packs the reference's published per-Tile target LLVM modules of its GEMM optimisation ladder into one fixture.

Source (read-only, only available where the reference checkout is mounted):
  docs/data/board-performance/gemm-optimization-ladder-20261020-ir/<plan>/target-llvm/tile_000NN.ll
seven plans x 16 Tiles of the same source program (out[4096,4096] = arg1[4096,1024] . arg0[1024,4096], bf16),
together with the kernel medians of the table in that folder's README. The modules are compiler OUTPUT (data), kept
byte for byte; they are the inputs of the Tile-program replay tests.

    python tests/golden/make_tile_module_fixture.py <reference checkout root>
"""
import json
import lzma
import re
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
LADDER = "docs/data/board-performance/gemm-optimization-ladder-20261020-ir"


def main():
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    root = Path(sys.argv[1]) / LADDER
    plans = {}
    for plan_dir in sorted(p for p in root.iterdir() if (p / "target-llvm").is_dir()):
        modules = [path.read_text() for path in sorted((plan_dir / "target-llvm").glob("tile_*.ll"))]
        assert len(modules) == 16, plan_dir
        plans[plan_dir.name] = modules
    medians = {}
    for line in (root / "README.md").read_text().splitlines():
        found = re.match(r"\|[^|]*\|\s*\[([^\]]+)\][^|]*\|\s*([0-9.]+)\s*\|", line)
        if found:
            medians[found.group(1)] = float(found.group(2))
    assert set(medians) == set(plans), (medians, list(plans))
    payload = {"program": {"m": 4096, "n": 4096, "k": 1024, "dtype": "bf16", "tiles": 16,
                           "expression": "out[1,4096,4096] = dot_general(arg1[1,4096,1024], arg0[1,1024,4096])"},
               "board_kernel_median_ms": medians, "plans": plans}
    out = HERE / "gemm_tile_modules.json.xz"
    out.write_bytes(lzma.compress(json.dumps(payload).encode(), preset=9))
    print(f"wrote {out}: {len(plans)} plans, {out.stat().st_size} bytes")


if __name__ == "__main__":
    main()
