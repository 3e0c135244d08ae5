"""Expected results of the correctly rounded function family over the COMPLETE 16-bit operand space.

For every function of oracle/formal_scalar.FUNCTIONS and both 16-bit formats, all 65 536 operand encodings are
evaluated with 200-bit arithmetic and rounded once; the fixture keeps the SHA-256 of the result table, the OR of all
flags, and 192 sampled operands (specials plus a seeded random draw) with their result and flags for per-element
checks. Takes about two minutes.

    python tests/golden/make_formal_function_expected.py
"""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import formal_scalar as F  # noqa: E402

SPECIALS = {"f16": [0x0000, 0x8000, 0x0001, 0x8001, 0x03ff, 0x0400, 0x3c00, 0xbc00, 0x4000, 0x4400, 0x4800, 0x7bff, 0xfbff, 0x7c00, 0xfc00, 0x7c01, 0x7e00, 0x3800, 0x4d00, 0xcd00],
            "bf16": [0x0000, 0x8000, 0x0001, 0x8001, 0x007f, 0x0080, 0x3f80, 0xbf80, 0x4000, 0x4080, 0x4100, 0x7f7f, 0xff7f, 0x7f80, 0xff80, 0x7f81, 0x7fc0, 0x3f00, 0x42b0, 0xc2b0]}


def main():
    expected = {}
    for fmt in ("f16", "bf16"):
        rng = np.random.default_rng(20260803)
        sample = sorted(set(SPECIALS[fmt]) | set(int(v) for v in rng.integers(0, 65536, 172)))
        for op in F.FUNCTIONS:
            table = np.empty(65536, dtype=np.uint16)
            flags_or, samples = 0, {}
            for bits in range(65536):
                result, flags = F.evaluate_function(op, fmt, bits)
                table[bits] = result
                flags_or |= flags
                if bits in sample:
                    samples[str(bits)] = [result, flags]
            expected[f"{fmt}:{op}"] = {"sha256": hashlib.sha256(table.tobytes()).hexdigest(), "flags_or": flags_or, "samples": samples}
            print(fmt, op, expected[f"{fmt}:{op}"]["sha256"][:16], flags_or, flush=True)
    (ROOT / "tests" / "golden" / "formal_function_expected.json").write_text(json.dumps(expected) + "\n")


if __name__ == "__main__":
    main()
