"""Golden vectors of the correctly rounded function family for binary32 and TF32 operands.

binary32: for each of the 11 functions, (1) every operand whose evaluation needs more than binary64 (found by scanning
the complete operand space with the library's own evaluator compiled for the host, formal_f32_scan.cpp: the operands
within 2^-46 of a rounding boundary, 46 to 905 per function), (2) the special operands and (3) 2^20 operands drawn from a
seed, all evaluated with 200-bit arithmetic (oracle/formal_scalar.evaluate_function: mpmath, exact rational, one
rounding). Kept: (1) and (2) element by element (operand, result, flags), (3) as the SHA-256 of the result and flag tables.
TF32: the complete space of 2^19 operand encodings per function, as SHA-256 of the result table and the OR of the flags.

    python tests/golden/make_formal_function_f32_expected.py          # about 25 minutes on 8 cores
    python tests/golden/make_formal_function_f32_expected.py --check   # host evaluator against the committed vectors
"""
import hashlib
import multiprocessing
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import formal_scalar as F  # noqa: E402

OUT = ROOT / "tests" / "golden" / "formal_function_f32_expected.npz"
SEED = 20260803
RANDOM_COUNT = 1 << 20
SPECIALS = [0x00000000, 0x80000000, 0x00000001, 0x80000001, 0x007fffff, 0x00800000, 0x3f800000, 0xbf800000, 0x40000000, 0x40800000,
            0x41000000, 0x7f7fffff, 0xff7fffff, 0x7f800000, 0xff800000, 0x7f800001, 0x7fc00000, 0x3f000000, 0x42b00000, 0xc2b00000,
            0x42000000, 0xc2000000, 0x41a00000, 0xc1a00000, 0x43000000, 0xc3160000, 0x42fe0000, 0xc2fc0000, 0x3fc90fdb, 0x40490fdb,
            0x4b000000, 0x7e800000, 0x3f490fdb, 0x33800000, 0xb3800000, 0x42d00000, 0xc2d00000, 0xc2ce0000]


def build_tool() -> Path:
    tool = Path(tempfile.gettempdir()) / "wb200_formal_f32_scan"
    subprocess.run(["g++", "-O2", "-std=c++17", "-pthread", "-o", str(tool), str(ROOT / "tests" / "golden" / "formal_f32_scan.cpp")], check=True)
    return tool


def host_eval(tool: Path, function: int, tf32: bool, operands: np.ndarray):
    raw = subprocess.run([str(tool), "eval", str(function), "1" if tf32 else "0"], input=operands.astype("<u4").tobytes(), capture_output=True, check=True).stdout
    pairs = np.frombuffer(raw, dtype="<u4").reshape(-1, 2)
    return pairs[:, 0].copy(), pairs[:, 1].copy()


def _oracle_chunk(args):
    op, fmt, operands = args
    results, flags = np.empty(len(operands), np.uint32), np.empty(len(operands), np.uint8)
    for i, bits in enumerate(operands):
        if fmt == "tf32":
            r, f = F.evaluate_function(op, "tf32", int(bits) >> 13)
            r <<= 13
        else:
            r, f = F.evaluate_function(op, "f32", int(bits))
        results[i], flags[i] = r, f
    return results, flags


def oracle_eval(pool, op: str, fmt: str, operands: np.ndarray):
    chunks = np.array_split(operands, max(1, min(len(operands) // 256, 512)))
    parts = pool.map(_oracle_chunk, [(op, fmt, c) for c in chunks])
    return np.concatenate([p[0] for p in parts]), np.concatenate([p[1] for p in parts])


def random_operands(function: int) -> np.ndarray:
    return np.random.default_rng(SEED + function).integers(0, 1 << 32, RANDOM_COUNT, dtype=np.uint64).astype(np.uint32)


def main():
    tool = build_tool()
    if "--check" in sys.argv:
        data = np.load(OUT)
        for function, op in enumerate(F.FUNCTIONS):
            listed = data[f"f32_{op}_operands"]
            got, got_flags = host_eval(tool, function, False, listed)
            assert np.array_equal(got, data[f"f32_{op}_results"]) and np.array_equal(got_flags.astype(np.uint8), data[f"f32_{op}_flags"]), op
            got, got_flags = host_eval(tool, function, False, random_operands(function))
            assert hashlib.sha256(got.astype("<u4").tobytes()).hexdigest() == str(data[f"f32_{op}_random_sha256"]), op
            assert hashlib.sha256(got_flags.astype(np.uint8).tobytes()).hexdigest() == str(data[f"f32_{op}_random_flags_sha256"]), op
            everything = (np.arange(1 << 19, dtype=np.uint32) << 13)
            got, got_flags = host_eval(tool, function, True, everything)
            assert hashlib.sha256(got.astype("<u4").tobytes()).hexdigest() == str(data[f"tf32_{op}_sha256"]), op
            assert int(np.bitwise_or.reduce(got_flags)) == int(data[f"tf32_{op}_flags_or"]), op
            print("host evaluator matches", op, flush=True)
        return
    quick = "--quick" in sys.argv          # development aid: fewer random operands, no TF32 table, nothing written
    out = {}
    with multiprocessing.Pool() as pool:
        for function, op in enumerate(F.FUNCTIONS):
            hard = np.frombuffer(subprocess.run([str(tool), "scan", str(function)], capture_output=True, check=True).stdout, dtype="<u4")
            listed = np.unique(np.concatenate([hard, np.array(SPECIALS, dtype=np.uint32)]))
            want, want_flags = oracle_eval(pool, op, "f32", listed)
            got, got_flags = host_eval(tool, function, False, listed)
            bad = np.nonzero((want != got) | (want_flags != got_flags.astype(np.uint8)))[0]
            print(op, "listed operands", len(listed), "host mismatches", len(bad), [(hex(int(listed[i])), hex(int(want[i])), hex(int(got[i])), int(want_flags[i]), int(got_flags[i])) for i in bad[:6]], flush=True)
            out[f"f32_{op}_operands"], out[f"f32_{op}_results"], out[f"f32_{op}_flags"] = listed, want, want_flags
            sample = random_operands(function)[: (20000 if quick else RANDOM_COUNT)]
            want, want_flags = oracle_eval(pool, op, "f32", sample)
            got, got_flags = host_eval(tool, function, False, sample)
            bad = np.nonzero((want != got) | (want_flags != got_flags.astype(np.uint8)))[0]
            print(op, "random operands", len(sample), "host mismatches", len(bad), [(hex(int(sample[i])), hex(int(want[i])), hex(int(got[i])), int(want_flags[i]), int(got_flags[i])) for i in bad[:6]], flush=True)
            out[f"f32_{op}_random_sha256"] = hashlib.sha256(want.astype("<u4").tobytes()).hexdigest()
            out[f"f32_{op}_random_flags_sha256"] = hashlib.sha256(want_flags.astype(np.uint8).tobytes()).hexdigest()
            out[f"f32_{op}_random_flags_or"] = int(np.bitwise_or.reduce(want_flags))
            if quick:
                continue
            everything = (np.arange(1 << 19, dtype=np.uint32) << 13)
            want, want_flags = oracle_eval(pool, op, "tf32", everything)
            got, got_flags = host_eval(tool, function, True, everything)
            bad = np.nonzero((want != got) | (want_flags != got_flags.astype(np.uint8)))[0]
            print(op, "tf32 complete space, host mismatches", len(bad), [(hex(int(everything[i])), hex(int(want[i])), hex(int(got[i])), int(want_flags[i]), int(got_flags[i])) for i in bad[:6]], flush=True)
            out[f"tf32_{op}_sha256"] = hashlib.sha256(want.astype("<u4").tobytes()).hexdigest()
            out[f"tf32_{op}_flags_or"] = int(np.bitwise_or.reduce(want_flags))
    if not quick:
        np.savez_compressed(OUT, **out)


if __name__ == "__main__":
    main()
