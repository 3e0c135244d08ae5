"""TEST INFRASTRUCTURE ONLY - CPU restatement of the command semantics a Tile-program trace carries.

Executes, on numpy byte images, the command list the library's device-free trace produces
(wb200_tile_program_trace), following the reference's functional model:
  strided layouts / DMA / gather-scatter  lib/Wafer/Simulator/Memory/TargetModelStridedMemory.cpp:121-152,
                                          lib/Wafer/Simulator/Kernel/TargetModelMovement.cpp:52-146
  memset                                  lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:874-899
  GEMM command (Cx operands, f32 psum)    lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:662-872 with the
                                          formal arithmetic of Reference/Numeric/FormalTensorNumeric.cpp:271-361
  Direct-DTE payload copy                 lib/Wafer/Simulator/SystemC/SystemCTargetModel.cpp:1182-1200
  elementwise forms, convert              lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:288-464 with the
                                          exact-rational scalar oracles (formal_scalar.py, formal_convert.py)
Pinned by the end-to-end identity the shipped modules must satisfy: out == arg1 . arg0 of the source dot_general.
Only tests may import this module.
"""
from __future__ import annotations

import numpy as np

from . import binding

DDR_BASE = 0x10000000
FORMAT_NAMES = {2: "f16", 3: "bf16", 5: "f32"}
FORMAT_BYTES = {0: 1, 1: 2, 2: 2, 3: 2, 4: 4, 5: 4, 6: 4, 8: 1, 9: 2, 10: 4}
NO_PSUM = 13


def _offsets(inner, strides, iterations):
    """Byte offset of every segment, dimension 0 fastest."""
    i0, i1, i2 = (np.arange(n, dtype=np.int64) for n in iterations)
    return (i2[:, None, None] * strides[2] + i1[None, :, None] * strides[1] + i0[None, None, :] * strides[0]).reshape(-1)


def _gather(image, base, address, inner, strides, iterations):
    starts = _offsets(inner, strides, iterations) + (address - base)
    index = starts[:, None] + np.arange(inner, dtype=np.int64)[None, :]
    return image[index.reshape(-1)]


def _scatter(image, base, address, inner, strides, iterations, payload):
    starts = _offsets(inner, strides, iterations) + (address - base)
    index = starts[:, None] + np.arange(inner, dtype=np.int64)[None, :]
    image[index.reshape(-1)] = payload


ELEMENTWISE_NAMES = ["abs", "recip", "square", "sqrt", "rsqrt", "neg", "max", "min", "add", "sub", "mul", None, "eq", "ne", "ge", "gt", "le",
                     "lt", "logic_not", "logic_and", "logic_or", "logic_xor", "log2", "ln", "pow2", "exp", "exp_lp", "sin", "cos", "tanh",
                     "sigmoid", "relu", "satrelu", "leakyrelu", "softplus"]
_FUNCTIONS = ("sqrt", "rsqrt", "log2", "ln", "pow2", "exp", "sin", "cos", "tanh", "sigmoid", "softplus")
_BOOL = 7
_WORD = {1: np.uint8, 2: np.uint16, 4: np.uint32}


def _read_vector(image, address, fmt, count):
    if fmt == _BOOL:
        return np.unpackbits(image[address:address + (count + 7) // 8], bitorder="little")[:count].astype(np.uint64)
    width = FORMAT_BYTES[fmt]
    return image[address:address + count * width].view(_WORD[width]).astype(np.uint64)


def _write_vector(image, address, fmt, values):
    if fmt == _BOOL:
        count = len(values)
        bits = np.unpackbits(image[address:address + (count + 7) // 8], bitorder="little")
        bits[:count] = np.asarray(values, dtype=np.uint8)
        image[address:address + (count + 7) // 8] = np.packbits(bits, bitorder="little")
        return
    width = FORMAT_BYTES[fmt]
    image[address:address + len(values) * width] = np.asarray(values, dtype=_WORD[width]).view(np.uint8)


def _elementwise(image, c):
    """One wafer_tx81_elementwise_* record -> flags. Operand expansion follows TargetModelTensorNumeric.cpp:347-372."""
    from . import formal_scalar as F
    a, op = c.args, ELEMENTWISE_NAMES[c.operation]
    unary, full = c.name.endswith("_unary"), c.name.endswith("_binary")
    rhs_at, dst_at, count, fmt = (0, a[1], a[2], a[3]) if unary else (a[1], a[2], a[3], a[4])
    unit, scalar, last = (a[5], a[6], a[7]) if full else (0, 0, 0)
    relation = op in ("eq", "ne", "ge", "gt", "le", "lt")
    logic = op.startswith("logic_")
    out_fmt = _BOOL if logic or (relation and not last) else fmt
    name = lambda f: "bool" if f == _BOOL else FORMAT_NAMES[f]
    lhs = _read_vector(image, a[0], fmt, count)
    if unary:
        rhs = np.zeros(count, dtype=np.uint64)
    elif scalar:
        rhs = np.full(count, rhs_at, dtype=np.uint64)
    elif not relation and last:
        rows = _read_vector(image, rhs_at, fmt, count)
        rhs = np.array([rows[i // last * 64 + i % 64] for i in range(count)], dtype=np.uint64)
    elif unit:
        rhs = np.resize(_read_vector(image, rhs_at, fmt, unit), count)
    else:
        rhs = _read_vector(image, rhs_at, fmt, count)
    out, flags = [], 0
    for x, y in zip(lhs, rhs):
        bits, f = F.evaluate_function(op, name(fmt), int(x)) if op in _FUNCTIONS else F.evaluate(op, name(fmt), name(out_fmt), int(x), int(y))
        out.append(bits)
        flags |= f
    _write_vector(image, dst_at, out_fmt, out)
    return flags


def _convert(image, c):
    from . import formal_convert as K
    a = c.args
    _, source, destination, _ = K.ROUTES[c.operation]
    codes = {"i8": 0, "i16": 1, "i32": 4, "f16": 2, "bf16": 3, "f32": 5, "tf32": 6}
    values = _read_vector(image, a[0], codes[source], a[2])
    out, flags = [], 0
    for x in values:
        bits, f = K.convert(c.operation, a[4], int(x))
        out.append(bits)
        flags |= f
    _write_vector(image, a[1], codes[destination], out)
    return flags


def _reduce(image, c):
    """One wafer_tx81_reduce record (NCx in and out) -> flags; the fold of FormalTensorNumeric.cpp:363-425."""
    from . import formal_scalar as F
    a = c.args
    shape, fmt = [int(v) for v in a[3:7]], FORMAT_NAMES[a[7]]
    reduced = {0: (3,), 1: (2,), 2: (1,), 3: (0,), 4: (1, 2), 5: (1, 2, 3)}[a[2]]
    out_shape = [1 if d in reduced else e for d, e in enumerate(shape)]
    size = binding.geometry(fmt, "ncx", shape)["physical_bytes"]
    compact = binding.unpack(fmt, "ncx", shape, image[a[0]:a[0] + size]).reshape(-1)
    infinity = {"f16": 0x7c00, "bf16": 0x7f80, "f32": 0x7f800000}[fmt]
    identity = {0: 0, 1: infinity | (0x80000000 if fmt == "f32" else 0x8000), 2: infinity}[c.operation]
    op = {0: "add", 1: "max", 2: "min"}[c.operation]
    out = [identity] * int(np.prod(out_shape))
    kept_shape = [e for d, e in enumerate(shape) if d not in reduced]
    flags = 0
    for index, bits in enumerate(compact):
        coordinates = np.unravel_index(index, shape)
        kept = [x for d, x in enumerate(coordinates) if d not in reduced]
        destination = int(np.ravel_multi_index(kept, kept_shape)) if kept else 0
        out[destination], f = F.evaluate(op, fmt, fmt, int(out[destination]), int(bits))
        flags |= f
    out_size = binding.geometry(fmt, "ncx", out_shape)["physical_bytes"]
    packed = binding.pack(fmt, "ncx", out_shape, np.array(out, dtype=compact.dtype), image[a[1]:a[1] + out_size].copy())
    image[a[1]:a[1] + out_size] = packed
    return flags


def _pool(image, c):
    """One wafer_tx81_pool record (NCx in and out, no padding) -> flags; the (kh, kw) fold of
    lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:466-583: max / min start from the first tap, sum from +0."""
    from . import formal_scalar as F
    a = c.args
    source_shape, destination_shape = [int(v) for v in a[3:7]], [int(v) for v in a[7:11]]
    kernel_w, kernel_h, stride_w, stride_h = (int(v) for v in a[15:19])
    fmt, op = FORMAT_NAMES[a[19]], {116: "add", 117: "max", 119: "min"}[c.operation]
    if any(a[11:15]):
        raise ValueError("plain pooling requires explicit input padding")
    size = binding.geometry(fmt, "ncx", source_shape)["physical_bytes"]
    compact = binding.unpack(fmt, "ncx", source_shape, image[a[0]:a[0] + size]).reshape(source_shape)
    out, flags = np.zeros(destination_shape, dtype=compact.dtype), 0
    for n, h, w, ch in np.ndindex(*destination_shape):
        result = 0
        for kh in range(kernel_h):
            for kw in range(kernel_w):
                tap = int(compact[n, h * stride_h + kh, w * stride_w + kw, ch])
                if kh == 0 and kw == 0 and op != "add":
                    result = tap
                else:
                    result, f = F.evaluate(op, fmt, fmt, result, tap)
                    flags |= f
        out[n, h, w, ch] = result
    out_size = binding.geometry(fmt, "ncx", destination_shape)["physical_bytes"]
    image[a[1]:a[1] + out_size] = binding.pack(fmt, "ncx", destination_shape, out.reshape(-1), image[a[1]:a[1] + out_size].copy())
    return flags


def replay(commands, ddr: np.ndarray, tile_count: int, spm_bytes: int = 3 << 20, threads: int = 1, report: dict = None):
    """commands: iterable of objects with .tile, .name, .args (the library's trace). `ddr` is the DDR arena (uint8,
    address DDR_BASE at index 0) with the inputs already in place; it is updated in place."""
    spm = [np.zeros(spm_bytes, dtype=np.uint8) for _ in range(tile_count)]
    numeric_flags = 0
    for c in commands:
        a, name = c.args, c.name
        if name.startswith("wafer_tx81_elementwise_"):
            numeric_flags |= _elementwise(spm[c.tile], c)
        elif name == "wafer_tx81_convert":
            numeric_flags |= _convert(spm[c.tile], c)
        elif name == "wafer_tx81_reduce":
            numeric_flags |= _reduce(spm[c.tile], c)
        elif name == "wafer_tx81_pool":
            numeric_flags |= _pool(spm[c.tile], c)
        elif name == "wafer_tx81_bit2fp":      # TargetModelTensorNumeric.cpp:198-236
            one = {2: 0x3c00, 3: 0x3f80, 5: 0x3f800000}[a[3]]
            bits = _read_vector(spm[c.tile], a[0], _BOOL, a[2])
            _write_vector(spm[c.tile], a[1], a[3], [one if b else 0 for b in bits])
        elif name == "wafer_tx81_mask_move":   # :238-286
            one = {2: 0x3c00, 3: 0x3f80, 5: 0x3f800000}[a[4]]
            source, mask = _read_vector(spm[c.tile], a[0], a[4], a[3]), _read_vector(spm[c.tile], a[1], a[4], a[3])
            destination = _read_vector(spm[c.tile], a[2], a[4], a[3])
            if any(m not in (0, one) for m in mask):
                raise ValueError("MaskMove requires canonical zero/one mask values")
            _write_vector(spm[c.tile], a[2], a[4], [x if m == one else d for x, m, d in zip(source, mask, destination)])
        elif name in ("wafer_tx81_rdma", "wafer_tx81_wdma"):
            inner, strides, iterations = a[3], a[4:7], a[7:10]
            segments = int(np.prod(iterations))
            assert inner * segments == a[2]
            if name == "wafer_tx81_rdma":
                spm[c.tile][a[1]:a[1] + a[2]] = _gather(ddr, DDR_BASE, a[0], inner, strides, iterations)
            else:
                _scatter(ddr, DDR_BASE, a[1], inner, strides, iterations, spm[c.tile][a[0]:a[0] + a[2]].copy())
        elif name == "wafer_tx81_gather_scatter":
            payload = _gather(spm[c.tile], 0, a[0], a[3], a[4:7], a[7:10])   # snapshot first
            _scatter(spm[c.tile], 0, a[1], a[3], a[10:13], a[13:16], payload)
        elif name == "wafer_tx81_memset":
            width = FORMAT_BYTES[a[3]]
            value = np.array([a[1] & ((1 << (8 * width)) - 1)], dtype={1: np.uint8, 2: np.uint16, 4: np.uint32}[width])
            spm[c.tile][a[0]:a[0] + a[2] * width] = np.tile(value.view(np.uint8), a[2])
        elif name == "direct_dte_transfer":
            spm[a[1]][a[3]:a[3] + a[4]] = spm[a[0]][a[2]:a[2] + a[4]]
        elif name in ("wafer_tx81_gemm", "wafer_tx81_gemm_oriented"):
            lhs_at, rhs_at, dst_at, psum_at, m, k, n, batch, in_fmt, out_fmt, psum_fmt = a[:11]
            lt, rt = (a[11], a[12]) if name.endswith("oriented") else (0, 0)
            fin, fout = FORMAT_NAMES[in_fmt], FORMAT_NAMES[out_fmt]
            layout = "cx" if batch == 1 else "ncx"
            lead = [] if batch == 1 else [batch]
            image = spm[c.tile]

            def load(address, fmt, rows, cols):
                shape = lead + [rows, cols]
                size = binding.geometry(fmt, layout, shape)["physical_bytes"]
                return binding.unpack(fmt, layout, shape, image[address:address + size])
            lhs = load(lhs_at, fin, k if lt else m, m if lt else k)
            rhs = load(rhs_at, fin, n if rt else k, k if rt else n)
            psum = None if psum_fmt == NO_PSUM else load(psum_at, "f32", m, n).view(np.uint32)
            out = binding.formal_gemm(fin, fout, batch, m, k, n, lhs, rhs, psum, bool(lt), bool(rt), threads=threads)
            shape = lead + [m, n]
            size = binding.geometry(fout, layout, shape)["physical_bytes"]
            image[dst_at:dst_at + size] = binding.pack(fout, layout, shape, out, image[dst_at:dst_at + size].copy())
        # joins, Direct-DTE lifecycle, prepares and waits carry no data
    if report is not None:
        report["numeric_flags"] = numeric_flags   # OR of the IEEE flags of the elementwise / convert commands
    return ddr
