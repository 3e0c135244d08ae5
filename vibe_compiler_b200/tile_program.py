"""Replay of the reference compiler's per-Tile target LLVM modules on the B200 backend.

`TileProgram` wraps the library's interpreter for the closed integer IR subset the reference admits for host
execution (lib/Wafer/Simulator/Invocation/TargetCallExecution.cpp:188-294): every `wafer_tx81_*` call of every Tile is
routed to a device executor where the reference routes it through waferTargetCallDispatch (:116-119) into its
functional model. Inputs and outputs are compact row-major arrays, like the reference's ProgramTensor files.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from . import _abi as abi
from .backend import B200TargetModelBackend, WB200Error



@dataclass
class ProgramTensor:
    format: int
    layout: int
    shape: tuple
    compact_bytes: int


@dataclass
class Command:
    tile: int
    name: str
    args: tuple
    operation: int = 0   # elementwise operation / convert opcode of the wafer_tx81_elementwise_* / convert_* families


def _stats(raw: abi.ProgramStats) -> dict:
    return {name: getattr(raw, name) for name, _ in abi.ProgramStats._fields_ }


class TileProgram:
    def __init__(self, modules: Sequence[str], backend: Optional[B200TargetModelBackend] = None, spm_bytes: int = 0):
        """`modules`: one LLVM-IR text per Tile, in any order (the Tile id comes from the module metadata).
        Without a backend the program can be inspected and traced, not run."""
        self._lib = abi.load()
        self._backend = backend   # keeps the backend alive
        texts = (C.c_char_p * len(modules))(*[m.encode() for m in modules])
        handle = C.c_void_p()
        status = self._lib.wb200_tile_program_load(backend._handle if backend else None, texts, len(modules), spm_bytes, C.byref(handle))
        if status != abi.OK:
            raise WB200Error(status, self._lib.wb200_last_error().decode())
        self._handle = handle
        if backend is not None:
            backend.adopt(self)
        n_in, n_out = C.c_uint32(), C.c_uint32()
        self._check(self._lib.wb200_tile_program_tensor_count(handle, C.byref(n_in), C.byref(n_out)))
        self.inputs = [self._info(0, i) for i in range(n_in.value)]
        self.outputs = [self._info(1, i) for i in range(n_out.value)]

    def _check(self, status: int):
        if status != abi.OK:
            raise WB200Error(status, self._lib.wb200_last_error().decode())

    def _info(self, is_output: int, index: int) -> ProgramTensor:
        desc, size = abi.TensorDesc(), C.c_uint64()
        self._check(self._lib.wb200_tile_program_tensor_info(self._handle, is_output, index, C.byref(desc), C.byref(size)))
        return ProgramTensor(desc.format, desc.layout, tuple(desc.shape[i] for i in range(desc.rank)), size.value)

    def placement(self, is_output: bool, index: int) -> dict:
        """DDR address and physical size the address plan gave an external tensor, plus the arena's base and size."""
        values = [C.c_uint64() for _ in range(4)]
        self._check(self._lib.wb200_tile_program_placement(self._handle, int(is_output), index, *[C.byref(v) for v in values]))
        return dict(zip(("address", "physical_bytes", "ddr_base", "ddr_bytes"), (v.value for v in values)))

    def close(self):
        if getattr(self, "_handle", None):
            self._lib.wb200_tile_program_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def trace(self):
        """Interprets every Tile without a device. Returns (commands in scheduling order, stats)."""
        count, stats = C.c_uint64(), abi.ProgramStats()
        self._check(self._lib.wb200_tile_program_trace(self._handle, None, 0, C.byref(count), C.byref(stats)))
        records = (abi.ProgramCommand * count.value)()
        self._check(self._lib.wb200_tile_program_trace(self._handle, records, count.value, C.byref(count), C.byref(stats)))
        names = {}
        commands: List[Command] = []
        for r in records:
            if r.kind not in names:
                names[r.kind] = self._lib.wb200_program_command_name(r.kind).decode()
            commands.append(Command(r.tile, names[r.kind], tuple(r.args[i] for i in range(r.argc)), r.operation))
        return commands, _stats(stats)

    def run(self, inputs: Sequence[np.ndarray], gemm_policy: int = abi.GEMM_FORMAL):
        """inputs: compact row-major arrays of the storage bits (uint16 for bf16 / f16, float32 / uint32 for f32).
        Returns (list of output bit arrays shaped like the program's outputs, stats)."""
        if len(inputs) != len(self.inputs):
            raise ValueError(f"the program takes {len(self.inputs)} inputs")
        held = []
        for array, info in zip(inputs, self.inputs):
            flat = np.ascontiguousarray(array).view(np.uint8).reshape(-1)
            if flat.size != info.compact_bytes:
                raise ValueError(f"input of {flat.size} bytes where the program expects {info.compact_bytes}")
            held.append(flat)
        outs = [np.empty(info.compact_bytes, dtype=np.uint8) for info in self.outputs]
        in_ptrs = (C.c_void_p * len(held))(*[a.ctypes.data for a in held])
        out_ptrs = (C.c_void_p * len(outs))(*[a.ctypes.data for a in outs])
        stats = abi.ProgramStats()
        self._check(self._lib.wb200_tile_program_run(self._handle, in_ptrs, out_ptrs, gemm_policy, C.byref(stats)))
        shaped = []
        for raw, info in zip(outs, self.outputs):
            elements = int(np.prod(info.shape)) if info.shape else 1
            width = info.compact_bytes // elements if elements and info.compact_bytes % elements == 0 else 1
            width = width if width in (1, 2, 4) else 1
            dtype = {1: np.uint8, 2: np.uint16, 4: np.uint32}[width]
            shaped.append(raw.view(dtype).reshape(info.shape))
        return shaped, _stats(stats)
