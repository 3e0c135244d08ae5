"""One Tile's scratch-pad image on the device and the `wafer_tx81_*` calls that execute on it.

`ScratchPad` is the host-side handle for the command-level seam (include/Wafer/Simulator/TargetCall.h:63-73): operands
live at byte addresses of a device-resident image, every method takes the arguments of the matching TargetCall
descriptor (lib/Wafer/Target/TargetCall.cpp:86-147) without the trailing NCC worker, and nothing is staged through the
host between calls. The Tile-program replayer drives the same entry points from the compiler's LLVM modules.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _abi as abi
from .backend import B200TargetModelBackend, WB200Error

POOL_KINDS = {"sum": 116, "max": 117, "min": 119}


class ScratchPad:
    def __init__(self, backend: B200TargetModelBackend, bytes: int = 3 << 20, base: int = 0):
        self._lib = abi.load()
        self._backend = backend
        handle = C.c_void_p()
        self._check(self._lib.wb200_spm_create(backend._handle, base, bytes, C.byref(handle)))
        self._handle = handle
        self.base, self.bytes = base, bytes
        backend.adopt(self)

    def _check(self, status: int):
        if status != abi.OK:
            raise WB200Error(status, self._lib.wb200_last_error().decode())

    def close(self):
        if getattr(self, "_handle", None):
            self._lib.wb200_spm_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def write(self, address: int, data: np.ndarray) -> None:
        flat = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        self._check(self._lib.wb200_spm_write(self._handle, address, flat.ctypes.data, flat.size))

    def read(self, address: int, bytes: int) -> np.ndarray:
        out = np.empty(bytes, dtype=np.uint8)
        self._check(self._lib.wb200_spm_read(self._handle, address, out.ctypes.data, bytes))
        return out

    def memset(self, destination: int, value_bits: int, element_count: int, format: int) -> None:
        self._check(self._lib.wb200_target_call_memset(self._handle, destination, value_bits, element_count, format))

    def gemm(self, lhs: int, rhs: int, dst: int, m: int, k: int, n: int, *, batch: int = 1, in_format: int = abi.BF16,
             out_format: int = abi.BF16, psum: int = 0, psum_format: int = abi.FORMAT_NONE, lhs_orientation: int = 0,
             rhs_orientation: int = 0, policy: int = abi.GEMM_FORMAL) -> None:
        self._check(self._lib.wb200_target_call_gemm(self._handle, lhs, rhs, dst, psum, m, k, n, batch, in_format, out_format,
                                                     psum_format, lhs_orientation, rhs_orientation, policy))

    def elementwise(self, operation: str, lhs: int, dst: int, count: int, format: int, *, rhs: Optional[int] = None,
                    rhs_unit_elements: int = 0, rhs_group_elements: int = 0, scalar_bits: Optional[int] = None,
                    numeric_result: bool = False) -> int:
        """`rhs` is an address; `scalar_bits` replaces it with an immediate. Returns the OR of the IEEE flags."""
        flags = C.c_uint32()
        second = scalar_bits if scalar_bits is not None else (rhs or 0)
        last = int(numeric_result) if operation in ("eq", "ne", "ge", "gt", "le", "lt") else rhs_group_elements
        self._check(self._lib.wb200_target_call_elementwise(self._handle, abi.ELEMENTWISE_OPS[operation], lhs, second, dst, count,
                                                            format, rhs_unit_elements, int(scalar_bits is not None), last,
                                                            C.byref(flags)))
        return flags.value

    def pool(self, kind: str, input: int, dst: int, source_shape: Sequence[int], destination_shape: Sequence[int],
             kernel_strides: Sequence[int], format: int, pads: Sequence[int] = (0, 0, 0, 0)) -> int:
        """`kernel_strides` = (kernel w, kernel h, stride w, stride h). Returns the OR of the IEEE flags."""
        four = lambda values: (C.c_uint32 * 4)(*[int(v) for v in values])
        flags = C.c_uint32()
        self._check(self._lib.wb200_target_call_pool(self._handle, POOL_KINDS.get(kind, 0) if isinstance(kind, str) else kind, input,
                                                     dst, four(source_shape), four(destination_shape), four(pads),
                                                     four(kernel_strides), format, C.byref(flags)))
        return flags.value

    def convert(self, opcode: int, source: int, destination: int, count: int, *, rounding_mode: int = 0, zero_point: int = 0) -> int:
        """`opcode`: a target convert route (139..174). Returns the OR of the IEEE flags; a refused element raises and
        leaves the destination untouched."""
        flags = C.c_uint32()
        self._check(self._lib.wb200_target_call_convert(self._handle, opcode, source, destination, count, zero_point, rounding_mode,
                                                        C.byref(flags)))
        return flags.value

    def reduce(self, operation: str, source: int, destination: int, dimension: str, nhwc: Sequence[int], format: int) -> int:
        """`operation`: "sum" | "max" | "min"; `dimension`: a key of _abi.REDUCE_DIMS. Returns the OR of the IEEE flags."""
        flags = C.c_uint32()
        shape = (C.c_uint32 * 4)(*[int(v) for v in nhwc])
        self._check(self._lib.wb200_target_call_reduce(self._handle, abi.REDUCE_OPS[operation], source, destination,
                                                       abi.REDUCE_DIMS[dimension], shape, format, C.byref(flags)))
        return flags.value

    def bit2fp(self, source: int, destination: int, count: int, format: int) -> None:
        """Packed Bool vector -> 1.0 / 0 of `format`."""
        self._check(self._lib.wb200_target_call_bit2fp(self._handle, source, destination, count, format))

    def mask_move(self, source: int, mask: int, destination: int, count: int, format: int) -> None:
        """destination[i] = source[i] where mask[i] is 1.0; a mask value other than 0 / 1.0 raises and writes nothing."""
        self._check(self._lib.wb200_target_call_mask_move(self._handle, source, mask, destination, count, format))
