"""Host-side mirror of the reference's numeric-backend interface over the libwb200 C ABI.

`B200TargetModelBackend` plays the role of the reference's `ManagedReferenceTargetModelBackend`
(include/Wafer/Simulator/Reference/TargetNumericBackend.h:55-87): `try_execute` for GEMM requests
(TargetModelOneDNNBackend::tryExecute) and `execute` for convert / elementwise / reduce requests
(TargetModelManagedReferenceBackend::execute), all on physical storage bytes. The region-level
methods (`attention_fa`, `attention_fd`, `gemm_epilogue`) run what a chain of lowered commands
computes as a whole. Every method calls the device library; nothing is computed in Python.
"""
from __future__ import annotations

import ctypes as C
import weakref
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from . import _abi as abi


class WB200Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"wb200 {abi.STATUS_NAMES[status] if status < len(abi.STATUS_NAMES) else status}: {message}")
        self.status = status
        self.message = message


_TORCH_FORMATS = {torch.bfloat16: abi.BF16, torch.float16: abi.F16, torch.float32: abi.F32}
FORMAT_BYTES = {abi.F16: 2, abi.BF16: 2, abi.F32: 4}


@dataclass
class PhysicalTensorDescriptor:
    """Mirror of wafer::PhysicalTensorDescriptor {format, layout, shape}."""
    format: int
    layout: int
    shape: Sequence[int]

    def c(self) -> abi.TensorDesc:
        return abi.make_desc(self.format, self.layout, self.shape)

    @property
    def element_count(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) if len(self.shape) else 1


@dataclass
class NumericTensor:
    """Mirror of TargetModelNumericTensor {key, storage}; storage is the full physical byte image."""
    key: PhysicalTensorDescriptor
    storage: np.ndarray  # uint8


@dataclass
class FormalGemmOperation:
    lhs: PhysicalTensorDescriptor
    rhs: PhysicalTensorDescriptor
    destination: PhysicalTensorDescriptor
    m: int
    k: int
    n: int
    batch_count: int = 1
    lhs_orientation: int = abi.NORMAL
    rhs_orientation: int = abi.NORMAL
    psum: Optional[PhysicalTensorDescriptor] = None


@dataclass
class Evidence:
    matmul_invocations: int = 0
    reorder_invocations: int = 0
    formal_fused_multiply_adds: int = 0
    scalar_evaluations: int = 0
    evidence_kind: int = 0
    flags: int = 0
    gpu_launches: int = 0
    digest: str = ""
    implementation: str = ""
    device_us: int = 0   # device time of the call's kernels (tensor commands only)


@dataclass
class BackendResult:
    destination: NumericTensor
    evidence: Evidence = field(default_factory=Evidence)


def _evidence(e: abi.Evidence) -> Evidence:
    return Evidence(e.matmul_invocations, e.reorder_invocations, e.formal_fused_multiply_adds, e.scalar_evaluations,
                    e.evidence_kind, e.flags, e.gpu_launches, e.digest.decode(), e.implementation.decode(), e.device_us)


def _u8(array: np.ndarray) -> np.ndarray:
    out = np.ascontiguousarray(array).view(np.uint8).reshape(-1)
    return out


def _ptr(array: Optional[np.ndarray]) -> Optional[int]:
    return None if array is None else array.ctypes.data


class B200TargetModelBackend:
    def __init__(self, device: int = 0):
        self._lib = abi.load()
        handle = C.c_void_p()
        status = self._lib.wb200_backend_create(device, C.byref(handle))
        if status != abi.OK:
            raise WB200Error(status, self._lib.wb200_last_error().decode())
        self._handle = handle
        self.device = device
        self._dependents = weakref.WeakSet()   # objects holding device state of this backend (images, programs)

    def adopt(self, dependent) -> None:
        """Registers an object whose `close()` must run before the backend is destroyed (finalisers of one garbage
        cycle run in no particular order)."""
        self._dependents.add(dependent)

    def close(self):
        if getattr(self, "_handle", None):
            for dependent in list(getattr(self, "_dependents", ())):
                dependent.close()
            self._lib.wb200_backend_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, status: int):
        if status != abi.OK:
            raise WB200Error(status, self._lib.wb200_last_error().decode())

    @property
    def launch_count(self) -> int:
        return int(self._lib.wb200_backend_launch_count(self._handle))

    def set_budget(self, max_total_bytes: int = 0, max_scratch_bytes: int = 0):
        self._check(self._lib.wb200_backend_set_budget(self._handle, max_total_bytes, max_scratch_bytes))

    def selftest_bounded_wait(self, cycle_limit: int) -> int:
        """Runs a kernel whose wait can never be satisfied, with a limit of `cycle_limit` SM clocks; returns the clocks it
        waited. The next poll() raises WB200Error(ERR_DEVICE_TIMEOUT)."""
        waited = C.c_uint64()
        self._check(self._lib.wb200_selftest_bounded_wait(self._handle, cycle_limit, C.byref(waited)))
        return waited.value

    def poll(self, stream: int = 0):
        self._check(self._lib.wb200_backend_poll(self._handle, C.c_void_p(stream)))

    # ------------------------------------------------------------------ layout / codec
    @staticmethod
    def physical_bytes(key: PhysicalTensorDescriptor) -> int:
        lib = abi.load()
        out = C.c_uint64()
        desc = key.c()
        status = lib.wb200_physical_bytes(C.byref(desc), C.byref(out))
        if status != abi.OK:
            raise WB200Error(status, lib.wb200_last_error().decode())
        return out.value

    @staticmethod
    def geometry(key: PhysicalTensorDescriptor) -> dict:
        lib = abi.load()
        geo = abi.Geometry()
        desc = key.c()
        status = lib.wb200_physical_geometry(C.byref(desc), C.byref(geo))
        if status != abi.OK:
            raise WB200Error(status, lib.wb200_last_error().decode())
        return {name: getattr(geo, name) for name, _ in abi.Geometry._fields_}

    def unpack(self, tensor: NumericTensor) -> np.ndarray:
        """Physical storage -> compact row-major bytes (uint8)."""
        desc = tensor.key.c()
        storage = _u8(tensor.storage)
        compact = np.empty(tensor.key.element_count * FORMAT_BYTES.get(tensor.key.format, 0) or
                           self.geometry(tensor.key)["compact_bytes"], dtype=np.uint8)
        self._check(self._lib.wb200_unpack(self._handle, C.byref(desc), storage.ctypes.data, storage.size,
                                           compact.ctypes.data, compact.size))
        return compact

    def pack(self, key: PhysicalTensorDescriptor, compact: np.ndarray, template: np.ndarray) -> np.ndarray:
        desc = key.c()
        compact = _u8(compact)
        template = _u8(template)
        out = np.empty_like(template)
        self._check(self._lib.wb200_pack(self._handle, C.byref(desc), compact.ctypes.data, compact.size,
                                         template.ctypes.data, out.ctypes.data, out.size))
        return out

    # ------------------------------------------------------------------ command level
    def try_execute(self, operation: FormalGemmOperation, lhs: NumericTensor, rhs: NumericTensor,
                    destination_template: NumericTensor, psum: Optional[NumericTensor] = None,
                    policy: int = abi.GEMM_TENSOR) -> Optional[BackendResult]:
        """GEMM request. Returns None when the request is outside the tensor backend's domain
        (the reference's successful null optional); raises WB200Error on failure."""
        req = abi.GemmRequest()
        req.lhs, req.rhs, req.destination = operation.lhs.c(), operation.rhs.c(), operation.destination.c()
        req.m, req.k, req.n, req.batch_count = operation.m, operation.k, operation.n, operation.batch_count
        req.lhs_orientation, req.rhs_orientation = operation.lhs_orientation, operation.rhs_orientation
        req.policy = policy
        lhs_s, rhs_s, tmpl = _u8(lhs.storage), _u8(rhs.storage), _u8(destination_template.storage)
        out = np.empty_like(tmpl)
        req.lhs_storage, req.lhs_bytes = lhs_s.ctypes.data, lhs_s.size
        req.rhs_storage, req.rhs_bytes = rhs_s.ctypes.data, rhs_s.size
        req.destination_template, req.destination_out, req.destination_bytes = tmpl.ctypes.data, out.ctypes.data, tmpl.size
        psum_s = None
        if operation.psum is not None:
            if psum is None:
                raise ValueError("operation has a psum descriptor but no psum tensor was given")
            psum_s = _u8(psum.storage)
            req.has_psum = 1
            req.psum = operation.psum.c()
            req.psum_storage, req.psum_bytes = psum_s.ctypes.data, psum_s.size
        handled = C.c_int(0)
        evidence = abi.Evidence()
        self._check(self._lib.wb200_gemm(self._handle, C.byref(req), C.byref(handled), C.byref(evidence)))
        if not handled.value:
            return None
        return BackendResult(NumericTensor(operation.destination, out), _evidence(evidence))

    def execute_elementwise(self, operation: str, inputs: Sequence[NumericTensor], destination_template: NumericTensor,
                            max_scalar_evaluations: int = 2 ** 62, formal: bool = False) -> BackendResult:
        """Managed-reference elementwise (NaN rejected, flags zero) or, with formal=True, the bit-exact formal family
        (relations, logic, NaN canonicalisation, IEEE flags in evidence.flags)."""
        req = abi.ElementwiseRequest()
        req.operation = abi.ELEMENTWISE_OPS[operation]
        req.input_count = len(inputs)
        keep = []
        for i, tensor in enumerate(inputs[:2]):
            storage = _u8(tensor.storage)
            keep.append(storage)
            req.inputs[i] = tensor.key.c()
            req.input_storage[i] = storage.ctypes.data
            req.input_bytes[i] = storage.size
        tmpl = _u8(destination_template.storage)
        out = tmpl.copy()
        req.destination = destination_template.key.c()
        req.destination_template, req.destination_out, req.destination_bytes = tmpl.ctypes.data, out.ctypes.data, tmpl.size
        req.max_scalar_evaluations = max_scalar_evaluations
        evidence = abi.Evidence()
        entry = self._lib.wb200_elementwise_formal if formal else self._lib.wb200_elementwise
        self._check(entry(self._handle, C.byref(req), C.byref(evidence)))
        return BackendResult(NumericTensor(destination_template.key, out), _evidence(evidence))

    def execute_convert(self, opcode: int, source: NumericTensor, destination_template: NumericTensor,
                        rounding_mode: int = 0, max_scalar_evaluations: int = 2 ** 62, formal: bool = False) -> BackendResult:
        """`formal` selects the bit-exact scalar conversion with the four rounding modes, integer routes and IEEE flags
        (wb200_convert_formal) instead of the managed nearest-even floating routes."""
        req = abi.ConvertRequest()
        req.opcode, req.rounding_mode = opcode, rounding_mode
        src, tmpl = _u8(source.storage), _u8(destination_template.storage)
        out = tmpl.copy()
        req.source, req.destination = source.key.c(), destination_template.key.c()
        req.source_storage, req.source_bytes = src.ctypes.data, src.size
        req.destination_template, req.destination_out, req.destination_bytes = tmpl.ctypes.data, out.ctypes.data, tmpl.size
        req.max_scalar_evaluations = max_scalar_evaluations
        evidence = abi.Evidence()
        entry = self._lib.wb200_convert_formal if formal else self._lib.wb200_convert
        self._check(entry(self._handle, C.byref(req), C.byref(evidence)))
        return BackendResult(NumericTensor(destination_template.key, out), _evidence(evidence))

    def execute_reduce(self, operation: str, dimension: str, source: NumericTensor, destination_template: NumericTensor,
                       max_scalar_evaluations: int = 2 ** 62, formal: bool = False) -> BackendResult:
        req = abi.ReduceRequest()
        req.operation, req.dimension = abi.REDUCE_OPS[operation], abi.REDUCE_DIMS[dimension]
        src, tmpl = _u8(source.storage), _u8(destination_template.storage)
        out = tmpl.copy()
        req.input, req.destination = source.key.c(), destination_template.key.c()
        req.input_storage, req.input_bytes = src.ctypes.data, src.size
        req.destination_template, req.destination_out, req.destination_bytes = tmpl.ctypes.data, out.ctypes.data, tmpl.size
        req.max_scalar_evaluations = max_scalar_evaluations
        evidence = abi.Evidence()
        entry = self._lib.wb200_reduce_formal if formal else self._lib.wb200_reduce
        self._check(entry(self._handle, C.byref(req), C.byref(evidence)))
        return BackendResult(NumericTensor(destination_template.key, out), _evidence(evidence))

    # ------------------------------------------------------------------ region level
    def _attention_params(self, q, k, v, out, scale, causal, zero_fully_masked, query_start, key_start, key_end,
                          lse, row_max, row_sum, stream) -> abi.AttentionParams:
        for name, tensor in (("q", q), ("k", k), ("v", v)):
            if tensor.dim() != 4 or not tensor.is_contiguous():
                raise ValueError(f"{name} must be a contiguous [batch, heads, length, head_dim] tensor")
        if q.dtype not in _TORCH_FORMATS or k.dtype != q.dtype or v.dtype != q.dtype or out.dtype != q.dtype:
            raise ValueError("q, k, v and out must share one of bfloat16 / float16 / float32")
        on_device = q.is_cuda
        for tensor in (k, v, out, lse, row_max, row_sum):
            if tensor is not None and tensor.is_cuda != on_device:
                raise ValueError("all attention buffers must live in the same memory space")
        p = abi.AttentionParams()
        p.batch, p.q_heads, p.q_len, p.head_dim = q.shape
        p.kv_heads, p.kv_len = k.shape[1], k.shape[2]
        p.format = _TORCH_FORMATS[q.dtype]
        p.causal, p.zero_fully_masked = int(causal), int(zero_fully_masked)
        p.memory = abi.MEM_DEVICE if on_device else abi.MEM_HOST
        p.scale = float(scale)
        p.query_start, p.key_start, p.key_end = int(query_start), int(key_start), int(key_end)
        p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
        p.lse = lse.data_ptr() if lse is not None else None
        p.row_max = row_max.data_ptr() if row_max is not None else None
        p.row_sum = row_sum.data_ptr() if row_sum is not None else None
        p.stream = stream
        return p

    def attention_fa(self, q, k, v, scale: float, causal: bool = False, *, out=None, lse=None, row_max=None,
                     row_sum=None, zero_fully_masked: bool = False, query_start: int = 0, key_start: int = 0,
                     key_end: int = 0, stream: Optional[int] = None, token_major_out: bool = False):
        """Flash-attention prefill. CPU tensors are staged by the library (copies inside the call);
        CUDA tensors are used in place and the kernel is enqueued on `stream` (default: current)."""
        if out is None:
            out = torch.empty(q.shape[0], q.shape[2], q.shape[1], q.shape[3], dtype=q.dtype, device=q.device) if token_major_out \
                else torch.empty_like(q)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream if q.is_cuda else 0
        p = self._attention_params(q, k, v, out, scale, causal, zero_fully_masked, query_start, key_start, key_end,
                                   lse, row_max, row_sum, stream)
        p.out_layout = abi.OUT_TOKEN_MAJOR if token_major_out else abi.OUT_HEAD_MAJOR
        self._check(self._lib.wb200_attention_fa(self._handle, C.byref(p)))
        return out

    def attention_fd(self, q, k, v, scale: float, *, kv_splits: int = 0, out=None, lse=None, row_max=None,
                     row_sum=None, zero_fully_masked: bool = False, causal: bool = False, query_start: int = 0,
                     key_start: int = 0, key_end: int = 0, stream: Optional[int] = None):
        if out is None:
            out = torch.empty_like(q)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream if q.is_cuda else 0
        p = self._attention_params(q, k, v, out, scale, causal, zero_fully_masked, query_start, key_start, key_end,
                                   lse, row_max, row_sum, stream)
        self._check(self._lib.wb200_attention_fd(self._handle, C.byref(p), kv_splits))
        return out

    def attention_fd_static(self, q, k, v, scale: float, *, kv_splits: int = 0, out=None, lse=None,
                            zero_fully_masked: bool = False, stream: Optional[int] = None):
        """Flash-decoding without any allocation inside the call (CUDA tensors only; `out` should be
        passed by callers that must not allocate either). The split-KV partial records use a fixed
        16 MiB array inside the library, shared by all calls: do not overlap two such calls on the GPU.
        Raises WB200Error (limit) when batch * q_heads * kv_splits * (head_dim + 2) exceeds 4 Mi floats."""
        if not q.is_cuda:
            raise ValueError("attention_fd_static takes CUDA tensors")
        if out is None:
            out = torch.empty_like(q)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        p = self._attention_params(q, k, v, out, scale, False, zero_fully_masked, 0, 0, 0, lse, None, None, stream)
        self._check(self._lib.wb200_attention_fd_static(self._handle, C.byref(p), kv_splits))
        return out

    def attention_fd_partial(self, q, k, v, scale: float, *, kv_splits: int = 0, state=None, key_start: int = 0,
                             key_end: int = 0, stream: Optional[int] = None):
        """One sequence shard's un-finalized (acc[D], m, l) state, [batch, q_heads, D + 2] float32."""
        if state is None:
            state = torch.empty(q.shape[0], q.shape[1], q.shape[3] + 2, dtype=torch.float32, device=q.device)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream if q.is_cuda else 0
        dummy_out = q  # not written
        p = self._attention_params(q, k, v, dummy_out, scale, False, False, 0, key_start, key_end, None, None, None, stream)
        self._check(self._lib.wb200_attention_fd_partial(self._handle, C.byref(p), kv_splits, state.data_ptr()))
        return state

    def fd_exchange_bytes(self, batch: int, q_heads: int, world: int) -> int:
        return int(self._lib.wb200_fd_exchange_bytes(batch, q_heads, world))

    def attention_fd_exchange(self, q, k, v, scale: float, *, rank: int, peer_pointers: Sequence[int], epoch: torch.Tensor,
                              kv_splits: int = 0, out=None, lse=None, stream: Optional[int] = None):
        """Sequence-sharded decode step of this rank (its KV shard in k, v) with the state exchange and the merge inside the
        kernel. `peer_pointers[r]` is rank r's exchange buffer as addressable from this GPU; `epoch` a zeroed int32[2]."""
        if out is None:
            out = torch.empty_like(q)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        p = self._attention_params(q, k, v, out, scale, False, False, 0, 0, 0, lse, None, None, stream)
        x = abi.FdExchange()
        x.rank, x.world = rank, len(peer_pointers)
        for r, pointer in enumerate(peer_pointers):
            x.peer_buffers[r] = pointer
        x.epoch = epoch.data_ptr()
        self._check(self._lib.wb200_attention_fd_exchange(self._handle, C.byref(p), kv_splits, C.byref(x)))
        return out

    def decoder_layer_timeline(self):
        """Device timeline of the last micro-batched decoder_layer call: a dict with, per part, the milliseconds (from the
        call's first kernel) at which each phase's partial sum was ready and its sum over shards was done, and `end`."""
        count = C.c_uint32(0)
        self._check(self._lib.wb200_decoder_layer_timeline(self._handle, None, 0, C.byref(count)))
        if count.value == 0:
            return None
        ms = (C.c_float * count.value)()
        self._check(self._lib.wb200_decoder_layer_timeline(self._handle, ms, count.value, C.byref(count)))
        parts = (count.value - 1) // 4
        return {"parts": [{"attention_ready": ms[4 * i], "attention_sum_done": ms[4 * i + 1], "ffn_ready": ms[4 * i + 2],
                           "ffn_sum_done": ms[4 * i + 3]} for i in range(parts)], "end": ms[4 * parts]}

    def switch_sum_signal_bytes(self, world: int) -> int:
        return int(self._lib.wb200_switch_sum_signal_bytes(world))

    def switch_sum(self, multicast_pointer: int, elements: int, dtype, *, rank: int, signal_pointers: Sequence[int],
                   epoch: torch.Tensor, blocks: int = 0, stream: Optional[int] = None, multicast_out: int = 0,
                   residual: Optional[torch.Tensor] = None) -> None:
        """In-place sum over the ranks of the buffer at `multicast_pointer` (an NVLink multicast address of a symmetric
        allocation) by one kernel per GPU: the switch adds and broadcasts (wb200_switch_sum). `signal_pointers[r]` are
        rank r's signal words as addressable from this GPU; `epoch` a zeroed int32[2] of this rank. `multicast_out`: store
        the sums there instead of in place; `residual`: this rank's copy of a tensor (identical on every rank) that is
        added to the sums before the store."""
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        x = abi.SwitchSumParams()
        x.rank, x.world = rank, len(signal_pointers)
        x.multicast, x.elements, x.format, x.blocks = multicast_pointer, elements, _TORCH_FORMATS[dtype], blocks
        for r, pointer in enumerate(signal_pointers):
            x.signals[r] = pointer
        x.epoch, x.stream = epoch.data_ptr(), stream
        x.multicast_out = multicast_out or None
        x.residual = residual.data_ptr() if residual is not None else None
        self._check(self._lib.wb200_switch_sum(self._handle, C.byref(x)))

    def attention_fd_merge(self, states, like_q, *, out=None, lse=None, zero_fully_masked: bool = False,
                           stream: Optional[int] = None):
        """Left-folds [shards, batch, q_heads, D + 2] states in ascending shard order and finalizes."""
        if out is None:
            out = torch.empty_like(like_q)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream if like_q.is_cuda else 0
        p = abi.AttentionParams()
        p.batch, p.q_heads, p.q_len, p.head_dim = like_q.shape
        p.kv_heads, p.kv_len = 1, 1
        p.format = _TORCH_FORMATS[like_q.dtype]
        p.zero_fully_masked = int(zero_fully_masked)
        p.memory = abi.MEM_DEVICE if like_q.is_cuda else abi.MEM_HOST
        p.out = out.data_ptr()
        p.lse = lse.data_ptr() if lse is not None else None
        p.stream = stream
        states = states.contiguous()
        self._check(self._lib.wb200_attention_fd_merge(self._handle, C.byref(p), states.data_ptr(), states.shape[0]))
        return out

    def gemm_epilogue(self, a, b, bias=None, *, epilogue: int = abi.EPI_NONE, out_dtype=None, out=None,
                      lhs_transposed: bool = False, rhs_transposed: bool = False, stream: Optional[int] = None):
        """out = epilogue(A x B): A[m,k] (or [k,m] transposed), B[k,n] (or [n,k] transposed)."""
        if a.dtype not in (torch.bfloat16, torch.float16) or b.dtype != a.dtype:
            raise ValueError("a and b must both be bfloat16 or float16")
        m, k = (a.shape[1], a.shape[0]) if lhs_transposed else a.shape
        n = b.shape[0] if rhs_transposed else b.shape[1]
        out_dtype = out_dtype or a.dtype
        if out is None:
            out = torch.empty(m, n // 2 if epilogue == abi.EPI_SWIGLU else n, dtype=out_dtype, device=a.device)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream if a.is_cuda else 0
        p = abi.GemmEpilogueParams()
        p.m, p.n, p.k = m, n, k
        p.in_format, p.out_format = _TORCH_FORMATS[a.dtype], _TORCH_FORMATS[out.dtype]
        p.lhs_orientation, p.rhs_orientation = int(lhs_transposed), int(rhs_transposed)
        p.epilogue = epilogue
        p.memory = abi.MEM_DEVICE if a.is_cuda else abi.MEM_HOST
        p.a, p.b, p.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
        p.bias = bias.data_ptr() if bias is not None else None
        p.stream = stream
        self._check(self._lib.wb200_gemm_epilogue(self._handle, C.byref(p)))
        return out

    # ------------------------------------------------------------------ decoder-layer pieces (CUDA tensors)
    def rmsnorm(self, x, gamma, eps: float, *, out=None, stream: Optional[int] = None):
        """y = round(round(x * rsqrt(mean(x^2) + eps)) * gamma) over the last dimension."""
        if out is None:
            out = torch.empty_like(x)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        rows = x.numel() // x.shape[-1]
        self._check(self._lib.wb200_rmsnorm(self._handle, _TORCH_FORMATS[x.dtype], x.data_ptr(), gamma.data_ptr(), out.data_ptr(),
                                            rows, x.shape[-1], float(eps), stream))
        return out

    def rope_split(self, qkv, batch: int, seq: int, q_heads: int, kv_heads: int, head_dim: int, theta: float,
                   position_offset: int = 0, stream: Optional[int] = None):
        """Token-major projection rows [q heads | k heads | v heads] -> head-major Q, K (rotary applied) and V."""
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        q = torch.empty(batch, q_heads, seq, head_dim, dtype=qkv.dtype, device=qkv.device)
        k = torch.empty(batch, kv_heads, seq, head_dim, dtype=qkv.dtype, device=qkv.device)
        v = torch.empty_like(k)
        self._check(self._lib.wb200_rope_split(self._handle, _TORCH_FORMATS[qkv.dtype], qkv.data_ptr(), q.data_ptr(), k.data_ptr(),
                                               v.data_ptr(), batch, seq, q_heads, kv_heads, head_dim, float(theta), position_offset, stream))
        return q, k, v

    def residual_add(self, a, b, *, out=None, stream: Optional[int] = None):
        if out is None:
            out = torch.empty_like(a)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        self._check(self._lib.wb200_residual_add(self._handle, _TORCH_FORMATS[a.dtype], a.data_ptr(), b.data_ptr(), out.data_ptr(),
                                                 a.numel(), stream))
        return out

    def decoder_layer(self, x, *, norm1, wqkv, wo, norm2, wgu, wdown, q_heads: int, kv_heads: int, head_dim: int, eps: float,
                      rope_theta: float, position_offset: int = 0, allreduce=None, workspace=None, out=None,
                      micro_batches: int = 1, reserved_sms: int = 0, stream: Optional[int] = None, workspace_factory=None,
                      switch_sum=None):
        """One shard of a Llama-style decoder layer forward through the single C-ABI call wb200_decoder_layer.
        x: [batch, seq, d_model] CUDA tensor. `allreduce(tensor)` must enqueue an in-place sum over the shards
        (torch.distributed.all_reduce); `workspace` is a uint8 CUDA tensor that is reused if large enough, else
        `workspace_factory(bytes)` (default: torch.empty) makes one. `switch_sum` (a sharding.SwitchSum whose allocate() is
        the workspace factory) instead of `allreduce`: the sums are done by the library's NVSwitch kernel inside the call.
        Returns (out, workspace)."""
        batch, seq, d_model = x.shape
        p = abi.DecoderLayerParams()
        p.batch, p.seq, p.d_model, p.head_dim = batch, seq, d_model, head_dim
        p.q_heads, p.kv_heads, p.ffn = q_heads, kv_heads, wdown.shape[0]
        p.format = _TORCH_FORMATS[x.dtype]
        p.eps, p.rope_theta, p.position_offset = eps, rope_theta, position_offset
        p.micro_batches = micro_batches if (allreduce is not None or switch_sum is not None) else 1
        p.reserved_sms = reserved_sms
        needed = self._lib.wb200_decoder_layer_workspace_bytes(C.byref(p))
        if needed == 0:
            raise WB200Error(abi.ERR_UNSUPPORTED, self._lib.wb200_last_error().decode())
        if workspace is None or workspace.numel() < needed:
            if workspace_factory is not None:
                workspace = workspace_factory(needed)
            else:
                workspace = torch.empty(needed, dtype=torch.uint8, device=x.device)
        if out is None:
            out = torch.empty_like(x)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        p.x, p.out = x.data_ptr(), out.data_ptr()
        p.norm1, p.wqkv, p.wo, p.norm2, p.wgu, p.wdown = (t.data_ptr() for t in (norm1, wqkv, wo, norm2, wgu, wdown))
        p.workspace, p.workspace_bytes, p.stream = workspace.data_ptr(), workspace.numel(), stream
        failure = []

        def reduce_callback(_user, pointer, elements, _format, part_stream):
            try:
                begin = pointer - workspace.data_ptr()
                view = workspace[begin:begin + elements * x.element_size()].view(x.dtype)
                if part_stream and part_stream != stream:
                    with torch.cuda.stream(torch.cuda.ExternalStream(part_stream)):
                        allreduce(view)
                else:
                    allreduce(view)
                return 0
            except Exception as error:   # must not propagate through the C frame
                failure.append(error)
                return 1
        callback = abi.ALLREDUCE_FN(reduce_callback) if allreduce is not None else abi.ALLREDUCE_FN()
        p.allreduce = callback
        if switch_sum is not None:
            native = abi.SwitchSumParams()
            native.rank, native.world = switch_sum.rank, switch_sum.world
            native.multicast = switch_sum.multicast_of(workspace)
            native.blocks = switch_sum.blocks
            for r, pointer in enumerate(switch_sum.signal_pointers):
                native.signals[r] = pointer
            native.epoch = switch_sum.epoch.data_ptr()
            p.switch_sum = C.pointer(native)
        status = self._lib.wb200_decoder_layer(self._handle, C.byref(p))
        if failure:
            raise failure[0]
        self._check(status)
        return out, workspace
