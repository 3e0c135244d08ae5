"""ctypes declarations of the C ABI in include/wb200.h.

The structures mirror the header field by field. Loading fails loudly when libwb200.so is absent:
there is no Python or CPU substitute for the device library.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
LIBRARY_PATH = PACKAGE_DIR / "libwb200.so"

MAX_RANK = 8

# wb200_status
OK, ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_NAN_DOMAIN, ERR_BUDGET, ERR_CUDA, ERR_DEVICE_TIMEOUT, ERR_NO_DEVICE, ERR_LIMIT, ERR_CALLBACK = range(10)
STATUS_NAMES = ["ok", "invalid-argument", "unsupported", "nan-domain", "budget", "cuda", "device-timeout", "no-device", "limit", "callback"]

# wb200_format (ordinals of the reference's LogicalFormat / Data_Format codes)
I8, I16, F16, BF16, I32, F32, TF32, BOOL, U8, U16, U32, I64, U64, FORMAT_NONE = range(14)
# wb200_layout
LAYOUT_TENSOR, LAYOUT_NTENSOR, LAYOUT_CX, LAYOUT_NCX = range(4)
# wb200_memory
MEM_HOST, MEM_DEVICE = 0, 1
# wb200_gemm_policy
GEMM_FORMAL, GEMM_TENSOR = 0, 1
# wb200_epilogue
EPI_NONE, EPI_BIAS, EPI_BIAS_GELU, EPI_SWIGLU = 0, 1, 2, 3
# wb200_out_layout
OUT_HEAD_MAJOR, OUT_TOKEN_MAJOR = 0, 1
# wb200_orientation
NORMAL, TRANSPOSE = 0, 1

ELEMENTWISE_OPS = {
    "abs": 0, "recip": 1, "square": 2, "sqrt": 3, "rsqrt": 4, "neg": 5, "max": 6, "min": 7, "add": 8,
    "sub": 9, "mul": 10, "eq": 12, "ne": 13, "ge": 14, "gt": 15, "le": 16, "lt": 17, "logic_not": 18,
    "logic_and": 19, "logic_or": 20, "logic_xor": 21, "log2": 22, "ln": 23, "pow2": 24, "exp": 25,
    "exp_lp": 26, "sin": 27, "cos": 28, "tanh": 29, "sigmoid": 30, "relu": 31, "satrelu": 32,
    "leakyrelu": 33, "softplus": 34,
}
REDUCE_OPS = {"sum": 0, "max": 1, "min": 2, "avg": 3}
REDUCE_DIMS = {"trailing0": 0, "trailing1": 1, "trailing2": 2, "trailing3": 3, "trailing2and1": 4, "trailing2and1and0": 5}


class TensorDesc(C.Structure):
    _fields_ = [("format", C.c_uint8), ("layout", C.c_uint8), ("rank", C.c_uint8), ("reserved", C.c_uint8 * 5),
                ("shape", C.c_uint64 * MAX_RANK)]


class Geometry(C.Structure):
    _fields_ = [(name, C.c_int64) for name in (
        "element_bytes", "compact_bytes", "physical_elements", "physical_bytes", "c_block", "cx_blocks", "c0",
        "aligned_c", "outer_elements", "block_outer_elements", "outer_slice_stride_elements", "bank_align_elements")]


class Evidence(C.Structure):
    _fields_ = [("matmul_invocations", C.c_uint64), ("reorder_invocations", C.c_uint64),
                ("formal_fused_multiply_adds", C.c_uint64), ("scalar_evaluations", C.c_uint64),
                ("evidence_kind", C.c_uint32), ("flags", C.c_uint32), ("gpu_launches", C.c_uint32),
                ("device_us", C.c_uint32), ("digest", C.c_char * 96), ("implementation", C.c_char * 64)]


class GemmRequest(C.Structure):
    _fields_ = [("lhs", TensorDesc), ("rhs", TensorDesc), ("destination", TensorDesc), ("psum", TensorDesc),
                ("m", C.c_uint32), ("k", C.c_uint32), ("n", C.c_uint32), ("batch_count", C.c_uint32),
                ("lhs_orientation", C.c_uint8), ("rhs_orientation", C.c_uint8), ("has_psum", C.c_uint8),
                ("policy", C.c_uint8), ("reserved", C.c_uint32),
                ("lhs_storage", C.c_void_p), ("lhs_bytes", C.c_uint64),
                ("rhs_storage", C.c_void_p), ("rhs_bytes", C.c_uint64),
                ("psum_storage", C.c_void_p), ("psum_bytes", C.c_uint64),
                ("destination_template", C.c_void_p), ("destination_out", C.c_void_p),
                ("destination_bytes", C.c_uint64)]


class ElementwiseRequest(C.Structure):
    _fields_ = [("operation", C.c_uint32), ("input_count", C.c_uint32), ("inputs", TensorDesc * 2),
                ("destination", TensorDesc), ("input_storage", C.c_void_p * 2), ("input_bytes", C.c_uint64 * 2),
                ("destination_template", C.c_void_p), ("destination_out", C.c_void_p),
                ("destination_bytes", C.c_uint64), ("max_scalar_evaluations", C.c_uint64)]


class ConvertRequest(C.Structure):
    _fields_ = [("opcode", C.c_uint32), ("rounding_mode", C.c_uint32), ("source", TensorDesc),
                ("destination", TensorDesc), ("source_storage", C.c_void_p), ("source_bytes", C.c_uint64),
                ("destination_template", C.c_void_p), ("destination_out", C.c_void_p),
                ("destination_bytes", C.c_uint64), ("max_scalar_evaluations", C.c_uint64)]


class ReduceRequest(C.Structure):
    _fields_ = [("operation", C.c_uint32), ("dimension", C.c_uint32), ("input", TensorDesc),
                ("destination", TensorDesc), ("input_storage", C.c_void_p), ("input_bytes", C.c_uint64),
                ("destination_template", C.c_void_p), ("destination_out", C.c_void_p),
                ("destination_bytes", C.c_uint64), ("max_scalar_evaluations", C.c_uint64)]


class AttentionParams(C.Structure):
    _fields_ = [("batch", C.c_uint32), ("q_heads", C.c_uint32), ("kv_heads", C.c_uint32),
                ("q_len", C.c_uint32), ("kv_len", C.c_uint32), ("head_dim", C.c_uint32),
                ("format", C.c_uint8), ("causal", C.c_uint8), ("zero_fully_masked", C.c_uint8), ("memory", C.c_uint8),
                ("scale", C.c_float),
                ("query_start", C.c_int64), ("key_start", C.c_int64), ("key_end", C.c_int64),
                ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
                ("lse", C.c_void_p), ("row_max", C.c_void_p), ("row_sum", C.c_void_p), ("stream", C.c_void_p),
                ("out_layout", C.c_uint32), ("reserved", C.c_uint32)]


class GemmEpilogueParams(C.Structure):
    _fields_ = [("m", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32),
                ("in_format", C.c_uint8), ("out_format", C.c_uint8), ("lhs_orientation", C.c_uint8),
                ("rhs_orientation", C.c_uint8), ("epilogue", C.c_uint8), ("memory", C.c_uint8),
                ("reserved", C.c_uint8 * 2),
                ("a", C.c_void_p), ("b", C.c_void_p), ("bias", C.c_void_p), ("out", C.c_void_p), ("stream", C.c_void_p)]


# Every exported symbol with its C signature; tests check the library exports exactly these.
ALLREDUCE_FN = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32, C.c_void_p)


class SwitchSumParams(C.Structure):
    _fields_ = [("rank", C.c_uint32), ("world", C.c_uint32), ("multicast", C.c_void_p), ("elements", C.c_uint64),
                ("format", C.c_uint32), ("blocks", C.c_uint32), ("signals", C.c_void_p * 16), ("epoch", C.c_void_p),
                ("stream", C.c_void_p), ("multicast_out", C.c_void_p), ("residual", C.c_void_p)]


class DecoderLayerParams(C.Structure):
    _fields_ = [("batch", C.c_uint32), ("seq", C.c_uint32), ("d_model", C.c_uint32), ("head_dim", C.c_uint32),
                ("q_heads", C.c_uint32), ("kv_heads", C.c_uint32), ("ffn", C.c_uint32), ("format", C.c_uint32),
                ("eps", C.c_float), ("rope_theta", C.c_float), ("position_offset", C.c_uint32), ("micro_batches", C.c_uint32), ("reserved_sms", C.c_uint32),
                ("x", C.c_void_p), ("out", C.c_void_p),
                ("norm1", C.c_void_p), ("wqkv", C.c_void_p), ("wo", C.c_void_p), ("norm2", C.c_void_p), ("wgu", C.c_void_p), ("wdown", C.c_void_p),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_uint64),
                ("allreduce", ALLREDUCE_FN), ("allreduce_user", C.c_void_p), ("stream", C.c_void_p),
                ("switch_sum", C.POINTER(SwitchSumParams))]


class FdExchange(C.Structure):
    _fields_ = [("rank", C.c_uint32), ("world", C.c_uint32), ("peer_buffers", C.c_void_p * 16), ("epoch", C.c_void_p)]


class ProgramStats(C.Structure):
    _fields_ = [("instructions", C.c_uint64), ("commands", C.c_uint64), ("gemm_commands", C.c_uint64), ("movement_commands", C.c_uint64),
                ("fill_commands", C.c_uint64), ("transfer_commands", C.c_uint64), ("sync_commands", C.c_uint64),
                ("gemm_fused_multiply_adds", C.c_uint64), ("bytes_moved", C.c_uint64), ("gpu_launches", C.c_uint64),
                ("device_ms", C.c_float), ("numeric_flags", C.c_uint32)]


class ProgramCommand(C.Structure):
    _fields_ = [("tile", C.c_uint32), ("kind", C.c_uint32), ("argc", C.c_uint32), ("operation", C.c_uint32), ("args", C.c_uint64 * 20)]


class Comparison(C.Structure):
    _fields_ = [("outcome", C.c_uint32), ("reserved", C.c_uint32), ("element", C.c_uint64),
                ("element_count", C.c_uint64), ("exact_count", C.c_uint64), ("mismatch_count", C.c_uint64),
                ("exact_fraction", C.c_double), ("mean_abs", C.c_double), ("p99_abs", C.c_double), ("p999_abs", C.c_double),
                ("max_abs", C.c_double), ("cosine", C.c_double), ("relative_l2", C.c_double), ("mean_ulp", C.c_double),
                ("p99_ulp", C.c_uint64), ("p999_ulp", C.c_uint64), ("max_ulp", C.c_uint64),
                ("first_mismatch", C.c_uint64), ("max_abs_mismatch", C.c_uint64), ("max_ratio_mismatch", C.c_uint64),
                ("detail", C.c_char * 512)]


CMP_MATCH, CMP_INVALID_TOLERANCE, CMP_ACTUAL_NONFINITE, CMP_EXPECTED_NONFINITE, CMP_NUMERIC_MISMATCH, CMP_EMPTY, CMP_RAW_MISMATCH = range(7)

_U32x3 = C.POINTER(C.c_uint32)

SIGNATURES = {
    "wb200_abi_version": (C.c_int, []),
    "wb200_last_error": (C.c_char_p, []),
    "wb200_backend_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "wb200_backend_destroy": (None, [C.c_void_p]),
    "wb200_backend_set_budget": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint64]),
    "wb200_backend_poll": (C.c_int, [C.c_void_p, C.c_void_p]),
    "wb200_backend_launch_count": (C.c_uint64, [C.c_void_p]),
    "wb200_physical_geometry": (C.c_int, [C.POINTER(TensorDesc), C.POINTER(Geometry)]),
    "wb200_physical_bytes": (C.c_int, [C.POINTER(TensorDesc), C.POINTER(C.c_uint64)]),
    "wb200_unpack": (C.c_int, [C.c_void_p, C.POINTER(TensorDesc), C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64]),
    "wb200_pack": (C.c_int, [C.c_void_p, C.POINTER(TensorDesc), C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_uint64]),
    "wb200_gemm": (C.c_int, [C.c_void_p, C.POINTER(GemmRequest), C.POINTER(C.c_int), C.POINTER(Evidence)]),
    "wb200_elementwise": (C.c_int, [C.c_void_p, C.POINTER(ElementwiseRequest), C.POINTER(Evidence)]),
    "wb200_elementwise_formal": (C.c_int, [C.c_void_p, C.POINTER(ElementwiseRequest), C.POINTER(Evidence)]),
    "wb200_convert": (C.c_int, [C.c_void_p, C.POINTER(ConvertRequest), C.POINTER(Evidence)]),
    "wb200_convert_formal": (C.c_int, [C.c_void_p, C.POINTER(ConvertRequest), C.POINTER(Evidence)]),
    "wb200_reduce": (C.c_int, [C.c_void_p, C.POINTER(ReduceRequest), C.POINTER(Evidence)]),
    "wb200_reduce_formal": (C.c_int, [C.c_void_p, C.POINTER(ReduceRequest), C.POINTER(Evidence)]),
    "wb200_attention_fa": (C.c_int, [C.c_void_p, C.POINTER(AttentionParams)]),
    "wb200_attention_fd": (C.c_int, [C.c_void_p, C.POINTER(AttentionParams), C.c_uint32]),
    "wb200_attention_fd_static": (C.c_int, [C.c_void_p, C.POINTER(AttentionParams), C.c_uint32]),
    "wb200_attention_fd_partial": (C.c_int, [C.c_void_p, C.POINTER(AttentionParams), C.c_uint32, C.c_void_p]),
    "wb200_attention_fd_merge": (C.c_int, [C.c_void_p, C.POINTER(AttentionParams), C.c_void_p, C.c_uint32]),
    "wb200_gemm_epilogue": (C.c_int, [C.c_void_p, C.POINTER(GemmEpilogueParams)]),
    "wb200_rmsnorm": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_float, C.c_void_p]),
    "wb200_rope_split": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_uint32] * 5 + [C.c_float, C.c_uint32, C.c_void_p]),
    "wb200_residual_add": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]),
    "wb200_selftest_bounded_wait": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(C.c_uint64)]),
    "wb200_fd_exchange_bytes": (C.c_uint64, [C.c_uint32, C.c_uint32, C.c_uint32]),
    "wb200_attention_fd_exchange": (C.c_int, [C.c_void_p, C.POINTER(AttentionParams), C.c_uint32, C.POINTER(FdExchange)]),
    "wb200_switch_sum_signal_bytes": (C.c_uint64, [C.c_uint32]),
    "wb200_switch_sum": (C.c_int, [C.c_void_p, C.POINTER(SwitchSumParams)]),
    "wb200_decoder_layer_workspace_bytes": (C.c_uint64, [C.POINTER(DecoderLayerParams)]),
    "wb200_decoder_layer": (C.c_int, [C.c_void_p, C.POINTER(DecoderLayerParams)]),
    "wb200_decoder_layer_timeline": (C.c_int, [C.c_void_p, C.POINTER(C.c_float), C.c_uint32, C.POINTER(C.c_uint32)]),
    "wb200_target_call_rdma": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, _U32x3, _U32x3]),
    "wb200_target_call_wdma": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, _U32x3, _U32x3]),
    "wb200_target_call_gather_scatter": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, _U32x3, _U32x3, _U32x3, _U32x3]),
    "wb200_target_call_memset": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32]),
    "wb200_tile_program_load": (C.c_int, [C.c_void_p, C.POINTER(C.c_char_p), C.c_uint32, C.c_uint64, C.POINTER(C.c_void_p)]),
    "wb200_tile_program_destroy": (None, [C.c_void_p]),
    "wb200_tile_program_tensor_count": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    "wb200_tile_program_tensor_info": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(TensorDesc), C.POINTER(C.c_uint64)]),
    "wb200_tile_program_placement": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32] + [C.POINTER(C.c_uint64)] * 4),
    "wb200_tile_program_trace": (C.c_int, [C.c_void_p, C.POINTER(ProgramCommand), C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(ProgramStats)]),
    "wb200_program_command_name": (C.c_char_p, [C.c_uint32]),
    "wb200_tile_program_run": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_uint32, C.POINTER(ProgramStats)]),
    "wb200_target_call_elementwise": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint64, C.c_uint64] + [C.c_uint32] * 5 + [C.POINTER(C.c_uint32)]),
    "wb200_target_call_bit2fp": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32]),
    "wb200_target_call_mask_move": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32]),
    "wb200_target_call_convert": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32)]),
    "wb200_target_call_reduce": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint64, C.c_uint32, _U32x3, C.c_uint32, C.POINTER(C.c_uint32)]),
    "wb200_target_call_pool": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint64, _U32x3, _U32x3, _U32x3, _U32x3, C.c_uint32, C.POINTER(C.c_uint32)]),
    "wb200_compare": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint64, C.c_void_p, C.c_void_p, C.c_uint32, C.c_double, C.c_double,
                                C.c_uint32, C.c_double, C.c_double, C.POINTER(Comparison)]),
    "wb200_compare_raw": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_uint32, C.POINTER(Comparison)]),
    "wb200_spm_create": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint64, C.POINTER(C.c_void_p)]),
    "wb200_spm_destroy": (None, [C.c_void_p]),
    "wb200_spm_write": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64]),
    "wb200_spm_read": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64]),
    "wb200_target_call_gemm": (C.c_int, [C.c_void_p] + [C.c_uint64] * 4 + [C.c_uint32] * 10),
}

_lib = None


def load():
    """Loads libwb200.so and attaches the signatures. Raises if the library has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    import os
    path = Path(os.environ.get("WB200_LIBRARY", LIBRARY_PATH))   # override: load another build of the same ABI
    if not path.exists():
        raise RuntimeError(f"{path} is missing: run `python -m vibe_compiler_b200.build`. "
                           "There is no fallback implementation.")
    lib = C.CDLL(str(path))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def make_desc(fmt: int, layout: int, shape) -> TensorDesc:
    desc = TensorDesc()
    desc.format, desc.layout, desc.rank = fmt, layout, len(shape)
    for i, extent in enumerate(shape):
        desc.shape[i] = int(extent)
    return desc
