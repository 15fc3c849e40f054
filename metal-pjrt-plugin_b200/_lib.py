"""ctypes binding of libb200graft.so (the C ABI of include/b200graft.h).

Nothing here computes: every function forwards raw device pointers to the
library.  There is no fallback: if the shared library is missing, loading
raises, and every entry point needs a CUDA device.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200graft.so")

OK, INVALID_ARGUMENT, UNIMPLEMENTED, INTERNAL, RESOURCE_EXHAUSTED, FAILED_PRECONDITION, TIMEOUT = range(7)
STATUS_NAMES = ["OK", "INVALID_ARGUMENT", "UNIMPLEMENTED", "INTERNAL", "RESOURCE_EXHAUSTED",
                "FAILED_PRECONDITION", "TIMEOUT"]
F32, F16, BF16 = 0, 1, 2
ROUTE_NONE, ROUTE_TCGEN05, ROUTE_FEWROW, ROUTE_SIMT = 0, 1, 2, 3
QMM_OUT_BF16, QMM_ADD_RESIDUAL, QMM_OUT_F32, QMM_OUT_F32_RAW, QMM_OUT_SILU_PAIR = 0, 1, 2, 3, 4
QMM_PRO_NONE, QMM_PRO_RMSNORM, QMM_PRO_SILU_MUL = 0, 1, 2
KIND_RMS, KIND_SOFTMAX, KIND_LOG_SOFTMAX, KIND_LAYERNORM = 0, 1, 2, 3
TP_ID_BYTES = 128
TP_PEER_HANDLE_BYTES = 64


class B200Error(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"{STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else status}: {message}")
        self.status = status


class Operand(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("ld", C.c_int64), ("batch_stride", C.c_int64),
                ("dtype", C.c_int32), ("transpose", C.c_int32)]


class GemmParamsC(C.Structure):
    _fields_ = [("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64), ("batch", C.c_int64),
                ("alpha", C.c_double), ("beta", C.c_double),
                ("a", Operand), ("b", Operand), ("c", Operand)]


class EpilogueC(C.Structure):
    _fields_ = [("act", C.c_int32), ("bias", C.c_void_p), ("aux", C.c_void_p)]


class MatrixLayoutC(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("order", C.c_int32), ("num_rows", C.c_int64), ("num_cols", C.c_int64),
                ("leading_dim_stride", C.c_int64), ("batch_size", C.c_int64), ("batch_stride", C.c_int64),
                ("transpose", C.c_int32)]


class MatmulConfigC(C.Structure):
    _fields_ = [("lhs", MatrixLayoutC), ("rhs", MatrixLayoutC), ("c", MatrixLayoutC), ("out", MatrixLayoutC),
                ("alpha_real", C.c_double), ("alpha_imag", C.c_double), ("beta", C.c_double)]


class EpilogueSpecC(C.Structure):
    _fields_ = [("bias", C.c_int32), ("act", C.c_int32), ("aux", C.c_int32)]


class MatmulPlanC(C.Structure):
    _fields_ = [("swap", C.c_int32), ("params", GemmParamsC), ("epi", EpilogueSpecC)]


ROW_MAJOR, COLUMN_MAJOR = 0, 1
(EPI_DEFAULT, EPI_RELU, EPI_BIAS, EPI_BIAS_RELU, EPI_GELU, EPI_GELU_AUX, EPI_BIAS_GELU, EPI_BIAS_GELU_AUX, EPI_SILU,
 EPI_SILU_AUX, EPI_BIAS_SILU, EPI_BIAS_SILU_AUX) = range(12)


class QmmParamsC(C.Structure):
    _fields_ = [("bits", C.c_int32), ("group", C.c_int32), ("nibble_order", C.c_int32),
                ("epilogue", C.c_int32), ("x", C.c_void_p), ("q", C.c_void_p), ("scale", C.c_void_p),
                ("bias", C.c_void_p), ("residual", C.c_void_p), ("out", C.c_void_p),
                ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64), ("ldx", C.c_int64), ("ldo", C.c_int64),
                ("prologue", C.c_int32), ("eps", C.c_float), ("prologue_gain", C.c_void_p)]


class DecoderConfigC(C.Structure):
    _fields_ = [("layers", C.c_int32), ("hidden", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("inter", C.c_int32), ("vocab", C.c_int32), ("max_len", C.c_int32),
                ("rope_theta", C.c_float), ("rms_eps", C.c_float), ("max_batch", C.c_int32)]


class QWeightC(C.Structure):
    _fields_ = [("q", C.c_void_p), ("scale", C.c_void_p), ("bias", C.c_void_p)]


class DecoderLayerC(C.Structure):
    _fields_ = [("attn_norm", C.c_void_p), ("qkv", QWeightC), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p),
                ("o", QWeightC), ("mlp_norm", C.c_void_p), ("gate_up", QWeightC), ("down", QWeightC),
                ("k_cache", C.c_void_p), ("v_cache", C.c_void_p)]


# name -> (restype, argtypes).  Every symbol include/b200graft.h declares.
_VP, _I, _I64, _D = C.c_void_p, C.c_int, C.c_int64, C.c_double
PROTOTYPES = {
    "b200_abi_version": (_I, []),
    "b200_context_create": (_I, [_I, C.POINTER(_VP)]),
    "b200_context_destroy": (None, [_VP]),
    "b200_last_error": (C.c_char_p, []),
    "b200_context_error": (_I, [_VP]),
    "b200_context_fail_launch_after": (None, [_VP, _I64]),
    "b200_context_launch_count": (_I64, [_VP]),
    "b200_context_wait_probe": (_I, [_VP, _VP, _I64]),
    "b200_gemm_validate": (_I, [C.POINTER(GemmParamsC), C.POINTER(EpilogueC)]),
    "b200_gemm": (_I, [_VP, _VP, C.POINTER(GemmParamsC), C.POINTER(EpilogueC)]),
    "b200_gemm_route": (_I, [C.POINTER(GemmParamsC), C.POINTER(EpilogueC)]),
    "b200_gemm_work": (C.c_uint64, [C.POINTER(GemmParamsC)]),
    "b200_gemm_force_route": (None, [_VP, _I]),
    "b200_qmm_force_route": (None, [_VP, _I]),
    "b200_probe_umma_rate": (_I, [_VP, _VP, _I, _I, _I, _I, _I, _I, _VP]),
    "b200_decode_epilogue": (_I, [C.c_int32, C.POINTER(EpilogueSpecC)]),
    "b200_matmul_plan_create": (_I, [C.POINTER(MatmulConfigC), C.c_int32, C.POINTER(MatmulPlanC)]),
    "b200_matmul_execute": (_I, [_VP, _VP, C.POINTER(MatmulPlanC), _VP, _VP, _VP, _VP, _VP, _VP, C.c_size_t, C.c_size_t,
                                 C.c_size_t]),
    "b200_qmm_validate": (_I, [C.POINTER(QmmParamsC)]),
    "b200_qmm_run": (_I, [_VP, _VP, C.POINTER(QmmParamsC)]),
    "b200_qmm": (_I, [_VP, _VP, _I, _I, _I, _VP, _VP, _VP, _VP, _VP, _I64, _I64, _I64, _I]),
    "b200_qmm_plan": (_I, [C.POINTER(QmmParamsC), C.POINTER(_I), C.POINTER(_I), C.POINTER(_I)]),
    "b200_dequantize": (_I, [_VP, _VP, _I, _I, _I, _VP, _VP, _VP, _VP, _I64, _I64, _I]),
    "b200_quantize": (_I, [_VP, _VP, _I, _I, _VP, _I, _VP, _VP, _VP, _I64, _I64]),
    "b200_quantize_int4_ref": (_I, [_VP, _VP, _VP, _I, _VP, _VP, _VP, _I64, _I64]),
    "b200_repack_int4": (_I, [_VP, _VP, _VP, _VP, _I64, _I64]),
    "b200_interleave_gate_up": (_I, [_VP, _VP, _VP, _VP, _I64, _I64]),
    "b200_rownorm": (_I, [_VP, _VP, _I, _VP, _VP, _VP, _VP, _I64, _I64, _I, _D]),
    "b200_decoder_create": (_I, [_VP, C.POINTER(DecoderConfigC), C.POINTER(DecoderLayerC), _VP, _VP, _VP, _VP,
                                 C.POINTER(_VP)]),
    "b200_decoder_destroy": (None, [_VP]),
    "b200_decoder_step": (_I, [_VP, _VP, _VP, _VP, _VP, _I]),
    "b200_decoder_launches_per_step": (_I64, [_VP, _I]),
    "b200_decoder_graphs_built": (_I64, [_VP]),
    "b200_decoder_trace": (_I, [_VP, _I]),
    "b200_decoder_trace_read": (_I, [_VP, _VP, _I64, C.POINTER(C.c_int32), C.POINTER(C.c_int32), _VP]),
    "b200_embed": (_I, [_VP, _VP, _VP, _VP, _VP, _I64, _I64, _I64]),
    "b200_qk_norm_rope_cache": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _I64, _I, _I, _I, _I64,
                                     C.c_float, C.c_float]),
    "b200_attention_scratch_bytes": (C.c_size_t, [_I64, _I, _I, _I64]),
    "b200_attention_decode": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _I64, _I, _I, _I, _I64]),
    "b200_attention_decode_static": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _I64, _I, _I, _I, _I64]),
    "b200_attention_step": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _I64, _I, _I, _I, _I64,
                                 C.c_float, C.c_float]),
    "b200_silu_mul": (_I, [_VP, _VP, _VP, _VP, _I64, _I64]),
    "b200_sample": (_I, [_VP, _VP, _VP, _I64, _I64, C.c_float, C.c_int32, C.c_float, _VP, _VP]),
    "b200_tp_make_id": (_I, [_VP]),
    "b200_tp_create": (_I, [_VP, _VP, _I, _I, C.POINTER(_VP)]),
    "b200_tp_destroy": (None, [_VP]),
    "b200_tp_all_reduce_bf16": (_I, [_VP, _VP, _VP, _I64]),
    "b200_tp_all_gather_f32": (_I, [_VP, _VP, _VP, _VP, _I64]),
    "b200_tp_peer_alloc": (_I, [_VP, _I64, _VP]),
    "b200_tp_peer_connect": (_I, [_VP, _VP]),
    "b200_tp_peer_partial": (_VP, [_VP, _I]),
    "b200_tp_sum_residual_norm": (_I, [_VP, _VP, _I, _VP, _VP, _VP, _I64, _I64, C.c_double]),
}

_lib = None


def lib():
    """The loaded library; raises if it was not built (python metal-pjrt-plugin_b200/build.py)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with metal-pjrt-plugin_b200/build.py "
                              "(there is no fallback path)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is absent
            fn.restype, fn.argtypes = res, args
        if handle.b200_abi_version() != 1:
            raise ImportError(f"{LIB_PATH}: ABI version {handle.b200_abi_version()} != 1")
        _lib = handle
    return _lib


def check(status):
    if status != OK:
        raise B200Error(status, lib().b200_last_error().decode("utf-8", "replace"))


def ptr(t):
    """Device pointer of a torch tensor (None -> NULL)."""
    return None if t is None else C.c_void_p(t.data_ptr())


def dtype_code(torch_dtype):
    import torch
    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[torch_dtype]


def current_stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)
