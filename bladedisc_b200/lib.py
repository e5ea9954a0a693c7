"""ctypes binding of libdisc_b200_ral.so (declared in include/disc_b200_ral.h).

There is no fallback: if the shared library has not been built, importing the
symbols raises.  Build it with ``python -m bladedisc_b200.build``.
"""
import ctypes
import os
from ctypes import (POINTER, Structure, c_char_p, c_float, c_int8, c_int32,
                    c_int64, c_size_t, c_void_p)
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libdisc_b200_ral.so"

ALLOC_FN = ctypes.CFUNCTYPE(c_void_p, c_void_p, c_size_t)
FREE_FN = ctypes.CFUNCTYPE(None, c_void_p, c_void_p)

# enums of include/disc_b200_ral.h
OUT_I8, OUT_F16, OUT_F32, OUT_I32 = 0, 1, 2, 3
ACT_NONE, ACT_GELU, ACT_SILU = 0, 1, 2
BIAS_NONE, BIAS_F32, BIAS_I8 = 0, 1, 2
SCALE_NONE, SCALE_SCALAR, SCALE_PER_COL, SCALE_PER_ROW = 0, 1, 2, 3
PATH_AUTO, PATH_TILED, PATH_SMALL_M, PATH_SIMT, PATH_PAIR, PATH_GEMV, PATH_SKINNY = 0, 1, 2, 3, 4, 5, 6
F32, F16 = 0, 1


class ContextOptions(Structure):
    _fields_ = [
        ("device", c_int32),
        ("stream", c_void_p),
        ("gpu_alloc", ALLOC_FN),
        ("gpu_free", FREE_FN),
        ("alloc_user", c_void_p),
        ("nccl_comm", c_void_p),
        ("comm_stream", c_void_p),
    ]


class QGemmArgs(Structure):
    _fields_ = [
        ("a", c_void_p), ("w", c_void_p), ("out", c_void_p),
        ("M", c_int64), ("N", c_int64), ("K", c_int64),
        ("lda", c_int64), ("ldw", c_int64), ("ldo", c_int64),
        ("x_scale", c_void_p), ("w_scale", c_void_p), ("out_scale", c_void_p),
        ("bias", c_void_p),
        ("x_scale_kind", c_int32), ("w_scale_kind", c_int32),
        ("out_scale_kind", c_int32), ("bias_kind", c_int32),
        ("fold_out_scale", c_int32), ("div_out_scale", c_int32),
        ("act", c_int32), ("out_dtype", c_int32),
        ("path", c_int32), ("split_k", c_int32),
        ("splitk_ws", c_void_p), ("splitk_ws_bytes", c_int64),
        ("a_slabs", c_int32), ("a_slab_cols", c_int64), ("a_slab_stride", c_int64),
        ("weights_static", c_int32), ("div_exact", c_int32),
    ]


class NormArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("residual", c_void_p), ("gamma", c_void_p), ("beta", c_void_p),
        ("y", c_void_p), ("sum_out", c_void_p), ("q_out", c_void_p),
        ("q_scale", c_void_p), ("q_row_scale", c_void_p),
        ("rows", c_int64), ("cols", c_int64),
        ("eps", c_float), ("type", c_int32), ("rms", c_int32),
        ("x_slab_cols", c_int64), ("x_slab_stride", c_int64),
    ]


class GatedQuantArgs(Structure):
    _fields_ = [
        ("gate", c_void_p), ("up", c_void_p), ("ld", c_int64),
        ("q", c_void_p), ("ldq", c_int64), ("row_scale", c_void_p),
        ("rows", c_int64), ("cols", c_int64), ("type", c_int32), ("pass_", c_int32),
    ]


class AttentionArgs(Structure):
    _fields_ = [
        ("qkv", c_void_p), ("tokens", c_int64), ("ld_qkv", c_int64), ("heads", c_int32),
        ("blocks", c_void_p), ("num_blocks", c_int32), ("scale", c_float),
        ("out", c_void_p), ("ld_out", c_int64), ("out_scale", c_void_p),
    ]


class WeightOnlyQGemmArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("w", c_void_p), ("scale", c_void_p), ("zero_point", c_void_p), ("bias", c_void_p),
        ("out", c_void_p), ("m", c_int64), ("n", c_int64), ("k", c_int64),
        ("ldx", c_int64), ("ldw", c_int64), ("ldo", c_int64), ("type", c_int32), ("path", c_int32),
    ]


class QConv2dArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("w", c_void_p), ("out", c_void_p),
        ("input_sizes", c_int64 * 4), ("kernel_sizes", c_int64 * 4), ("output_sizes", c_int64 * 4),
        ("padding", c_int32 * 4), ("metadata", c_int32 * 16),
        ("x_scale", c_void_p), ("w_scale", c_void_p), ("w_scale_per_channel", c_int32), ("out_scale", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_int64), ("splitk_ws", c_void_p), ("splitk_ws_bytes", c_int64),
    ]


# name -> (restype, argtypes): every function include/disc_b200_ral.h declares.
SIGNATURES = {
    "tao_ral_call_impl": (None, [c_void_p, c_void_p, POINTER(c_void_p)]),
    "tao_ral_last_error": (c_int32, [c_void_p, POINTER(c_char_p)]),
    "tao_ral_clear_error": (None, [c_void_p]),
    "disc_b200_context_create": (c_void_p, [POINTER(ContextOptions)]),
    "disc_b200_context_destroy": (None, [c_void_p]),
    "disc_b200_exec_create": (c_void_p, [c_void_p]),
    "disc_b200_exec_destroy": (None, [c_void_p]),
    "disc_b200_exec_bind_input": (c_int32, [c_void_p, c_int32, c_void_p, c_int32, POINTER(c_int64)]),
    "disc_b200_exec_get_output": (c_int32, [c_void_p, c_int32, POINTER(c_void_p), POINTER(c_int32),
                                            POINTER(c_int64), POINTER(c_int32)]),
    "disc_b200_exec_free_output": (None, [c_void_p, c_void_p]),
    "disc_b200_registry_size": (c_int32, []),
    "disc_b200_registry_name": (c_char_p, [c_int32]),
    "disc_b200_registry_has": (c_int32, [c_char_p]),
    "disc_b200_qgemm": (c_int32, [POINTER(QGemmArgs), c_void_p]),
    "disc_b200_qgemm_scratch_bytes": (c_int64, [c_int64, c_int64, c_int64]),
    "disc_b200_qgemm_small_m_noalloc": (c_int32, [POINTER(QGemmArgs), c_void_p]),
    "disc_b200_qgemm_small_m_noalloc_capacity": (c_int64, []),
    "disc_b200_qgemm_path": (c_int32, [POINTER(QGemmArgs)]),
    "disc_b200_host_linear_create": (c_void_p, [c_int64, c_int64, c_int64, c_int32, c_int32]),
    "disc_b200_host_linear_run": (c_int32, [c_void_p, POINTER(QGemmArgs), c_void_p, c_void_p, c_int64, c_void_p]),
    "disc_b200_host_linear_chunks": (c_int64, [c_void_p, c_int64]),
    "disc_b200_host_linear_destroy": (None, [c_void_p]),
    "disc_b200_quantize": (c_int32, [c_void_p, c_int32, c_void_p, c_int64, c_void_p, c_void_p,
                                     c_int64, c_int64, c_int32, c_int32, c_void_p]),
    "disc_b200_dequantize": (c_int32, [c_void_p, c_void_p, c_int32, c_int64, c_void_p, c_void_p,
                                       c_int64, c_int64, c_void_p]),
    "disc_b200_dynamic_quantize": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_int64, c_int64,
                                             c_void_p]),
    "disc_b200_norm": (c_int32, [POINTER(NormArgs), c_void_p]),
    "disc_b200_gated_quantize": (c_int32, [POINTER(GatedQuantArgs), c_void_p]),
    "disc_b200_rope_kv_append": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                           c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "disc_b200_softmax": (c_int32, [c_void_p, c_void_p, c_int32, c_int64, c_int64, c_int64, c_void_p,
                                    c_void_p, c_float, c_int32, c_void_p]),
    "disc_b200_attention": (c_int32, [POINTER(AttentionArgs), c_void_p]),
    "disc_b200_nccl_available": (c_int32, []),
    "disc_b200_nccl_unique_id": (c_int32, [c_void_p]),
    "disc_b200_nccl_comm_create": (c_int32, [c_void_p, c_int32, c_int32, POINTER(c_void_p)]),
    "disc_b200_nccl_comm_destroy": (c_int32, [c_void_p]),
    "disc_b200_all_gather": (c_int32, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "disc_b200_all_gather_rows": (c_int32, [c_void_p, c_void_p, c_int32, c_int64, c_int64, c_int64, c_void_p]),
    "disc_b200_all_reduce_f32": (c_int32, [c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_void_p]),
    "disc_b200_exec_free_host_output": (None, [c_void_p]),
    "disc_b200_executable_open": (c_void_p, [c_char_p, c_char_p, POINTER(ContextOptions)]),
    "disc_b200_executable_context": (c_void_p, [c_void_p]),
    "disc_b200_executable_run": (c_void_p, [c_void_p, c_int32, c_void_p]),
    "disc_b200_executable_close": (None, [c_void_p]),
    "disc_b200_context_load_metadata": (c_int32, [c_void_p, c_char_p]),
    "disc_b200_context_share_metadata": (c_int32, [c_void_p, c_char_p]),
    "disc_b200_metadata_write": (c_int32, [c_char_p, c_int32, POINTER(c_char_p), POINTER(c_int32),
                                           POINTER(c_void_p), POINTER(c_int64)]),
    "disc_b200_const_name_info": (c_int32, [c_char_p, POINTER(c_int32), POINTER(c_int64), POINTER(c_int64)]),
    "disc_b200_weight_only_qgemm": (c_int32, [POINTER(WeightOnlyQGemmArgs), c_void_p]),
    "disc_b200_weight_only_qgemm_plan": (c_int32, [c_int64, c_int64, c_int64, c_int32, c_int32, POINTER(c_int64)]),
    "disc_b200_qconv2d_workspace_bytes": (c_int64, [POINTER(QConv2dArgs)]),
    "disc_b200_qconv2d": (c_int32, [POINTER(QConv2dArgs), c_void_p]),
    "disc_b200_qconv2d_plan": (c_int32, [c_char_p, POINTER(c_int64), c_int32, POINTER(c_int64), c_int32, c_char_p,
                                         POINTER(c_int64), c_int32, c_int32, POINTER(c_int64), POINTER(c_int64),
                                         POINTER(c_int32), POINTER(c_int64), POINTER(c_int32)]),
    "disc_b200_observe_minmax_scratch_floats": (c_int64, [c_int64, c_int64, c_int64]),
    "disc_b200_observe_minmax": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                           c_int64, c_void_p]),
    "disc_b200_observe_histogram": (c_int32, [c_void_p, c_int32, c_int64, c_float, c_float, c_int32, c_void_p,
                                              c_void_p]),
    "disc_b200_minmax_qparams": (c_int32, [c_void_p, c_void_p, c_int64, c_int32, c_int32, c_int32, c_int32, c_void_p,
                                           c_void_p, c_void_p]),
    "disc_b200_select_device_image": (c_int32, [c_int64, c_int32, c_int32]),
    "disc_b200_last_error_string": (c_char_p, []),
    "disc_b200_kernel_status": (c_int32, []),
    "disc_b200_selftest_wait_expiry": (c_int32, [ctypes.c_uint64, POINTER(c_int64), c_void_p]),
    "disc_b200_version": (c_char_p, []),
    "disc_b200_attrs_describe": (c_int32, [c_void_p, c_char_p, c_int32]),
    "disc_b200_attrs_describe_bounded": (c_int32, [c_void_p, c_int64, c_char_p, c_int32]),
}

_lib = None


def library_path() -> Path:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Loads the shared library once and types every exported function."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} is missing: the CUDA extension has not been built "
            "(run `python -m bladedisc_b200.build`); there is no CPU fallback")
    lib = ctypes.CDLL(os.fspath(_LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int) -> None:
    """Raises with the library's message when a section-3 call failed."""
    if code != 0:
        msg = load().disc_b200_last_error_string().decode()
        raise RuntimeError(f"disc_b200 call failed ({code}): {msg}")
