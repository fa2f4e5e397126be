"""ctypes binding of the C ABI declared in include/lutmac_b200.h.

The shared library is built in-tree (lutmac_b200/liblutmac_b200.so).  There is no fallback:
importing this module without the library raises, and every compute call fails with
LMB_ERR_CUDA on a machine without a B200-class GPU.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# LMB_DEBUG_BOUNDS=1 selects the range-checking build (python -m lutmac_b200.build --debug-bounds)
LIB_PATH = os.path.join(HERE, "liblutmac_b200_dbg.so" if os.environ.get("LMB_DEBUG_BOUNDS") == "1" else "liblutmac_b200.so")

OK = 0
ERR_ARG, ERR_CUDA, ERR_ALLOC, ERR_TIMEOUT, ERR_FORMAT, ERR_LIMIT, ERR_STATE = 1, 2, 3, 4, 5, 6, 7

ROTATE = 1
AUTO_ROTATE = 2
OPT_TERNARY_LUT = 1
OPT_PDL = 2
OPT_SCRATCH_FLOATS = 3

f32p = C.POINTER(C.c_float)
vp = C.c_void_p
sz = C.c_size_t


class ModelConfig(C.Structure):
    _fields_ = [("vocab_size", sz), ("hidden_size", sz), ("intermediate_size", sz), ("num_hidden_layers", sz),
                ("num_attention_heads", sz), ("num_key_value_heads", sz), ("head_dim", sz), ("max_seq_len", sz),
                ("rope_theta", C.c_float), ("rope_scaling_factor", C.c_float), ("rms_norm_eps", C.c_float),
                ("max_batch", sz), ("tp_rank", C.c_int), ("tp_size", C.c_int), ("gemma", C.c_int), ("activation", C.c_int)]


# name -> (restype, argtypes); every symbol include/lutmac_b200.h declares
SIGNATURES = {
    "lmb_strerror": (C.c_char_p, [C.c_int]),
    "lmb_last_error": (C.c_char_p, []),
    "lmb_block_bytes": (sz, [C.c_int]),
    "lmb_ctx_create": (C.c_int, [C.c_int, C.POINTER(vp)]),
    "lmb_ctx_destroy": (C.c_int, [vp]),
    "lmb_ctx_set_stream": (C.c_int, [vp, vp]),
    "lmb_ctx_sync": (C.c_int, [vp]),
    "lmb_ctx_set_option": (C.c_int, [vp, C.c_int, C.c_int]),
    "lmb_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "lmb_ctx_launch_count": (C.c_int, [vp, C.POINTER(C.c_uint64)]),
    "lmb_malloc": (C.c_int, [vp, sz, C.POINTER(vp)]),
    "lmb_free": (C.c_int, [vp, vp]),
    "lmb_memcpy_h2d": (C.c_int, [vp, vp, vp, sz]),
    "lmb_memcpy_d2h": (C.c_int, [vp, vp, vp, sz]),
    "lmb_memset": (C.c_int, [vp, vp, C.c_int, sz]),
    "lmb_host_alloc_pinned": (C.c_int, [sz, C.POINTER(vp)]),
    "lmb_host_free_pinned": (C.c_int, [vp]),
    "lmb_timer_start": (C.c_int, [vp]),
    "lmb_timer_stop": (C.c_int, [vp, f32p]),
    "lmb_graph_begin": (C.c_int, [vp]),
    "lmb_graph_end": (C.c_int, [vp, C.POINTER(vp)]),
    "lmb_graph_launch": (C.c_int, [vp, vp]),
    "lmb_graph_destroy": (C.c_int, [vp]),
    "lmb_weight_upload": (C.c_int, [vp, C.c_int, vp, sz, sz, C.POINTER(vp)]),
    "lmb_weight_upload_shard": (C.c_int, [vp, C.c_int, vp, sz, sz, sz, sz, sz, sz, C.POINTER(vp)]),
    "lmb_weight_free": (C.c_int, [vp]),
    "lmb_weight_info": (C.c_int, [vp, C.POINTER(C.c_int), C.POINTER(sz), C.POINTER(sz), C.POINTER(sz)]),
    "lmb_weight_download": (C.c_int, [vp, vp, vp]),
    "lmb_tiled_bytes": (sz, [C.c_int, sz, sz]),
    "lmb_retile_host": (C.c_int, [C.c_int, vp, sz, sz, vp]),
    "lmb_untile_host": (C.c_int, [C.c_int, vp, sz, sz, vp]),
    "lmb_quantize": (C.c_int, [vp, C.c_int, vp, sz, sz, vp]),
    "lmb_quantize_host": (C.c_int, [vp, C.c_int, vp, sz, sz, C.c_int, vp]),
    "lmb_linear": (C.c_int, [vp, vp, vp, vp, sz, sz, vp, sz, C.c_uint]),
    "lmb_linear_static_scratch": (C.c_int, [vp, vp, vp, sz, vp, C.c_uint, vp]),
    "lmb_group_create": (C.c_int, [vp, sz, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.c_uint, C.POINTER(vp)]),
    "lmb_group_launch": (C.c_int, [vp, vp]),
    "lmb_group_create_host": (C.c_int, [vp, sz, C.POINTER(vp), C.c_uint, C.POINTER(vp)]),
    "lmb_group_run_host": (C.c_int, [vp, vp, C.POINTER(vp), C.POINTER(vp)]),
    "lmb_group_host_io": (C.c_int, [vp, sz, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "lmb_group_destroy": (C.c_int, [vp]),
    "lmb_gemv_host": (C.c_int, [C.c_int, vp, sz, vp, vp, sz, sz]),
    "lmb_linear_host": (C.c_int, [vp, vp, vp, vp, vp, sz, C.c_uint]),
    "lmb_linear_host_multi": (C.c_int, [vp, sz, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.c_uint]),
    "lmb_fwht256": (C.c_int, [vp, vp, sz]),
    "lmb_apply_hadamard_rotation_host": (C.c_int, [vp, sz]),
    "lmb_debug_plan": (C.c_int, [C.c_int, sz, sz, sz, sz, C.c_int, C.POINTER(C.c_int)]),
    "lmb_debug_plan_weight": (C.c_int, [vp, C.c_int, C.POINTER(C.c_int)]),
    "lmb_debug_launch_timeline": (C.c_int, [vp, sz, vp, C.POINTER(sz)]),
    "lmb_debug_force_plan": (C.c_int, [C.c_int, C.c_int, C.c_int]),
    "lmb_debug_bounds": (C.c_int, [vp, C.POINTER(C.c_ulonglong)]),
    "lmb_debug_bounds_shrink": (C.c_int, [sz]),
    "lmb_debug_luts": (C.c_int, [vp, vp, sz, C.c_uint, vp]),
    "lmb_debug_ternary_indices": (C.c_int, [vp, vp, vp]),
    "lmb_model_create": (C.c_int, [vp, C.POINTER(ModelConfig), C.POINTER(vp)]),
    "lmb_model_destroy": (C.c_int, [vp]),
    "lmb_model_set_weight": (C.c_int, [vp, C.c_int, C.c_int, C.c_int, C.c_int, vp, sz, sz]),
    "lmb_model_tie_head": (C.c_int, [vp]),
    "lmb_model_set_vector": (C.c_int, [vp, C.c_int, C.c_int, vp, sz]),
    "lmb_model_forward": (C.c_int, [vp, C.POINTER(C.c_int), C.POINTER(sz), sz, vp]),
    "lmb_debug_model_timeline": (C.c_int, [vp, C.POINTER(C.c_uint64), C.POINTER(C.c_int), C.POINTER(C.c_int), sz, C.POINTER(sz)]),
    "lmb_debug_model_waits": (C.c_int, [vp, C.c_int, C.c_uint]),
    "lmb_model_logits_dev": (C.c_int, [vp, C.POINTER(vp)]),
    "lmb_model_reset": (C.c_int, [vp]),
    "lmb_model_kv_export": (C.c_int, [vp, sz, vp]),
    "lmb_model_kv_import": (C.c_int, [vp, sz, vp]),
    "lmb_model_step_bytes": (C.c_int, [vp, sz, C.POINTER(C.c_uint64)]),
    "lmb_file_open": (C.c_int, [C.c_char_p, C.POINTER(vp)]),
    "lmb_file_close": (C.c_int, [vp]),
    "lmb_file_config": (C.c_int, [vp, C.POINTER(ModelConfig)]),
    "lmb_file_tensor_count": (C.c_int, [vp, C.POINTER(sz)]),
    "lmb_file_tensor_info": (C.c_int, [vp, sz, C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                       C.POINTER(sz), C.POINTER(sz), C.POINTER(sz)]),
    "lmb_file_read_tensor": (C.c_int, [vp, sz, vp, sz]),
    "lmb_model_load": (C.c_int, [vp, C.c_char_p, sz, sz, C.c_int, C.c_int, C.POINTER(vp)]),
    "lmb_tp_unique_id": (C.c_int, [vp]),
    "lmb_tp_init": (C.c_int, [vp, vp, C.c_int, C.c_int]),
    "lmb_tp_destroy": (C.c_int, [vp]),
    "lmb_tp_peer_create": (C.c_int, [vp, sz, vp]),
    "lmb_tp_peer_open": (C.c_int, [vp, vp]),
    "lmb_tp_peer_status": (C.c_int, [vp, C.POINTER(C.c_int)]),
    "lmb_debug_tp_wait": (C.c_int, [vp, C.c_int, C.c_int, sz, C.c_uint, C.POINTER(C.c_int)]),
    "lmb_debug_tp_wait_prepare": (C.c_int, [vp, C.c_int, C.c_int, sz, C.c_uint, C.POINTER(C.c_int)]),
    "lmb_allreduce_sum": (C.c_int, [vp, vp, sz]),
    "lmb_allgather": (C.c_int, [vp, vp, vp, sz]),
}


class LutmacError(RuntimeError):
    def __init__(self, status: int, text: str, detail: str):
        super().__init__(f"lutmac_b200: {text} (status {status}){': ' + detail if detail else ''}")
        self.status = status


_lib = None


def lib() -> C.CDLL:
    """Load the shared library (once) and attach the signatures."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m lutmac_b200.build` "
                "(there is no CPU fallback for the CUDA path)")
        L = C.CDLL(LIB_PATH)
        missing = [name for name in SIGNATURES if not hasattr(L, name)]
        if missing:
            raise ImportError(f"{LIB_PATH} does not export {missing}: rebuild it (python -m lutmac_b200.build --force)")
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != OK:
        L = lib()
        raise LutmacError(status, L.lmb_strerror(status).decode(), L.lmb_last_error().decode())
