"""ctypes binding of ``liblrqk_sm100.so`` (declarations: ``include/lrqk_sm100.h``).

The library is the only compute path of this package.  If it has not been built
the import fails with instructions; there is no Python or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "liblrqk_sm100.so")

LRQK_F32, LRQK_BF16 = 0, 1
OK, EINVAL, ECAPACITY, EUNSUPPORTED, ELAUNCH, ETIMEOUT, ENODEVICE, ENOMEM = 0, -1, -2, -3, -4, -5, -6, -7


class LrqkError(RuntimeError):
    def __init__(self, code: int, where: str, detail: str = ""):
        self.code = code
        super().__init__(f"{where}: {detail}")


class Layer(C.Structure):
    """struct lrqk_layer."""
    _fields_ = [
        ("dtype", C.c_int32), ("bsz", C.c_int32), ("q_heads", C.c_int32), ("kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("r", C.c_int32), ("k", C.c_int32), ("m", C.c_int32),
        ("a_capacity", C.c_int64), ("host_capacity", C.c_int64),
        ("A_K", C.c_void_p), ("B_Q", C.c_void_p), ("B_K", C.c_void_p),
        ("K_res", C.c_void_p), ("V_res", C.c_void_p),
        ("table", C.c_void_p), ("lite_pos", C.c_void_p), ("host_kv", C.c_void_p),
        ("weights", C.c_float * 4),
    ]


class Miss(C.Structure):
    """struct lrqk_miss."""
    _fields_ = [("head", C.c_int32), ("slot", C.c_int32), ("pos", C.c_int32)]


class StepArgs(C.Structure):
    """struct lrqk_step_args."""
    _fields_ = [
        ("q", C.c_void_p), ("k_new", C.c_void_p), ("v_new", C.c_void_p), ("attn_out", C.c_void_p),
        ("lite_slot", C.c_int32), ("position", C.c_int32), ("flush_rows", C.c_int32),
        ("host_row", C.c_int64), ("candidates", C.c_int64),
        ("max_iter", C.c_int32), ("tol", C.c_float), ("scale", C.c_float),
        ("q_hat", C.c_void_p), ("wanted", C.c_void_p), ("mask", C.c_void_p), ("miss_count", C.c_void_p),
        ("miss_list", C.c_void_p), ("counters", C.c_void_p),
        ("project_workspace", C.c_void_p), ("attn_workspace", C.c_void_p),
        ("peers", C.c_void_p), ("push_seq", C.c_int32),
        ("score_workspace", C.c_void_p), ("score_workspace_bytes", C.c_size_t),
        ("gathered_out", C.c_void_p), ("wait_status", C.c_void_p),
    ]


MAX_PEERS = 8


class PeerGroup(C.Structure):
    """struct lrqk_peer_group."""
    _fields_ = [
        ("world", C.c_int32), ("rank", C.c_int32), ("heads_per_rank", C.c_int32), ("head_dim", C.c_int32),
        ("dtype", C.c_int32), ("base", C.c_void_p * MAX_PEERS), ("local_counter", C.c_void_p),
    ]


_SIGNATURES = {
    # name: (restype, argtypes)
    "lrqk_version": (C.c_char_p, []),
    "lrqk_strerror": (C.c_char_p, [C.c_int]),
    "lrqk_device_supported": (C.c_int, []),
    "lrqk_last_cuda_error": (C.c_char_p, []),
    "lrqk_host_alloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "lrqk_host_free": (C.c_int, [C.c_void_p]),
    "lrqk_host_device_ptr": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "lrqk_lite_append": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                   C.c_int64, C.c_void_p]),
    "lrqk_decode_project_update_workspace_bytes": (C.c_size_t, [C.POINTER(Layer), C.c_int32]),
    "lrqk_decode_project_update": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_int32, C.c_float,
                                             C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "lrqk_decode_project": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_void_p,
                                      C.c_void_p, C.c_void_p]),
    "lrqk_decode_update": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_int32, C.c_float,
                                     C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "lrqk_score_topk_workspace_bytes": (C.c_size_t, [C.POINTER(Layer), C.c_int64]),
    "lrqk_score_topk": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64,
                                  C.c_void_p, C.c_size_t, C.c_void_p]),
    "lrqk_slot_diff": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_void_p, C.c_void_p]),
    "lrqk_miss_gather": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_void_p]),
    "lrqk_flash_decode_workspace_bytes": (C.c_size_t, [C.POINTER(Layer), C.c_int32]),
    "lrqk_flash_decode": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_int32, C.c_float, C.c_void_p,
                                    C.c_void_p]),
    "lrqk_flash_decode_static_capacity_bytes": (C.c_size_t, []),
    "lrqk_flash_decode_static_status": (C.c_int, [C.c_void_p, C.c_void_p]),
    "lrqk_flash_decode_status_word": (C.c_void_p, [C.POINTER(Layer), C.c_void_p]),
    "lrqk_decode_project_update_status_word": (C.c_void_p, [C.POINTER(Layer), C.c_int32, C.c_void_p]),
    "lrqk_flash_decode_static": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_int32, C.c_float,
                                           C.c_void_p]),
    "lrqk_peer_buffer_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "lrqk_peer_buffer_create": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]),
    "lrqk_peer_buffer_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "lrqk_peer_buffer_close": (C.c_int, [C.c_void_p]),
    "lrqk_peer_buffer_destroy": (C.c_int, [C.c_void_p]),
    "lrqk_flash_decode_push": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_int32, C.c_float, C.c_void_p,
                                         C.POINTER(PeerGroup), C.c_int32, C.c_void_p]),
    "lrqk_fetch_attend": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p,
                                    C.POINTER(PeerGroup), C.c_int32, C.c_void_p]),
    "lrqk_peer_set_wait_polls": (C.c_int, [C.c_uint32]),
    "lrqk_allgather_wait": (C.c_int, [C.POINTER(PeerGroup), C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "lrqk_layer_step": (C.c_int, [C.POINTER(Layer), C.POINTER(StepArgs), C.c_void_p]),
    "lrqk_layer_step_launches": (C.c_int, [C.POINTER(Layer), C.POINTER(StepArgs)]),
    "lrqk_d0_indices_select": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                         C.c_void_p]),
    "lrqk_take_along_dim_with_mask_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int64, C.c_int64]),
    "lrqk_take_along_dim_with_mask": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                                C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                                C.c_void_p, C.c_void_p]),
    "lrqk_rope_qkv": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                C.c_void_p]),
    "lrqk_add_rmsnorm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int32, C.c_int32, C.c_int32,
                                   C.c_void_p, C.c_void_p, C.c_void_p]),
    "lrqk_swiglu": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "lrqk_kv_pack_host": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "lrqk_prefill_fill_resident": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "lrqk_prefill_factorize_workspace_bytes": (C.c_size_t, [C.POINTER(Layer), C.c_int64]),
    "lrqk_prefill_factor_maps": (C.c_int, [C.POINTER(Layer), C.c_int64, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                           C.c_void_p, C.c_void_p]),
    "lrqk_prefill_factorize": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_int64, C.c_int32, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_void_p]),
}

_lib = None


def exported_names():
    """Names every build of the library must export (those declared in the header)."""
    return sorted(_SIGNATURES)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m lrqk_b200.build` (needs nvcc). "
                "lrqk_b200 has no fallback path.")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if a declared symbol is missing
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(code: int, where: str) -> None:
    if code == OK:
        return
    L = lib()
    msg = L.lrqk_strerror(code).decode()
    if code == ELAUNCH:
        msg += " -- " + L.lrqk_last_cuda_error().decode()
    raise LrqkError(code, where, msg)
