"""ctypes loader of liboptengine.so and the C structs of include/optengine.h."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboptengine.so")

OE_ERR_INVALID, OE_ERR_NO_DRIVER, OE_ERR_NOT_INIT, OE_ERR_ARCH, OE_ERR_LIMIT, OE_ERR_DEVICE = -1, -2, -3, -4, -5, -6
OE_CLIP_DEVFORM, OE_WRITE_SHADOW, OE_ZERO_GRAD, OE_NESTEROV, OE_MAXIMIZE, OE_PARTIAL_ONLY = 1, 2, 4, 8, 16, 32
OE_ACCUMULATE = 64


class oe_tensor_desc(C.Structure):
    _fields_ = [("param", C.c_uint64), ("grad", C.c_uint64), ("state1", C.c_uint64), ("state2", C.c_uint64),
                ("shadow", C.c_uint64), ("numel", C.c_uint64), ("lr_scale", C.c_float), ("weight_decay", C.c_float)]


class oe_adamw_hparams(C.Structure):
    _fields_ = [("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
                ("bc1", C.c_float), ("bc2", C.c_float), ("max_norm", C.c_float), ("flags", C.c_uint32),
                ("step_dev", C.c_uint64), ("lr_dev", C.c_uint64)]


class oe_sgd_hparams(C.Structure):
    _fields_ = [("lr", C.c_float), ("momentum", C.c_float), ("dampening", C.c_float), ("max_norm", C.c_float),
                ("flags", C.c_uint32), ("reserved", C.c_uint32), ("step_dev", C.c_uint64), ("lr_dev", C.c_uint64)]


class oe_zero1_desc(C.Structure):
    _fields_ = [("rank", C.c_uint32), ("world", C.c_uint32), ("first_elem", C.c_uint64), ("numel", C.c_uint64),
                ("grad_bases", C.c_uint64 * 8), ("shadow_deltas", C.c_int64 * 8), ("shadow_mc_delta", C.c_int64),
                ("sync_blocks", C.c_uint64 * 8), ("timeout_ms", C.c_uint32), ("flags", C.c_uint32),
                ("staging", C.c_uint64), ("staging_bytes", C.c_uint64), ("ce_pull_sources", C.c_uint32),
                ("ce_push_targets", C.c_uint32), ("staging_bases", C.c_uint64 * 8)]


OE_ZERO1_SYNC_BYTES = 512
OE_ZERO1_NO_ENTRY_EXCHANGE = 1
OE_ZERO1_CE_NONE = 0xffffffff
OE_TUNE_PEER_REDUCE_GRID, OE_TUNE_PEER_UPDATE_GRID, OE_TUNE_PEER_REDUCE_FIRST, OE_TUNE_PEER_PUSH_WARP_ROTATE = 1, 2, 3, 4
OE_TUNE_STEP_GRID, OE_TUNE_PEER_UPDATE_VECTORS, OE_TUNE_PEER_REDUCE_WARP_ROTATE = 5, 6, 7


class EngineError(RuntimeError):
    """A C-ABI call returned non-zero; carries the code and oe_last_error()."""

    def __init__(self, code: int, message: str):
        super().__init__(f"optengine error {code}: {message}")
        self.code = code
        self.message = message


_u64, _u32, _i, _vp = C.c_uint64, C.c_uint32, C.c_int, C.c_void_p
_plan = C.c_void_p

# name -> (restype, argtypes); the list the symbol-export test walks.
PROTOTYPES = {
    "oe_abi_version": (_i, []),
    "oe_last_error": (C.c_char_p, []),
    "oe_init": (_i, [_i]),
    "oe_shutdown": (_i, []),
    "oe_device_sm_count": (_i, [_i]),
    "oe_device_count": (_i, [C.POINTER(_i)]),
    "oe_enable_peer_access": (_i, [_i, _i]),
    "oe_plan_create": (_i, [_i, C.POINTER(oe_tensor_desc), _u32, _u32, C.POINTER(_plan)]),
    "oe_plan_update": (_i, [_plan, C.POINTER(oe_tensor_desc), _u32, _u64]),
    "oe_plan_destroy": (_i, [_plan]),
    "oe_plan_info": (C.c_int64, [_plan, _i]),
    "oe_plan_norm_address": (_u64, [_plan]),
    "oe_plan_set_variant": (_i, [_plan, C.c_char_p]),
    "oe_plan_set_grad_scale": (_i, [_plan, C.POINTER(C.c_float)]),
    "oe_grad_norm": (_i, [_plan, _u32, _u64]),
    "oe_norm_finalize": (_i, [_plan, _u64]),
    "oe_clip_grad_norm": (_i, [_plan, C.POINTER(C.c_float), _u32, _u64]),
    "oe_read_norm": (_i, [_plan, C.POINTER(C.c_float), C.POINTER(C.c_double), _u64]),
    "oe_adamw_step": (_i, [_plan, C.POINTER(oe_adamw_hparams), _u64]),
    "oe_adamw_step_chunks": (_i, [_plan, C.POINTER(oe_adamw_hparams), _u64, _u64, _u64]),
    "oe_sgd_step": (_i, [_plan, C.POINTER(oe_sgd_hparams), _u64]),
    "oe_zero_grads": (_i, [_plan, _u64]),
    "oe_cast_bf16": (_i, [_i, _u64, _u64, _u64, _u64]),
    "oe_adamw_step_from_host": (_i, [_plan, C.POINTER(oe_adamw_hparams), C.POINTER(_vp), _u32,
                                     C.POINTER(C.c_float), _u64]),
    "oe_peer_reduce_grads": (_i, [_plan, C.POINTER(_u64), _u32, _u64, _u64, _u64, C.POINTER(C.c_float), _u32, _u64]),
    "oe_adamw_step_peers": (_i, [_plan, C.POINTER(oe_adamw_hparams), C.POINTER(C.c_int64), _u32, _u64]),
    "oe_sgd_step_peers": (_i, [_plan, C.POINTER(oe_sgd_hparams), C.POINTER(C.c_int64), _u32, _u64]),
    "oe_adamw_step_multicast": (_i, [_plan, C.POINTER(oe_adamw_hparams), C.POINTER(C.c_int64), _u32,
                                     C.POINTER(C.c_int64), _u64]),
    "oe_sgd_step_multicast": (_i, [_plan, C.POINTER(oe_sgd_hparams), C.POINTER(C.c_int64), _u32,
                                   C.POINTER(C.c_int64), _u64]),
    "oe_plan_set_tuning": (_i, [_plan, _i, _u64]),
    "oe_link_probe_reads": (_i, [_plan, C.POINTER(_u64), _u32, _u64, _u64, _u64]),
    "oe_link_probe_stores": (_i, [_plan, _u64, C.POINTER(C.c_int64), _u32, _u64, _u64]),
    "oe_zero1_create": (_i, [_plan, C.POINTER(oe_zero1_desc), C.POINTER(_vp)]),
    "oe_zero1_destroy": (_i, [_vp]),
    "oe_zero1_adamw_step": (_i, [_vp, C.POINTER(oe_adamw_hparams), _u64]),
    "oe_zero1_sgd_step": (_i, [_vp, C.POINTER(oe_sgd_hparams), _u64]),
    "oe_zero1_exchange": (_i, [_vp, _u32, _u64]),
    "oe_zero1_reduce": (_i, [_vp, _u64]),
    "oe_zero1_info": (C.c_int64, [_vp, _i]),
    "oe_zero1_adamw_update": (_i, [_vp, C.POINTER(oe_adamw_hparams), _u64]),
    "oe_zero1_sgd_update": (_i, [_vp, C.POINTER(oe_sgd_hparams), _u64]),
    "oe_zero1_status": (_i, [_vp, C.POINTER(_u32), _u64]),
    "oe_ipc_export": (_i, [_i, _u64, _vp, C.POINTER(_u64)]),
    "oe_ipc_import": (_i, [_i, _vp, C.POINTER(_u64)]),
    "oe_ipc_close": (_i, [_i, _u64]),
    "oe_grad_norm_static": (_i, [_i, _u64, _u64, _u64, _u64]),
    "oe_launch_count": (C.c_int64, [C.c_char_p]),
    "oe_launch_count_reset": (None, []),
    "oe_profile_enable": (None, [_i]),
    "oe_profile_get": (_i, [C.c_char_p, C.POINTER(C.c_int64), C.POINTER(C.c_double)]),
    "oe_mem_alloc": (_i, [_i, _u64, C.POINTER(_u64)]),
    "oe_mem_free": (_i, [_i, _u64]),
    "oe_mem_info": (_i, [_i, C.POINTER(_u64), C.POINTER(_u64)]),
    "oe_memcpy_h2d": (_i, [_i, _u64, _vp, _u64, _u64]),
    "oe_memcpy_d2h": (_i, [_i, _vp, _u64, _u64, _u64]),
    "oe_memcpy_d2d": (_i, [_i, _u64, _u64, _u64, _u64]),
    "oe_memset_u32": (_i, [_i, _u64, _u32, _u64, _u64]),
    "oe_host_alloc": (_i, [_i, _u64, C.POINTER(_vp)]),
    "oe_host_free": (_i, [_i, _vp]),
    "oe_stream_create": (_i, [_i, C.POINTER(_u64)]),
    "oe_stream_destroy": (_i, [_i, _u64]),
    "oe_stream_sync": (_i, [_i, _u64]),
    "oe_event_create": (_i, [_i, C.POINTER(_u64)]),
    "oe_event_destroy": (_i, [_i, _u64]),
    "oe_event_record": (_i, [_i, _u64, _u64]),
    "oe_event_sync": (_i, [_i, _u64]),
    "oe_event_elapsed_ms": (_i, [_i, _u64, _u64, C.POINTER(C.c_float)]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library. Raises if it was not built: there is no fallback path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `make -C gograd_b200/csrc` "
                "(or __graft_entry__.build()); the engine has no CPU fallback")
        handle = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(code: int) -> None:
    if code != 0:
        raise EngineError(code, lib().oe_last_error().decode("utf-8", "replace"))
