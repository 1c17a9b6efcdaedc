"""ctypes binding of libb200moe.so (the C ABI of include/b200moe.h). There is no fallback: a missing or stale library
raises, and every non-zero return code raises with the library's own message."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

_PKG = Path(__file__).resolve().parent
# B200MOE_LIB: load another build of the same library (the diagnostic build of `build.py --diag`); default: the product build
LIB_PATH = Path(os.environ["B200MOE_LIB"]) if os.environ.get("B200MOE_LIB") else _PKG / "libb200moe.so"
_lib = None

ERR_ARG, ERR_SHAPE, ERR_CUDA, ERR_DEVICE, ERR_TIMEOUT, ERR_WORKSPACE, ERR_LIMIT, ERR_RANGE, ERR_ORDER = -1, -2, -3, -4, -5, -6, -7, -8, -9

_P, _I, _LL = C.c_void_p, C.c_int, C.c_longlong
SIGNATURES = {
    "b200moe_version": (_I, []),
    "b200moe_error_string": (C.c_char_p, [_I]),
    "b200moe_last_cuda_error": (C.c_char_p, []),
    "b200moe_to_128x4": (_I, [_P, _P, _I, _I, _I, _P]),
    "b200moe_from_128x4": (_I, [_P, _P, _I, _I, _I, _P]),
    "b200moe_global_scale": (_I, [_P, _I, _LL, _P, _P, _P]),
    "b200moe_global_scale_grouped": (_I, [_P, _I, _I, _LL, _P, _P, _P]),
    "b200moe_quantize_nvfp4": (_I, [_P, _I, _P, _I, _I, _P, _I, _P, _P, _I, _P]),
    "b200moe_route_workspace_bytes": (_LL, [_I, _I]),
    "b200moe_route": (_I, [_P, _I, _I, _I, _P, _P, _P, _P, _LL, _P]),
    "b200moe_route_status": (_I, [_P, _I, _I, _P]),
    "b200moe_route_static": (_I, [_P, _I, _I, _I, _P, _P, _P, _P]),
    "b200moe_route_static_status": (_I, [_I, _I, _P]),
    "b200moe_layer_create": (_I, [C.POINTER(_P), _I, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "b200moe_layer_destroy": (None, [_P]),
    "b200moe_layer_workspace_bytes": (_LL, [_P]),
    "b200moe_layer_workspace_init": (_I, [_P, _P, _LL, _P]),
    "b200moe_layer_sm_count": (_I, [_P]),
    "b200moe_layer_workspace_map": (_I, [_P, _P]),
    "b200moe_layer_prepack_bytes": (_LL, [_P]),
    "b200moe_layer_prepack": (_I, [_P, _P, _LL, _P]),
    "b200moe_layer_set_decode_impl": (_I, [_P, _I]),
    "b200moe_layer_release_checkpoint": (_I, [_P]),
    "b200moe_layer_set_act_scale": (_I, [_P, C.c_float]),
    "b200moe_prefill_workspace_bytes": (_LL, [_P, _I]),
    "b200moe_prefill_forward": (_I, [_P, _P, _P, _P, _I, _P, _P, _LL, _I, C.c_float, C.c_float, _P]),
    "b200moe_prefill_status": (_I, [_P, _P, _I, _P]),
    "b200moe_prefill_workspace_map": (_I, [_P, _I, _P]),
    "b200moe_decode_forward": (_I, [_P, _P, _P, _P, _I, _P, _P, _LL, _P]),
    "b200moe_decode_forward_ex": (_I, [_P, _P, _P, _P, _I, _P, _P, _LL, _I, _P]),
    "b200moe_decode_forward_host": (_I, [_P, _P, _P, _P, _I, _P, _P, _LL, _P]),
    "b200moe_decode_fc1": (_I, [_P, _P, _P, _P, _I, _P, _P, _LL, _P]),
    "b200moe_decode_fc2": (_I, [_P, _P, _P, _P, _I, _P, _P, _LL, _P]),
    "b200moe_layer_route_tables": (_I, [_P, _P, _I, _P, _P, _P, _P]),
    "b200moe_layer_status": (_I, [_P, _P, _P]),
    "b200moe_stream_probe": (_I, [_P, _LL, _I, _I, _I, _I, _I, _I, _P, _P]),
    "b200moe_mid_workspace_bytes": (_LL, [_P, _I]),
    "b200moe_mid_forward": (_I, [_P, _P, _P, _P, _I, _P, _P, _LL, _I, _P]),
    "b200moe_mid_status": (_I, [_P, _P, _I, _P]),
    "b200moe_ep_dispatch": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "b200moe_ep_dispatch_wait": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P]),
    "b200moe_ep_return_combine": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _P, _P]),
    "b200moe_ep_dispatch_ll": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P]),
    "b200moe_ep_return_combine_ll": (_I, [_P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P, _I, _P, _P, _P, _P]),
    "b200moe_ep_unpack": (_I, [_P, _LL, _I, _I, _I, _I, _P, _P, _P, _P]),
    "b200moe_ep_wait": (_I, [_P, _I, _I, _P, _P, _P]),
    "b200moe_ep_return": (_I, [_P, _I, _I, _I, _I, _P, _P, _P]),
    "b200moe_ep_combine": (_I, [_P, _I, _I, _I, _I, _P, _P]),
    "b200moe_ep_plan": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "b200moe_ep_gather": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P]),
    "b200moe_ep_combine_rows": (_I, [_P, _P, _I, _I, _I, _P, _P]),
    "b200moe_umma_probe": (_I, [_P, _P, _P, _P, _I, _I, _P, _I, _P, _P]),
    "b200moe_umma_pair_probe": (_I, [_P, _P, _P, _P, _I, _P, _P, _P]),
}
# exported only by a diagnostic build (include/b200moe_diag.h); bound when present
DIAG_SIGNATURES = {
    "b200moe_layer_debug_counters": (_I, [_P, _P, _P, _I, _P]),
    "b200moe_umma_cost": (_I, [_I, _I, _I, _I, _I, _I, _P, _P]),
}


class B200MoEError(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = code
        super().__init__(what)


def lib() -> C.CDLL:
    """Load the shared object once. Raises if it has not been built (python sm120-fp4_b200/build.py)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} is missing: build it with `python {_PKG / 'build.py'}`; there is no fallback path")
        h = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(h, name)     # AttributeError if the library does not export a declared symbol
            fn.restype, fn.argtypes = res, args
        for name, (res, args) in DIAG_SIGNATURES.items():
            if hasattr(h, name):
                fn = getattr(h, name)
                fn.restype, fn.argtypes = res, args
        _lib = h
    return _lib


def check(code: int, what: str = "") -> None:
    if code == 0:
        return
    h = lib()
    msg = h.b200moe_error_string(code).decode()
    if code == ERR_CUDA:
        msg += f": {h.b200moe_last_cuda_error().decode()}"
    raise B200MoEError(code, f"{what or 'b200moe'}: {msg} ({code})")


def ptr(t) -> int:
    """Device (or host) address of a torch tensor, 0 for None."""
    return 0 if t is None else t.data_ptr()


def stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream
