"""Loads the kernel library through ctypes and declares its entry points.

The entry points are plain C functions over device pointers, sizes and a stream; each returns 0
or a negative code, and ``tk_last_error`` gives the message. There is no other implementation
behind them: if the library cannot be built or loaded, the import of an op raises.
"""

from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p

from tokenomos_b200.csrc import build as _build

F32, BF16 = 0, 1

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None

P, I, L, F = c_void_p, c_int, c_int64, c_float

_SIGNATURES = {
    "tk_check_device": [],
    "tk_built_for": [],
    "tk_set_pdl": [I],
    "tk_checks_enabled": [],
    "tk_checks_set_bounds": [I, I],
    "tk_checks_status": [P],
    "tk_gather_rows": [P, P, P, I, I, I, I, P],
    "tk_gather_rows_select": [P, P, P, P, P, P, I, I, I, I, P],
    "tk_add_rmsnorm": [P, L, P, P, F, P, F, P, P, I, I, I, P],
    "tk_swiglu": [P, P, I, I, I, I, P],
    "tk_head_gate": [P, P, L, I, I, I, I, P],
    "tk_qk_norm_rope_write": [P, L, P, P, P, P, F, P, P, P, P, I, I, I, I, I, I, I, I, P],
    "tk_attn_generic_rows": [],
    "tk_attn_generic": [P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, I, P],
    "tk_attn_mma_supported": [I, I, I],
    "tk_attn_prefill_mma_tokens": [I, I],
    "tk_attn_prefill_mma": [P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, P, L, P],
    "tk_attn_prefill_tc_supported": [I, I, I],
    "tk_attn_prefill_tc_tokens": [I, I],
    "tk_attn_prefill_tc_status": [],
    "tk_attn_prefill_tc": [P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, P, L, I, P, P, P],
    "tk_attn_decode_mma": [P, P, P, P, P, P, I, P, I, I, I, I, I, I, F, I, P, P, L, P],
    "tk_attn_decode_fused_supported": [I, I, I, I],
    "tk_attn_decode_fused_max_splits": [I, I, I],
    "tk_attn_decode_fused": [P, L, P, P, P, P, F, P, I, P, L, P, P, P, I, I, I, I, I, I, I, F, I, P, P, I, I, P],
    "tk_conv_min_tile": [I],
    "tk_conv_gated": [P, L, I, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, P],
    "tk_gemm_skinny_conv": [P, L, P, L, P, P, L, I, I, I, P, P, P, P, P, I, F, P],
    "tk_gemm_simt": [P, L, P, L, P, P, L, I, I, I, I, I, P],
    "tk_gemm_skinny": [P, L, P, L, P, P, L, I, I, I, I, I, F, P, L, P],
    "tk_sample": [P, L, I, I, P, P, P, P, P, P, P, P, P, P],
    "tk_scale_rows": [P, L, F, I, P],
    "tk_logit_options": [P, L, I, I, F, P, I, P],
    "tk_gemm_tc_status": [],
    "tk_sample_status": [],
    "tk_gemm_tc_decode": [P, L, P, L, P, P, L, I, I, I, I, I, I, P],
}


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or failed to launch."""


def lib() -> ctypes.CDLL:
    """The loaded library, built on first use."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = _build.build()
            loaded = ctypes.CDLL(str(path))
            loaded.tk_last_error.restype = c_char_p
            loaded.tk_last_error.argtypes = []
            for name, args in _SIGNATURES.items():
                fn = getattr(loaded, name)
                fn.restype = c_int
                fn.argtypes = args
            if os.environ.get("TOKENOMOS_B200_PDL", "1") == "0":
                loaded.tk_set_pdl(0)
            _lib = loaded
    return _lib


def declare(name: str, args: list) -> None:
    """Declare one more entry point (used by modules that add kernels to the table above)."""
    _SIGNATURES[name] = args
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype = c_int
        fn.argtypes = args


_calls = 0


def calls() -> int:
    """How many kernel entry points have been called in this process (each launches one
    kernel of this library; queries such as ``tk_conv_min_tile`` are not counted)."""
    return _calls


_QUERIES = {"tk_check_device", "tk_built_for", "tk_set_pdl", "tk_checks_enabled", "tk_checks_set_bounds", "tk_checks_status", "tk_attn_generic_rows", "tk_conv_min_tile",
            "tk_attn_mma_supported", "tk_attn_decode_fused_supported", "tk_attn_decode_fused_max_splits", "tk_attn_prefill_mma_tokens", "tk_attn_prefill_tc_supported",
            "tk_attn_prefill_tc_tokens", "tk_attn_prefill_tc_status", "tk_gemm_tc_status", "tk_sample_status"}


_fns: dict = {}


def call(name: str, *args) -> int:
    """Call an entry point; a negative return raises ``KernelError`` with the library's message."""
    global _calls
    fn = _fns.get(name)
    if fn is None:
        fn = _fns[name] = (getattr(lib(), name), name not in _QUERIES)
    if fn[1]:
        _calls += 1
    rc = fn[0](*args)
    if rc < 0:
        raise KernelError(f"{name}: {lib().tk_last_error().decode()}")
    return rc
