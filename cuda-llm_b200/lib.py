"""ctypes binding of the C ABI in include/b2ops.h (lib/libb2ops.so).

There is no fallback of any kind: if the shared library has not been built, or does
not export a declared symbol, loading fails with an error that says so.
"""
from __future__ import annotations

import ctypes as C
import os
import re

PKG = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(os.path.dirname(PKG), "include", "b2ops.h")
LIB_PATH = os.path.join(PKG, "lib", "libb2ops.so")

F32, F16 = 0, 1
FAST, DETERMINISTIC = 0, 1
OK = 0


class B2Error(RuntimeError):
    """A C ABI call returned a negative status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"b2ops status {status}: {message}")
        self.status = status


class InvalidArgument(B2Error, ValueError):
    """B2_ERR_INVALID: the counterpart of the std::invalid_argument the reference's wrappers throw."""


class AllocStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("malloc_calls", "free_calls", "allocated_bytes_total",
                                          "freed_bytes_total", "live_bytes", "peak_live_bytes")]


P2P_MAX_WORLD = 16


class P2PExchange(C.Structure):
    """b2_p2p_exchange of include/b2ops.h."""
    _fields_ = [("buffers", C.c_void_p * P2P_MAX_WORLD), ("world", C.c_int32), ("rank", C.c_int32),
                ("max_rows", C.c_int64), ("timeout_ms", C.c_uint32), ("trace", C.c_void_p)]


def declared_symbols(header: str = HEADER):
    """Names of every B2_API function the header declares."""
    text = open(header).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"B2_API\s+[\w\s\*]+?\b(b2_\w+)\s*\(", text)))


_p, _i64, _i, _f, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_size_t
_SIGNATURES = {
    "b2_version": (C.c_int, []),
    "b2_last_error": (C.c_char_p, []),
    "b2_status_string": (C.c_char_p, [_i]),
    "b2_rms_norm": (_i, [_p, _p, _p, _i64, _i64, _f, _i, _i, _p]),
    "b2_add_rms_norm": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _f, _i, _i, _p]),
    "b2_add": (_i, [_p, _p, _p, _i64, _i, _p]),
    "b2_swiglu": (_i, [_p, _p, _p, _i64, _i, _i, _p]),
    "b2_rope": (_i, [_p, _p, _p, _i64, _i64, _i64, _f, _i, _i, _p, _p]),
    "b2_rope_batched": (_i, [_p, _p, _p, _i64, _i64, _i64, _i64, _f, _i, _i, _p, _p]),
    "b2_qk_norm_rope": (_i, [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f, _f, _i, _p, _p]),
    "b2_bulk_copy_timeouts": (_i, [C.POINTER(C.c_uint32)]),
    "b2_set_programmatic_launch": (None, [_i]),
    "b2_get_programmatic_launch": (_i, []),
    "b2_embedding_gather": (_i, [_p, _p, _p, _i64, _i64, _i64, _i, _p, _p]),
    "b2_argmax_workspace_bytes": (_sz, [_i64]),
    "b2_argmax_workspace_init": (_i, [_p, _i64, _p]),
    "b2_argmax_rows": (_i, [_p, _i64, _i64, _i64, _i, _p, _p, _p]),
    "b2_argmax_rows_static": (_i, [_p, _i64, _i64, _i64, _i, _p, _p]),
    "b2_argmax_keys": (_i, [_p, _i64, _i64, _i64, _i, _i64, _p, _p, _p]),
    "b2_argmax_keys_exchange": (_i, [_p, _i64, _p, _p, _p, _p]),
    "b2_lm_head_argmax": (_i, [_p, _p, _i64, _i64, _i64, _i, _i, _i64, _p, _i64, _p, _p, _p, _p]),
    "b2_argmax_decode_keys": (_i, [_p, _i64, _p, _p]),
    "b2_softmax_workspace_bytes": (_sz, [_i64]),
    "b2_softmax_rows": (_i, [_p, _p, _i64, _i64, _i, _i, _p, _p]),
    "b2_softmax_stats": (_i, [_p, _i64, _i64, _i, _p, _p, _p]),
    "b2_softmax_rebase": (_i, [_p, _p, _p, _i64, _p]),
    "b2_softmax_apply": (_i, [_p, _p, _i64, _i64, _i, _p, _p, _p]),
    "b2_paged_kv_write_decode_batch": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i, _p, _p]),
    "b2_paged_kv_write_decode": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i, _p, _p]),
    "b2_paged_kv_prefill_copy": (_i, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i, _p, _p]),
    "b2_qk_norm_rope_paged": (_i, [_p] * 10 + [_i64, _i64, _i64, _i64, _f, _f, _i64, _i64, _i64, _i64, _i64, _i64, _i, _p, _p]),
    "b2_select_last_valid_rows": (_i, [_p, _p, _p, _i64, _i64, _i64, _i, _p, _p]),
    "b2_sampler_workspace_bytes": (_sz, [_i64, _i64]),
    "b2_ordered_sums": (_i, [_p, _i64, _i64, _p, _p]),
    "b2_sample_rows": (_i, [_p, _i64, _i64, _i64, _i, _f, C.c_int32, _f, C.c_uint64, _p, _p, _p, _p]),
    "b2_p2p_exchange_bytes": (_sz, [_i, _i64]),
    "b2_p2p_exchange_init": (_i, [_p, _i, _i64, _p]),
    "b2_ipc_export": (_i, [_p, _p]),
    "b2_ipc_open": (_i, [_p, C.POINTER(C.c_void_p)]),
    "b2_ipc_close": (_i, [_p]),
    "b2_argmax_rows_sharded": (_i, [_p, _i64, _i64, _i64, _i, _i64, _p, _p, _p, _p, _p]),
    "b2_softmax_stats_sharded": (_i, [_p, _i64, _i64, _i, _p, _p, _p, _p, _p]),
    "b2_alloc": (_p, [_sz]),
    "b2_free": (_i, [_p]),
    "b2_get_alloc_stats": (None, [C.POINTER(AllocStats)]),
    "b2_reset_alloc_stats": (None, []),
}

_lib = None


def load(path: str = LIB_PATH) -> C.CDLL:
    """Load the shared library and bind every declared entry point."""
    global _lib
    if _lib is not None and path == LIB_PATH:
        return _lib
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m cuda_llm_b200.build` "
            "(there is no CPU or library fallback for these operators)")
    lib = C.CDLL(path)
    for name in declared_symbols():
        if not hasattr(lib, name):
            raise ImportError(f"{path} does not export {name}, which include/b2ops.h declares")
        if name in _SIGNATURES:
            res, args = _SIGNATURES[name]
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
    if path == LIB_PATH:
        _lib = lib
    return lib


def check(status: int) -> None:
    """Raise for a negative status, with the library's message."""
    if status == OK:
        return
    msg = load().b2_last_error().decode(errors="replace")
    raise (InvalidArgument if status == -1 else B2Error)(status, msg)
