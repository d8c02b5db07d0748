"""The host runtime library (``csrc/host/runtime.cpp``) through ctypes: pools,
block tables and the step packer live in C++; this module loads the library,
declares the signatures and turns its error classes into exceptions."""

from __future__ import annotations

import ctypes
import threading

_lib = None
_lock = threading.Lock()

I = ctypes.c_int
P = ctypes.c_void_p
IP = ctypes.POINTER(ctypes.c_int)


class PoolError(RuntimeError):
    pass


class OutOfPages(PoolError):
    pass


_ERRORS = {1: PoolError, 2: OutOfPages, 3: ValueError, 4: IndexError, 5: RuntimeError}

_SIGNATURES = {
    "li_pool_create": (P, [I, ctypes.c_char_p]),
    "li_pool_destroy": (None, [P]),
    "li_pool_alloc": (I, [P, I, IP]),
    "li_pool_free": (I, [P, I, I]),
    "li_pool_num_free": (I, [P]),
    "li_pool_owner": (I, [P, I]),
    "li_pool_check": (I, [P]),
    "li_cm_create": (P, [I, IP, I, I, I]),
    "li_cm_destroy": (None, [P]),
    "li_cm_num_free": (I, [P, I]),
    "li_cm_owner": (I, [P, I, I]),
    "li_cm_pool_check": (I, [P, I]),
    "li_cm_admit": (I, [P, I, IP]),
    "li_cm_pages_needed": (I, [P, I, I, IP]),
    "li_cm_extend": (I, [P, I, I]),
    "li_cm_commit": (I, [P, I, I]),
    "li_cm_commit_many": (I, [P, I, P, P]),
    "li_cm_release": (I, [P, I]),
    "li_cm_length": (I, [P, I]),
    "li_cm_table": (I, [P, I, I, IP, I]),
    "li_cm_check": (I, [P]),
    "li_sched_create": (P, [P, I, I, I, I]),
    "li_sched_destroy": (None, [P]),
    "li_sched_set_eos": (I, [P, P, I]),
    "li_sched_add": (I, [P, I, I, I]),
    "li_sched_counts": (I, [P, IP, IP, IP]),
    "li_sched_schedule": (I, [P, P, I, IP, P, I, IP]),
    "li_sched_update": (I, [P, I, P, P, P, P]),
    "li_sched_abort": (I, [P, I, IP]),
    "li_sched_forget": (I, [P, I]),
    "li_cm_pack_step": (I, [P, I, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P, ctypes.c_longlong, P, I]),
    "li_cm_table_updates_bound": (I, [P, I, P, P, P, P]),
}


def library() -> ctypes.CDLL:
    """The host runtime, compiled with the system's C++ compiler on first use."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                from ..csrc.build import ensure_host_built

                lib = ctypes.CDLL(str(ensure_host_built()))
                lib.li_host_last_error.restype = ctypes.c_char_p
                for name, (res, args) in _SIGNATURES.items():
                    fn = getattr(lib, name)
                    fn.restype = res
                    fn.argtypes = args
                _lib = lib
    return _lib


def check(code: int) -> None:
    """Raise what the library reported: a class per kind of fault, its own words as the message."""
    if code:
        raise _ERRORS.get(code, RuntimeError)(library().li_host_last_error().decode("utf-8", "replace"))
