"""ctypes face of the cache manager's bookkeeping in C++ (``csrc/host/cache_core.cpp``): page pools, block
tables and request slots.  It has no CUDA in it, so it is built with the C++ compiler and runs where there is
no GPU."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_int, c_int32, c_int64, c_longlong, c_void_p

import numpy as np

from ..csrc import build

OK, EXHAUSTED, CONTEXT, SLOT_NOT_LIVE, NOT_OWNED, NO_SLOT, TABLE_FULL, BAD_ARG = range(8)

_lib = None


def lib():
    global _lib
    if _lib is None:
        l = build.load_library("host")
        P, I, LL = c_void_p, c_int, c_longlong
        IP, LP = POINTER(c_int), POINTER(c_longlong)
        sig = {
            "glint_pool_create": (P, [I]), "glint_pool_destroy": (None, [P]),
            "glint_pool_take": (I, [P, I, IP]), "glint_pool_give": (I, [P, IP, I, IP]),
            "glint_pool_stats": (None, [P, LP]), "glint_pool_free_list": (I, [P, IP, I]),
            "glint_cache_create": (P, [I, IP, I, I, I, I]), "glint_cache_destroy": (None, [P]),
            "glint_cache_pool": (P, [P, I]), "glint_cache_table": (POINTER(c_int32), [P, I]),
            "glint_cache_first_live": (POINTER(c_int64), [P, I]), "glint_cache_end_live": (POINTER(c_int64), [P, I]),
            "glint_cache_lengths": (POINTER(c_int64), [P]), "glint_cache_max_pages": (I, [P]),
            "glint_cache_free_slots": (I, [P]), "glint_cache_alloc_slot": (I, [P, IP]),
            "glint_cache_free_slot": (I, [P, I, IP]), "glint_cache_slot_live": (I, [P, I]),
            "glint_cache_pages_short": (I, [P, IP, IP, I, IP, LP, LP]),
            "glint_cache_reserve": (I, [P, IP, IP, I, IP, IP, LP, LP]),
            "glint_cache_advance": (None, [P, IP, IP, I]),
            "glint_cache_release_behind": (I, [P, I, I, LL]),
            "glint_cache_plan": (I, [P, I, I, I, IP, IP, IP, I, IP, IP, IP]),
        }
        for name, (res, args) in sig.items():
            f = getattr(l, name)
            f.restype, f.argtypes = res, args
        _lib = l
    return _lib


def int_array(values):
    """A C int array of ``values`` (kept alive by the caller for the call's duration)."""
    n = len(values)
    return (c_int * max(n, 1))(*values), n


def as_array(pointer, shape):
    """A numpy view of memory that the C++ side owns (no copy): it changes as the C++ side changes it."""
    return np.ctypeslib.as_array(pointer, shape=shape)
