"""The host runtime: the C++ library of ``csrc/host`` (cache accounting, step packer, scheduler),
loaded with ctypes.  ``lib()`` builds it on first use; there is no Python stand-in."""
from __future__ import annotations

import ctypes
from typing import Optional

_I, _L, _P = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p
_IP = ctypes.POINTER(ctypes.c_int)
_LP = ctypes.POINTER(ctypes.c_int64)

# Status codes (csrc/host/cache.h).
UNKNOWN_REQUEST, ALREADY_OPEN, OUT_OF_PAGES, OUT_OF_SLOTS = -1, -2, -3, -4
BAD_ARGUMENT, RELEASED_PAGE, NOT_HELD, INCONSISTENT, TOO_SMALL = -5, -6, -7, -8, -9

_SIGNATURES = {
    "ph_freelist_new": (_P, [_I]), "ph_freelist_delete": (None, [_P]), "ph_freelist_take": (_I, [_P]),
    "ph_freelist_give": (_I, [_P, _I]), "ph_freelist_n": (_I, [_P]), "ph_freelist_n_free": (_I, [_P]),
    "ph_freelist_held": (_I, [_P, _I]),
    "ph_cache_new": (_P, [_I, _IP, _IP, _I, _I]), "ph_cache_delete": (None, [_P]),
    "ph_open": (_I, [_P, _L]), "ph_has": (_I, [_P, _L]), "ph_length": (_I, [_P, _L]), "ph_state_slot": (_I, [_P, _L]),
    "ph_n_logical_pages": (_I, [_P, _L]), "ph_pages_to_append": (_I, [_P, _L, _I, _IP]), "ph_reclaimable": (_I, [_P, _L, _IP]),
    "ph_can_append": (_I, [_P, _L, _I]), "ph_can_admit": (_I, [_P, _I]), "ph_release_passed": (_I, [_P, _L]),
    "ph_append": (_I, [_P, _L, _I]), "ph_close": (_I, [_P, _L]), "ph_check": (_I, [_P]),
    "ph_n_free_pages": (_I, [_P, _I]), "ph_n_pages": (_I, [_P, _I]), "ph_page_held": (_I, [_P, _I, _I]),
    "ph_n_free_slots": (_I, [_P]), "ph_slot_held": (_I, [_P, _I]),
    "ph_table": (_I, [_P, _L, _I, _IP, _I]), "ph_slots": (_I, [_P, _L, _I, _I, _I, _IP]),
    "ph_set_resident_tables": (None, [_P, _I]),
    "ph_step_plan": (_I, [_P, _I, _LP, _IP, _IP, _IP, _IP, _IP, _I, _I, _I, _IP, _IP, _IP, _IP]),
    "ph_step_pack": (_I, [_P, _I, _LP, _IP, _IP, _IP, _IP, _IP, _IP, _IP, _IP, _P, _I, _IP, _IP]),
}

_lib: Optional[ctypes.CDLL] = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        from .csrc.build import host_library
        loaded = host_library()
        for name, (res, args) in _SIGNATURES.items():
            f = getattr(loaded, name)
            f.restype, f.argtypes = res, args
        _lib = loaded
    return _lib


def ints(values) -> ctypes.Array:
    return (ctypes.c_int * len(values))(*values)


def longs(values) -> ctypes.Array:
    return (ctypes.c_int64 * len(values))(*values)
