"""ctypes binding of the native host core (csrc/host_core.cpp): page pools, cache manager, scheduler.

The functions live in the same shared library as the kernels; loading it needs no GPU."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_int64, c_uint64, c_void_p

from . import build as _build

OK, ERR_NO_PAGES, ERR_NO_SLOT, ERR_STATE, ERR_NO_PROGRESS, ERR_POOL_TOO_SMALL = 0, -1, -2, -3, -4, -5

_lib = None
_IP = POINTER(c_int)
_LP = POINTER(c_int64)
_UP = POINTER(c_uint64)

_PROTOS = {
    "nvh_last_error": (c_char_p, []),
    "nvh_chain_hash": (c_uint64, [_IP, c_int, c_int, c_uint64]),
    "nvh_pool_create": (c_void_p, [c_int, c_int]),
    "nvh_pool_destroy": (None, [c_void_p]),
    "nvh_pool_num_pages": (c_int, [c_void_p]),
    "nvh_pool_num_free": (c_int, [c_void_p]),
    "nvh_pool_ref_count": (c_int, [c_void_p, c_int]),
    "nvh_pool_allocate": (c_int, [c_void_p]),
    "nvh_pool_share": (c_int, [c_void_p, c_int]),
    "nvh_pool_release": (c_int, [c_void_p, c_int]),
    "nvh_pool_lookup": (c_int, [c_void_p, c_uint64, _IP, c_int]),
    "nvh_pool_set_hash": (None, [c_void_p, c_int, c_uint64, _IP, c_int]),
    "nvh_pool_check": (c_int, [c_void_p, _IP]),
    "nvh_manager_create": (c_void_p, [_IP, _IP, c_int, c_int, c_int, c_int, c_int]),
    "nvh_manager_destroy": (None, [c_void_p]),
    "nvh_manager_pool": (c_void_p, [c_void_p, c_int]),
    "nvh_manager_groups": (c_int, [c_void_p]),
    "nvh_manager_prefix_caching": (c_int, [c_void_p]),
    "nvh_manager_free_slots": (c_int, [c_void_p]),
    "nvh_manager_num_requests": (c_int, [c_void_p]),
    "nvh_has": (c_int, [c_void_p, c_int64]),
    "nvh_open": (c_int, [c_void_p, c_int64]),
    "nvh_close": (c_int, [c_void_p, c_int64]),
    "nvh_extend": (c_int, [c_void_p, c_int64, c_int, c_int]),
    "nvh_can_extend": (c_int, [c_void_p, c_int64, c_int, c_int]),
    "nvh_pages_needed": (c_int, [c_void_p, c_int64, c_int, c_int, _IP]),
    "nvh_commit": (c_int, [c_void_p, c_int64, c_int, _IP, c_int]),
    "nvh_request_info": (c_int, [c_void_p, c_int64, c_int]),
    "nvh_table": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_int]),
    "nvh_match_prefix": (c_int, [c_void_p, _IP, c_int, _IP, _UP, c_int]),
    "nvh_adopt_prefix": (c_int, [c_void_p, c_int64, _IP, _UP, c_int]),
    "nvh_new_pages_for": (c_int, [c_void_p, c_int, _IP, c_int]),
    "nvh_manager_check": (c_int, [c_void_p]),
    "nvh_commit_many": (c_int, [c_void_p, c_int, _LP, _IP]),
    "nvh_step_layout": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, _IP, _IP]),
    "nvh_prepare_step": (c_int, [c_void_p, c_int, _LP, _IP, _IP, _IP, _IP, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                 _IP, _IP, _IP]),
    "nvh_touch_tables": (None, [c_void_p]),
    "nvs_create": (c_void_p, [c_void_p, c_int, c_int, c_int, c_int, c_int]),
    "nvs_destroy": (None, [c_void_p]),
    "nvs_add": (c_int, [c_void_p, c_int64, _IP, c_int, c_int, c_int, c_int]),
    "nvs_is_finished": (c_int, [c_void_p]),
    "nvs_num_preemptions": (c_int, [c_void_p]),
    "nvs_queue_sizes": (c_int, [c_void_p, _IP, _IP]),
    "nvs_seq_info": (c_int, [c_void_p, c_int64, c_int]),
    "nvs_forget": (c_int, [c_void_p, c_int64]),
    "nvs_schedule": (c_int, [c_void_p, _LP, _IP, _IP, _IP, c_int]),
    "nvs_postprocess": (c_int, [c_void_p, _IP, _LP, c_int]),
    "nvs_patch_token": (c_int, [c_void_p, c_int64, c_int, c_int]),
    "nvs_finish_late": (c_int, [c_void_p, c_int64]),
}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        L = ctypes.CDLL(_build.library_path())
        for name, (res, args) in _PROTOS.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib


def last_error() -> str:
    return lib().nvh_last_error().decode()


def ints(values):
    """A C int array of the values (kept alive by the caller for the duration of the call)."""
    n = len(values)
    return (c_int * max(n, 1))(*values), n
