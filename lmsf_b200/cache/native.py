"""ctypes face of csrc/host_runtime.cpp (compiled with g++ on first use)."""
from __future__ import annotations

from ctypes import POINTER, c_double, c_int, c_int64, c_longlong, c_void_p

from ..csrc.build import load_library

_lib = None
P_INT = POINTER(c_int)
P_I64 = POINTER(c_int64)


def lib():
    global _lib
    if _lib is None:
        l = load_library("host_runtime.cpp")
        sig = {
            "lmsf_cm_create": (c_void_p, [c_int, P_INT, P_INT, c_int, c_int]),
            "lmsf_cm_destroy": (None, [c_void_p]),
            "lmsf_cm_has": (c_int, [c_void_p, c_int64]),
            "lmsf_cm_can_add": (c_int, [c_void_p]),
            "lmsf_cm_add": (c_int, [c_void_p, c_int64]),
            "lmsf_cm_free": (c_int, [c_void_p, c_int64]),
            "lmsf_cm_take_fresh_slots": (c_int, [c_void_p, P_INT, c_int]),
            "lmsf_cm_pages_needed": (c_int, [c_void_p, c_int64, c_int, P_INT]),
            "lmsf_cm_can_reserve": (c_int, [c_void_p, c_int64, c_int, c_int]),
            "lmsf_cm_reserve": (c_int, [c_void_p, c_int64, c_int]),
            "lmsf_cm_commit": (c_int, [c_void_p, c_int64, c_int]),
            "lmsf_cm_rollback": (c_int, [c_void_p, c_int64]),
            "lmsf_cm_query": (c_int, [c_void_p, c_int64, c_int, c_int]),
            "lmsf_cm_table": (c_int, [c_void_p, c_int64, c_int, P_INT, c_int]),
            "lmsf_cm_num_free": (c_int, [c_void_p, c_int]),
            "lmsf_cm_num_total": (c_int, [c_void_p, c_int]),
            "lmsf_cm_num_live": (c_int, [c_void_p]),
            "lmsf_cm_live": (c_int, [c_void_p, P_I64, c_int]),
            "lmsf_cm_check": (c_int, [c_void_p]),
            "lmsf_cm_build_batch": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_int, c_int, c_int, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p]),
            "lmsf_sched_create": (c_void_p, [c_void_p, c_int, c_int, c_int]),
            "lmsf_sched_destroy": (None, [c_void_p]),
            "lmsf_sched_add": (c_int, [c_void_p, c_int64, c_double, c_int]),
            "lmsf_sched_update": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
            "lmsf_sched_remove": (c_int, [c_void_p, c_int64]),
            "lmsf_sched_queue": (c_int, [c_void_p, c_int, c_void_p, c_int]),
            "lmsf_sched_num_preemptions": (c_longlong, [c_void_p]),
            "lmsf_sched_watermark": (c_int, [c_void_p, c_int]),
            "lmsf_sched_schedule": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_void_p]),
        }
        for name, (res, args) in sig.items():
            f = getattr(l, name)
            f.restype, f.argtypes = res, args
        _lib = l
    return _lib
