"""ctypes binding of libmechta_kv.so, the C-ABI library declared in include/mechta_kv.h.

The library is built in-tree (mechta_b200/csrc/Makefile, or build() below). There is no fallback: if the
shared object is missing or a symbol is absent the import of the product path fails with a clear error.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
# MKV_LIB_PATH names another build of the same library to load instead (e.g. the measurement build, `make measure`)
SO_PATH = os.environ.get("MKV_LIB_PATH") or os.path.join(_HERE, "libmechta_kv.so")
HEADER = os.path.join(os.path.dirname(_HERE), "include", "mechta_kv.h")

OK, ERR_INVALID, ERR_CAPACITY, ERR_CUDA, ERR_NOMEM, ERR_UNSUPPORTED, ERR_STATE, ERR_FORMAT, ERR_IO = range(9)
F16, F32 = 0, 1
REC = 258


class MkvError(RuntimeError):
    """A call into libmechta_kv returned a status other than MKV_OK."""

    def __init__(self, status: int, text: str):
        super().__init__(f"mkv status {status}: {text}")
        self.status = status


class StepIn(C.Structure):
    """mkv_step_in of include/mechta_kv.h."""
    _fields_ = [("qf_dev", C.c_void_p), ("kb_dev", C.c_void_p), ("vb_dev", C.c_void_p), ("q_norm_dev", C.c_void_p),
                ("k_norm_dev", C.c_void_p), ("rope_tab_dev", C.c_void_p), ("eps", C.c_float)]


class VerifyItem(C.Structure):
    """mkv_verify_item of include/mechta_kv.h."""
    _fields_ = [("cache", C.c_void_p), ("layer", C.c_int32), ("first_pos", C.c_uint32), ("pos", C.c_uint32),
                ("ntok", C.c_uint32), ("q_dev", C.c_void_p), ("out_dev", C.c_void_p)]


def build(force: bool = False) -> str:
    """Compile the library for sm_100a with nvcc (no GPU needed to build)."""
    csrc = os.path.join(_HERE, "csrc")
    cmd = ["make", "-C", csrc, "-j8"] + (["-B"] if force else [])
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building libmechta_kv.so failed:\n" + r.stdout[-4000:] + r.stderr[-4000:])
    return SO_PATH


def build_checks() -> str:
    """Compile the checked build (every cache buffer between canary bytes): libmechta_kv_checks.so beside the library."""
    r = subprocess.run(["make", "-C", os.path.join(_HERE, "csrc"), "checks"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building libmechta_kv_checks.so failed:\n" + r.stdout[-4000:] + r.stderr[-4000:])
    return os.path.join(_HERE, "libmechta_kv_checks.so")


_SIGS = {
    # name: (restype, argtypes)
    "mkv_strerror": (C.c_char_p, [C.c_int]),
    "mkv_last_error": (C.c_char_p, []),
    "mkv_version": (C.c_char_p, []),
    "mkv_ctx_create": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(C.c_void_p)]),
    "mkv_ctx_destroy": (None, [C.c_void_p]),
    "mkv_sync": (C.c_int, [C.c_void_p]),
    "mkv_launch_count": (C.c_uint64, [C.c_void_p]),
    "mkv_prof_enable": (C.c_int, [C.c_void_p, C.c_int]),
    "mkv_prof_read": (C.c_int, [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_uint64)]),
    "mkv_cache_create": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_void_p)]),
    "mkv_cache_destroy": (None, [C.c_void_p]),
    "mkv_checks_enabled": (C.c_int, []),
    "mkv_cache_check_guards": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "mkv_checks_touch_guard": (C.c_int, [C.c_void_p]),
    "mkv_cache_buffers": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "mkv_cache_len": (C.c_uint32, [C.c_void_p]),
    "mkv_cache_set_len": (C.c_int, [C.c_void_p, C.c_uint32]),
    "mkv_need_bytes": (C.c_uint64, [C.c_uint32, C.c_int, C.c_int]),
    "mkv_cache_device_bytes": (C.c_uint64, [C.c_void_p]),
    "mkv_append": (C.c_int, [C.c_void_p, C.c_int, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "mkv_append_layers": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "mkv_rope_table": (None, [C.c_int32, C.c_uint32, C.c_void_p]),
    "mkv_truncate": (C.c_int, [C.c_void_p, C.c_uint32, C.c_int]),
    "mkv_attn_verify": (C.c_int, [C.c_void_p, C.c_int, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]),
    "mkv_attn_verify_partial": (C.c_int, [C.c_void_p, C.c_int, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]),
    "mkv_attn_verify_static": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                                         C.c_uint32, C.c_void_p, C.c_void_p]),
    "mkv_static_status": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(C.c_uint32)]),
    "mkv_exchange_create": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "mkv_exchange_handle": (C.c_int, [C.c_void_p, C.c_void_p]),
    "mkv_exchange_connect": (C.c_int, [C.c_void_p, C.c_void_p]),
    "mkv_exchange_destroy": (None, [C.c_void_p]),
    "mkv_attn_verify_exchange": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p,
                                           C.c_void_p]),
    "mkv_combine_shards": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_uint32, C.c_void_p]),
    "mkv_attn_verify_batch": (C.c_int, [C.c_void_p, C.POINTER(VerifyItem), C.c_int]),
    "mkv_cache_create_ring": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_uint32, C.c_uint32, C.POINTER(C.c_void_p)]),
    "mkv_attn_verify_window": (C.c_int, [C.c_void_p, C.c_int, C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]),
    "mkv_attn_step": (C.c_int, [C.c_void_p, C.c_int, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(StepIn), C.c_void_p, C.c_void_p]),
    "mkv_attn_prefill": (C.c_int, [C.c_void_p, C.c_int, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_int, C.c_void_p]),
    "mkv_snapshot_bytes": (C.c_size_t, [C.c_void_p, C.c_uint32]),
    "mkv_snapshot": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "mkv_snapshot_wait": (C.c_int, [C.c_void_p]),
    "mkv_restore": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_size_t]),
    "mkv_host_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "mkv_host_free": (None, [C.c_void_p]),
    "mkv_root_write": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.c_uint32, C.c_void_p, C.c_void_p, C.c_size_t]),
    "mkv_root_read": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_uint32), C.c_void_p, C.c_size_t, C.c_void_p,
                                C.c_size_t, C.POINTER(C.c_size_t)]),
    "mkv_root_key": (C.c_uint64, [C.c_void_p, C.c_size_t]),
    "mkv_dispatch": (C.c_int, [C.c_void_p, C.c_int, C.c_char_p, C.POINTER(C.c_uint32), C.c_void_p, C.c_void_p, C.c_void_p]),
}

_lib = None


def lib() -> C.CDLL:
    """Loads the library and types every entry point; raises if the library or a symbol is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise ImportError(f"{SO_PATH} is missing: build it with `make -C mechta_b200/csrc` "
                              "(or __graft_entry__.build()); there is no fallback path")
        L = C.CDLL(SO_PATH)
        for name, (res, args) in _SIGS.items():
            fn = getattr(L, name)  # AttributeError if the symbol is absent
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def exported_symbols() -> list[str]:
    return sorted(_SIGS)


def check(status: int) -> None:
    if status != OK:
        raise MkvError(status, lib().mkv_last_error().decode("utf-8", "replace"))
