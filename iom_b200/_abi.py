"""ctypes binding of libiom_b200.so (the declarations of include/iom_b200.h).

The library is mandatory: importing the operator layer without it raises, and
nothing in this package computes on the CPU instead.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
# IOMB_LIBRARY names another build of the same library (a variant compiled with other
# flags, for side-by-side measurements); the default is the in-tree build.
LIBRARY_PATH = Path(os.environ.get("IOMB_LIBRARY") or PACKAGE_DIR / "libiom_b200.so")

MAX_RANK = 8
MAX_LEADING = 6


class IombView(ctypes.Structure):
    """struct iomb_view."""

    _fields_ = [
        ("base", ctypes.c_void_p),
        ("storage_bytes", ctypes.c_uint64),
        ("dtype", ctypes.c_uint32),
        ("rank", ctypes.c_uint32),
        ("dims", ctypes.c_uint64 * MAX_RANK),
        ("plane_offset", ctypes.c_uint64),
        ("plane_strides", ctypes.c_uint64 * MAX_LEADING),
    ]


class IombSdpaStages(ctypes.Structure):
    """struct iomb_sdpa_stages."""

    _fields_ = [
        ("scores", ctypes.c_void_p),
        ("probability", ctypes.c_void_p),
        ("planes", ctypes.c_uint64), ("Hq", ctypes.c_uint64), ("Hkv", ctypes.c_uint64),
        ("R", ctypes.c_uint64), ("C", ctypes.c_uint64), ("D", ctypes.c_uint64),
        ("a", ctypes.c_uint64), ("L", ctypes.c_uint64),
    ]


# name -> (restype, argtypes); every symbol include/iom_b200.h declares.
_VIEW = ctypes.POINTER(IombView)
_U64P = ctypes.POINTER(ctypes.c_uint64)
PROTOTYPES = {
    "iomb_last_error": (ctypes.c_char_p, []),
    "iomb_last_launch": (ctypes.c_char_p, []),
    "iomb_rmsnorm_copy_timeouts": (ctypes.c_int, [ctypes.POINTER(ctypes.c_uint)]),
    "iomb_abi_version": (ctypes.c_uint32, []),
    "iomb_dtype_bits": (ctypes.c_uint32, [ctypes.c_uint32]),
    "iomb_tiled_storage_nbytes": (ctypes.c_int, [_U64P, ctypes.c_uint32, ctypes.c_uint32, _U64P]),
    "iomb_logical_nbytes": (ctypes.c_int, [_U64P, ctypes.c_uint32, ctypes.c_uint32, _U64P]),
    "iomb_plane_slot": (ctypes.c_uint64, [ctypes.c_uint64] * 5),
    "iomb_binary": (ctypes.c_int, [ctypes.c_int, _VIEW, _VIEW, _VIEW, ctypes.c_void_p]),
    "iomb_binary_supported": (ctypes.c_int, [ctypes.c_uint32]),
    "iomb_prepare_device": (ctypes.c_int, [ctypes.c_void_p]),
    "iomb_rmsnorm": (ctypes.c_int, [_VIEW, _VIEW, _VIEW, ctypes.c_float, ctypes.c_int, ctypes.c_void_p]),
    "iomb_add_rmsnorm": (ctypes.c_int, [_VIEW, _VIEW, _VIEW, _VIEW, _VIEW, ctypes.c_float,
                                        ctypes.c_int, ctypes.c_void_p]),
    "iomb_copy": (ctypes.c_int, [_VIEW, _VIEW, ctypes.c_void_p]),
    "iomb_cast": (ctypes.c_int, [_VIEW, _VIEW, ctypes.c_void_p]),
    "iomb_rope_angles": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64,
                                        ctypes.c_uint64, ctypes.c_double]),
    "iomb_rope": (ctypes.c_int, [_VIEW, _VIEW, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]),
    "iomb_silu": (ctypes.c_int, [_VIEW, _VIEW, ctypes.c_void_p]),
    "iomb_silu_mul": (ctypes.c_int, [_VIEW, _VIEW, _VIEW, _VIEW, ctypes.c_void_p]),
    "iomb_embedding": (ctypes.c_int, [_VIEW, _VIEW, _VIEW, ctypes.c_void_p, ctypes.c_void_p]),
    "iomb_cache_append": (ctypes.c_int, [_VIEW, _VIEW, ctypes.c_uint64, ctypes.c_void_p]),
    "iomb_cache_append_batched": (ctypes.c_int, [_VIEW, _VIEW, ctypes.c_void_p, ctypes.c_void_p,
                                                 ctypes.c_void_p]),
    "iomb_sumsq_scratch_bytes": (ctypes.c_uint64, []),
    "iomb_sumsq": (ctypes.c_int, [_VIEW, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "iomb_sumsq_static": (ctypes.c_int, [_VIEW, ctypes.c_void_p, ctypes.c_void_p]),
    "iomb_scatter": (ctypes.c_int, [_VIEW, ctypes.c_void_p, ctypes.c_void_p]),
    "iomb_gather": (ctypes.c_int, [_VIEW, ctypes.c_void_p, ctypes.c_void_p]),
    "iomb_sdpa_scale_mask": (ctypes.c_int, [ctypes.POINTER(IombSdpaStages), ctypes.c_void_p]),
    "iomb_sdpa_softmax": (ctypes.c_int, [ctypes.POINTER(IombSdpaStages), ctypes.c_void_p]),
    "iomb_sdpa_scale_mask_softmax": (ctypes.c_int, [ctypes.POINTER(IombSdpaStages), ctypes.c_int,
                                                    ctypes.c_void_p]),
    "iomb_sdpa_canonicalize_output": (ctypes.c_int, [_VIEW, ctypes.c_void_p]),
}

_library = None


def load_library() -> ctypes.CDLL:
    """Loads the kernel library; raises when it has not been built."""
    global _library
    if _library is None:
        if not LIBRARY_PATH.exists():
            raise RuntimeError(
                f"{LIBRARY_PATH} is missing: build it with `python -m iom_b200.build` "
                "(there is no CPU fallback)")
        library = ctypes.CDLL(str(LIBRARY_PATH))
        for name, (restype, argtypes) in PROTOTYPES.items():
            function = getattr(library, name)
            function.restype = restype
            function.argtypes = argtypes
        _library = library
    return _library


def last_error() -> str:
    text = load_library().iomb_last_error()
    return text.decode() if text else ""
