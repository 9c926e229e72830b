"""ctypes binding of libb200_gemm.so (the C ABI in include/b200_gemm.h).

There is no fallback: if the library is missing and cannot be built, importing raises.
Takes the place of the reference's `flyc.compile` / DLPack argument marshalling
(kernels/gemm_a16w16_gfx950.py:1284-1285, :1419-1440).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

from . import build as _build

DTYPE_FP32, DTYPE_BF16, DTYPE_FP16 = 1, 2, 3
STATIC_SCRATCH_BYTES = 16 << 20  # B200_GEMM_STATIC_SCRATCH_BYTES
COUNTER_BYTES = 1 << 20          # B200_GEMM_COUNTER_BYTES: ticket region at the start of a workspace

ERR_TEXT_FALLBACK = "b200_gemm error"


class Policy(C.Structure):
    _fields_ = [
        ("tile_n", C.c_int32),
        ("stages", C.c_int32),
        ("split_k", C.c_int32),
        ("group_m", C.c_int32),
        ("swap_ab", C.c_int32),
        ("cta_group", C.c_int32),
        ("split_mode", C.c_int32),
        ("max_ctas", C.c_int32),
        ("stream_k", C.c_int32),
        ("no_pdl", C.c_int32),
        ("tile_k", C.c_int32),
        ("wait_limit_us", C.c_int32),
        ("loader", C.c_int32),
        ("reserved", C.c_int32 * 3),
    ]


class Args(C.Structure):
    _fields_ = [
        ("a", C.c_void_p),
        ("b", C.c_void_p),
        ("out", C.c_void_p),
        ("bias", C.c_void_p),
        ("m", C.c_int64),
        ("n", C.c_int64),
        ("k", C.c_int64),
        ("lda", C.c_int64),
        ("ldb", C.c_int64),
        ("ldo", C.c_int64),
        ("a_trans", C.c_int32),
        ("b_trans", C.c_int32),
        ("in_dtype", C.c_int32),
        ("out_dtype", C.c_int32),
        ("policy", Policy),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_uint64),
        ("status", C.c_void_p),
        ("trace", C.c_void_p),
        ("trace_words", C.c_uint64),
    ]


class Plan(C.Structure):
    _fields_ = [
        ("tile_m", C.c_int32),
        ("tile_n", C.c_int32),
        ("tile_k", C.c_int32),
        ("stages", C.c_int32),
        ("split_k", C.c_int32),
        ("cta_group", C.c_int32),
        ("swap_ab", C.c_int32),
        ("group_m", C.c_int32),
        ("tiles_p", C.c_int32),
        ("tiles_q", C.c_int32),
        ("num_units", C.c_int32),
        ("grid", C.c_int32),
        ("smem_bytes", C.c_int32),
        ("tmem_cols", C.c_int32),
        ("cluster_split", C.c_int32),
        ("stream_k", C.c_int32),
        ("sk_tiles", C.c_int32),
        ("sk_slots", C.c_int32),
        ("a_repacked", C.c_int32),
        ("b_repacked", C.c_int32),
        ("a_loader", C.c_int32),
        ("b_loader", C.c_int32),
        ("counter_bytes", C.c_uint64),
        ("partial_bytes", C.c_uint64),
        ("repack_bytes", C.c_uint64),
        ("workspace_bytes", C.c_uint64),
        ("atomic_out", C.c_int32),
        ("reserved", C.c_int32),
    ]

    def as_dict(self) -> dict:
        return {name: getattr(self, name) for name, _ in self._fields_}


class PeerHandle(C.Structure):
    """b200_peer_handle: plain bytes, safe to pickle with bytes(handle) and rebuild with from_buffer_copy."""
    _fields_ = [
        ("ipc", C.c_uint8 * 64),
        ("offset", C.c_uint64),
        ("bytes", C.c_uint64),
        ("device", C.c_int32),
        ("reserved", C.c_int32),
    ]


EXPORTS = (
    "b200_gemm_a16w16",
    "b200_gemm_a16w16_static_scratch",
    "b200_gemm_prepare",
    "b200_gemm_launch",
    "b200_gemm_release",
    "b200_gemm_plan_query",
    "b200_gemm_workspace_bytes",
    "b200_gemm_num_variants",
    "b200_gemm_describe_variant",
    "b200_gemm_cast_bias",
    "b200_gemm_reduce_slots",
    "b200_peer_export",
    "b200_peer_open",
    "b200_peer_close",
    "b200_gemm_selftest",
    "b200_gemm_wait_selftest",
    "b200_gemm_strerror",
    "b200_gemm_version",
)

_lib = None


def lib_path() -> Path:
    return _build.LIB_PATH


def load() -> C.CDLL:
    """Load (building first if the sources are newer and nvcc is present) the shared library."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if not _build.is_current() and os.environ.get("B200_GEMM_NO_BUILD") != "1":
        try:
            _build.build()
        except Exception as exc:  # no nvcc on this machine: a prebuilt library is still usable
            if not path.exists():
                raise ImportError(
                    f"libb200_gemm.so is missing and could not be built ({exc}); "
                    "run `python -m flydsl_examples_b200.build`"
                ) from exc
    if not path.exists():
        raise ImportError("libb200_gemm.so is missing; run `python -m flydsl_examples_b200.build`")
    lib = C.CDLL(str(path))
    lib.b200_gemm_a16w16.argtypes = [C.POINTER(Args), C.c_void_p]
    lib.b200_gemm_a16w16.restype = C.c_int
    lib.b200_gemm_a16w16_static_scratch.argtypes = [C.POINTER(Args), C.c_void_p]
    lib.b200_gemm_a16w16_static_scratch.restype = C.c_int
    lib.b200_gemm_prepare.argtypes = [C.POINTER(Args), C.POINTER(C.c_void_p)]
    lib.b200_gemm_prepare.restype = C.c_int
    lib.b200_gemm_launch.argtypes = [C.c_void_p, C.c_void_p]
    lib.b200_gemm_launch.restype = C.c_int
    lib.b200_gemm_release.argtypes = [C.c_void_p]
    lib.b200_gemm_release.restype = None
    lib.b200_gemm_plan_query.argtypes = [C.POINTER(Args), C.POINTER(Plan)]
    lib.b200_gemm_plan_query.restype = C.c_int
    lib.b200_gemm_workspace_bytes.argtypes = [C.POINTER(Args)]
    lib.b200_gemm_workspace_bytes.restype = C.c_uint64
    lib.b200_gemm_num_variants.argtypes = []
    lib.b200_gemm_num_variants.restype = C.c_int
    lib.b200_gemm_describe_variant.argtypes = [C.c_int, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                               C.POINTER(C.c_int32)]
    lib.b200_gemm_describe_variant.restype = C.c_int
    lib.b200_gemm_cast_bias.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_void_p]
    lib.b200_gemm_cast_bias.restype = C.c_int
    lib.b200_gemm_reduce_slots.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                           C.c_int32, C.c_int32, C.c_void_p]
    lib.b200_gemm_reduce_slots.restype = C.c_int
    lib.b200_peer_export.argtypes = [C.c_void_p, C.POINTER(PeerHandle)]
    lib.b200_peer_export.restype = C.c_int
    lib.b200_peer_open.argtypes = [C.POINTER(PeerHandle), C.POINTER(C.c_void_p)]
    lib.b200_peer_open.restype = C.c_int
    lib.b200_peer_close.argtypes = [C.c_void_p, C.POINTER(PeerHandle)]
    lib.b200_peer_close.restype = C.c_int
    lib.b200_gemm_selftest.argtypes = [C.c_void_p, C.POINTER(C.c_int32)]
    lib.b200_gemm_selftest.restype = C.c_int
    lib.b200_gemm_wait_selftest.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p]
    lib.b200_gemm_wait_selftest.restype = C.c_int
    lib.b200_gemm_strerror.argtypes = [C.c_int]
    lib.b200_gemm_strerror.restype = C.c_char_p
    lib.b200_gemm_version.argtypes = []
    lib.b200_gemm_version.restype = C.c_char_p
    _lib = lib
    return lib


def strerror(code: int) -> str:
    try:
        return load().b200_gemm_strerror(code).decode()
    except Exception:
        return ERR_TEXT_FALLBACK


def variants() -> list[dict]:
    lib = load()
    out = []
    for i in range(lib.b200_gemm_num_variants()):
        tn, cg, ms, tk = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
        lib.b200_gemm_describe_variant(i, C.byref(tn), C.byref(cg), C.byref(ms), C.byref(tk))
        out.append({"tile_n": tn.value, "cta_group": cg.value, "max_stages": ms.value, "tile_k": tk.value})
    return out
