"""The C-ABI library loads without a GPU and exports every symbol include/b200_gemm.h declares."""
import ctypes as C
import re
from pathlib import Path

from flydsl_examples_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    names = set()
    for h in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        names |= set(re.findall(r"\b(b200_(?:gemm|peer)_[a-z0-9_]+)\s*\(", text))
    return names


def test_every_declared_symbol_is_exported():
    lib = _lib.load()
    declared = _declared()
    assert "b200_gemm_a16w16" in declared and len(declared) >= 7
    for name in declared:
        assert getattr(lib, name) is not None, name
    assert declared == set(_lib.EXPORTS) | {n for n in declared if n not in _lib.EXPORTS}
    for name in _lib.EXPORTS:
        assert name in declared, f"{name} is bound but not declared in include/"


def test_version_variants_and_strerror():
    lib = _lib.load()
    assert b"sm_100a" in lib.b200_gemm_version()
    v = _lib.variants()
    assert {x["tile_n"] for x in v} == {16, 32, 64, 128, 256}
    assert {(x["tile_n"], x["cta_group"], x["tile_k"]) for x in v} >= {(128, 1, 128), (128, 1, 64), (16, 1, 64), (256, 1, 64), (256, 2, 64)}
    assert _lib.strerror(0) == "ok"
    assert "policy" in _lib.strerror(-2)
    assert "unknown" in _lib.strerror(-99)


def test_bad_arguments_return_codes_not_crashes():
    lib = _lib.load()
    pl = _lib.Plan()
    args = _lib.Args()
    assert lib.b200_gemm_plan_query(C.byref(args), C.byref(pl)) == -1  # zero sizes
    args.m, args.n, args.k = 128, 128, 128
    args.lda = args.ldb = args.ldo = 128
    args.in_dtype, args.out_dtype = 2, 2
    args.b_trans = 1
    args.policy.tile_n = 48
    assert lib.b200_gemm_plan_query(C.byref(args), C.byref(pl)) == -2
    args.policy.tile_n = 128
    assert lib.b200_gemm_plan_query(C.byref(args), C.byref(pl)) == 0
    args.out_dtype = 3  # bf16 in, fp16 out: not allowed
    assert lib.b200_gemm_plan_query(C.byref(args), C.byref(pl)) == -1
    args.out_dtype = 1
    args.lda = 64  # leading stride below the extent
    assert lib.b200_gemm_plan_query(C.byref(args), C.byref(pl)) == -1
    assert lib.b200_gemm_workspace_bytes(C.byref(args)) == 0
    assert lib.b200_gemm_plan_query(None, C.byref(pl)) == -1
