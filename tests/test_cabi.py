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
    assert declared == set(_lib.EXPORTS), (sorted(declared - set(_lib.EXPORTS)), sorted(set(_lib.EXPORTS) - declared))


def test_version_variants_and_strerror():
    lib = _lib.load()
    assert b"sm_100a" in lib.b200_gemm_version()
    v = _lib.variants()
    assert {x["tile_n"] for x in v} == {16, 32, 64, 128, 192, 256, 512}
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


def test_multi_gpu_entry_points_validate_before_touching_a_device():
    lib = _lib.load()
    h = _lib.PeerHandle()
    assert C.sizeof(_lib.PeerHandle) == 88  # 64-byte IPC handle + offset + bytes + device + reserved
    ptr = C.c_void_p()
    assert lib.b200_peer_export(None, C.byref(h)) == -1
    assert lib.b200_peer_export(C.c_void_p(4096), None) == -1
    assert lib.b200_peer_open(None, C.byref(ptr)) == -1
    assert lib.b200_peer_open(C.byref(h), None) == -1
    assert lib.b200_peer_close(None, C.byref(h)) == -1
    # reduce_slots: null pointers, no slots, cols not a multiple of 4, slots closer together than one image,
    # misaligned base, unknown dtype: all refused with BAD_ARG, nothing launched
    ok = (C.c_void_p(4096), 1024, 2, C.c_void_p(8192), None, 4, 256, 2, 0, None)
    def call(**kw):
        names = ("slots", "stride", "n", "out", "bias", "rows", "cols", "odt", "bdt", "stream")
        vals = dict(zip(names, ok))
        vals.update(kw)
        return lib.b200_gemm_reduce_slots(*[vals[k] for k in names])
    assert call(slots=None) == -1 and call(out=None) == -1
    assert call(n=0) == -1
    assert call(cols=254) == -1
    assert call(stride=512) == -1          # two 4x256 images cannot be 512 elements apart
    assert call(stride=1026) == -1         # not a multiple of 4 elements
    assert call(slots=C.c_void_p(4100)) == -1
    assert call(odt=7) == -1
    assert call(bias=C.c_void_p(64), bdt=1) == -1  # bias must be bf16 or fp16
    assert call(rows=0) == 0               # nothing to do is not an error


def test_wait_selftest_validates_its_arguments():
    lib = _lib.load()
    assert lib.b200_gemm_wait_selftest(None, 100, None) == -1
    assert lib.b200_gemm_wait_selftest(C.c_void_p(4096), 0, None) == -1         # no limit given
    assert lib.b200_gemm_wait_selftest(C.c_void_p(4096), 2_000_000, None) == -1  # beyond one second


def test_ctypes_structures_match_the_header(tmp_path):
    """The Python binding restates the header's structs by hand: compile the header with the host C compiler and compare
    sizes and the offsets of the last members, so that a field added on one side only is caught here and not on a GPU."""
    import shutil
    import subprocess

    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        import pytest

        pytest.skip("no host C compiler")
    src = tmp_path / "layout.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "b200_gemm.h"\n'
        "int main(void) {\n"
        '  printf("%zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(b200_gemm_policy), sizeof(b200_gemm_args), sizeof(b200_gemm_plan),\n'
        "         sizeof(b200_peer_handle), offsetof(b200_gemm_policy, reserved), offsetof(b200_gemm_args, trace_words),\n"
        "         offsetof(b200_gemm_plan, atomic_out), offsetof(b200_gemm_args, policy));\n"
        "  return 0;\n}\n")
    exe = tmp_path / "layout"
    subprocess.run([cc, "-std=c99", f"-I{ROOT / 'include'}", "-o", str(exe), str(src)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    want = [C.sizeof(_lib.Policy), C.sizeof(_lib.Args), C.sizeof(_lib.Plan), C.sizeof(_lib.PeerHandle),
            _lib.Policy.reserved.offset, _lib.Args.trace_words.offset, _lib.Plan.atomic_out.offset, _lib.Args.policy.offset]
    assert got == want, (got, want)
