#!/usr/bin/env python
"""Policy tuner CLI; same flags as the reference's gemm_tune.py (:409-448), Blackwell search space.

    python gemm_tune.py --single --dtype bf16 --m 2048 --n 4096 --k 4096
    python gemm_tune.py --tune_all --enable_split_k --out gemm_a16w16_tuned
"""
import argparse
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from flydsl_examples_b200 import tuner  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser(description="Tune gemm_a16w16 policies on B200")
    ap.add_argument("--out", type=str, default="gemm_a16w16_tuned", help="output prefix; '.jsonl' is appended")
    ap.add_argument("--dtype", type=str, default="bf16", choices=("bf16", "f16", "fp16"))
    ap.add_argument("--layout", choices=("nn", "nt", "tn", "tt"), default="nt")
    ap.add_argument("--single", action="store_true")
    ap.add_argument("--tune_all", action="store_true")
    ap.add_argument("--enable_split_k", "--enable-split-k", action="store_true")
    ap.add_argument("--shapes", type=str, default=None, help="semicolon-separated m,n,k triples for --tune_all")
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--quiet", action="store_true")
    a = ap.parse_args()
    dtype = "fp16" if a.dtype in ("f16", "fp16") else "bf16"
    out = Path(a.out + ".jsonl")
    if a.single:
        rec = tuner.tune_single(tuner.TuneArgs(dtype=dtype, m=a.m, n=a.n, k=a.k, layout=a.layout, enable_split_k=a.enable_split_k),
                                out, verbose=not a.quiet)
        print(rec)
    elif a.tune_all:
        shapes = tuner.DEFAULT_SHAPES
        if a.shapes:
            shapes = [tuple(int(x) for x in s.split(",")) for s in a.shapes.split(";") if s]
        tuner.tune_all(dtype, out, a.layout, shapes, a.enable_split_k, verbose=not a.quiet)
    else:
        ap.print_help()


if __name__ == "__main__":
    main()
