"""Policy search for the B200 A16W16 GEMM.

Retargets the reference's tuner (gemm_tune.py: search space :235-249, tile-fit pruner :60-92, validity filter
:257-300, per-policy correctness + timing :187-226, JSONL writer :392-406) to Blackwell parameters. There is no
compile step: every candidate is a row of the library's ahead-of-time variant table, so the reference's parallel
compile pool (:126-184) has no counterpart. Output rows keep the reference's schema
{arch, dtype, layout, m, n, k, config, duration (us), tflops}; `arch` is "sm_100a".
"""
from __future__ import annotations

import itertools
import json
import statistics
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Optional

from . import policy as P

ARCH = "sm_100a"


@dataclass
class TuneArgs:
    dtype: str          # "bf16" | "fp16"
    m: int
    n: int
    k: int
    layout: str = "nt"
    enable_split_k: bool = False
    has_bias: bool = True
    out_dtype: Optional[str] = None


def tile_fit(m: int, n: int, k: int, cfg: dict) -> float:
    """Useful fraction of the work a tiling performs: logical volume / volume after padding M, N to whole tiles
    and every K slice to whole K blocks (same idea as the reference's tile-IoU pruner, gemm_tune.py:60-92)."""
    p_ext, q = (n, m) if cfg.get("swap_ab") else (m, n)
    tm = P.TILE_M * cfg.get("cta_group", 1)
    pad_p = -(-p_ext // tm) * tm
    pad_q = -(-q // cfg["tile_n"]) * cfg["tile_n"]
    tk = P.tile_k(cfg["tile_n"], cfg.get("cta_group", 1), cfg.get("tile_k", 0))
    pad_k = sum(nb for _, nb in P.split_k_slices(k, cfg.get("split_k", 1), tk)) * tk
    return (m * n * k) / (pad_p * pad_q * pad_k)


def candidate_configs(args: TuneArgs, num_sms: int = P.NUM_SMS_DEFAULT) -> list[dict]:
    """Every runnable policy worth timing for this problem."""
    variants = [(1, t, tk) for t in P.TILE_N_MENU for tk in ((64, 128) if t <= 128 else (64,))]
    variants += [(2, t, 64) for t in P.MAX_STAGES_PAIR]
    # run-time widths of the 512-column pair variant: worth timing where whole waves matter (few tiles per CTA pair)
    if args.m > 2 * P.TILE_M and -(-args.m // (2 * P.TILE_M)) * -(-args.n // 256) <= 6 * (num_sms // 2):
        variants += [(2, t, 64) for t in range(288, 512, 32)]
    out = []
    for (cg, tile_n, tk), swap in itertools.product(variants, (False, True)):
        if swap and (cg == 2 or args.m > 256):
            continue
        p_ext, q = (args.n, args.m) if swap else (args.m, args.n)
        if tile_n > max(64, 2 * (1 << (max(q, 1) - 1).bit_length())):
            continue  # tile far wider than the problem
        tiles = -(-p_ext // (P.TILE_M * cg)) * -(-q // tile_n)
        walkers = num_sms // cg
        kb = -(-args.k // tk)  # K blocks of this variant's stage depth
        max_stages = P.max_stages(tile_n, cg, tk)
        stage_opts = sorted({max_stages, max(2, max_stages - 2)})
        splits = [(1, False, "ticket")]
        if tiles % walkers != 0:
            splits.append((1, True, "ticket"))  # stream-K
        if args.enable_split_k or tiles * 2 <= walkers:
            for s in (2, 3, 4, 6, 8, 12, 16, 24, 32, 48):
                if s <= kb and tiles * s <= 4 * walkers:
                    splits.append((s, False, "ticket"))
            if cg == 1:
                for s in (2, 4, 8, 16):  # K slices as one thread-block cluster
                    if s <= kb and tiles * s <= 2 * walkers:
                        splits.append((s, False, "cluster"))
        if args.out_dtype == "fp32" and not swap and tile_n >= 64:
            # fp32 outputs: K-parallel units may add their tiles straight into C (no workspace, no second pass)
            splits += [(s, sk, "atomic") for (s, sk, mode) in list(splits) if mode == "ticket" and (s > 1 or sk)]
        groups = (0, 4, 8) if tiles >= 2 * walkers else (0,)
        for stages, (split_k, stream_k, mode), group_m in itertools.product(stage_opts, splits, groups):
            cfg = {"tile_n": tile_n, "cta_group": cg, "stages": stages, "split_k": split_k, "stream_k": stream_k,
                   "group_m": group_m, "swap_ab": swap, "split_mode": mode, "tile_k": tk}
            pol = P.Policy(tile_n=tile_n, stages=stages, split_k=split_k, group_m=group_m, swap_ab=swap, cta_group=cg,
                           stream_k=stream_k, split_mode=mode, tile_k=tk)
            if P.validate(pol, args.m, args.n, args.k, args.layout) is None:
                out.append(cfg)
    if not out:
        return out
    keep = 0.5 if args.m <= 32 else 0.7 if args.m <= 128 else 0.85
    best = max(tile_fit(args.m, args.n, args.k, c) for c in out)
    return [c for c in out if tile_fit(args.m, args.n, args.k, c) >= keep * best]


def already_tuned(path: Path) -> set[tuple]:
    done = set()
    if path.exists():
        for line in path.read_text().splitlines():
            if line.strip():
                r = json.loads(line)
                done.add((r.get("arch"), r["dtype"], r["layout"], r["m"], r["n"], r["k"]))
    return done


def append_result(path: Path, args: TuneArgs, config: dict, duration_us: float) -> dict:
    rec = {"arch": ARCH, "dtype": args.dtype, "layout": args.layout, "m": args.m, "n": args.n, "k": args.k,
           "config": config, "duration": duration_us, "tflops": 2.0 * args.m * args.n * args.k / duration_us * 1e-6}
    path.parent.mkdir(parents=True, exist_ok=True)
    with path.open("a", encoding="utf-8") as f:
        f.write(json.dumps(rec) + "\n")
    return rec


# --------------------------------------------------------------------------------------------- GPU part
def _make_inputs(args: TuneArgs, copies: int):
    import torch

    dt = {"bf16": torch.bfloat16, "fp16": torch.float16}[args.dtype]

    def mat(rows, cols, is_t):
        t = torch.empty((cols, rows) if is_t else (rows, cols), dtype=dt, device="cuda").uniform_(-1, 1)
        return t.t() if is_t else t

    sets = []
    for _ in range(copies):
        a = mat(args.m, args.k, args.layout[0] == "t")
        b = mat(args.k, args.n, args.layout[1] == "t")
        bias = torch.empty(args.n, dtype=dt, device="cuda").uniform_(-1, 1) if args.has_bias else None
        out_dt = torch.float32 if args.out_dtype == "fp32" else dt
        sets.append((a, b, bias, torch.empty((args.m, args.n), dtype=out_dt, device="cuda")))
    return sets


def time_config(args: TuneArgs, cfg: dict, sets, iters: int = 30) -> float:
    """Check one policy against torch.addmm on the same GPU (the reference tuner's gate, gemm_tune.py:187-203),
    then return its median device time in microseconds over rotating buffers."""
    import math

    import torch

    from .gemm_a16w16 import check_status, gemm_a16w16

    a, b, bias, out = sets[0]
    out.fill_(float("nan"))
    gemm_a16w16(a, b, out, bias=bias, user_kwargs=cfg, layout=args.layout)
    check_status()
    ref = torch.matmul(a.float(), b.float())
    if bias is not None:
        ref += bias.float()
    scale = math.sqrt(max(args.k, 1) / 1024.0)
    rtol, atol = (2e-3, 2e-3 * scale) if out.dtype is torch.float32 else (1e-2, 1e-2 * scale)
    if not torch.allclose(out.float(), ref.to(out.dtype).float(), rtol=rtol, atol=atol):
        raise AssertionError("result outside tolerance")
    for i in range(3):
        s = sets[i % len(sets)]
        gemm_a16w16(s[0], s[1], s[3], bias=s[2], user_kwargs=cfg, layout=args.layout)
    # Device time per call from CUDA-graph replay (no host launch overhead, like the reference's profiler-based
    # kernel times); plain stream loop if the capture fails.
    side = torch.cuda.Stream()
    graph = None
    try:
        with torch.cuda.stream(side):
            for i in range(2):
                s = sets[i % len(sets)]
                gemm_a16w16(s[0], s[1], s[3], bias=s[2], user_kwargs=cfg, layout=args.layout, stream=side)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(iters):
                    s = sets[i % len(sets)]
                    gemm_a16w16(s[0], s[1], s[3], bias=s[2], user_kwargs=cfg, layout=args.layout, stream=side)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
    except Exception:
        graph = None
    times = []
    for rep in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        if graph is not None:
            graph.replay()
        else:
            for i in range(iters):
                s = sets[i % len(sets)]
                gemm_a16w16(s[0], s[1], s[3], bias=s[2], user_kwargs=cfg, layout=args.layout)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / iters * 1e3)
    check_status()
    return statistics.median(times)


def tune_single(args: TuneArgs, out_path: Optional[Path] = None, verbose: bool = True, max_configs: int = 0) -> Optional[dict]:
    import torch

    configs = candidate_configs(args, torch.cuda.get_device_properties(0).multi_processor_count)
    if max_configs:
        configs = configs[:max_configs]
    if not configs:
        raise RuntimeError(f"no runnable policy for {args}")
    per_set = 2 * (args.m * args.k + args.k * args.n + args.m * args.n)
    copies = max(1, min(16, (300 << 20) // max(per_set, 1)))
    sets = _make_inputs(args, copies)
    best, best_us = None, float("inf")
    for cfg in configs:
        try:
            us = time_config(args, cfg, sets)
        except Exception as exc:  # a failing candidate is skipped, as in the reference's tuner
            if verbose:
                print(f"  skip {cfg}: {exc}", flush=True)
            continue
        if verbose:
            print(f"  {us:9.2f} us  {2.0 * args.m * args.n * args.k / us * 1e-6:8.1f} TF  {cfg}", flush=True)
        if us < best_us:
            best, best_us = cfg, us
    if best is None:
        return None
    rec = {"arch": ARCH, "dtype": args.dtype, "layout": args.layout, "m": args.m, "n": args.n, "k": args.k,
           "config": best, "duration": best_us, "tflops": 2.0 * args.m * args.n * args.k / best_us * 1e-6}
    if out_path is not None:
        append_result(out_path, args, best, best_us)
    return rec


# Shapes the reference tunes (gemm_tune.py:348-391) plus the benchmark configurations.
DEFAULT_SHAPES = [
    (8, 4096, 4096), (16, 4096, 4096), (32, 4096, 4096), (64, 4096, 4096), (128, 4096, 4096), (256, 4096, 4096),
    (512, 4096, 4096), (1024, 4096, 4096), (2048, 4096, 4096), (1024, 1024, 1024), (2048, 2048, 2048),
    (4096, 4096, 4096), (4096, 4096, 8192), (8192, 8192, 8192), (8, 7168, 2048), (32, 384, 7168), (32, 14336, 4096),
    (16, 28672, 4096), (4096, 256, 4096), (1, 5120, 2880), (16, 5120, 2880), (48, 5120, 2880), (32, 384, 16384),
    (800, 384, 7168), (32, 7168, 2048), (32, 2880, 2048), (256, 512, 1024), (16384, 3584, 8192),
]


def tune_all(dtype: str, out_path: Path, layout: str, shapes: Iterable[tuple] = DEFAULT_SHAPES, enable_split_k: bool = False,
             verbose: bool = True) -> list[dict]:
    done = already_tuned(out_path)
    results = []
    for m, n, k in shapes:
        if (ARCH, dtype, layout, m, n, k) in done:
            continue  # resume: finished shapes are not repeated
        rec = tune_single(TuneArgs(dtype=dtype, m=m, n=n, k=k, layout=layout, enable_split_k=enable_split_k), out_path, verbose)
        if rec:
            results.append(rec)
            print(rec, flush=True)
    return results
