"""In-kernel role timelines of one GEMM call (profiling aid).

Every CTA of the GEMM kernel can record %globaltimer stamps of its producer, MMA and epilogue roles for its first
work items (see `trace` in include/b200_gemm.h). This module runs one call with that buffer attached and prints, per
role and work item, the minimum / median / maximum over the CTAs of each stamp, in microseconds after the first
stamp of the launch (and, from clock64 read next to two of the stamps, the SM clock the call ran at):

    producer  s0 work item taken      s1 first load issued          s2 last load issued
    mma       s0 accumulator free     s1 first stage seen full      s2 last MMA issued
    epilogue  s0 accumulator complete s1 tile read out and sent off s2 done (after a split-K second pass)

    python -m flydsl_examples_b200.trace --m 2048 --n 4096 --k 4096 --layout nt --dtype bf16 --bias \
        --policy '{"tile_n": 256, "cta_group": 2}' [--out-dtype fp32] [--warm] [--detail]

The MMA rows end with the number of K blocks whose operands were not yet complete when the MMA warp first asked
(`stalls`). With `--detail` the MMA warp also counts its cycles per work item: waiting for operands, issuing the
MMAs, committing (this slows the kernel down a little, so the stamps of a `--detail` run are not the ones to quote).

By default a buffer larger than L2 is written before the traced call, so that the operands come from HBM; `--warm`
leaves them in L2. The reference has no counterpart (it times whole kernels with torch.profiler, gemm_tune.py:205-226).
"""
from __future__ import annotations

import argparse
import json

import torch

from . import gemm_a16w16 as G

ROLES = ("producer", "mma", "epilogue")
_DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def _operand(rows: int, cols: int, dtype: torch.dtype, is_t: bool, device) -> torch.Tensor:
    t = torch.randn((cols, rows) if is_t else (rows, cols), device=device, dtype=torch.float32).to(dtype)
    return t.t() if is_t else t


def timeline(m: int, n: int, k: int, user_kwargs: dict, layout: str = "nt", dtype: torch.dtype = torch.bfloat16,
             out_dtype: torch.dtype | None = None, bias: bool = False, cold: bool = True, items: int = 3,
             device: str = "cuda", detail: bool = False) -> dict:
    """Run one traced call; return {"span_us", "plan", "stamps": {role: [[(min, median, max) x 3] per item]},
    "mma": [{"stalls", "wait", "issue", "commit"} per item] (medians over the MMA-issuing CTAs; cycles only with detail)}."""
    out_dtype = out_dtype or dtype
    a = _operand(m, k, dtype, layout[0] == "t", device)
    b = _operand(k, n, dtype, layout[1] == "t", device)
    bias_t = torch.randn(n, device=device).to(dtype) if bias else None
    out = torch.empty(m, n, device=device, dtype=out_dtype)
    pl = G.plan(a, b, layout, user_kwargs, out_dtype=out_dtype, bias=bias_t)
    for _ in range(3):
        G.gemm_a16w16(a, b, out, bias=bias_t, user_kwargs=user_kwargs, layout=layout)
    torch.cuda.synchronize()
    words = torch.zeros(pl["grid"] * 4 * 16 * 4 * (2 if detail else 1), dtype=torch.int64, device=device)
    G.set_trace_buffer(words)
    try:
        if cold:
            torch.empty(256 << 20, dtype=torch.uint8, device=device).fill_(1)  # evict the operands from L2
        torch.cuda.synchronize()
        G.gemm_a16w16(a, b, out, bias=bias_t, user_kwargs=user_kwargs, layout=layout)
        torch.cuda.synchronize()
        G.check_status()
    finally:
        G.set_trace_buffer(None)
    t = words.cpu()[: pl["grid"] * 4 * 16 * 4].view(pl["grid"], 4, 16, 4)
    stamps = t[:, :3, :, :3]
    t0 = int(stamps[stamps > 0].min())
    result = {"span_us": (int(stamps.max()) - t0) / 1e3, "plan": pl, "stamps": {}}
    for r, role in enumerate(ROLES):
        rows = []
        for it in range(items):
            cols = []
            for s in range(3):
                x = t[:, r, it, s]
                x = x[x > 0]
                if x.numel() == 0:
                    cols.append(None)
                else:
                    x = (x - t0).double() / 1e3
                    cols.append((float(x.min()), float(x.median()), float(x.max())))
            rows.append({"ctas": int((t[:, r, it, 0] > 0).sum()), "s": cols})
        result["stamps"][role] = rows
    # SM clock: the producer (first item) and the epilogue (each item) both store globaltimer and clock64 together
    n_items = (t[:, 2, :, 0] > 0).sum(dim=1)
    rows_ok = (n_items > 0) & (t[:, 0, 0, 0] > 0)
    if bool(rows_ok.any()):
        idx = (n_items.clamp(min=1) - 1)[rows_ok]
        sel_t = t[rows_ok]
        ar = torch.arange(sel_t.shape[0])
        d_ns = (sel_t[ar, 2, idx, 0] - sel_t[:, 0, 0, 0]).double()
        d_clk = (sel_t[ar, 2, idx, 3] - sel_t[:, 0, 0, 3]).double()
        good = d_ns > 1000
        if bool(good.any()):
            result["sm_mhz"] = float((d_clk[good] / d_ns[good] * 1e3).median())
    issuing = t[:, 1, :, 0] > 0  # CTAs (pair leaders) whose MMA warp ran this item
    result["mma"] = []
    for it in range(items):
        sel = issuing[:, it]
        if not bool(sel.any()):
            break
        med = lambda x: float(x[sel].double().median())
        rec = {"stalls": med(t[:, 1, it, 3])}
        if detail:
            rec.update(wait=med(t[:, 3, it, 0]), issue=med(t[:, 3, it, 2]), commit=med(t[:, 3, it, 3]))
        result["mma"].append(rec)
    return result


def format_timeline(res: dict) -> str:
    pl = res["plan"]
    lines = [f"span {res['span_us']:.2f} us; grid {pl['grid']}, tile {pl['tile_m']}x{pl['tile_n']}, stages {pl['stages']}, "
             f"split_k {pl['split_k']}, stream-K tiles {pl['sk_tiles']}"
             + (f"; SM clock {res['sm_mhz']:.0f} MHz" if "sm_mhz" in res else "")]
    for role in ROLES:
        for it, row in enumerate(res["stamps"][role]):
            if row["ctas"] == 0:
                continue
            cells = ["      -      " if c is None else f"{c[0]:5.1f}/{c[1]:5.1f}/{c[2]:5.1f}" for c in row["s"]]
            tail = ""
            if role == "mma" and it < len(res.get("mma", [])):
                rec = res["mma"][it]
                tail = f"   stalls {rec['stalls']:.0f}"
                if "wait" in rec:
                    tail += f", cycles waiting {rec['wait']:.0f} / issuing {rec['issue']:.0f} / committing {rec['commit']:.0f}"
            lines.append(f"  {role:8s} item {it} ({row['ctas']:3d} CTAs)  s0 {cells[0]}   s1 {cells[1]}   s2 {cells[2]}{tail}")
    return "\n".join(lines)


def main() -> None:
    ap = argparse.ArgumentParser(description="role timelines of one gemm_a16w16 call (min/median/max over CTAs, us)")
    ap.add_argument("--m", type=int, required=True)
    ap.add_argument("--n", type=int, required=True)
    ap.add_argument("--k", type=int, required=True)
    ap.add_argument("--layout", default="nt", choices=("nn", "nt", "tn", "tt"))
    ap.add_argument("--dtype", default="bf16", choices=("bf16", "fp16"))
    ap.add_argument("--out-dtype", default=None, choices=("bf16", "fp16", "fp32"))
    ap.add_argument("--bias", action="store_true")
    ap.add_argument("--policy", default="{}", help="JSON dict of user_kwargs")
    ap.add_argument("--warm", action="store_true", help="leave the operands in L2 before the traced call")
    ap.add_argument("--items", type=int, default=3)
    ap.add_argument("--detail", action="store_true", help="also count the MMA warp's cycles (wait / issue / commit)")
    a = ap.parse_args()
    kw = json.loads(a.policy)
    res = timeline(a.m, a.n, a.k, kw, a.layout, _DT[a.dtype], None if a.out_dtype is None else _DT[a.out_dtype], a.bias,
                   cold=not a.warm, items=a.items, detail=a.detail)
    print(f"{a.m}x{a.n}x{a.k} {a.dtype} '{a.layout}' {json.dumps(kw)} ({'warm' if a.warm else 'cold'} L2)")
    print(format_timeline(res))


if __name__ == "__main__":
    main()
