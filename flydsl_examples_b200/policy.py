"""Blackwell tile policy: defaults, validation and the shape heuristic.

Takes the place of the reference's compile-time policy struct and its validators
(kernels/gemm_a16w16_gfx950.py:33-61 GemmA16W16Gfx950Param, :64-245 make_gemm_a16w16_gfx950_param,
:1213-1236 make_gemm_a16w16_param_and_validate, :1239-1274 assert_no_k_tail). The reference keys are still
accepted so that its call sites run unchanged; the keys that describe gfx950 wave layouts have no meaning on
sm_100a and are ignored.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, asdict
from pathlib import Path
from typing import Optional

TILE_M = 128  # rows per CTA on the MMA M axis (TMEM lanes)
TILE_K = 64   # one TMA box: a 128-byte swizzle span of 16-bit data
TILE_N_MENU = (16, 32, 64, 128, 256)
MAX_STAGES = {16: 5, 32: 5, 64: 4, 128: 3, 256: 4}            # one CTA per tile, default stage depth
MAX_STAGES_K64 = {16: 8, 32: 8, 64: 8, 128: 6, 256: 4}        # one CTA per tile, 64-deep stages
MAX_STAGES_PAIR = {128: 8, 192: 6, 256: 6, 512: 4}            # a CTA pair per 256-row tile (cta_group 2)


def tile_k(tile_n: int, cta_group: int = 1, requested: int = 0) -> int:
    """K elements per pipeline stage of a variant. Single-CTA tiles up to 128 wide exist with 64- and 128-deep
    stages (two 64-deep boxes per operand and stage, so that the fixed per-stage cost — barrier poll, election,
    commit — is paid once per 128); 128 is their default. 256-wide tiles and CTA pairs are 64-deep only."""
    if cta_group == 1 and tile_n <= 128:
        return requested if requested in (64, 128) else 128
    return 64


def variant_width(tile_n: int, cta_group: int = 1) -> int:
    """Width of the kernel variant that runs tiles of tile_n columns: the 512-column pair variant takes its tile
    width at run time (any multiple of 32 above 256), every other variant has exactly one width."""
    return 512 if (cta_group == 2 and 256 < tile_n <= 512 and tile_n % 32 == 0) else tile_n


def max_stages(tile_n: int, cta_group: int = 1, requested_tile_k: int = 0) -> int:
    if cta_group == 2:
        return MAX_STAGES_PAIR[variant_width(tile_n, 2)]
    return (MAX_STAGES_K64 if tile_k(tile_n, 1, requested_tile_k) == 64 else MAX_STAGES)[tile_n]
SMEM_LIMIT = 232448
TMEM_COLUMNS = 512
NUM_SMS_DEFAULT = 148

# Keys of the reference's policy dict (kernels/gemm_a16w16_gfx950.py:1390-1401).
REFERENCE_KEYS = (
    "block_m", "block_n", "block_k", "stages", "split_k", "m_waves", "n_waves", "k_waves", "group_m",
    "use_half_tile_interleaved",
)
# Keys that only exist here.
BLACKWELL_KEYS = ("tile_n", "swap_ab", "cta_group", "split_mode", "max_ctas", "stream_k", "tile_k")
# Keys that switch behaviour without describing a tiling (they do not make a dict a "Blackwell policy").
CONTROL_KEYS = ("strict_reference_envelope", "pdl", "wait_limit_us", "loader")
SPLIT_MODES = {"ticket": 0, "atomic": 1, "cluster": 2}


@dataclass(frozen=True)
class Policy:
    tile_n: int
    stages: int = 0          # 0 = deepest ring that fits
    split_k: int = 1
    group_m: int = 0
    swap_ab: bool = False
    cta_group: int = 1
    split_mode: str = "ticket"
    max_ctas: int = 0
    stream_k: bool = False
    pdl: bool = True         # programmatic dependent launch: set-up overlaps the previous kernel in the stream
    tile_k: int = 0          # K elements per pipeline stage; 0 = the tile's default (see tile_k())
    wait_limit_us: int = 0   # time limit of the kernel's waits in microseconds; 0 = 2 s
    loader: bool = False     # True: K-contiguous operands TMA cannot describe (8- but not 16-byte aligned rows) are fetched
                             # by loader warps inside the kernel (no scratch, one launch, much slower) instead of being
                             # copied into an aligned image first

    def as_dict(self) -> dict:
        return asdict(self)


def smem_bytes(tile_n: int, stages: int, cta_group: int = 1, requested_tile_k: int = 0) -> int:
    """Dynamic shared memory of one CTA: the ring, the bias slice, the barriers and alignment slack. In a pair
    each CTA holds 128 of the tile's 256 rows and half of its tile_n columns."""
    tile_n = variant_width(tile_n, cta_group)  # shared memory is laid out for the variant's full width
    staging = 4 * 2 * 32 * 128 if tile_n >= 64 else 0  # epilogue images for TMA stores
    staging = max(staging, TILE_M * tile_n * 4 if tile_n <= 64 else 0)  # rows received in cluster split-K mode
    tk = tile_k(tile_n, cta_group, requested_tile_k)
    bias = tile_n * 2 if tile_n > 256 else 256 * 4  # a 512-wide tile keeps its bias slice in 16 bits
    v_rows = tile_n // cta_group
    if v_rows > 64:
        v_rows = -(-v_rows // 64) * 64  # whole 64-row boxes (the 192-wide pair tile: 96 -> 128)
    return stages * (TILE_M * tk * 2 + v_rows * tk * 2) + staging + bias + (2 * stages + 4) * 8 + 32 + 1024


def split_k_slices(k: int, split_k: int, tk: int = TILE_K) -> list[tuple[int, int]]:
    """K-block ranges [(first_block, n_blocks)] of each slice, in blocks of `tk` elements (the variant's stage
    depth): uneven slices allowed, none empty."""
    kb = (k + tk - 1) // tk
    split_k = max(1, min(split_k, kb))
    base, rem = divmod(kb, split_k)
    out = []
    for s in range(split_k):
        out.append((s * base + min(s, rem), base + (1 if s < rem else 0)))
    return out


def raster(tile: int, tiles_p: int, tiles_q: int, group: int) -> tuple[int, int]:
    """Tile id -> (tile row, tile column). Groups of `group` tile rows are walked row-fastest, like the
    GROUP_M part of the reference's BlockSwizzle (kernels/gemm_a16w16_gfx950_utils.py:84-92)."""
    if group > 0:
        per_group = group * tiles_q
        g = tile // per_group
        first = g * group
        rows = min(tiles_p - first, group)
        r = tile - g * per_group
        return first + r % rows, r // rows
    return tile // tiles_q, tile % tiles_q


def stream_k_plan(tiles: int, kb_total: int, cap: int, min_span: int = 4) -> tuple[int, int, int]:
    """(grid, sk_tiles, sk_slots) of the stream-K schedule; sk_tiles == 0 means plain data-parallel.
    The tiles that do not fill a whole wave of `cap` CTAs are cut into equal contiguous spans of K blocks, one
    span per CTA; a remainder whose spans would be shorter than half a tile borrows one full wave (so a cut tile
    has at most three contributors); with less than one wave of tiles, spans shorter than `min_span` blocks make
    the grid shrink instead. Mirrors the planner in csrc/gemm_api.cu."""
    g = cap
    sk = tiles % g if tiles >= g else tiles
    if sk > 0 and tiles > g and sk * kb_total // g < max(min_span, kb_total // 2):
        sk += g
    elif sk > 0 and sk * kb_total // g < min_span:
        g = min(cap, sk * kb_total // min_span)
    if sk > 0 and g >= 1 and sk * kb_total // g >= min_span:
        span_min = sk * kb_total // g
        return g, sk, (kb_total + span_min - 1) // span_min + 1
    return min(tiles, cap), 0, 0


def stream_k_walk(cta: int, grid: int, tiles: int, kb_total: int, sk_tiles: int) -> list[dict]:
    """Work items of one CTA, in order, exactly as the device-side walk produces them: first its span of the
    stream-K region (may cross tile boundaries), then whole tiles sk_tiles + cta, + grid, ..."""
    total = sk_tiles * kb_total

    def owner(x: int) -> int:
        return ((x + 1) * grid + total - 1) // total - 1

    items = []
    cur, end = total * cta // grid, total * (cta + 1) // grid
    while cur < end:
        tile = cur // kb_total
        kb0 = cur - tile * kb_total
        kbn = min(kb_total - kb0, end - cur)
        item = {"tile": tile, "kb0": kb0, "kbn": kbn, "partial": kbn != kb_total}
        if item["partial"]:
            first, last = owner(tile * kb_total), owner((tile + 1) * kb_total - 1)
            item.update(n_contrib=last - first + 1, ordinal=cta - first)
        items.append(item)
        cur += kbn
    t = sk_tiles + cta
    while sk_tiles > 0 and t < tiles:
        items.append({"tile": t, "kb0": 0, "kbn": kb_total, "partial": False})
        t += grid
    return items


def validate(pol: Policy, m: int, n: int, k: int, layout: str) -> Optional[str]:
    """Return None when the policy is runnable for this problem, else the reason."""
    width = variant_width(pol.tile_n, pol.cta_group)
    if pol.tile_n not in TILE_N_MENU and not (pol.cta_group == 2 and width in MAX_STAGES_PAIR):
        return (f"tile_n must be one of {TILE_N_MENU} (or {tuple(MAX_STAGES_PAIR)} or a multiple of 32 between 288 and 512 "
                f"with cta_group 2), got {pol.tile_n}")
    if pol.cta_group not in (1, 2):
        return f"cta_group must be 1 or 2, got {pol.cta_group}"
    stage_menu = MAX_STAGES if pol.cta_group == 1 else MAX_STAGES_PAIR
    if width not in stage_menu:
        return f"cta_group 2 needs tile_n in {tuple(MAX_STAGES_PAIR)} (or a multiple of 32 between 288 and 512), got {pol.tile_n}"
    if pol.stages < 0 or pol.stages == 1:
        return f"stages must be 0 (auto) or >= 2, got {pol.stages} (more than fit are clamped)"
    if pol.tile_k not in (0, tile_k(pol.tile_n, pol.cta_group, pol.tile_k)):
        return f"tile_k {pol.tile_k} is not built for tile_n {pol.tile_n}, cta_group {pol.cta_group}"
    if pol.split_k < 1:
        return f"split_k must be >= 1, got {pol.split_k}"
    if pol.split_mode not in SPLIT_MODES:
        return f"split_mode must be one of {tuple(SPLIT_MODES)}, got {pol.split_mode!r}"
    if pol.group_m < 0:
        return f"group_m must be >= 0, got {pol.group_m}"
    if pol.wait_limit_us < 0:
        return f"wait_limit_us must be >= 0, got {pol.wait_limit_us}"
    if pol.split_mode == "cluster" and pol.split_k > 1 and (pol.cta_group != 1 or pol.stream_k):
        return "cluster split-K needs cta_group 1 and no stream_k"
    if pol.split_mode == "cluster" and pol.split_k > 1 and pol.tile_n > 64:
        # wide tiles receive the cluster's rows (128 x tile_n floats) in the operand ring
        tk = tile_k(pol.tile_n, 1, pol.tile_k)
        stages = min(pol.stages or 99, max_stages(pol.tile_n, 1, pol.tile_k))
        if stages * (TILE_M + pol.tile_n) * tk * 2 < TILE_M * pol.tile_n * 4:
            return f"cluster split-K with tile_n {pol.tile_n} needs a ring of at least {TILE_M * pol.tile_n * 4} bytes"
    # The operand on the MMA N axis, when it is contiguous along N (or M after a swap), is fetched as 64-wide boxes.
    a_mn = layout[0] == "t"
    b_mn = layout[1] == "n"
    v_mn = a_mn if pol.swap_ab else b_mn
    if v_mn and width // pol.cta_group < 64:
        return "a tile_n-side operand that is not K-contiguous needs at least 64 tile_n columns per CTA"
    if pol.tile_n > TMEM_COLUMNS:
        return "the accumulator does not fit in 512 TMEM columns"
    return None


# Rough cost of one 64-deep K block of a tile, in SM cycles, used only to rank candidate tilings. Two bounds, both
# measured: the tensor pipe needs 128 cycles per 128 x 256 x 16 MMA, and one SM takes in about 64 bytes per clock
# from L2, i.e. 2 * (128 + tile_n) cycles for the 128 + tile_n operand rows of a block (a CTA of a pair loads half of
# the tile_n rows). Every single-CTA tile is bound by the second; the 256 x 256 pair balances the two (its main loop
# runs 8-15 % above the tensor time), the 256 x 512 pair is tensor-bound (3 % above).
_KBLOCK_CYCLES = {(1, 256): 800.0, (2, 256): 590.0, (2, 512): 1060.0, (2, 192): 530.0, (1, 128): 540.0, (1, 64): 400.0, (1, 32): 340.0,
                  (1, 16): 310.0}
_FIXED_CYCLES = 6000.0  # launch tail, pipeline fill, last epilogue


def _kblock_cycles(cta_group: int, tile_n: int) -> float:
    if cta_group == 2 and tile_n > 256:
        # the 512-column variant at a run-time width: per K = 16 step one MMA of 256 columns (128 cycles) and one of
        # tile_n - 256, which cannot be issued in less than about 90 cycles however narrow it is (measured: 288 to 416
        # columns all take about 900 cycles per K block, 512 columns 1060)
        return 4.0 * (128.0 + max(90.0, (tile_n - 256) / 2.0)) + 36.0
    return _KBLOCK_CYCLES[(cta_group, tile_n)]


def _auto_split(tiles: int, kb: int, walkers: int, cluster_ok: bool = False) -> tuple[int, str]:
    """(K slices per tile, reduction mode) when the tiles alone cannot occupy the machine. Narrow single-CTA tiles
    reduce inside a thread-block cluster (2..16 CTAs, through distributed shared memory); the rest use tickets."""
    if tiles * 2 <= walkers and kb >= 8:
        if cluster_ok:
            s = 16
            while s > 1 and (s > walkers // tiles or s > kb // 2):
                s //= 2
            if s >= 2:
                return s, "cluster"
        return max(1, min(walkers // tiles, kb // 4, 64)), "ticket"
    return 1, "ticket"


def _estimate_cycles(p_ext: int, q: int, kb: int, cta_group: int, tile_n: int, num_sms: int) -> float:
    walkers = max(1, num_sms // cta_group)
    tiles = -(-p_ext // (TILE_M * cta_group)) * -(-q // tile_n)
    split, _ = _auto_split(tiles, kb, walkers, cta_group == 1 and tile_n <= 64)
    waves = -(-(tiles * split) // walkers)
    # per tile, outside the main loop: the hand-over between tiles; a 512-wide tile has a single accumulator, so its
    # whole epilogue (5 to 6 us at 512 columns) stands between two main loops
    epilogue = 9000.0 * tile_n / 512 if tile_n > 256 else 1000.0 + 500.0 * tile_n / 256
    # after the main loop: a cluster exchange of a narrow tile costs about 1 us, a reduction through global memory
    # (partial write, fences and ticket, read-back) about 5 us
    # (the last arriver reads split slabs of 128 x tile_n floats at about 24 bytes per clock)
    fixup = 0.0 if split <= 1 else (1500.0 + 200.0 * split) if (cta_group == 1 and tile_n <= 64) else (8000.0 + 21.0 * split * tile_n)
    pair_start = 2500.0 if cta_group == 2 else 0.0  # a cluster launch reaches its first MMA about 1.5 us later
    return _FIXED_CYCLES + pair_start + waves * (-(-kb // split) * _kblock_cycles(cta_group, tile_n) + epilogue) + fixup


def heuristic(m: int, n: int, k: int, layout: str = "nt", num_sms: int = NUM_SMS_DEFAULT) -> Policy:
    """Shape-driven default used when the caller passes no Blackwell keys and the tuned table has no entry."""
    a_mn = layout[0] == "t"
    b_mn = layout[1] == "n"
    kb = max(1, (k + TILE_K - 1) // TILE_K)
    swap = m <= 64 and n > m
    if swap:
        q, v_mn, p_ext = m, a_mn, n
    else:
        q, v_mn, p_ext = n, b_mn, m
    menu = [t for t in TILE_N_MENU if not (v_mn and t < 64)]
    cta_group = 1
    if swap:
        tile_n = next((t for t in menu if t >= q), menu[-1])
    else:
        cands = [(1, t) for t in menu if t <= max(64, 1 << (max(q, 1) - 1).bit_length())]
        if p_ext > TILE_M and q > 128:
            cands.append((2, 256))
            if q > 256:
                # the 512-column variant at the widths that may fill whole waves better: up to a quarter less operand
                # traffic per flop, but an epilogue that no main loop hides
                cands += [(2, t) for t in range(288, 513, 32)]
            cands.append((2, 192))
        best = min(cands, key=lambda c: (_estimate_cycles(p_ext, q, kb, c[0], c[1], num_sms), -c[1], -c[0]))
        cta_group, tile_n = best
    walkers = num_sms // cta_group
    tiles = -(-p_ext // (TILE_M * cta_group)) * -(-q // tile_n)
    split, mode = _auto_split(tiles, kb, walkers, cta_group == 1 and tile_n <= 64)
    group = 8 if (tiles >= 2 * walkers and not swap) else 0
    # 128-wide single-CTA tiles that stream their whole K run 5-7 % faster with six 64-deep stages than with three
    # 128-deep ones (measured on 384 and 512 rows against 4096 x 4096 weights); the cluster split-K shapes prefer 128
    stage_k = 64 if (cta_group == 1 and tile_n == 128 and mode != "cluster") else 0
    return Policy(tile_n=tile_n, split_k=split, group_m=group, swap_ab=swap, cta_group=cta_group, split_mode=mode, tile_k=stage_k)


def from_user_kwargs(user_kwargs: dict, m: int, n: int, k: int, layout: str, num_sms: int = NUM_SMS_DEFAULT) -> Policy:
    """Merge a caller's dict over the heuristic. Unknown keys raise ValueError."""
    known = set(REFERENCE_KEYS) | set(BLACKWELL_KEYS) | set(CONTROL_KEYS)
    unknown = [key for key in user_kwargs if key not in known]
    if unknown:
        raise ValueError(f"unknown gemm_a16w16 policy keys: {sorted(unknown)}")
    base = heuristic(m, n, k, layout, num_sms)
    native = any(key in user_kwargs for key in BLACKWELL_KEYS)
    fields = base.as_dict()
    if native:
        # A Blackwell policy is taken literally: nothing the caller left out is second-guessed by the heuristic
        # except the tile, which falls back to the heuristic's choice.
        fields.update(split_k=1, group_m=0, swap_ab=False, stages=0, cta_group=1, split_mode="ticket", tile_k=0)
        for key in BLACKWELL_KEYS + ("stages", "split_k", "group_m"):
            if key in user_kwargs:
                fields[key] = user_kwargs[key]
        if "tile_n" not in user_kwargs and "swap_ab" in user_kwargs and bool(user_kwargs["swap_ab"]) != base.swap_ab:
            q = m if fields["swap_ab"] else n
            v_mn = (layout[0] == "t") if fields["swap_ab"] else (layout[1] == "n")
            menu = [t for t in TILE_N_MENU if not (v_mn and t < 64)]
            fields["tile_n"] = next((t for t in menu if t >= q), menu[-1])
    else:
        # Reference policy: its split_k / group_m requests carry over, wave and block shapes do not apply.
        if "split_k" in user_kwargs:
            fields["split_k"] = int(user_kwargs["split_k"])
        if "group_m" in user_kwargs:
            fields["group_m"] = int(user_kwargs["group_m"])
    for key in ("pdl", "wait_limit_us", "loader"):
        if key in user_kwargs:
            fields[key] = user_kwargs[key]
    fields["swap_ab"] = bool(fields["swap_ab"])
    fields["stream_k"] = bool(fields["stream_k"])
    fields["pdl"] = bool(fields["pdl"])
    fields["wait_limit_us"] = int(fields["wait_limit_us"])
    fields["loader"] = bool(fields["loader"])
    pol = Policy(**fields)
    return pol


# ------------------------------------------------------------------ tuned table (JSONL written by gemm_tune.py)
_TUNED: dict[tuple, dict] = {}
_TUNED_LOADED = False
TUNED_PATH = Path(__file__).resolve().parent.parent / "gemm_a16w16_tuned.jsonl"


def load_tuned(path: Optional[Path] = None) -> dict[tuple, dict]:
    """Read the tuner's JSONL ({arch,dtype,layout,m,n,k,config,duration,tflops} per line; same schema as the
    reference's gemm_a16w16_tuned.jsonl) keeping only sm_100a rows."""
    global _TUNED_LOADED
    path = Path(path) if path else TUNED_PATH
    table: dict[tuple, dict] = {}
    if path.exists():
        for line in path.read_text().splitlines():
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            if rec.get("arch") != "sm_100a":
                continue
            table[(rec["dtype"], rec["layout"], rec["m"], rec["n"], rec["k"])] = rec["config"]
    if path == TUNED_PATH:
        _TUNED.clear()
        _TUNED.update(table)
        _TUNED_LOADED = True
    return table


def tuned_lookup(dtype: str, layout: str, m: int, n: int, k: int) -> Optional[dict]:
    """Tuned policy for this exact problem, if the table has one. fp16 and bf16 run the same kernels at the same
    speed, so a row tuned for one serves the other."""
    if not _TUNED_LOADED:
        load_tuned()
    other = "fp16" if dtype == "bf16" else "bf16"
    # Rows tuned for another layout of the same problem are the next best thing (the main loop differs only in the
    # shared-memory image of an operand); the caller checks that the policy is valid for its own layout.
    layouts = [layout] + [l for l in (layout[0] + "t", "nt", "tt", "nn", "tn") if l != layout]
    for lay in dict.fromkeys(layouts):
        for dt in (dtype, other):
            rec = _TUNED.get((dt, lay, m, n, k))
            if rec is not None:
                return rec
    return None
