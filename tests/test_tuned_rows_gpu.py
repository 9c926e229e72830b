"""Every row of the shipped policy table (gemm_a16w16_tuned.jsonl) through the CUDA path, by name.

The table steers every call that passes no policy of its own, so a bad row would silently break the default path
of its shape. Mirrors test_gemm_a16w16_acc_tuned_policies of the reference (test_gemm_a16w16_gfx950.py:428-524),
which runs every tuned policy on 'nn' and 'nt': here each row runs through the *default-policy* call (empty
user_kwargs, so the lookup itself is exercised) in its own layout and dtype and in 'nn' with the other 16-bit
dtype, against the CPU oracle: the whole product for shapes the CPU finishes quickly, sampled full rows and columns
for the large ones. Where the row's policy is valid for the call, the resolved policy must be the row's.
"""
import json

import pytest
import torch

from flydsl_examples_b200 import gemm_a16w16 as G
from flydsl_examples_b200 import policy as P
from kernels.gemm_a16w16_gfx950 import gemm_a16w16
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"bf16": torch.bfloat16, "fp16": torch.float16}
ROWS = [json.loads(line) for line in P.TUNED_PATH.read_text().splitlines() if line.strip()]
FULL_ORACLE_FLOPS = 2 * 2048 * 4096 * 4096  # above this the oracle checks sampled rows and columns only


def _row_id(rec):
    return f"{rec['dtype']}-{rec['layout']}-{rec['m']}x{rec['n']}x{rec['k']}"


def _operand(rows, cols, dtype, is_t, seed, std):
    g = torch.Generator(device=DEV).manual_seed(seed)
    t = (torch.randn((cols, rows) if is_t else (rows, cols), generator=g, device=DEV, dtype=torch.float32) * std).to(dtype)
    return t.t() if is_t else t


@pytest.mark.parametrize("rec", ROWS, ids=_row_id)
def test_shipped_tuned_row(rec):
    m, n, k, cfg = rec["m"], rec["n"], rec["k"], rec["config"]
    assert rec["arch"] == "sm_100a"
    other = "fp16" if rec["dtype"] == "bf16" else "bf16"
    for dt_name, layout in ((rec["dtype"], rec["layout"]), (other, "nn")):
        dtype = DT[dt_name]
        # the row itself for its own (dtype, layout); for the other combination whichever row the lookup prefers
        # (one of the same layout, if the table has it)
        looked = P.tuned_lookup(dt_name, layout, m, n, k)
        if (dt_name, layout) == (rec["dtype"], rec["layout"]):
            assert looked == cfg
        want = P.from_user_kwargs(looked, m, n, k, layout)
        got_pol = G.resolve_policy(m, n, k, dtype, layout, {})
        if P.validate(want, m, n, k, layout) is None:
            assert got_pol == want, f"the default call did not pick the shipped row: {got_pol} != {want}"
        std = 1.0 if max(m, n) * k < (1 << 26) else 0.05
        a = _operand(m, k, dtype, layout[0] == "t", 7 * m + k, std)
        b = _operand(k, n, dtype, layout[1] == "t", 11 * n + k, std)
        bias = _operand(1, n, dtype, False, n, 0.5).reshape(n)
        out = torch.full((m, n), float("nan"), dtype=dtype, device=DEV)
        res = gemm_a16w16(a, b, out, bias=bias, user_kwargs={}, layout=layout)
        G.check_status()
        assert res.data_ptr() == out.data_ptr()
        what = f"tuned row {_row_id(rec)} run as {dt_name} {layout}"
        if 2 * m * n * k <= FULL_ORACLE_FLOPS:
            O.assert_close(out, O.reference_matmul(a, b, bias, dtype), k, what)
        else:
            g = torch.Generator().manual_seed(m + n)
            rows = torch.unique(torch.cat([torch.tensor([0, m - 1]), torch.randint(0, m, (14,), generator=g)]))
            cols = torch.unique(torch.cat([torch.tensor([0, n - 1]), torch.randint(0, n, (14,), generator=g)]))
            rd, cd = rows.to(DEV), cols.to(DEV)
            O.assert_close(out[rd], O.reference_matmul(a[rd], b, bias, dtype), k, what + " (sampled rows)")
            O.assert_close(out[:, cd], O.reference_matmul(a, b[:, cd], bias[cd], dtype), k, what + " (sampled columns)")
        del a, b, out
    torch.cuda.empty_cache()


# The large shapes of the reference's main-loop accuracy test (test_gemm_a16w16_gfx950.py:262-283) with its own policy
# dicts, in all four layouts: full 256-row tiles, ragged 8160-wide edges, K = 8192 + 64 (an odd K block at the end) and
# 2048 - 64. The dtype alternates over (shape, layout) and every shape runs with and without bias.
REFERENCE_MAIN_LOOP = [  # m, n, k, block_m, block_n, block_k, stages, m_waves, n_waves, group_m, has_bias, hti
    (8192, 8192, 8192, 256, 256, 64, 2, 2, 4, 4, True, False),
    (8160, 8160, 8192, 256, 256, 64, 2, 2, 4, 0, False, True),
    (8192, 8192, 8192 + 64, 256, 256, 64, 2, 2, 4, 0, True, False),
    (8160, 8160, 8192 + 64, 256, 256, 64, 2, 2, 4, 0, False, False),
    (2048, 2048, 2048, 128, 128, 64, 4, 4, 4, 0, True, False),
    (2048, 2048, 2048 - 64, 128, 128, 64, 2, 4, 4, 0, False, False),
]


@pytest.mark.parametrize("layout", ["nn", "nt", "tn", "tt"])
@pytest.mark.parametrize("idx", range(len(REFERENCE_MAIN_LOOP)))
def test_reference_main_loop_large_shapes(layout, idx):
    m, n, k, bm, bn, bk, stages, mw, nw, gm, has_bias, hti = REFERENCE_MAIN_LOOP[idx]
    kw = {"block_m": bm, "block_n": bn, "block_k": bk, "stages": stages, "m_waves": mw, "n_waves": nw, "group_m": gm,
          "use_half_tile_interleaved": hti}
    dt_name = ("bf16", "fp16")[(idx + ["nn", "nt", "tn", "tt"].index(layout)) % 2]
    dtype = DT[dt_name]
    a = _operand(m, k, dtype, layout[0] == "t", 3 * idx + 1, 0.05)
    b = _operand(k, n, dtype, layout[1] == "t", 3 * idx + 2, 0.05)
    bias = _operand(1, n, dtype, False, idx, 0.5).reshape(n) if has_bias else None
    out = torch.randn((m, n), device=DEV).to(dtype)  # the reference pre-fills outputs with randn (:76-79)
    gemm_a16w16(a, b, out, bias=bias, user_kwargs=kw, layout=layout)
    G.check_status()
    g = torch.Generator().manual_seed(idx)
    rows = torch.unique(torch.cat([torch.tensor([0, m - 1]), torch.randint(0, m, (14,), generator=g)]))
    cols = torch.unique(torch.cat([torch.tensor([0, n - 1]), torch.randint(0, n, (14,), generator=g)]))
    rd, cd = rows.to(DEV), cols.to(DEV)
    what = f"main loop {m}x{n}x{k} {dt_name} {layout}"
    O.assert_close(out[rd], O.reference_matmul(a[rd], b, bias, dtype), k, what + " (sampled rows)")
    O.assert_close(out[:, cd], O.reference_matmul(a, b[:, cd], None if bias is None else bias[cd], dtype), k, what + " (sampled columns)")


# The reference's workgroup slice-K tests (test_gemm_a16w16_gfx950.py:769-790, :912-931): its `k_waves` key has no
# counterpart here (accepted, ignored); split_k carries over. fp32 output without bias, and a biased 16-bit run.
@pytest.mark.parametrize("k_waves, split_k, k, has_bias, fp32_out", [(2, 1, 2048, False, True), (2, 2, 2048, False, True), (4, 1, 1024, True, False)])
def test_reference_slice_k_policies(k_waves, split_k, k, has_bias, fp32_out):
    kw = {"block_m": 32, "block_n": 64, "block_k": 128, "stages": 4, "m_waves": 1, "n_waves": 2, "k_waves": k_waves, "group_m": 0,
          "use_half_tile_interleaved": False, "split_k": split_k}
    case = O.Case("slice_k", "bf16", "nt", 64, 128, k, seed=800 + k_waves + split_k, bias_std=0.5 if has_bias else None,
                  out_dtype="fp32" if fp32_out else None, user_kwargs=kw)
    a, b, bias, a_l, b_l, bias_l = O.build_inputs(case, device=DEV)
    out = torch.randn((case.m, case.n), device=DEV).to(case.torch_out_dtype)
    got = gemm_a16w16(a, b, out, bias=bias, user_kwargs=kw, layout="nt")
    G.check_status()
    O.assert_close(got, O.reference_matmul(a_l, b_l, bias_l, case.torch_out_dtype), k, f"slice-K policy {kw}")


# The reference's split-K benchmark list with its half-tile-interleaved policies (test_gemm_a16w16_gfx950.py:1036-1048;
# the shapes of gemm_tune.py:350-355): tall-skinny outputs whose K is cut 2 to 8 ways.
REFERENCE_SPLIT_K_BENCH = [  # m, n, k, block_m, block_n, block_k, stages, split_k, m_waves, n_waves, k_waves, group_m, bias
    (4096, 128, 6144, 64, 64, 256, 2, 2, 2, 2, 1, 0, False),
    (512, 2560, 6144, 128, 128, 128, 2, 3, 2, 4, 1, 4, False),
    (576, 256, 4096, 64, 64, 256, 2, 4, 2, 2, 1, 0, True),
    (1024, 128, 6144, 64, 64, 256, 2, 6, 2, 2, 1, 0, True),
    (1216, 64, 7168, 64, 64, 256, 2, 7, 2, 2, 1, 0, False),
    (1280, 64, 4096, 64, 64, 256, 2, 8, 2, 2, 1, 0, False),
]


@pytest.mark.parametrize("idx", range(len(REFERENCE_SPLIT_K_BENCH)))
def test_reference_split_k_bench_list(idx):
    m, n, k, bm, bn, bk, stages, split_k, mw, nw, kwv, gm, has_bias = REFERENCE_SPLIT_K_BENCH[idx]
    kw = {"block_m": bm, "block_n": bn, "block_k": bk, "stages": stages, "split_k": split_k, "m_waves": mw, "n_waves": nw,
          "k_waves": kwv, "group_m": gm, "use_half_tile_interleaved": True}
    for dt_name in ("bf16", "fp16"):
        dtype = DT[dt_name]
        a = _operand(m, k, dtype, False, 5 * idx + 1, 1.0)
        b = _operand(k, n, dtype, True, 5 * idx + 2, 1.0)
        bias = _operand(1, n, dtype, False, idx, 0.5).reshape(n) if has_bias else None
        pl = G.plan(a, b, "nt", kw, bias=bias)
        assert pl["split_k"] == split_k or pl["cluster_split"] > 0, pl  # the reference's split_k request carries over
        for rep in range(2):
            out = torch.randn((m, n), device=DEV).to(dtype)
            gemm_a16w16(a, b, out, bias=bias, user_kwargs=kw, layout="nt")
            G.check_status()
            O.assert_close(out, O.reference_matmul(a, b, bias, dtype), k, f"split-K bench {m}x{n}x{k} {dt_name} call {rep}")


def test_reference_bench_smoke_largest_shape():
    # 16384^3 of the reference's benchmark smoke list (test_gemm_a16w16_gfx950.py:1083) with its own policy: one run,
    # sampled full rows and columns against the CPU oracle
    m = n = k = 16384
    kw = {"block_m": 256, "block_n": 256, "block_k": 64, "stages": 2, "m_waves": 2, "n_waves": 4, "group_m": 4,
          "use_half_tile_interleaved": True}
    a = _operand(m, k, torch.bfloat16, False, 91, 0.05)
    b = _operand(k, n, torch.bfloat16, True, 92, 0.05)
    bias = _operand(1, n, torch.bfloat16, False, 93, 0.5).reshape(n)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    gemm_a16w16(a, b, out, bias=bias, user_kwargs=kw, layout="nt")
    G.check_status()
    assert bool(torch.isfinite(out).all())
    g = torch.Generator().manual_seed(16384)
    rows = torch.unique(torch.cat([torch.tensor([0, m - 1]), torch.randint(0, m, (10,), generator=g)]))
    cols = torch.unique(torch.cat([torch.tensor([0, n - 1]), torch.randint(0, n, (10,), generator=g)]))
    rd, cd = rows.to(DEV), cols.to(DEV)
    O.assert_close(out[rd], O.reference_matmul(a[rd], b, bias, torch.bfloat16), k, "16384^3 (sampled rows)")
    O.assert_close(out[:, cd], O.reference_matmul(a, b[:, cd], bias[cd], torch.bfloat16), k, "16384^3 (sampled columns)")
