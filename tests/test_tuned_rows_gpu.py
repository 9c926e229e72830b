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
        want = P.from_user_kwargs(cfg, m, n, k, layout)
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
