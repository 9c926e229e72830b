"""GPU parity of the CUDA path against the CPU oracle, through the public call (one ctypes hop into the C ABI).

Tolerance is the build contract's: rtol 1e-2 / atol 1e-2*sqrt(K/1024) for 16-bit outputs, rtol 2e-3 /
atol 2e-3*sqrt(K/1024) for fp32 outputs, the same bound with split-K. Case lists follow the reference's tests
(test_gemm_a16w16_gfx950.py:253-1031) re-parametrised by Blackwell policies, plus the five benchmark configs.
"""
import functools

import pytest
import torch

from flydsl_examples_b200.gemm_a16w16 import check_status, plan
from kernels.gemm_a16w16_gfx950 import gemm_a16w16
from oracle import oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda"
DT = {"bf16": torch.bfloat16, "fp16": torch.float16}
LAYOUTS = ("nn", "nt", "tn", "tt")


def run_case(case: O.Case, repeats: int = 1, prefill="nan"):
    a, b, bias, a_l, b_l, bias_l = O.build_inputs(case, device=DEV)
    ref = O.reference_matmul(a_l, b_l, bias_l, case.torch_out_dtype)
    res = None
    for _ in range(repeats):
        if prefill == "nan":
            out = torch.full((case.m, case.n), float("nan"), dtype=case.torch_out_dtype, device=DEV)
        else:  # the reference pre-fills outputs with randn (test_gemm_a16w16_gfx950.py:76-79)
            out = torch.randn((case.m, case.n), dtype=case.torch_out_dtype, device=DEV)
        got = gemm_a16w16(a, b, out, bias=bias, user_kwargs=case.user_kwargs, layout=case.layout)
        check_status()
        assert got.data_ptr() == out.data_ptr()
        res = O.assert_close(got, ref, case.k, f"{case.name} {case.user_kwargs}")
    return res


def sampled_check(got, a_l, b_l, bias_l, k, out_dtype, n_rows=64, n_cols=64, seed=0):
    """Full rows and full columns of the product against the CPU oracle (for shapes whose full fp32 CPU matmul
    would take minutes)."""
    m, n = got.shape
    g = torch.Generator().manual_seed(seed)
    rows = torch.unique(torch.cat([torch.tensor([0, m - 1]), torch.randint(0, m, (n_rows,), generator=g)]))
    cols = torch.unique(torch.cat([torch.tensor([0, n - 1]), torch.randint(0, n, (n_cols,), generator=g)]))
    ref_rows = O.reference_matmul(a_l[rows], b_l, bias_l, out_dtype)
    O.assert_close(got[rows.to(got.device)], ref_rows, k, "sampled rows")
    ref_cols = O.reference_matmul(a_l, b_l[:, cols], None if bias_l is None else bias_l[cols], out_dtype)
    O.assert_close(got[:, cols.to(got.device)], ref_cols, k, "sampled cols")


# ------------------------------------------------------------------------------------------ benchmark configs
def test_config1_bf16_nt_256x512x1024():
    run_case(O.CONFIGS["c1"], repeats=3)


@pytest.mark.parametrize("kw", [{}, {"tile_n": 256, "group_m": 8}, {"tile_n": 128, "stages": 6}, {"tile_n": 256, "stream_k": True},
                                {"tile_n": 128, "stream_k": True, "group_m": 4}])
def test_config2_bf16_nt_bias(kw):
    case = O.CONFIGS["c2"]
    run_case(O.Case(**{**case.__dict__, "user_kwargs": kw}))


@pytest.mark.parametrize("split_k", [1, 8, 14, 16, 28, 32])
@pytest.mark.parametrize("swap", [True, False])
def test_config3_small_m_split_k_fp32(split_k, swap):
    case = O.CONFIGS["c3"]
    kw = {"tile_n": 32 if swap else 128, "swap_ab": swap, "split_k": split_k}
    run_case(O.Case(**{**case.__dict__, "user_kwargs": kw}), repeats=2)


@pytest.mark.parametrize("split_k", [2, 4, 8, 16])
@pytest.mark.parametrize("swap", [True, False])
def test_config3_cluster_split_k(split_k, swap):
    # the K slices of a tile form one thread-block cluster and reduce through distributed shared memory
    case = O.CONFIGS["c3"]
    kw = {"tile_n": 32 if swap else 64, "swap_ab": swap, "split_k": split_k, "split_mode": "cluster"}
    run_case(O.Case(**{**case.__dict__, "user_kwargs": kw}), repeats=3, prefill="randn")


CLUSTER_SPLIT = [
    (3, 5120, 2880, {"tile_n": 16, "swap_ab": True, "split_k": 4, "split_mode": "cluster"}),
    (17, 300, 1000, {"tile_n": 32, "swap_ab": True, "split_k": 8, "split_mode": "cluster"}),
    (64, 64, 768, {"tile_n": 64, "split_k": 4, "split_mode": "cluster"}),
    (129, 136, 1536, {"tile_n": 64, "split_k": 16, "split_mode": "cluster"}),
    (48, 5120, 2880, {"tile_n": 64, "swap_ab": True, "split_k": 2, "split_mode": "cluster"}),
    (200, 328, 333, {"tile_n": 32, "split_k": 16, "split_mode": "cluster"}),   # 6 K blocks: rounds down to 4 slices
    (256, 4096, 4096, {"tile_n": 128, "split_k": 2, "split_mode": "cluster"}),  # wide tiles receive into the idle ring
    (300, 700, 2048, {"tile_n": 256, "split_k": 8, "split_mode": "cluster"}),
    (800, 384, 7168, {"tile_n": 128, "split_k": 4, "split_mode": "cluster"}),
    (100, 600, 1000, {"tile_n": 128, "swap_ab": True, "split_k": 4, "split_mode": "cluster"}),
]


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("idx", range(len(CLUSTER_SPLIT)))
def test_cluster_split_k_shapes(dtype, idx):
    m, n, k, kw = CLUSTER_SPLIT[idx]
    for out_dtype in (None, "fp32"):
        run_case(O.Case("cluster", dtype, "nt", m, n, k, seed=500 + idx, bias_std=0.5, out_dtype=out_dtype, user_kwargs=kw),
                 repeats=2, prefill="randn")
    if kw["tile_n"] >= 64:  # operands contiguous along M / N need 64-wide boxes on the tile_n side
        run_case(O.Case("cluster_tn", dtype, "tn" if not kw.get("swap_ab") else "nn", m, n, k, seed=600 + idx, bias_std=0.5, user_kwargs=kw))


def test_config3_default_policy():
    run_case(O.CONFIGS["c3"], repeats=5, prefill="randn")


@functools.lru_cache(maxsize=1)
def _c4_reference():
    case = O.CONFIGS["c4_nn"]
    a_l, b_l, bias_l = O.draw_logical(case)
    return a_l, b_l, bias_l, O.reference_matmul(a_l, b_l, bias_l, torch.float32)


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("kw", [{}, {"tile_n": 128, "split_k": 2}, {"tile_n": 256, "stream_k": True}])
def test_config4_fp16_padded_offset_ktail(layout, kw):
    case = O.CONFIGS[f"c4_{layout}"]
    a_l, b_l, bias_l, ref = _c4_reference()
    a = O.place(a_l, layout[0] == "t", case.pad, case.offset, DEV)
    b = O.place(b_l, layout[1] == "t", case.pad, case.offset, DEV)
    # K-contiguous operands have an 8328-byte pitch here: TMA cannot describe them, so they are copied into an
    # aligned image first; their rows start on 8-byte boundaries, so on request the kernel's loader warps fetch them
    # instead (one launch, no scratch). Both ways must give the oracle's result.
    for loader in (False, True):
        kw2 = {**kw, "loader": True} if loader else kw
        pl = plan(a, b, layout, kw2, out_dtype=torch.float32)
        assert pl["a_loader" if loader else "a_repacked"] == (1 if layout[0] == "n" else 0)
        assert pl["b_loader" if loader else "b_repacked"] == (1 if layout[1] == "t" else 0)
        assert pl["b_repacked" if loader else "b_loader"] == 0 and pl["a_repacked" if loader else "a_loader"] == 0
        out = torch.full((case.m, case.n), float("nan"), dtype=torch.float32, device=DEV)
        got = gemm_a16w16(a, b, out, bias=bias_l.to(DEV), user_kwargs=kw2, layout=layout)
        check_status()
        O.assert_close(got, ref, case.k, f"c4 {layout} {kw2}")


def test_config5_large_bf16_sampled_and_consistent():
    case = O.CONFIGS["c5"]
    a_l, b_l, bias_l = O.draw_logical(case)
    a, b = a_l.to(DEV), b_l.t().contiguous().to(DEV).t()
    out = torch.full((case.m, case.n), float("nan"), dtype=torch.bfloat16, device=DEV)
    got = gemm_a16w16(a, b, out, layout="nt")
    check_status()
    assert bool(torch.isfinite(got).all())
    sampled_check(got, a_l, b_l, None, case.k, torch.bfloat16, n_rows=48, n_cols=48)
    # size-independent property: an N-slab computed on its own (what one rank of the N-sharded mode does) equals the
    # same columns of the full product -- bit for bit when both use the same tiling, within tolerance otherwise
    n0, n1 = 7168, 7168 + 3584
    pol = {"tile_n": 256, "cta_group": 2, "group_m": 8}
    full_fixed = gemm_a16w16(a, b, layout="nt", user_kwargs=pol)
    slab_fixed = gemm_a16w16(a, b[:, n0:n1], layout="nt", user_kwargs=pol)
    check_status()
    assert torch.equal(slab_fixed, full_fixed[:, n0:n1])
    slab = gemm_a16w16(a, b[:, n0:n1], layout="nt")
    check_status()
    O.assert_close(slab, got[:, n0:n1], case.k, "slab vs full product")
    # secondary cross-check of the whole matrix against the library GEMM on the same GPU
    lib = torch.matmul(a, b)
    O.assert_close(got, lib, case.k, "c5 vs torch.matmul (secondary)")


def test_golden_fixtures_through_the_cuda_path(golden):
    # the committed vectors come from the reference's own ref_func (tests/golden/make_golden.py)
    for name in (str(n) for n in golden["names"]):
        dt, layout, fp32 = (str(x) for x in golden[f"{name}.meta"])
        dtype = DT[dt]
        a_l = torch.from_numpy(golden[f"{name}.a"].copy()).view(dtype)
        b_l = torch.from_numpy(golden[f"{name}.b"].copy()).view(dtype)
        bias_l = torch.from_numpy(golden[f"{name}.bias"].copy()).view(dtype) if f"{name}.bias" in golden.files else None
        want = torch.from_numpy(golden[f"{name}.c"].copy())
        want = want if fp32 == "1" else want.view(dtype)
        a = O.place(a_l, layout[0] == "t", device=DEV)
        b = O.place(b_l, layout[1] == "t", device=DEV)
        got = gemm_a16w16(a, b, bias=None if bias_l is None else bias_l.to(DEV), layout=layout, out_dtype=want.dtype)
        check_status()
        O.assert_close(got, want, a_l.shape[1], f"golden {name}")


# ------------------------------------------------------------------------------------------ reference case lists
MAIN_LOOP = [  # (m, n, k, kw)  cf. test_gemm_a16w16_gfx950.py:262-283
    (1024, 1024, 1024, {"tile_n": 256}),
    (1024, 1024, 1024, {"tile_n": 128, "group_m": 4}),
    (1056, 1056, 2048 - 64, {"tile_n": 256, "group_m": 4}),   # boundary tiles, odd K-tile count
    (1056, 1056, 1024 + 64, {"tile_n": 64, "stages": 3}),
    (512, 768, 4096, {"tile_n": 128, "stages": 2}),
    (2048, 2048, 512, {}),
]


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("idx", range(len(MAIN_LOOP)))
def test_main_loop_shapes(layout, dtype, idx):
    m, n, k, kw = MAIN_LOOP[idx]
    run_case(O.Case("main", dtype, layout, m, n, k, seed=100 + idx, bias_std=(0.5 if idx % 2 else None), user_kwargs=kw))


SPLIT_K = [  # cf. test_gemm_a16w16_gfx950.py:327-385
    (32, 384, 7168, {"tile_n": 64, "split_k": 8}),
    (3, 5120, 2880, {"tile_n": 64, "split_k": 3}),
    (65, 96, 1024, {"tile_n": 64, "split_k": 2}),
    (129, 136, 1536, {"tile_n": 128, "split_k": 3}),
    (257, 264, 2048, {"tile_n": 64, "split_k": 4}),
    (257, 264, 2048, {"tile_n": 256, "split_k": 8}),
    (800, 384, 7168, {"tile_n": 128, "split_k": 4}),
    (64, 64, 512, {"tile_n": 64, "split_k": 2}),
    (576, 256, 4096, {"tile_n": 64, "split_k": 7, "group_m": 2}),
]


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("idx", range(len(SPLIT_K)))
def test_split_k_shapes(layout, dtype, idx):
    m, n, k, kw = SPLIT_K[idx]
    for out_dtype in (None, "fp32"):
        run_case(O.Case("split", dtype, layout, m, n, k, seed=200 + idx, bias_std=0.5, out_dtype=out_dtype, user_kwargs=kw),
                 repeats=2, prefill="randn")


# The reference's benchmark list with the reference's own policy dicts (test_gemm_a16w16_gfx950.py:628-649): the
# gfx950 wave/tile keys are accepted and ignored, group_m carries over, the tiling comes from the shipped table or the
# heuristic. Shapes whose full fp32 CPU product would take minutes are checked on sampled full rows and columns.
REFERENCE_BENCH = [  # m, n, k, block_m, block_n, block_k, stages, m_waves, n_waves, group_m, hti
    (8, 4096, 4096, 16, 16, 128, 8, 1, 1, 4, False),
    (16, 4096, 4096, 16, 16, 128, 8, 1, 1, 4, False),
    (32, 4096, 4096, 16, 16, 64, 8, 1, 1, 0, False),
    (64, 4096, 4096, 32, 32, 64, 8, 2, 2, 4, False),
    (128, 4096, 4096, 64, 32, 128, 4, 4, 2, 4, False),
    (256, 4096, 4096, 64, 64, 64, 7, 4, 2, 4, False),
    (512, 4096, 4096, 64, 128, 64, 6, 2, 4, 4, False),
    (1024, 4096, 4096, 128, 128, 64, 4, 2, 4, 4, False),
    (2048, 4096, 4096, 128, 256, 64, 3, 4, 4, 4, False),
    (1024, 1024, 1024, 64, 64, 64, 4, 2, 4, 0, False),
    (2048, 2048, 2048, 128, 128, 64, 3, 4, 2, 0, False),
    (4096, 4096, 4096, 256, 256, 64, 2, 2, 4, 4, True),
    (4096, 4096, 8192, 256, 256, 64, 2, 2, 4, 4, True),
    (8192, 8192, 8192, 256, 256, 64, 2, 2, 4, 0, True),
    (8, 7168, 2048, 16, 16, 128, 8, 1, 1, 4, False),
    (32, 384, 7168, 16, 16, 128, 8, 1, 1, 0, False),
    (32, 14336, 4096, 32, 64, 64, 8, 2, 2, 0, False),
    (16, 28672, 4096, 16, 64, 128, 3, 1, 4, 4, False),
    (4096, 256, 4096, 64, 64, 64, 6, 4, 2, 4, False),
]


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("idx", range(len(REFERENCE_BENCH)))
def test_reference_bench_list_with_reference_policies(dtype, idx):
    m, n, k, bm, bn, bk, stages, mw, nw, gm, hti = REFERENCE_BENCH[idx]
    kw = {"block_m": bm, "block_n": bn, "block_k": bk, "stages": stages, "m_waves": mw, "n_waves": nw, "group_m": gm,
          "use_half_tile_interleaved": hti}
    big = m * n * k > 1 << 34
    if big and dtype == "fp16":
        pytest.skip("the large shapes run once (bf16): their CPU check dominates the test time")
    layouts = ("nt",) if big else (("nt", "nn") if m * n * k > 1 << 31 else LAYOUTS)
    for layout in layouts:
        if (layout[0] == "t" and m % 8) or (layout[1] == "n" and n % 8):
            continue
        case = O.Case("refbench", dtype, layout, m, n, k, seed=600 + idx, bias_std=0.5, user_kwargs=kw)
        if not big:
            run_case(case)
            continue
        a, b, bias, a_l, b_l, bias_l = O.build_inputs(case, device=DEV)
        out = torch.full((m, n), float("nan"), dtype=case.torch_out_dtype, device=DEV)
        got = gemm_a16w16(a, b, out, bias=bias, user_kwargs=kw, layout=layout)
        check_status()
        assert bool(torch.isfinite(got).all())
        sampled_check(got, a_l, b_l, bias_l, k, case.torch_out_dtype, n_rows=24, n_cols=24, seed=idx)


PAIR = [  # a CTA pair per 256-row tile (tcgen05 cta_group::2)
    (256, 256, 64, {"tile_n": 256, "cta_group": 2}),
    (1024, 1024, 512, {"tile_n": 256, "cta_group": 2}),
    (512, 384, 512, {"tile_n": 128, "cta_group": 2}),
    (700, 900, 520, {"tile_n": 256, "cta_group": 2}),              # ragged: second CTA of a pair partly / fully out of range
    (130, 300, 1000, {"tile_n": 128, "cta_group": 2}),
    (512, 512, 4096, {"tile_n": 256, "cta_group": 2, "split_k": 4}),
    (1000, 3000, 4100, {"tile_n": 256, "cta_group": 2, "stream_k": True}),
    (4096, 4096, 1024, {"tile_n": 256, "cta_group": 2, "group_m": 4}),
    (2048, 4096, 4096, {"tile_n": 256, "cta_group": 2, "stream_k": True, "group_m": 8}),
]


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("idx", range(len(PAIR)))
def test_cta_pair_shapes(dtype, idx):
    m, n, k, kw = PAIR[idx]
    for layout in (LAYOUTS if m * n * k <= 1 << 32 else ("nt", "tn")):
        for out_dtype in (None, "fp32"):
            run_case(O.Case("pair", dtype, layout, m, n, k, seed=400 + idx, bias_std=0.5, out_dtype=out_dtype, user_kwargs=kw),
                     repeats=2, prefill="randn")


PAIR_192 = [  # 256 x 192 pair tiles: 96 columns per CTA (one and a half 64-row boxes of an N-contiguous B)
    (512, 768, 520, {"tile_n": 192, "cta_group": 2}),
    (700, 500, 1000, {"tile_n": 192, "cta_group": 2}),                      # ragged in M and N
    (1000, 3000, 4100, {"tile_n": 192, "cta_group": 2}),                    # config 4's shape: 64 pair tiles
    (1000, 3000, 4100, {"tile_n": 192, "cta_group": 2, "stream_k": True}),
    (512, 384, 4096, {"tile_n": 192, "cta_group": 2, "split_k": 3}),
    (2048, 1920, 512, {"tile_n": 192, "cta_group": 2, "group_m": 4, "stages": 3}),
]


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("idx", range(len(PAIR_192)))
def test_cta_pair_192_wide_tiles(dtype, idx):
    m, n, k, kw = PAIR_192[idx]
    for layout in LAYOUTS:
        for out_dtype in (None, "fp32"):
            run_case(O.Case("pair192", dtype, layout, m, n, k, seed=450 + idx, bias_std=0.5, out_dtype=out_dtype, user_kwargs=kw),
                     repeats=2, prefill="randn")


def test_cta_pair_192_exact_integers_all_layouts():
    # small integers: a misplaced box of the one-and-a-half-box V share shows as a wrong integer
    g = torch.Generator().manual_seed(7)
    m, n, k = 512, 1000, 1096
    a_l = torch.randint(-2, 3, (m, k), generator=g).to(torch.float16)
    b_l = torch.randint(-2, 3, (k, n), generator=g).to(torch.float16)
    ref = (a_l.double() @ b_l.double()).float()
    for layout in LAYOUTS:
        a = O.place(a_l, layout[0] == "t", 0, 0, DEV)
        b = O.place(b_l, layout[1] == "t", 0, 0, DEV)
        for kw in ({"tile_n": 192, "cta_group": 2}, {"tile_n": 192, "cta_group": 2, "stages": 3, "stream_k": True}):
            got = gemm_a16w16(a, b, layout=layout, out_dtype=torch.float32, user_kwargs=kw)
            check_status()
            assert torch.equal(got.cpu(), ref), (layout, kw)


PAIR_512 = [  # 256 x 512 pair tiles: two MMAs per K step into one accumulator that fills TMEM
    (512, 1024, 520, {"tile_n": 512, "cta_group": 2}),
    (700, 900, 1000, {"tile_n": 512, "cta_group": 2}),                      # ragged in M and N, second half-tile partly empty
    (300, 200, 328, {"tile_n": 512, "cta_group": 2}),                       # N inside the first accumulator half
    (2048, 4096, 4096, {"tile_n": 512, "cta_group": 2}),                    # config 2's shape: 64 pair tiles, one wave
    (2048, 4096, 1024, {"tile_n": 512, "cta_group": 2, "max_ctas": 32}),    # four tiles per pair: the accumulator is reused
    (1000, 3000, 4100, {"tile_n": 512, "cta_group": 2, "stream_k": True}),
    (512, 1024, 4096, {"tile_n": 512, "cta_group": 2, "split_k": 3}),
    (2048, 2048, 512, {"tile_n": 512, "cta_group": 2, "group_m": 4, "stages": 3}),
    (1024, 1024, 4096, {"tile_n": 512, "cta_group": 2, "split_k": 4, "split_mode": "atomic"}),
    # widths chosen at run time: any multiple of 32 above 256 (an odd number of 32-column chunks when not a multiple of 64)
    (2048, 4096, 4096, {"tile_n": 480, "cta_group": 2}),                    # config 2 as 72 tiles for 74 pairs
    (512, 1024, 520, {"tile_n": 288, "cta_group": 2}),
    (700, 900, 1000, {"tile_n": 352, "cta_group": 2}),
    (1000, 3000, 1100, {"tile_n": 416, "cta_group": 2, "stream_k": True}),
    (512, 960, 4096, {"tile_n": 320, "cta_group": 2, "split_k": 3}),
    (1024, 1344, 2048, {"tile_n": 448, "cta_group": 2, "split_k": 2, "split_mode": "atomic"}),
    (2048, 1536, 512, {"tile_n": 384, "cta_group": 2, "group_m": 4, "stages": 3, "max_ctas": 16}),
]


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("idx", range(len(PAIR_512)))
def test_cta_pair_512_wide_tiles(dtype, idx):
    m, n, k, kw = PAIR_512[idx]
    for layout in LAYOUTS:
        for out_dtype in (None, "fp32"):
            case = O.Case("pair512", dtype, layout, m, n, k, seed=470 + idx, bias_std=0.5, out_dtype=out_dtype, user_kwargs=kw)
            run_case(case, repeats=2, prefill="randn")


@pytest.mark.parametrize("width", [512, 480, 352, 288])
def test_pair_512_other_exits(width):
    """The wide pair variant away from its TMA-store path: D written transposed (swap_ab, bias along the rows), C rows that
    are not 16-byte aligned (direct vector / scalar stores, including the lone last chunk of an odd chunk count),
    operands that need the aligned copy first, and exact small integers (a misplaced accumulator half or V box shows as
    a wrong integer)."""
    kw = {"tile_n": width, "cta_group": 2}
    run_case(O.Case("wide_swap", "bf16", "nt", 600, 520, 700, seed=31, bias_std=0.5, user_kwargs={**kw, "swap_ab": True}), repeats=2)
    run_case(O.Case("wide_swap32", "fp16", "tn", 600, 520, 700, seed=32, bias_std=0.5, out_dtype="fp32", user_kwargs={**kw, "swap_ab": True}))
    run_case(O.Case("wide_pad", "bf16", "nt", 520, 1000, 333, seed=33, bias_std=0.5, pad=3, offset=1, user_kwargs=kw))
    # C rows that are not 16-byte aligned (N odd): no TMA stores
    for out_dtype in (None, "fp32"):
        run_case(O.Case("wide_oddc", "bf16", "nt", 520, 1031, 520, seed=34, bias_std=0.5, out_dtype=out_dtype, user_kwargs=kw), repeats=2)
    g = torch.Generator().manual_seed(width)
    m, n, k = 512, 2 * width + 40, 1100
    a_l = torch.randint(-2, 3, (m, k), generator=g).to(torch.bfloat16)
    b_l = torch.randint(-2, 3, (k, n), generator=g).to(torch.bfloat16)
    ref = (a_l.double() @ b_l.double()).float()
    for layout in LAYOUTS:
        a = O.place(a_l, layout[0] == "t", 0, 0, DEV)
        b = O.place(b_l, layout[1] == "t", 0, 0, DEV)
        got = gemm_a16w16(a, b, layout=layout, out_dtype=torch.float32, user_kwargs=kw)
        check_status()
        assert torch.equal(got.cpu(), ref), (layout, kw)


@pytest.mark.parametrize("shape", [(1536, 4096, 4096), (2304, 2304, 8192), (5000, 3000, 8000), (3000, 5000, 2000)])
def test_heuristic_run_time_widths_through_the_default_path(shape):
    # shapes outside the shipped table for which the heuristic picks a run-time width of the 512-column variant
    m, n, k = shape
    a = (torch.randn(m, k, device=DEV) * 0.05).to(torch.bfloat16)
    b = (torch.randn(n, k, device=DEV) * 0.05).to(torch.bfloat16).t()
    bias = torch.randn(n, device=DEV).to(torch.bfloat16)
    pl = plan(a, b, "nt", {}, bias=bias)
    assert pl["cta_group"] == 2 and 256 < pl["tile_n"] <= 512 and pl["tile_n"] % 32 == 0, pl
    out = gemm_a16w16(a, b, bias=bias, layout="nt")
    check_status()
    sampled_check(out, a.cpu(), b.cpu(), bias.cpu(), k, torch.bfloat16, n_rows=24, n_cols=24, seed=m)
    # an fp32 output of the same problem falls back to 256-wide pair tiles
    assert plan(a, b, "nt", {}, out_dtype=torch.float32, bias=bias)["tile_n"] == 256


def test_pair_512_plan():
    a = torch.empty(2048, 4096, dtype=torch.bfloat16, device=DEV)
    b = torch.empty(4096, 4096, dtype=torch.bfloat16, device=DEV).t()
    pl = plan(a, b, "nt", {"tile_n": 512, "cta_group": 2})
    assert (pl["tile_m"], pl["tile_n"], pl["tmem_cols"], pl["stages"], pl["grid"]) == (256, 512, 512, 4, 128)
    assert pl["smem_bytes"] <= 232448


def test_default_policy_picks_a_pair_for_large_shapes():
    a = torch.empty(8192, 4096, dtype=torch.bfloat16, device=DEV)
    b = torch.empty(4096, 4096, dtype=torch.bfloat16, device=DEV).t()
    pl = plan(a, b, "nt", {})
    assert pl["cta_group"] == 2 and pl["tile_m"] == 256 and pl["tile_n"] == 256
    run_case(O.Case("pair_default", "bf16", "nt", 4096, 4096, 2048, seed=9, bias_std=0.5))


STREAM_K = [  # shapes whose tile count is not a multiple of the SM count, or smaller than it
    (2048, 4096, 4096, {"tile_n": 256, "stream_k": True}),                 # 256 tiles: 108 cut into spans
    (1000, 3000, 4100, {"tile_n": 256, "stream_k": True}),                 # 96 tiles: all cut
    (1000, 3000, 4100, {"tile_n": 128, "stream_k": True, "group_m": 2}),
    (32, 384, 7168, {"tile_n": 32, "swap_ab": True, "stream_k": True}),    # 3 tiles over 84 CTAs
    (4096, 4736, 512, {"tile_n": 128, "stream_k": True}),                  # remainder wave with short K: borrows a wave
    (129, 136, 1536, {"tile_n": 64, "stream_k": True}),
    (640, 640, 8192, {"tile_n": 128, "stream_k": True}),
    (1, 5120, 2880, {"tile_n": 64, "stream_k": True}),
]


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("idx", range(len(STREAM_K)))
def test_stream_k_shapes(dtype, idx):
    m, n, k, kw = STREAM_K[idx]
    layouts = ("nt",) if kw["tile_n"] < 64 else (("nt", "nn") if m * n * k > 1 << 32 else LAYOUTS)
    for layout in layouts:
        for out_dtype in (None, "fp32"):
            run_case(O.Case("streamk", dtype, layout, m, n, k, seed=300 + idx, bias_std=0.5, out_dtype=out_dtype, user_kwargs=kw),
                     repeats=2, prefill="randn")


def test_stream_k_is_deterministic():
    case = O.Case("sk_det", "bf16", "nt", 1000, 3000, 4100, seed=5, bias_std=0.5, user_kwargs={"tile_n": 256, "stream_k": True})
    a, b, bias, *_ = O.build_inputs(case, device=DEV)
    outs = [gemm_a16w16(a, b, bias=bias, user_kwargs=case.user_kwargs, layout="nt").clone() for _ in range(4)]
    check_status()
    assert all(torch.equal(outs[0], o) for o in outs[1:])


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("split_k", [1, 3])
def test_fp32_output_64x64x768(layout, dtype, bias, split_k):
    run_case(O.Case("fp32out", dtype, layout, 64, 64, 768, seed=7, bias_std=1.0 if bias else None, out_dtype="fp32",
                    user_kwargs={"tile_n": 64, "split_k": split_k}))


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("m", [1, 3, 8, 17])
def test_small_m(layout, dtype, m):
    # M = 3 with a column-major A is rejected by the reference (M % 8); it runs here.
    for kw in ({}, {"tile_n": 64}, {"tile_n": 64, "swap_ab": True, "split_k": 2}):
        run_case(O.Case("small_m", dtype, layout, m, 32, 512, seed=m, bias_std=0.5, user_kwargs=kw))
        run_case(O.Case("small_m_wide", dtype, layout, m, 1000, 200, seed=m, user_kwargs=kw))


@pytest.mark.parametrize("tile_n", [16, 32])
@pytest.mark.parametrize("swap", [False, True])
def test_narrow_tiles_k_contiguous(tile_n, swap):
    layout = "nt"
    m, n = (24, 300) if swap else (300, 24)
    for dtype in ("bf16", "fp16"):
        run_case(O.Case("narrow", dtype, layout, m, n, 640, seed=5, bias_std=0.3, user_kwargs={"tile_n": tile_n, "swap_ab": swap}))
        run_case(O.Case("narrow_split", dtype, layout, m, n, 2000, seed=6, bias_std=0.3, out_dtype="fp32",
                        user_kwargs={"tile_n": tile_n, "swap_ab": swap, "split_k": 5}))


@pytest.mark.parametrize("tile_k", [64, 128])
@pytest.mark.parametrize("tile_n", [16, 32, 64, 128])
def test_both_stage_depths(tile_n, tile_k):
    # Single-CTA tiles up to 128 wide are built with 64- and 128-deep pipeline stages; K = 1000 leaves a ragged
    # last stage in both, and the split and cluster modes see uneven slices.
    for layout in (LAYOUTS if tile_n >= 64 else ("nt",)):
        for extra in ({}, {"split_k": 3}, {"split_k": 4, "split_mode": "cluster"}):
            kw = {"tile_n": tile_n, "tile_k": tile_k, **extra}
            case = O.Case("depth", "bf16", layout, 200, 264, 1000, seed=tile_n + tile_k, bias_std=0.2,
                          out_dtype="fp32" if extra else None, user_kwargs=kw)
            run_case(case)


@pytest.mark.parametrize("layout", LAYOUTS)
def test_exhaustive_edge_residues(layout):
    # every residue class of M mod 8 and N mod 8 around one tile, K around one K block
    for m in (121, 128, 129, 135):
        for n in (57, 64, 65, 71, 72):
            for k in (1, 8, 63, 64, 65, 72):
                run_case(O.Case("edge", "fp16", layout, m, n, k, seed=m * n + k, bias_std=0.2, out_dtype="fp32",
                                pad=8 if layout == "nt" else 0, user_kwargs={"tile_n": 64}))


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("split_k", [1, 2])
def test_padded_stride_and_storage_offset(layout, split_k):
    # cf. test_gemm_a16w16_gfx950.py:688-766: one leading row skipped, 8 leading columns skipped, pitch padded
    m = n = 64
    k = 256
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(9)

    def padded(rows, cols, padding, is_t):
        lead, other = (rows, cols) if is_t else (cols, rows)
        storage = torch.full((other + 1, lead + padding), float("nan"), dtype=dtype, device=DEV)
        logical = (torch.rand(rows, cols, generator=g) * 2 - 1).to(dtype)
        view = storage[1:, 8:8 + lead]
        view.copy_((logical.t() if is_t else logical).to(DEV))
        return (view.t() if is_t else view), logical

    a, a_l = padded(m, k, 32, layout[0] == "t")
    b, b_l = padded(k, n, 48, layout[1] == "t")
    assert not a.is_contiguous() and not b.is_contiguous() and a.storage_offset() > 0
    bias_l = (torch.rand(n, generator=g) * 2 - 1).to(dtype)
    out = torch.empty((m, n), dtype=dtype, device=DEV)
    kw = {"block_m": 64, "block_n": 64, "block_k": 64, "stages": 2, "split_k": split_k, "m_waves": 2, "n_waves": 2,
          "group_m": 0, "use_half_tile_interleaved": True}
    res = gemm_a16w16(a, b, out, bias=bias_l.to(DEV), user_kwargs=kw, layout=layout)
    check_status()
    assert res.data_ptr() == out.data_ptr()
    O.assert_close(out, O.reference_matmul(a_l, b_l, bias_l, dtype), k, f"padded {layout}")


@pytest.mark.parametrize("layout", LAYOUTS)
def test_unaligned_base_and_odd_pitch(layout):
    # base pointer 2 bytes off a 16-byte boundary and an odd pitch: the reference rejects this, the repack path runs it
    run_case(O.Case("unaligned", "bf16", layout, 150, 200, 333, seed=21, bias_std=0.5, pad=3, offset=1, user_kwargs={"tile_n": 64}))
    run_case(O.Case("unaligned_split", "fp16", layout, 150, 200, 1333, seed=22, out_dtype="fp32", pad=1, offset=7,
                    user_kwargs={"tile_n": 128, "split_k": 3}))


LOADER_POLICIES = [
    {"tile_n": 16, "swap_ab": True}, {"tile_n": 32, "tile_k": 64}, {"tile_n": 64}, {"tile_n": 64, "tile_k": 64, "split_k": 3},
    {"tile_n": 128}, {"tile_n": 128, "tile_k": 64, "stream_k": True}, {"tile_n": 256}, {"tile_n": 128, "cta_group": 2},
    {"tile_n": 192, "cta_group": 2}, {"tile_n": 256, "cta_group": 2}, {"tile_n": 256, "cta_group": 2, "stream_k": True},
    {"tile_n": 32, "swap_ab": True, "split_k": 4, "split_mode": "cluster"},
]


@pytest.mark.parametrize("pad", [6, 14, 22])
@pytest.mark.parametrize("idx", range(len(LOADER_POLICIES)))
def test_loader_warps_fetch_8_byte_aligned_rows(pad, idx):
    """Operands whose K-contiguous rows start on 8- but not 16-byte boundaries (pitch = K + pad = 1036, 1044 or 1052
    elements, i.e. 8 mod 16 bytes) go through the cp.async loader warps of every tile family: ragged M, N and K (K = 1030 leaves a
    6-element tail in the last 64-deep box, so pieces are cut at 4 and at 12 bytes), NaN-poisoned padding, both
    dtypes, one or both operands on the loader, bit-equal to the aligned-copy path."""
    kw = LOADER_POLICIES[idx]
    small_n = kw["tile_n"] < 64 and not kw.get("swap_ab")
    layouts = ("nt",) if (small_n or kw.get("swap_ab")) else ("nt", "tt") if kw["tile_n"] == 192 else ("nt", "nn", "tt")
    for dtype, layout in [(d, l) for d in ("bf16", "fp16") for l in layouts]:
        case = O.Case("loader", dtype, layout, 300, 456, 1030, seed=900 + idx + pad, bias_std=0.3, out_dtype="fp32" if idx % 2 else None,
                      pad=pad, offset=4 * (idx % 3), user_kwargs=kw)
        a, b, bias, a_l, b_l, bias_l = O.build_inputs(case, device=DEV)
        pl = plan(a, b, layout, {**kw, "loader": True}, out_dtype=case.torch_out_dtype)
        assert pl["a_loader"] == (1 if layout[0] == "n" else 0) and pl["b_loader"] == (1 if layout[1] == "t" else 0), pl
        assert pl["a_repacked"] == 0 or layout[0] == "t"
        ref = O.reference_matmul(a_l, b_l, bias_l, case.torch_out_dtype)
        outs = []
        for loader in (True, False):
            out = torch.full((case.m, case.n), float("nan"), dtype=case.torch_out_dtype, device=DEV)
            got = gemm_a16w16(a, b, out, bias=bias, user_kwargs={**kw, "loader": loader}, layout=layout)
            check_status()
            O.assert_close(got, ref, case.k, f"loader={loader} {dtype} {layout} pad {pad} {kw}")
            outs.append(got.clone())
        if not kw.get("stream_k") and kw.get("split_k", 1) == 1:
            assert torch.equal(outs[0], outs[1])  # same tiles, same order of accumulation


def test_loader_warps_exact_integers_full_tiles():
    # small integers: fp32 accumulation is exact, so any misplaced 16-byte piece shows as a wrong integer
    g = torch.Generator().manual_seed(5)
    m, n, k = 512, 768, 2052
    a_l = torch.randint(-2, 3, (m, k), generator=g).to(torch.bfloat16)
    b_l = torch.randint(-2, 3, (k, n), generator=g).to(torch.bfloat16)
    ref = (a_l.double() @ b_l.double()).float()
    for layout in ("nt", "nn", "tt"):
        a = O.place(a_l, layout[0] == "t", 8, 8, DEV)   # K pitch 2060 elements = 4120 bytes: 8 mod 16
        b = O.place(b_l, layout[1] == "t", 8, 8, DEV)
        for kw in ({"tile_n": 256, "cta_group": 2}, {"tile_n": 128}, {"tile_n": 192, "cta_group": 2} if layout[1] == "t" else {"tile_n": 64}):
            kw = {**kw, "loader": True}
            pl = plan(a, b, layout, kw, out_dtype=torch.float32)
            assert pl["a_loader"] + pl["b_loader"] >= 1
            got = gemm_a16w16(a, b, layout=layout, out_dtype=torch.float32, user_kwargs=kw)
            check_status()
            assert torch.equal(got.cpu(), ref), (layout, kw)


ATOMIC_POLICIES = [
    {"tile_n": 64, "split_k": 3}, {"tile_n": 128, "split_k": 2}, {"tile_n": 128, "tile_k": 64, "stream_k": True},
    {"tile_n": 256, "split_k": 4}, {"tile_n": 256, "stream_k": True}, {"tile_n": 128, "cta_group": 2, "split_k": 2},
    {"tile_n": 256, "cta_group": 2, "stream_k": True}, {"tile_n": 256, "cta_group": 2, "split_k": 3},
    {"tile_n": 192, "cta_group": 2, "stream_k": True},
]


@pytest.mark.parametrize("idx", range(len(ATOMIC_POLICIES)))
def test_atomic_split_mode_adds_partial_tiles_into_fp32_output(idx):
    """split_mode 'atomic': K slices / stream-K spans add their fp32 tiles into C with TMA reduce-add after a small
    kernel has put the bias (or zero) there. No workspace; the result is within the split-K bound of the contract
    (the order of the additions is not fixed). Ragged M, N, K; outputs pre-filled with NaN; repeated calls."""
    kw = {**ATOMIC_POLICIES[idx], "split_mode": "atomic"}
    layouts = ("nt", "tt") if kw["tile_n"] == 192 else LAYOUTS
    for dtype, layout, bias in [("bf16", layouts[0], 0.5), ("fp16", layouts[-1], None), ("bf16", layouts[1], 0.5)]:
        case = O.Case("atomic", dtype, layout, 700, 936, 2100, seed=300 + idx, bias_std=bias, out_dtype="fp32", user_kwargs=kw)
        a, b, bias_d, a_l, b_l, bias_l = O.build_inputs(case, device=DEV)
        pl = plan(a, b, layout, kw, out_dtype=torch.float32, bias=bias_d)
        assert pl["atomic_out"] == 1 and pl["partial_bytes"] == 0, pl  # no partial tiles in the workspace
        run_case(case, repeats=3)


def test_atomic_split_mode_falls_back_where_it_cannot_apply():
    # 16-bit output, or C written transposed (swap_ab), or a C row pitch TMA cannot take: the ticket mode runs
    a = torch.empty(300, 2048, dtype=torch.bfloat16)
    b = torch.empty(520, 2048, dtype=torch.bfloat16).t()
    kw = {"tile_n": 128, "split_k": 4, "split_mode": "atomic"}
    assert plan(a, b, "nt", kw, out_dtype=torch.float32)["atomic_out"] == 1
    pl = plan(a, b, "nt", kw, out_dtype=torch.bfloat16)
    assert pl["atomic_out"] == 0 and pl["partial_bytes"] > 0
    assert plan(a, b, "nt", {**kw, "tile_n": 64, "swap_ab": True}, out_dtype=torch.float32)["atomic_out"] == 0
    assert plan(a, b[:, :518], "nt", kw, out_dtype=torch.float32)["atomic_out"] == 0  # N = 518: rows of C not 16-byte aligned
    run_case(O.Case("atomic_bf16", "bf16", "nt", 300, 520, 2048, seed=41, bias_std=0.5, user_kwargs=kw))
    run_case(O.Case("atomic_odd_n", "bf16", "nt", 300, 518, 2048, seed=42, bias_std=0.5, out_dtype="fp32", user_kwargs=kw))


def test_config4_atomic_stream_k():
    a_l, b_l, bias_l, ref = _c4_reference()
    for layout in LAYOUTS:
        case = O.CONFIGS[f"c4_{layout}"]
        a = O.place(a_l, layout[0] == "t", case.pad, case.offset, DEV)
        b = O.place(b_l, layout[1] == "t", case.pad, case.offset, DEV)
        kw = {"tile_n": 256, "cta_group": 2, "stream_k": True, "split_mode": "atomic"}
        for rep in range(2):
            out = torch.full((case.m, case.n), float("nan"), dtype=torch.float32, device=DEV)
            got = gemm_a16w16(a, b, out, bias=bias_l.to(DEV), user_kwargs=kw, layout=layout)
            check_status()
            O.assert_close(got, ref, case.k, f"c4 {layout} atomic stream-K call {rep}")


def test_allocates_output_with_default_policy():
    a_l = torch.randn(64, 256).to(torch.bfloat16)
    b_l = torch.randn(256, 64).to(torch.bfloat16)
    a = a_l.to(DEV)
    b = b_l.t().contiguous().to(DEV).t()
    out = gemm_a16w16(a, b)
    check_status()
    assert out.shape == (64, 64) and out.dtype is torch.bfloat16 and out.device == a.device
    O.assert_close(out, O.reference_matmul(a_l, b_l, None, torch.bfloat16), 256)
    out32 = gemm_a16w16(a, b, out_dtype=torch.float32)
    assert out32.dtype is torch.float32
    O.assert_close(out32, O.reference_matmul(a_l, b_l, None, torch.float32), 256)


def test_out_may_be_nd_and_result_aliases_it():
    a_l = torch.randn(96, 128).to(torch.float16)
    b_l = torch.randn(128, 80).to(torch.float16)
    out = torch.full((4, 24, 80), float("nan"), dtype=torch.float16, device=DEV)
    got = gemm_a16w16(a_l.to(DEV), b_l.to(DEV), out, layout="nn")
    check_status()
    assert got.shape == (96, 80) and got.data_ptr() == out.data_ptr()
    O.assert_close(out.view(96, 80), O.reference_matmul(a_l, b_l, None, torch.float16), 128)


def test_strided_bias_is_made_contiguous():
    a_l = torch.randn(64, 256).to(torch.bfloat16)
    b_l = torch.randn(256, 64).to(torch.bfloat16)
    bias_storage = torch.randn(128).to(torch.bfloat16)
    bias = bias_storage.to(DEV)[::2]
    assert not bias.is_contiguous()
    out = gemm_a16w16(a_l.to(DEV), b_l.t().contiguous().to(DEV).t(), bias=bias, layout="nt")
    check_status()
    O.assert_close(out, O.reference_matmul(a_l, b_l, bias_storage[::2], torch.bfloat16), 256)


@pytest.mark.parametrize("n", [4096, 4032])
def test_grouped_raster_boundary_paths(n):
    # cf. test_gemm_a16w16_gfx950.py:890-909: ragged last group of tile rows
    run_case(O.Case("raster", "bf16", "nt", 320, n, 256, seed=n, user_kwargs={"tile_n": 64, "group_m": 4}), repeats=2)
    run_case(O.Case("raster2", "bf16", "nt", 5 * 128 + 7, 777, 192, seed=n, user_kwargs={"tile_n": 64, "group_m": 3}))


def test_split_k_workspaces_are_per_stream():
    # cf. test_gemm_a16w16_gfx950.py:933-998: two streams running split-K at once must not share tickets/partials
    case = O.Case("streams", "bf16", "nt", 256, 512, 4096, seed=31, bias_std=0.5, user_kwargs={"tile_n": 64, "split_k": 8})
    a, b, bias, a_l, b_l, bias_l = O.build_inputs(case, device=DEV)
    ref = O.reference_matmul(a_l, b_l, bias_l, torch.bfloat16)
    outs = [torch.full((256, 512), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    for rep in range(10):
        for s, o in zip(streams, outs):
            with torch.cuda.stream(s):
                gemm_a16w16(a, b, o, bias=bias, user_kwargs=case.user_kwargs, layout="nt", stream=s)
    for s in streams:
        s.synchronize()
    check_status()
    for o in outs:
        O.assert_close(o, ref, case.k, "two streams")


def test_repeated_calls_leave_tickets_clean():
    case = O.Case("repeat", "fp16", "tn", 300, 200, 3000, seed=41, bias_std=0.5, out_dtype="fp32", user_kwargs={"tile_n": 64, "split_k": 6})
    run_case(case, repeats=5, prefill="randn")
    # a different split-K shape right after, on the same workspace
    run_case(O.Case("repeat2", "fp16", "nt", 100, 700, 1000, seed=42, user_kwargs={"tile_n": 128, "split_k": 4}), repeats=2)


def test_prepared_call_cache_tracks_workspace_growth_and_new_tensors():
    from flydsl_examples_b200 import gemm_a16w16 as G

    G.clear_prepared_calls()
    case = O.Case("cache", "bf16", "nt", 130, 200, 2048, seed=51, bias_std=0.5, out_dtype="fp32", user_kwargs={"tile_n": 64, "split_k": 4})
    a, b, bias, a_l, b_l, bias_l = O.build_inputs(case, device=DEV)
    ref = O.reference_matmul(a_l, b_l, bias_l, torch.float32)
    out = torch.empty((130, 200), dtype=torch.float32, device=DEV)
    for _ in range(3):  # first call prepares, the next two reuse the handle
        out.fill_(float("nan"))
        gemm_a16w16(a, b, out, bias=bias, user_kwargs=case.user_kwargs, layout="nt")
        check_status()
        O.assert_close(out, ref, case.k, "cached call")
    assert len(G._prepared) == 1
    # a call that needs a much larger workspace makes it grow; the old handle must not be reused with the stale pointer
    big = O.Case("cache_big", "bf16", "nt", 1024, 2048, 8192, seed=52, out_dtype="fp32", user_kwargs={"tile_n": 128, "split_k": 16})
    run_case(big)
    out.fill_(float("nan"))
    gemm_a16w16(a, b, out, bias=bias, user_kwargs=case.user_kwargs, layout="nt")
    check_status()
    O.assert_close(out, ref, case.k, "after workspace growth")
    # same storage, new contents: the cached launch reads the new data
    a.copy_((a_l * 2).to(DEV))
    gemm_a16w16(a, b, out, bias=bias, user_kwargs=case.user_kwargs, layout="nt")
    check_status()
    O.assert_close(out, O.reference_matmul(a_l * 2, b_l, bias_l, torch.float32), case.k, "new contents")


def test_zero_sized_and_k_zero():
    a = torch.empty(0, 64, dtype=torch.bfloat16, device=DEV)
    b = torch.empty(64, 32, dtype=torch.bfloat16, device=DEV)
    assert gemm_a16w16(a, b, layout="nn").shape == (0, 32)
    bias = torch.randn(32).to(torch.bfloat16)
    out = gemm_a16w16(torch.empty(5, 0, dtype=torch.bfloat16, device=DEV), torch.empty(0, 32, dtype=torch.bfloat16, device=DEV),
                      bias=bias.to(DEV), layout="nn")
    assert torch.equal(out.cpu(), bias.expand(5, 32))


def test_integer_inputs_are_exact_in_every_layout():
    g = torch.Generator().manual_seed(2)
    a_l = torch.randint(-3, 4, (200, 328), generator=g).float()
    b_l = torch.randint(-3, 4, (328, 264), generator=g).float()
    want = a_l @ b_l
    for layout in LAYOUTS:
        for dt in (torch.bfloat16, torch.float16):
            a = O.place(a_l.to(dt), layout[0] == "t", device=DEV)
            b = O.place(b_l.to(dt), layout[1] == "t", device=DEV)
            got = gemm_a16w16(a, b, layout=layout, out_dtype=torch.float32, user_kwargs={"tile_n": 64, "split_k": 2})
            check_status()
            assert torch.equal(got.cpu(), want), (layout, dt)


def test_linearity_at_full_config2_size():
    # size-independent property: (A1 + A2) B == A1 B + A2 B when the sums are exact (integers)
    g = torch.Generator().manual_seed(8)
    m, n, k = 2048, 4096, 4096
    a1 = torch.randint(-2, 3, (m, k), generator=g).to(torch.bfloat16).to(DEV)
    a2 = torch.randint(-2, 3, (m, k), generator=g).to(torch.bfloat16).to(DEV)
    b = torch.randint(-2, 3, (n, k), generator=g).to(torch.bfloat16).to(DEV).t()
    f = lambda x: gemm_a16w16(x, b, layout="nt", out_dtype=torch.float32)
    lhs = f(a1 + a2)
    rhs = f(a1) + f(a2)
    check_status()
    assert torch.equal(lhs, rhs)


def test_bounded_wait_runs_out_and_is_reported():
    """The liveness guarantee of every kernel here: a wait that nobody satisfies ends at its time limit, the kernel
    returns normally with a note in the status block, and the context stays usable. Exercised on the wait primitive
    alone (one thread, one barrier nobody signals, 200 us limit): no GEMM is made to fail."""
    import ctypes as C

    from flydsl_examples_b200 import _lib
    from flydsl_examples_b200 import gemm_a16w16 as G

    lib = _lib.load()
    # a split-K call first, so that this stream has a workspace whose tickets check_status() must clear
    case = O.Case("before", "bf16", "nt", 200, 328, 1000, seed=77, bias_std=0.5, user_kwargs={"tile_n": 64, "split_k": 3})
    run_case(case)
    stream = torch.cuda.current_stream()
    ws = G._workspace_for(torch.device("cuda", torch.cuda.current_device()), stream)
    ws.buf[:64].fill_(7)  # tickets as a kernel that gave up could have left them
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = lib.b200_gemm_wait_selftest(ws.status.data_ptr(), 200, C.c_void_p(stream.cuda_stream))
    t1.record()
    assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 50.0  # milliseconds: the limit ended the wait (200 us at 2 GHz; longer at low clocks)
    assert ws.status.tolist() == [1, 0, 9, -1]
    with pytest.raises(RuntimeError, match="gave up a bounded wait: code=1 cta=0 role=9"):
        check_status()
    assert ws.status.tolist() == [0, 0, 0, 0] or ws.status.tolist()[0] == 0
    assert int(ws.buf[:64].sum()) == 0  # the ticket region was cleared
    check_status()                      # nothing pending any more
    run_case(case, repeats=2)           # and the next split-K call on this stream is right
