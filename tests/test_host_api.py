"""Host-side logic on CPU: policy resolution, validation, the error contract of the public call (the reference's
negative tests, test_gemm_a16w16_gfx950.py:810-858 and :1001-1031), scheduler arithmetic. No GPU, no kernels."""
import pytest
import torch

from flydsl_examples_b200 import policy as P
from flydsl_examples_b200.gemm_a16w16 import gemm_a16w16, make_gemm_a16w16_param_and_validate, plan
from kernels.gemm_a16w16_gfx950 import GEMM_A16W16_DTYPE_BF16, GEMM_A16W16_DTYPE_FP16, GEMM_A16W16_DTYPE_FP32
from kernels.gemm_a16w16_gfx950_utils import GFX950_DMA_BYTES

REF_KW = {"block_m": 64, "block_n": 64, "block_k": 64, "stages": 2, "m_waves": 2, "n_waves": 2, "group_m": 0}


def _mat(rows, cols, dtype, is_t):
    return torch.empty(cols, rows, dtype=dtype).t() if is_t else torch.empty(rows, cols, dtype=dtype)


def test_reexported_names():
    assert (GEMM_A16W16_DTYPE_FP32, GEMM_A16W16_DTYPE_BF16, GEMM_A16W16_DTYPE_FP16) == (1, 2, 3)
    assert GFX950_DMA_BYTES == 16


def test_bad_layout_is_value_error():
    a, b = torch.empty(8, 8, dtype=torch.bfloat16), torch.empty(8, 8, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="unsupported GEMM layout"):
        gemm_a16w16(a, b, layout="xy")


@pytest.mark.parametrize(("operand", "layout"), [("A", "nn"), ("A", "tn"), ("B", "nn"), ("B", "nt")])
def test_rejects_wrong_contiguous_dim(operand, layout):
    m = n = 64
    k = 256
    dt = torch.bfloat16
    a = _mat(m, k, dt, layout[0] == "t")
    b = _mat(k, n, dt, layout[1] == "t")
    if operand == "A":
        a = torch.empty(m, k, dtype=dt) if layout[0] == "t" else torch.empty(m, 2 * k, dtype=dt)[:, ::2]
    else:
        b = torch.empty(k, n, dtype=dt) if layout[1] == "t" else torch.empty(k, 2 * n, dtype=dt)[:, ::2]
    with pytest.raises(ValueError, match=rf"^{operand} does not satisfy"):
        gemm_a16w16(a, b, layout=layout)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_strict_mode_rejects_unaligned_m_for_column_major_a(dtype):
    vec = GFX950_DMA_BYTES // 2
    m, n, k = vec + 1, 64, 256
    a = torch.empty(k, 2 * vec, dtype=dtype)[:, :m].t()
    b = torch.empty(k, n, dtype=dtype)
    with pytest.raises(ValueError, match=rf"M divisible by {vec}"):
        gemm_a16w16(a, b, layout="tn", user_kwargs={"strict_reference_envelope": True})


@pytest.mark.parametrize(("k", "hti", "message"), [(480, False, "K-tail is unsupported"), (64, True, "HTI requires at least two"), (192, True, "HTI requires at least two")])
def test_strict_mode_rejects_k_partitioning(k, hti, message):
    a = torch.empty(64, k, dtype=torch.bfloat16)
    b = _mat(k, 64, torch.bfloat16, True)
    kw = dict(REF_KW, use_half_tile_interleaved=hti, strict_reference_envelope=True)
    with pytest.raises(AssertionError, match=message):
        gemm_a16w16(a, b, user_kwargs=kw, layout="nt")


def test_default_mode_has_no_cpu_path():
    a = torch.empty(64, 480, dtype=torch.bfloat16)
    b = _mat(480, 64, torch.bfloat16, True)
    with pytest.raises(AssertionError, match="CUDA tensors only"):
        gemm_a16w16(a, b)


def test_dtype_and_shape_asserts():
    a = torch.empty(8, 16, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        gemm_a16w16(a, torch.empty(16, 8, dtype=torch.float16), layout="nn")
    with pytest.raises(AssertionError):
        gemm_a16w16(a, torch.empty(12, 8, dtype=torch.bfloat16), layout="nn")
    with pytest.raises(AssertionError):
        gemm_a16w16(torch.empty(8, 16), torch.empty(16, 8), layout="nn")
    with pytest.raises(ValueError, match="unsupported output dtype"):
        gemm_a16w16(a, torch.empty(16, 8, dtype=torch.bfloat16), layout="nn", out_dtype=torch.float16)
    with pytest.raises(AssertionError):  # out not contiguous
        gemm_a16w16(a, torch.empty(16, 8, dtype=torch.bfloat16), out=torch.empty(8, 16, dtype=torch.bfloat16)[:, ::2], layout="nn")
    with pytest.raises(AssertionError):  # bias length
        gemm_a16w16(a, torch.empty(16, 8, dtype=torch.bfloat16), bias=torch.empty(7, dtype=torch.bfloat16), layout="nn")
    with pytest.raises(ValueError, match="unknown gemm_a16w16 policy keys"):
        P.from_user_kwargs({"tile_q": 3}, 8, 8, 8, "nt")


def test_reference_policy_keys_are_accepted():
    kw = dict(REF_KW, split_k=2, k_waves=1, use_half_tile_interleaved=True)
    pol = P.from_user_kwargs(kw, 64, 64, 512, "nt")
    assert pol.split_k == 2 and pol.tile_n in P.TILE_N_MENU
    assert P.validate(pol, 64, 64, 512, "nt") is None
    assert make_gemm_a16w16_param_and_validate(64, 64, 512, dict(kw, a_is_transposed=False, b_is_transposed=True)) is not None
    assert make_gemm_a16w16_param_and_validate(64, 64, 512, {"tile_n": 48}) is None
    assert make_gemm_a16w16_param_and_validate(64, 64, 512, {"tile_n": 256, "stages": 1}) is None


def test_blackwell_policy_is_taken_literally():
    pol = P.from_user_kwargs({"tile_n": 128, "stages": 3, "split_k": 5, "group_m": 2}, 4096, 4096, 4096, "nt")
    assert (pol.tile_n, pol.stages, pol.split_k, pol.group_m, pol.swap_ab) == (128, 3, 5, 2, False)
    pol = P.from_user_kwargs({"tile_n": 32, "swap_ab": True}, 32, 384, 7168, "nt")
    assert pol.swap_ab and pol.split_k == 1


def test_validate_rules():
    assert P.validate(P.Policy(tile_n=32), 32, 384, 512, "nn") is not None  # N-contiguous B on a 32-wide tile
    assert P.validate(P.Policy(tile_n=64), 32, 384, 512, "nn") is None
    assert P.validate(P.Policy(tile_n=32, swap_ab=True), 32, 384, 512, "tn") is not None  # M-contiguous A after swap
    assert P.validate(P.Policy(tile_n=256, stages=1), 512, 512, 512, "nt") is not None
    assert P.validate(P.Policy(tile_n=256, stages=4), 512, 512, 512, "nt") is None
    assert P.validate(P.Policy(tile_n=256, stages=9), 512, 512, 512, "nt") is None  # clamped to what fits
    assert P.validate(P.Policy(tile_n=128, split_k=0), 512, 512, 512, "nt") is not None
    for t in P.TILE_N_MENU:
        assert P.smem_bytes(t, P.MAX_STAGES[t]) <= P.SMEM_LIMIT
        assert P.smem_bytes(t, P.MAX_STAGES_K64[t], 1, 64) <= P.SMEM_LIMIT
    for t, st in P.MAX_STAGES_PAIR.items():
        assert P.smem_bytes(t, st, 2) <= P.SMEM_LIMIT
    assert (P.tile_k(128), P.tile_k(256), P.tile_k(128, 2), P.tile_k(128, 1, 64)) == (128, 64, 64, 64)
    assert P.validate(P.Policy(tile_n=256, tile_k=128), 512, 512, 512, "nt") is not None
    assert P.validate(P.Policy(tile_n=64, tile_k=64), 512, 512, 512, "nt") is None
    assert (P.max_stages(128), P.max_stages(128, 1, 64), P.max_stages(128, 2)) == (3, 6, 8)
    # 512 columns: one accumulator that fills TMEM, CTA pairs only, four 48 KB stages
    assert P.validate(P.Policy(tile_n=512), 512, 1024, 512, "nt") is not None
    assert P.validate(P.Policy(tile_n=512, cta_group=2), 512, 1024, 512, "nt") is None
    assert P.validate(P.Policy(tile_n=512, cta_group=2), 512, 1024, 512, "nn") is None
    assert P.validate(P.Policy(tile_n=512, cta_group=2, split_k=2, split_mode="cluster"), 512, 1024, 512, "nt") is not None
    assert P.max_stages(512, 2) == 4 and P.smem_bytes(512, 5, 2) > P.SMEM_LIMIT


def test_heuristic_is_always_valid():
    shapes = [(1, 5120, 2880), (3, 32, 256), (32, 384, 7168), (256, 512, 1024), (2048, 4096, 4096), (1000, 3000, 4100),
              (16384, 28672, 8192), (16384, 3584, 8192), (65, 96, 192), (4096, 128, 6144), (8, 7168, 2048), (8192, 8192, 8192),
              (6000, 6000, 6000)]
    for m, n, k in shapes:
        for layout in ("nn", "nt", "tn", "tt"):
            pol = P.heuristic(m, n, k, layout)
            assert P.validate(pol, m, n, k, layout) is None, (m, n, k, layout, pol)


def test_heuristic_is_valid_on_random_shapes():
    import random

    rng = random.Random(1234)
    seen_wide = 0
    for _ in range(400):
        m = rng.choice([1, 7, 33, 130, 300, 700, 1536, 2304, 5000, 9000, rng.randint(1, 12000)])
        n = rng.choice([16, 100, 384, 2000, 4096, 5120, 7000, rng.randint(8, 30000)])
        k = rng.choice([64, 200, 1000, 4100, 8192, rng.randint(1, 16384)])
        layout = rng.choice(["nn", "nt", "tn", "tt"])
        pol = P.heuristic(m, n, k, layout)
        assert P.validate(pol, m, n, k, layout) is None, (m, n, k, layout, pol)
        if pol.cta_group == 2 and pol.tile_n > 256:
            seen_wide += 1
            assert pol.tile_n % 32 == 0 and pol.tile_n <= 512
            assert P.smem_bytes(pol.tile_n, P.max_stages(pol.tile_n, 2), 2) <= P.SMEM_LIMIT
    assert seen_wide > 0  # the run-time widths of the 512-column variant are among the picks


def test_split_k_slices_cover_k_exactly_once():
    for k, tk in ((1, 64), (63, 64), (64, 128), (65, 64), (1000, 128), (4100, 64), (4100, 128), (7168, 128)):
        for s in (1, 2, 3, 7, 8, 16, 32, 200):
            sl = P.split_k_slices(k, s, tk)
            kb = (k + tk - 1) // tk
            assert len(sl) == min(s, kb)
            assert all(n >= 1 for _, n in sl)
            assert sl[0][0] == 0 and sum(n for _, n in sl) == kb
            for (f0, n0), (f1, _) in zip(sl, sl[1:]):
                assert f0 + n0 == f1


@pytest.mark.parametrize("group", [0, 1, 3, 4, 8, 100])
def test_raster_is_a_bijection(group):
    for tp, tq in ((1, 1), (5, 7), (16, 16), (3, 64), (13, 2)):
        seen = {P.raster(t, tp, tq, group) for t in range(tp * tq)}
        assert seen == {(i, j) for i in range(tp) for j in range(tq)}


def test_raster_groups_rows_like_group_m():
    # group_m = 4 over 8x3 tiles: the first 12 tile ids cover rows 0..3 only, row index fastest
    ids = [P.raster(t, 8, 3, 4) for t in range(12)]
    assert {r for r, _ in ids} == {0, 1, 2, 3}
    assert ids[:5] == [(0, 0), (1, 0), (2, 0), (3, 0), (0, 1)]


def test_plan_query_on_cpu_tensors():
    a = torch.empty(2048, 4096, dtype=torch.bfloat16)
    b = torch.empty(4096, 4096, dtype=torch.bfloat16).t()
    pl = plan(a, b, "nt", {"tile_n": 256, "group_m": 8})
    assert (pl["tile_m"], pl["tile_n"], pl["tile_k"], pl["stages"]) == (128, 256, 64, 4)
    assert plan(a, b, "nt", {"tile_n": 128})["tile_k"] == 128 and plan(a, b, "nt", {"tile_n": 128, "cta_group": 2})["tile_k"] == 64
    pl64 = plan(a, b, "nt", {"tile_n": 128, "tile_k": 64})
    assert (pl64["tile_k"], pl64["stages"]) == (64, 6)
    assert pl["tiles_p"] * pl["tiles_q"] == 256 and pl["num_units"] == 256
    assert pl["workspace_bytes"] == 0 and pl["tmem_cols"] == 512
    assert pl["smem_bytes"] == P.smem_bytes(256, 4) <= P.SMEM_LIMIT
    pl = plan(torch.empty(32, 7168, dtype=torch.bfloat16), torch.empty(384, 7168, dtype=torch.bfloat16).t(), "nt",
              {"tile_n": 32, "swap_ab": True, "split_k": 16}, out_dtype=torch.float32)
    assert pl["swap_ab"] == 1 and pl["tiles_p"] == 3 and pl["tiles_q"] == 1 and pl["num_units"] == 48
    assert pl["partial_bytes"] == 48 * 128 * 32 * 4 and pl["counter_bytes"] == 1 << 20
    plw = plan(a, b, "nt", {"tile_n": 512, "cta_group": 2})
    assert (plw["tile_m"], plw["tile_n"], plw["stages"], plw["tmem_cols"], plw["grid"]) == (256, 512, 4, 512, 128)
    assert plw["smem_bytes"] == P.smem_bytes(512, 4, 2) <= P.SMEM_LIMIT
    with pytest.raises(RuntimeError, match="unsupported policy"):
        plan(a, b, "nt", {"tile_n": 512})
    # split_k larger than the number of K blocks (128 deep for this tile) is clamped
    pl = plan(torch.empty(64, 300, dtype=torch.float16), torch.empty(300, 64, dtype=torch.float16), "nn", {"tile_n": 64, "split_k": 9})
    assert pl["split_k"] == 3


def test_plan_flags_operands_tma_cannot_describe():
    # K = 4100 fp16 with +64 padding: a K-contiguous operand has an 8328-byte pitch (not a multiple of 16)
    buf = torch.empty(1000 * 4164 + 256, dtype=torch.float16)
    a = torch.as_strided(buf, (1000, 4100), (4164, 1), 128)
    bbuf = torch.empty(4100 * 3064 + 256, dtype=torch.float16)
    b = torch.as_strided(bbuf, (4100, 3000), (3064, 1), 128)
    # TMA cannot describe it: by default it is copied into an aligned image first
    pl = plan(a, b, "nn", {"tile_n": 128}, out_dtype=torch.float32)
    assert (pl["a_loader"], pl["a_repacked"]) == (0, 1)
    assert pl["repack_bytes"] >= 1000 * 4104 * 2
    if b.data_ptr() % 16 == 0:
        assert (pl["b_loader"], pl["b_repacked"]) == (0, 0)
    # its rows start on 8-byte boundaries, so on request the loader warps of the kernel fetch it: no copy, no scratch
    pl = plan(a, b, "nn", {"tile_n": 128, "loader": True}, out_dtype=torch.float32)
    assert (pl["a_loader"], pl["a_repacked"], pl["repack_bytes"]) == (1, 0, 0)
    assert pl["stages"] == 3  # the one ring depth the loader variant of this tile is built with
    # rows that start on odd 4-byte boundaries (pitch 4102 elements) are beyond the loader: copied
    buf2 = torch.empty(1000 * 4102 + 256, dtype=torch.float16)
    a2 = torch.as_strided(buf2, (1000, 4100), (4102, 1), 128)
    pl = plan(a2, b, "nn", {"tile_n": 128, "loader": True}, out_dtype=torch.float32)
    assert (pl["a_loader"], pl["a_repacked"]) == (0, 1)
    # an M-contiguous operand TMA cannot take (pitch 1001 elements) is copied too
    a3 = torch.as_strided(torch.empty(4100 * 1001 + 256, dtype=torch.float16), (1000, 4100), (1, 1001), 128)
    pl = plan(a3, b, "tn", {"tile_n": 128, "loader": True}, out_dtype=torch.float32)
    assert (pl["a_loader"], pl["a_repacked"]) == (0, 1)


def test_tuned_table_roundtrip(tmp_path):
    import json
    rec = {"arch": "sm_100a", "dtype": "bf16", "layout": "nt", "m": 32, "n": 384, "k": 7168,
           "config": {"tile_n": 32, "swap_ab": True, "split_k": 16, "stages": 8}, "duration": 3.2, "tflops": 55.0}
    other = dict(rec, arch="gfx950")
    path = tmp_path / "t.jsonl"
    path.write_text(json.dumps(other) + "\n" + json.dumps(rec) + "\n\n")
    table = P.load_tuned(path)
    assert list(table) == [("bf16", "nt", 32, 384, 7168)]
    pol = P.from_user_kwargs(table[("bf16", "nt", 32, 384, 7168)], 32, 384, 7168, "nt")
    assert pol.swap_ab and pol.split_k == 16 and pol.stages == 8


def test_tuned_rows_serve_other_layouts_only_when_valid():
    import torch

    from flydsl_examples_b200.gemm_a16w16 import resolve_policy

    # the shipped table has config 3 tuned for 'nt' only (tile 16, swapped, 16-CTA cluster)
    nt = resolve_policy(32, 384, 7168, torch.bfloat16, "nt", {})
    assert (nt.tile_n, nt.swap_ab, nt.split_mode) == (16, True, "cluster")
    # 'nn' keeps A K-contiguous, which is all a swapped narrow tile needs: the row is reused
    nn = resolve_policy(32, 384, 7168, torch.float16, "nn", {})
    assert (nn.tile_n, nn.swap_ab, nn.split_k) == (nt.tile_n, True, nt.split_k)
    # with an M-contiguous A the narrow tile is not runnable: the heuristic answers instead, with a valid policy
    tn = resolve_policy(32, 384, 7168, torch.bfloat16, "tn", {})
    assert tn.tile_n >= 64 and P.validate(tn, 32, 384, 7168, "tn") is None
    # config 4: 'nt' and 'nn' have rows of their own
    assert resolve_policy(1000, 3000, 4100, torch.float16, "tt", {}).tile_n == 192
    assert resolve_policy(1000, 3000, 4100, torch.float16, "nn", {}).tile_n == 256
    # rows and heuristic picks with pair tiles wider than 256 columns are for 16-bit outputs; fp32 outputs get 256
    wide = resolve_policy(16384, 28672, 8192, torch.bfloat16, "nt", {})
    assert (wide.tile_n, wide.cta_group, wide.group_m) == (512, 2, 8)
    narrow = resolve_policy(16384, 28672, 8192, torch.bfloat16, "nt", {}, out_dtype=torch.float32)
    assert (narrow.tile_n, narrow.cta_group, narrow.group_m) == (256, 2, 8)
    assert 256 < resolve_policy(6000, 6000, 6000, torch.bfloat16, "nt", {}).tile_n <= 512
    assert resolve_policy(6000, 6000, 6000, torch.bfloat16, "nt", {}, out_dtype=torch.float32).tile_n == 256
    # the heuristic may pick a run-time width that fills whole waves: 1536 x 4096 as one wave of 256 x 352 tiles
    assert resolve_policy(1536, 4096, 4096, torch.bfloat16, "nt", {}).tile_n in (352, 384)
    assert resolve_policy(6000, 6000, 6000, torch.bfloat16, "nt", {"tile_n": 480, "cta_group": 2}, out_dtype=torch.float32).tile_n == 480


@pytest.mark.parametrize(("tiles", "kb", "cap"), [(256, 64, 148), (96, 65, 148), (3, 112, 148), (1792, 128, 148), (149, 2, 148),
                                                  (148, 64, 148), (1, 1000, 148), (300, 5, 148), (7, 3, 148), (14336, 128, 148)])
def test_stream_k_walk_covers_every_k_block_once(tiles, kb, cap):
    grid, sk_tiles, sk_slots = P.stream_k_plan(tiles, kb, cap)
    if sk_tiles == 0:
        assert tiles % cap == 0 or tiles * kb < 4 * 1 or (tiles % cap) * kb // cap < 4
        return
    assert 1 <= grid <= cap and sk_tiles <= tiles
    seen = {}
    contrib = {}
    for cta in range(grid):
        items = P.stream_k_walk(cta, grid, tiles, kb, sk_tiles)
        assert items, "every CTA gets work"
        for it in items:
            for blk in range(it["kb0"], it["kb0"] + it["kbn"]):
                assert (it["tile"], blk) not in seen
                seen[(it["tile"], blk)] = cta
            if it["partial"]:
                contrib.setdefault(it["tile"], []).append((it["ordinal"], it["n_contrib"], cta))
    assert len(seen) == tiles * kb
    for tile, lst in contrib.items():
        n = lst[0][1]
        assert all(x[1] == n for x in lst) and n <= sk_slots
        assert sorted(x[0] for x in lst) == list(range(n))  # ordinals are exactly 0..n-1: the ticket completes
    # spans are balanced to within one K block
    loads = [sum(it["kbn"] for it in P.stream_k_walk(c, grid, tiles, kb, sk_tiles) if it["tile"] < sk_tiles) for c in range(grid)]
    assert max(loads) - min(loads) <= 1


def test_stream_k_plan_matches_the_library():
    cases = [((2048, 4096, 4096), 256), ((1000, 3000, 4100), 256), ((16384, 3584, 8192), 256), ((32, 384, 7168), 64), ((4096, 4736, 512), 128)]
    for (m, n, k), tile_n in cases:
        a = torch.empty(m, k, dtype=torch.bfloat16)
        b = torch.empty(n, k, dtype=torch.bfloat16).t()
        pl = plan(a, b, "nt", {"tile_n": tile_n, "stream_k": True})
        tiles = pl["tiles_p"] * pl["tiles_q"]
        tk = P.tile_k(tile_n)
        grid, sk_tiles, sk_slots = P.stream_k_plan(tiles, (k + tk - 1) // tk, 148)
        assert (pl["grid"], pl["sk_tiles"], pl["sk_slots"]) == (grid, sk_tiles, sk_slots), (m, n, k)
        assert pl["stream_k"] == (1 if sk_tiles else 0)
        if sk_tiles:
            assert pl["partial_bytes"] == sk_tiles * sk_slots * 128 * tile_n * 4 and pl["counter_bytes"] == 1 << 20


def test_call_key_tells_output_strides_apart():
    # A prepared launch is reused only for an identical call. Two outputs with the same address, shape and dtype but
    # different strides are different calls: the second one must reach the `out.is_contiguous()` assertion
    # (kernels/gemm_a16w16_gfx950.py:1381) instead of hitting the cache.
    from flydsl_examples_b200 import gemm_a16w16 as G

    a = torch.empty(8, 16, dtype=torch.bfloat16)
    b = torch.empty(4, 16, dtype=torch.bfloat16).t()
    big = torch.empty(8, 8, dtype=torch.bfloat16)
    contiguous = big.view(-1)[:32].view(8, 4)
    strided = big[:, :4]
    assert contiguous.data_ptr() == strided.data_ptr() and contiguous.shape == strided.shape
    key1 = G._call_key(a, b, contiguous, None, (), 0, "nt", None)
    key2 = G._call_key(a, b, strided, None, (), 0, "nt", None)
    assert key1 != key2
    with pytest.raises(AssertionError):
        G.gemm_a16w16(a, b, strided, layout="nt")


def test_wait_limit_is_a_control_key():
    # it rides along with a tuned or heuristic tiling instead of replacing it
    pol = P.from_user_kwargs({"wait_limit_us": 50}, 2048, 4096, 4096, "nt")
    base = P.from_user_kwargs({}, 2048, 4096, 4096, "nt")
    assert pol.wait_limit_us == 50 and base.wait_limit_us == 0
    assert (pol.tile_n, pol.cta_group, pol.split_k) == (base.tile_n, base.cta_group, base.split_k)
    assert P.validate(P.Policy(tile_n=64, wait_limit_us=-1), 64, 64, 64, "nt") is not None
