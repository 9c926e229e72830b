"""Tuner host logic on CPU: candidate enumeration, pruning, JSONL schema and resume."""
import json

from flydsl_examples_b200 import policy as P
from flydsl_examples_b200 import tuner as T


def test_candidates_are_valid_and_cover_the_variant_table():
    args = T.TuneArgs("bf16", 2048, 4096, 4096, "nt")
    cfgs = T.candidate_configs(args)
    assert cfgs
    for c in cfgs:
        pol = P.Policy(tile_n=c["tile_n"], stages=c["stages"], split_k=c["split_k"], group_m=c["group_m"], swap_ab=c["swap_ab"],
                       cta_group=c["cta_group"], stream_k=c["stream_k"], split_mode=c["split_mode"])
        assert P.validate(pol, args.m, args.n, args.k, args.layout) is None
    assert any(c["cta_group"] == 2 and c["tile_n"] == 256 for c in cfgs)
    assert any(c["stream_k"] for c in cfgs)  # 256 tiles do not fill whole waves of 148
    assert all(not c["swap_ab"] for c in cfgs)


def test_small_m_candidates_include_swap_and_split():
    args = T.TuneArgs("bf16", 32, 384, 7168, "nt", enable_split_k=True)
    cfgs = T.candidate_configs(args)
    assert any(c["swap_ab"] and c["tile_n"] == 32 and c["split_k"] >= 8 for c in cfgs)
    assert any(c["split_mode"] == "cluster" and c["split_k"] == 16 for c in cfgs)
    # an N-contiguous operand on the tile_n axis cannot use tiles narrower than 64
    assert all(c["tile_n"] >= 64 for c in T.candidate_configs(T.TuneArgs("bf16", 200, 384, 1024, "nn")) if not c["swap_ab"])


def test_tile_fit():
    assert T.tile_fit(256, 256, 128, {"tile_n": 256, "cta_group": 2}) == 1.0
    assert T.tile_fit(128, 256, 64, {"tile_n": 256, "cta_group": 2}) == 0.5
    assert abs(T.tile_fit(32, 384, 7168, {"tile_n": 32, "swap_ab": True, "split_k": 16}) - 1.0) < 1e-9
    assert T.tile_fit(100, 100, 100, {"tile_n": 128}) < 0.5


def test_jsonl_schema_and_resume(tmp_path):
    path = tmp_path / "tuned.jsonl"
    args = T.TuneArgs("bf16", 32, 384, 7168, "nt")
    rec = T.append_result(path, args, {"tile_n": 32, "swap_ab": True, "split_k": 16}, 10.0)
    assert set(rec) == {"arch", "dtype", "layout", "m", "n", "k", "config", "duration", "tflops"}
    assert rec["arch"] == "sm_100a" and abs(rec["tflops"] - 2 * 32 * 384 * 7168 / 10.0 * 1e-6) < 1e-9
    assert json.loads(path.read_text().splitlines()[0]) == rec
    assert ("sm_100a", "bf16", "nt", 32, 384, 7168) in T.already_tuned(path)
    # the runtime lookup reads the same file format
    table = P.load_tuned(path)
    assert table[("bf16", "nt", 32, 384, 7168)]["split_k"] == 16
