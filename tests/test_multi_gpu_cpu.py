"""Partition arithmetic and the chunked K-shard exchange with two gloo ranks on CPU. The compute function and the
exchange are injected (the oracle's matmul, a gloo all-reduce): what is tested is the host logic — who owns which
columns / K range / rows, buffer rotation, row bookkeeping — not a CPU GEMM of the product (there is none)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flydsl_examples_b200 import multi_gpu as MG
from oracle import oracle as O


def test_shard_bounds_cover_exactly():
    for extent in (1, 255, 256, 257, 3584, 28672, 8192, 4100):
        for world in (1, 2, 3, 4, 8):
            for align in (64, 256):
                spans = [MG.shard_bounds(extent, world, r, align) for r in range(world)]
                assert spans[0][0] == 0 and spans[-1][1] == extent
                for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                    assert a1 == b0 and a0 <= a1
    assert [MG.shard_bounds(28672, 8, r) for r in range(8)] == [(r * 3584, (r + 1) * 3584) for r in range(8)]
    assert [MG.shard_bounds(8192, 4, r, 64) for r in range(4)] == [(r * 2048, (r + 1) * 2048) for r in range(4)]


def test_shard_views_do_not_copy():
    b = torch.empty(512, 128, dtype=torch.bfloat16).t()  # 'nt' B: logical [K=128, N=512]
    v, n0, n1 = MG.shard_b_along_n(b, 2, 1)
    assert (n0, n1) == (256, 512) and v.shape == (128, 256)
    assert v.data_ptr() == b.data_ptr() + 256 * 128 * 2 and v.stride() == b.stride()
    a = torch.empty(64, 256, dtype=torch.bfloat16)
    bk = torch.empty(512, 256, dtype=torch.bfloat16).t()
    a_r, b_r, k0, k1 = MG.shard_along_k(a, bk, 2, 1)
    assert (k0, k1) == (128, 256) and a_r.stride() == (256, 1) and b_r.stride() == (1, 256)
    assert a_r.data_ptr() == a.data_ptr() + 128 * 2 and b_r.data_ptr() == bk.data_ptr() + 128 * 2


def test_row_ranges():
    assert MG.k_shard_row_ranges(16, 2, 0, 2) == [(0, 4), (8, 12)]
    assert MG.k_shard_row_ranges(16, 2, 1, 2) == [(4, 8), (12, 16)]
    with pytest.raises(AssertionError):
        MG.k_shard_row_ranges(10, 4, 0, 1)


class _GlooExchange:
    """Test double for the NCCL exchange: all-reduce the partial, keep this rank's rows, round once."""

    def __init__(self, rank, world, bias):
        self.rank, self.world, self.bias, self.calls = rank, world, bias, []

    def before_gemm(self, buf):
        self.calls.append(("gemm", buf))

    def reduce(self, buf, partial, reduced, dst):
        dist.all_reduce(partial, op=dist.ReduceOp.SUM)
        per = partial.shape[0] // self.world
        red = partial[self.rank * per:(self.rank + 1) * per]
        if self.bias is not None:
            red = red + self.bias.float()
        dst.copy_(red.to(dst.dtype))
        self.calls.append(("reduce", buf))

    def finish(self):
        self.calls.append(("finish",))


def _oracle_gemm(a, b, out, bias=None, user_kwargs={}, layout="nt"):
    res = O.reference_matmul(a, b, bias, out.dtype if out is not None else a.dtype)
    if out is None:
        return res
    out.copy_(res)
    return out


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = O.Case("mg", "bf16", "nt", 64, 512, 256, seed=77, bias_std=0.5)
        a, b, bias = O.draw_logical(case)
        full = O.reference_matmul(a, b, bias, torch.bfloat16)
        # N-shard: no communication
        b_loc, n0, n1 = MG.shard_b_along_n(b, world, rank)
        c_loc = MG.gemm_n_sharded(a, b_loc, None, bias[n0:n1], "nt", gemm_fn=_oracle_gemm)
        ok_n = torch.equal(c_loc, full[:, n0:n1])
        # K-shard: chunked exchange
        a_r, b_r, k0, k1 = MG.shard_along_k(a, b, world, rank)
        ex = _GlooExchange(rank, world, bias)
        res = MG.gemm_k_sharded(a_r, b_r, torch.bfloat16, bias=bias, layout="nt", chunks=4, gemm_fn=_oracle_gemm, exchange=ex)
        ok_k = True
        for blk, (r0, r1) in enumerate(res.row_ranges):
            got = res.out[blk * (r1 - r0):(blk + 1) * (r1 - r0)]
            ok_k &= bool(O.compare(got, full[r0:r1], case.k)["ok"])
        ok_order = ex.calls == [("gemm", 0), ("reduce", 0), ("gemm", 1), ("reduce", 1), ("gemm", 0), ("reduce", 0),
                                ("gemm", 1), ("reduce", 1), ("finish",)]
        ret[rank] = (ok_n, ok_k, ok_order, res.reduce_bytes, res.row_ranges)
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_n_shard_and_k_shard():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    rows = set()
    for r in range(world):
        ok_n, ok_k, ok_order, reduce_bytes, ranges = ret[r]
        assert ok_n and ok_k and ok_order
        assert reduce_bytes == 4 * 64 * 512 // 2
        for r0, r1 in ranges:
            rows |= set(range(r0, r1))
    assert rows == set(range(64))  # every row of C is owned by exactly one rank


# ------------------------------------------------------------------------------------------- fused K-shard schedule
class _SharedSlots:
    """Test double for PeerSlots: every rank's receive slots live in one shared-memory tensor
    [rank, set, slot, rows, cols], so a 'peer store' is a plain write by another process."""

    def __init__(self, shared, rank):
        self.shared, self.rank = shared, rank
        self.world, self.sets, _, self.rows, self.cols = (shared.shape[0], shared.shape[1], shared.shape[2],
                                                          shared.shape[3], shared.shape[4])
        self.calls = 0

    def next_set(self):
        s = self.calls % self.sets
        self.calls += 1
        return s

    def target(self, dest, set_idx, src):
        return self.shared[dest, set_idx, src]

    def local_set(self, set_idx):
        return self.shared[self.rank, set_idx]


def _fused_worker(rank, world, port, shared, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        slots = _SharedSlots(shared, rank)
        log = []

        def gemm_into(a_rows, b, target):
            log.append(("gemm", int(a_rows.storage_offset() // a_rows.stride(0))))
            target.copy_(O.reference_matmul(a_rows, b, None, torch.float32))

        def reduce_fn(local_set, dst, bias):
            acc = local_set[0].clone()
            for s in range(1, local_set.shape[0]):
                acc += local_set[s]
            if bias is not None:
                acc += bias.float()
            dst.copy_(acc.to(dst.dtype))
            log.append(("reduce",))

        oks = []
        for call in range(3):  # three calls: both slot sets are used and the first one is reused
            case = O.Case("mgf", "bf16", "nt", 96, 256, 384, seed=90 + call, bias_std=0.5)
            a, b, bias = O.draw_logical(case)
            full = O.reference_matmul(a, b, bias, torch.bfloat16)
            a_r, b_r, k0, k1 = MG.shard_along_k(a, b, world, rank)
            res = MG.gemm_k_sharded_fused(a_r, b_r, torch.bfloat16, slots, bias=bias, layout="nt", gemm_into=gemm_into,
                                          barrier=dist.barrier, reduce_fn=reduce_fn)
            (r0, r1), = res.row_ranges
            oks.append(bool(O.compare(res.out, full[r0:r1], case.k)["ok"]) and res.out.shape == (r1 - r0, 256))
        ret[rank] = (all(oks), log[:world + 1], res.row_ranges, res.reduce_bytes, slots.calls)
    finally:
        dist.destroy_process_group()


def test_fused_send_order():
    assert MG.fused_send_order(4, 1) == [2, 3, 0, 1]
    assert MG.fused_send_order(1, 0) == [0]
    for world in (2, 3, 8):  # at every step the ranks address distinct destinations
        for step in range(world):
            assert len({MG.fused_send_order(world, r)[step] for r in range(world)}) == world


def test_three_rank_gloo_fused_k_shard():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    world, per, n = 3, 32, 256
    shared = torch.full((world, 2, world, per, n), float("nan")).share_memory_()
    ret = mp.Manager().dict()
    mp.spawn(_fused_worker, args=(world, port, shared, ret), nprocs=world, join=True)
    rows = set()
    for r in range(world):
        ok, log, ranges, reduce_bytes, calls = ret[r]
        assert ok and calls == 3
        # rows served in the order of the right-hand neighbours, own rows last, then the reduction
        assert log == [("gemm", d * per) for d in MG.fused_send_order(world, r)] + [("reduce",)]
        assert reduce_bytes == 4 * per * n * (world - 1)
        rows |= set(range(*ranges[0]))
    assert rows == set(range(world * per))
