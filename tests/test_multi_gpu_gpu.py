"""Multi-GPU modes on real GPUs: two ranks (one process per GPU, NCCL), compared with the CPU oracle. Skipped on a
box with fewer than two GPUs. The fused K-shard ranks store into each other's memory over NVLink; nothing here waits
on another GPU inside a kernel, and NVLS is switched off for the NCCL barrier."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from flydsl_examples_b200 import multi_gpu as MG
        from flydsl_examples_b200.gemm_a16w16 import check_status

        oks = {}
        slots = None
        for call, (m, n, k, kw) in enumerate([(512, 1024, 2048, {}), (512, 1024, 2048, {"tile_n": 128}),
                                              (512, 1024, 2048, {"tile_n": 256, "cta_group": 2})]):
            case = O.Case("mgf", "bf16", "nt", m, n, k, seed=40 + call, bias_std=0.5)
            a, b, bias = O.draw_logical(case)
            full = O.reference_matmul(a, b, bias, torch.bfloat16)
            ad, bd, biasd = a.to(dev), b.t().contiguous().to(dev).t(), bias.to(dev)
            a_r, b_r, _, _ = MG.shard_along_k(ad, bd, world, rank)
            if slots is None:
                slots = MG.PeerSlots(m // world, n, dev)
                slots.local.fill_(float("nan"))
                torch.cuda.synchronize(dev)
                dist.barrier()
            res = MG.gemm_k_sharded_fused(a_r, b_r, torch.bfloat16, slots, bias=biasd, layout="nt", user_kwargs=kw)
            check_status(dev)
            (r0, r1), = res.row_ranges
            oks[f"fused{call}"] = bool(O.compare(res.out, full[r0:r1], case.k)["ok"])
            nccl = MG.gemm_k_sharded(a_r, b_r, torch.bfloat16, bias=biasd, layout="nt", chunks=2)
            check_status(dev)
            per = nccl.out.shape[0] // len(nccl.row_ranges)
            oks[f"nccl{call}"] = all(bool(O.compare(nccl.out[i * per:(i + 1) * per], full[q0:q1], case.k)["ok"])
                                     for i, (q0, q1) in enumerate(nccl.row_ranges))
        dist.barrier()
        slots.close()
        ret[rank] = oks
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_k_shard_fused_and_nccl():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    for r in range(world):
        assert all(ret[r].values()), (r, dict(ret[r]))
