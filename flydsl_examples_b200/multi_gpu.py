"""Single-box multi-GPU partitioning of one large GEMM (one process per GPU, torch.distributed for plumbing).

Two modes, neither present in the reference (xytpai/flydsl-examples is single-GPU; its op is
kernels/gemm_a16w16_gfx950.py:1288):

  N-shard  rank r owns B[:, n0:n1] and computes C[:, n0:n1]. A is replicated. No communication at all.
  K-shard  rank r owns A[:, k0:k1] and B[k0:k1, :], computes a full-size fp32 partial product with the same CUDA
           kernel (fp32-output path), and the partials are summed across GPUs with an NCCL reduce-scatter over
           NVLink, chunk by chunk along M so the reduce of chunk i overlaps the GEMM of chunk i+1. Each rank ends up
           with 1/world of the rows of every chunk, rounded once (bias added) by a small cast kernel.

`gemm_fn` is the product call everywhere; the CPU tests inject their own function to exercise the partition and
exchange logic with gloo ranks.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from . import _lib

SHARD_ALIGN = 256  # shard boundaries fall on multiples of the widest tile where the size allows


def shard_bounds(extent: int, world: int, rank: int, align: int = SHARD_ALIGN) -> tuple[int, int]:
    """[begin, end) of `rank`'s slab of `extent`: as even as possible in units of `align`; the last ranks may
    get less (or nothing) when extent is small."""
    assert 0 <= rank < world
    units = -(-extent // align)
    base, rem = divmod(units, world)
    begin_u = rank * base + min(rank, rem)
    end_u = begin_u + base + (1 if rank < rem else 0)
    return min(begin_u * align, extent), min(end_u * align, extent)


def shard_b_along_n(b: torch.Tensor, world: int, rank: int) -> tuple[torch.Tensor, int, int]:
    """View of B[K, N] (any layout) restricted to this rank's columns. For an 'nt' B (stored [N, K]) that is a
    contiguous slab of rows of the stored matrix: a plain pointer offset, no copy."""
    n0, n1 = shard_bounds(b.shape[1], world, rank)
    return b[:, n0:n1], n0, n1


def shard_along_k(a: torch.Tensor, b: torch.Tensor, world: int, rank: int, align: int = 64):
    """Views A[:, k0:k1], B[k0:k1, :]: strided views with the original leading strides (no copy)."""
    k0, k1 = shard_bounds(a.shape[1], world, rank, align)
    return a[:, k0:k1], b[k0:k1, :], k0, k1


def gemm_n_sharded(a, b_local, out_local=None, bias_local=None, layout="nt", user_kwargs={}, gemm_fn: Optional[Callable] = None):
    """C[:, n0:n1] = A @ B[:, n0:n1] (+ bias[n0:n1]) on this rank. No collective."""
    if gemm_fn is None:
        from .gemm_a16w16 import gemm_a16w16 as gemm_fn
    return gemm_fn(a, b_local, out_local, bias=bias_local, user_kwargs=user_kwargs, layout=layout)


def cast_bias(src_f32: torch.Tensor, dst: torch.Tensor, bias: Optional[torch.Tensor], stream: torch.cuda.Stream) -> None:
    """dst = cast(src + bias) with the library's own kernel (one rounding, like the GEMM epilogue)."""
    ids = {torch.float32: 1, torch.bfloat16: 2, torch.float16: 3}
    rows, cols = src_f32.shape
    rc = _lib.load().b200_gemm_cast_bias(
        src_f32.data_ptr(), dst.data_ptr(), None if bias is None else bias.data_ptr(), rows, cols, ids[dst.dtype],
        0 if bias is None else ids[bias.dtype], C.c_void_p(stream.cuda_stream))
    if rc != 0:
        raise RuntimeError(f"b200_gemm_cast_bias failed ({rc}): {_lib.strerror(rc)}")


@dataclass
class KShardResult:
    out: torch.Tensor           # [sum over chunks of rows_per_rank, N]: this rank's rows, chunk after chunk
    row_ranges: list            # global [begin, end) row range of each block of `out`
    reduce_bytes: int           # fp32 bytes this rank sent into the reduce-scatter


def k_shard_row_ranges(m: int, world: int, rank: int, chunks: int) -> list[tuple[int, int]]:
    """Rows of C this rank owns after the chunked reduce-scatter: chunk c covers rows [c*mc, (c+1)*mc) and is
    split evenly over ranks, so mc must be divisible by world."""
    assert m % chunks == 0, "M must divide into equal chunks"
    mc = m // chunks
    assert mc % world == 0, "chunk rows must divide by the number of ranks"
    per = mc // world
    return [(c * mc + rank * per, c * mc + (rank + 1) * per) for c in range(chunks)]


class NcclChunkExchange:
    """Sums one chunk's fp32 partial across ranks (NCCL reduce-scatter over NVLink) and rounds this rank's rows,
    on a side stream so that it overlaps the next chunk's GEMM. CUDA only."""

    def __init__(self, device: torch.device, group, bias: Optional[torch.Tensor]):
        assert device.type == "cuda", "the K-sharded exchange runs on CUDA devices only"
        self.group = group
        self.bias = bias
        self.main = torch.cuda.current_stream(device)
        self.side = torch.cuda.Stream(device)
        self.done: dict[int, torch.cuda.Event] = {}

    def before_gemm(self, buf: int) -> None:
        ev = self.done.get(buf)
        if ev is not None:
            self.main.wait_event(ev)  # the reduce that read this partial buffer two chunks ago

    def reduce(self, buf: int, partial: torch.Tensor, reduced: torch.Tensor, dst: torch.Tensor) -> None:
        import torch.distributed as dist

        ready = torch.cuda.Event()
        ready.record(self.main)
        with torch.cuda.stream(self.side):
            self.side.wait_event(ready)
            dist.reduce_scatter_tensor(reduced, partial, op=dist.ReduceOp.SUM, group=self.group)
            cast_bias(reduced, dst, self.bias, self.side)
            ev = torch.cuda.Event()
            ev.record(self.side)
            self.done[buf] = ev

    def finish(self) -> None:
        self.main.wait_stream(self.side)


def gemm_k_sharded(a_local, b_local, out_dtype, bias=None, layout="nt", user_kwargs={}, group=None, chunks: int = 4,
                   gemm_fn: Optional[Callable] = None, exchange=None) -> KShardResult:
    """Row-sharded C = sum over ranks of A[:, k_r] @ B[k_r, :] (+ bias), rounded once to out_dtype.

    Each chunk's fp32 partial is produced on the current stream and handed to `exchange` (default: NCCL on a side
    stream); two partial buffers alternate so chunk i+1's GEMM never overwrites data the exchange still reads."""
    import torch.distributed as dist

    if gemm_fn is None:
        from .gemm_a16w16 import gemm_a16w16 as gemm_fn
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    m, n = a_local.shape[0], b_local.shape[1]
    ranges = k_shard_row_ranges(m, world, rank, chunks)
    mc = m // chunks
    per = mc // world
    dev = a_local.device
    if exchange is None:
        exchange = NcclChunkExchange(dev, group, bias)
    out = torch.empty((per * chunks, n), dtype=out_dtype, device=dev)
    nbuf = min(2, chunks)
    partial = [torch.empty((mc, n), dtype=torch.float32, device=dev) for _ in range(nbuf)]
    reduced = [torch.empty((per, n), dtype=torch.float32, device=dev) for _ in range(nbuf)]
    for c in range(chunks):
        buf = c % nbuf
        exchange.before_gemm(buf)
        gemm_fn(a_local[c * mc:(c + 1) * mc], b_local, partial[buf], bias=None, user_kwargs=user_kwargs, layout=layout)
        exchange.reduce(buf, partial[buf], reduced[buf], out[c * per:(c + 1) * per])
    exchange.finish()
    return KShardResult(out=out, row_ranges=ranges, reduce_bytes=4 * m * n * (world - 1) // world)
