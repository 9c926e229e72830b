#!/usr/bin/env python
"""Benchmark of the A16W16 GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4_nt|...|c5|c5_nshard|c5_kshard|c5_kshard_fused]
                    [--impl ours|reference]

Prints ONE JSON line. A step is one pass of the hot path (one GEMM call) over one batch of synthetic input.
  N = 1  default workload c5: bf16 'nt' 16384x28672x8192, the whole GEMM on one GPU (the largest configuration of the
         benchmark list that fits one GPU, and the very GEMM the N > 1 runs shard). The same line carries a `configs`
         dict with device-timed records of the small configurations (c1, c2, c3, c4 in its four layouts), each with its
         own roofline entry, and a `sustained` record (the same step looped for more than a second).
  N > 1  default workload c5_nshard: the same GEMM with B sharded along N over the ranks, no collective; `value` is
         total FLOPs of the whole GEMM / max-over-ranks time (fixed total work: strong scaling). The line also carries
         `kshard` and `kshard_fused` records: the K-sharded modes (NCCL reduce-scatter of fp32 partials; partial sums
         stored into the owner's memory over NVLink by the GEMM epilogue), each with a sampled-row parity check
         against the CPU oracle.
`value`   device-timed (CUDA events on the launching stream) with inputs resident in HBM; inputs rotate over a set
          of buffers larger than L2 for the small configs, and are larger than L2 by themselves for c5.
`e2e`     same metric through the public Python call with HOST (pinned) inputs: host->device copies of A, B, bias
          and the device->host read of C are inside the timed region.
`--impl reference`: the reference has no CPU implementation of its kernel; its tests check against torch.mm on
the same tensors (test_gemm_a16w16_gfx950.py:82-94). That CPU computation (oracle.reference_matmul: fp32
torch.matmul + bias) is what the reference arm times, on all host threads this process may use, on a bounded sample.
"""
from __future__ import annotations

import argparse
import gc
import json
import math
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

L2_BYTES_NOMINAL = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the GEMM kernel, from ncu captures of these workloads
# (None where no capture exists). The c4 figures are the GEMM launch alone; its repack launch moves 33.9 MB more.
NCU_TRAFFIC_BYTES = {"c2": 53.2e6, "c3": 6.04e6, "c4_nt": 32.9e6, "c4_tn": 33.9e6, "c5": 7.55e9}
SMALL_CONFIGS = ("c1", "c2", "c3", "c4_nn", "c4_nt", "c4_tn", "c4_tt")
SHARDED = ("c5_nshard", "c5_kshard", "c5_kshard_fused")
PLAN_KEYS = ("tile_m", "tile_n", "tile_k", "stages", "split_k", "cluster_split", "swap_ab", "group_m", "grid", "num_units",
             "stream_k", "sk_tiles", "a_repacked", "b_repacked")


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def host_threads() -> int:
    """Threads this process may run on (its CPU affinity), not what OMP_NUM_THREADS says: torch.distributed.run sets
    that variable to 1 for every rank."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self.index, self.period = index, period_s
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


def cpu_reference_run(case, seconds_budget: float = 12.0, max_reps: int = 20) -> dict:
    """Time the CPU computation the reference's tests use as ground truth (fp32 torch.matmul + bias) on a bounded
    sample of `case`: all of it when one pass is short, else a slab of rows scaled to fit the budget. Uses every host
    thread this process may run on."""
    from oracle import oracle as O

    torch.set_num_threads(host_threads())
    m = case.m
    flops_full = case.flops
    # probe speed on a small slab to size the sample
    g = torch.Generator().manual_seed(case.seed)
    rows_probe = min(m, 128)
    a = (torch.randn(rows_probe, case.k, generator=g) * case.a_std).to(case.torch_dtype)
    b = (torch.randn(case.k, case.n, generator=g) * case.b_std).to(case.torch_dtype)
    bias = None if case.bias_std is None else (torch.randn(case.n, generator=g) * case.bias_std).to(case.torch_dtype)
    O.reference_matmul(a, b, bias, case.torch_out_dtype)
    t0 = time.perf_counter()
    O.reference_matmul(a, b, bias, case.torch_out_dtype)
    t_probe = max(time.perf_counter() - t0, 1e-6)
    rate = 2.0 * rows_probe * case.n * case.k / t_probe
    rows = int(min(m, max(rows_probe, (rate * seconds_budget / 4) / (2.0 * case.n * case.k))))
    rows = max(1, rows)
    if rows != rows_probe:
        a = (torch.randn(rows, case.k, generator=g) * case.a_std).to(case.torch_dtype)
    times = []
    t_start = time.perf_counter()
    for _ in range(max_reps):
        t0 = time.perf_counter()
        O.reference_matmul(a, b, bias, case.torch_out_dtype)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_start > seconds_budget and len(times) >= 3:
            break
    best = min(times)
    flops = 2.0 * rows * case.n * case.k
    return {
        "tflops": flops / best / 1e12,
        "seconds_per_pass": best,
        "rows": rows,
        "reps": len(times),
        "cores": torch.get_num_threads(),
        "cpu_count": os.cpu_count(),
        "sample": f"fp32 torch.matmul(+bias) of {rows} of {m} rows x N={case.n} x K={case.k}, best of {len(times)} passes",
        "full_pass_seconds_est": best * m / rows,
        "flops_full": flops_full,
    }


def flat_storage_view(t: torch.Tensor) -> torch.Tensor:
    """1-D view of everything `t`'s storage holds (padding included)."""
    n = t.untyped_storage().nbytes() // t.element_size()
    return torch.as_strided(t, (n,), (1,), 0)


def clone_with_layout(t: torch.Tensor) -> torch.Tensor:
    """A copy of `t` in fresh storage with the same shape, strides and storage offset."""
    flat = flat_storage_view(t).clone()
    return torch.as_strided(flat, t.shape, t.stride(), t.storage_offset())


def workload_label(workload: str, case) -> str:
    return (f"{workload}: {case.dtype} '{case.layout}' M={case.m} N={case.n} K={case.k}"
            f"{' +bias' if case.bias_std is not None else ''} -> {case.out_dtype or case.dtype}")


class Workload:
    """One benchmark workload on one rank: resident-input step, host-input step, and the numbers that describe it."""

    def __init__(self, name, args, world, rank, device):
        from flydsl_examples_b200 import multi_gpu as MG
        from flydsl_examples_b200.gemm_a16w16 import gemm_a16w16, plan
        from oracle import oracle as O

        self.name, self.world, self.rank, self.device = name, world, rank, device
        self.extra = {}
        big = name in ("c5",) + SHARDED
        self.case = case = O.CONFIGS["c5" if big else name]
        if args.policy:
            import dataclasses
            self.case = case = dataclasses.replace(case, user_kwargs=json.loads(args.policy))
        out_es = 4 if case.torch_out_dtype is torch.float32 else 2
        if big:
            # Synthetic N(0, 0.02) operands drawn on the device; C5's operands and output exceed L2 by themselves.
            # A is the same on every rank (same seed); a rank's slab of B comes from a seed of its own.
            torch.manual_seed(case.seed)
            a_full = (torch.randn(case.m, case.k, device=device, dtype=torch.float32) * case.a_std).to(torch.bfloat16)
            self.a_full = a_full
            self.rotation = "inputs larger than L2"
            self.total_flops = float(case.flops)
            torch.manual_seed(case.seed + 1000 * (rank + 1))
            if name in ("c5_kshard", "c5_kshard_fused") and world > 1:
                k0, k1 = MG.shard_bounds(case.k, world, rank, 64)
                b_store = (torch.randn(case.n, k1 - k0, device=device, dtype=torch.float32) * case.b_std).to(torch.bfloat16)
                self.b_store, self.k_range = b_store, (k0, k1)
                a_loc, b_loc, chunks = a_full[:, k0:k1], b_store.t(), args.chunks
                self.result = None
                self.per_rank_flops = 2.0 * case.m * case.n * (k1 - k0)
                self.extra["reduce_bytes_per_rank"] = 4 * case.m * case.n * (world - 1) // world
                if name == "c5_kshard":
                    def step():
                        self.result = MG.gemm_k_sharded(a_loc, b_loc, torch.bfloat16, layout="nt", chunks=chunks)

                    self.plan = plan(a_loc[: case.m // chunks], b_loc, "nt", {}, out_dtype=torch.float32)
                    self.launches_per_step = 2 * chunks
                    self.gemm_launches_per_step = chunks
                    self.partition = f"K sharded over {world} GPUs, NCCL fp32 reduce-scatter in {chunks} M-chunks"
                else:
                    per = case.m // world
                    self.slots = MG.PeerSlots(per, case.n, device)
                    out_loc = torch.empty((per, case.n), dtype=torch.bfloat16, device=device)

                    def step():
                        self.result = MG.gemm_k_sharded_fused(a_loc, b_loc, torch.bfloat16, self.slots, layout="nt",
                                                              user_kwargs=case.user_kwargs, out=out_loc)

                    self.plan = plan(a_loc[:per], b_loc, "nt", case.user_kwargs, out_dtype=torch.float32)
                    self.launches_per_step = world + 1
                    self.gemm_launches_per_step = world
                    self.partition = (f"K sharded over {world} GPUs, GEMM epilogues store fp32 tiles into the owner's slots "
                                      "over NVLink (peer memory), owner-side slot reduction")
                ins = [a_loc, b_loc]
                out_getter = lambda: self.result.out
            else:
                n0, n1 = MG.shard_bounds(case.n, world, rank)
                b_store = (torch.randn(n1 - n0, case.k, device=device, dtype=torch.float32) * case.b_std).to(torch.bfloat16)
                b_loc = b_store.t()
                out = torch.empty((case.m, n1 - n0), dtype=torch.bfloat16, device=device)

                def step():
                    gemm_a16w16(a_full, b_loc, out, user_kwargs=case.user_kwargs, layout="nt")

                self.per_rank_flops = 2.0 * case.m * (n1 - n0) * case.k
                self.plan = plan(a_full, b_loc, "nt", case.user_kwargs)
                self.launches_per_step = self.gemm_launches_per_step = 1
                self.partition = (f"B sharded along N over {world} GPUs, no collective" if world > 1 else "whole GEMM on one GPU")
                ins = [a_full, b_loc]
                out_getter = lambda: out
            self.step = step
            self.algorithmic_bytes = None
            e2e_kwargs, e2e_layout, bias = case.user_kwargs, "nt", None
        else:
            a, b, bias, *_ = O.build_inputs(case, device=device)
            per = a.untyped_storage().nbytes() + b.untyped_storage().nbytes() + case.m * case.n * out_es
            n_slots = max(1, min(64, -(-(2 * L2_BYTES_NOMINAL + (1 << 20)) // per)))
            slots = [(a, b)] + [(clone_with_layout(a), clone_with_layout(b)) for _ in range(n_slots - 1)]
            outs = [torch.empty((case.m, case.n), dtype=case.torch_out_dtype, device=device) for _ in range(n_slots)]
            cursor = [0]

            def step(stream=None):
                i = cursor[0] % n_slots
                cursor[0] += 1
                gemm_a16w16(slots[i][0], slots[i][1], outs[i], bias=bias, user_kwargs=case.user_kwargs, layout=case.layout,
                            stream=stream)

            self.step = step
            self.rotation = f"{n_slots} rotating input/output sets of {per} bytes each (together > 2x L2)"
            self.total_flops = float(case.flops) * world
            self.per_rank_flops = float(case.flops)
            self.plan = plan(a, b, case.layout, case.user_kwargs, out_dtype=case.torch_out_dtype, bias=bias)
            self.gemm_launches_per_step = 1
            self.launches_per_step = 1 + (1 if self.plan["a_repacked"] or self.plan["b_repacked"] else 0)  # one repack launch covers both operands
            self.partition = "one GEMM per GPU" + (" (independent replicas)" if world > 1 else "")
            self.algorithmic_bytes = case.algorithmic_bytes
            ins = [a, b]
            out_getter = lambda: outs[0]
            e2e_kwargs, e2e_layout = case.user_kwargs, case.layout

        # ---- host-input variant: pinned host images of every input, copied in each step; result read back each step
        self._ins, self._bias, self._out_getter = ins, bias, out_getter
        self._e2e_kwargs, self._e2e_layout = e2e_kwargs, e2e_layout
        self._e2e_ready = False

    def prepare_e2e(self):
        from flydsl_examples_b200 import multi_gpu as MG
        from flydsl_examples_b200.gemm_a16w16 import gemm_a16w16

        dev = self.device
        self.host_in, self.dev_in_flat, self.dev_in = [], [], []
        for t in self._ins:
            flat = flat_storage_view(t) if t.untyped_storage().nbytes() <= 1.5 * t.numel() * t.element_size() + 4096 else None
            if flat is None:  # a narrow view into a much larger buffer (K-shard of A): ship only the view
                h = t.contiguous().cpu().pin_memory() if t.stride(-1) == 1 else t.t().contiguous().cpu().pin_memory().t()
                d = torch.empty_like(h, device=dev)
                self.host_in.append(h), self.dev_in_flat.append(d), self.dev_in.append(d)
            else:
                h = flat.cpu().pin_memory()
                d = torch.empty_like(flat)
                self.host_in.append(h), self.dev_in_flat.append(d)
                self.dev_in.append(torch.as_strided(d, t.shape, t.stride(), t.storage_offset()))
        self.bias_h = None if self._bias is None else self._bias.cpu().pin_memory()
        self.bias_d = None if self._bias is None else torch.empty_like(self._bias)
        out0 = self._out_getter()
        if out0 is None:
            self.step()
            out0 = self._out_getter()
        self.out_d = torch.empty_like(out0)
        self.out_h = torch.empty(out0.shape, dtype=out0.dtype).pin_memory()
        self.h2d = sum(h.numel() * h.element_size() for h in self.host_in) + (0 if self.bias_h is None else self.bias_h.numel() * 2)
        self.d2h = self.out_h.numel() * self.out_h.element_size()
        kshard = self.name in ("c5_kshard", "c5_kshard_fused") and self.world > 1

        # Three streams, two device copies of every buffer: the host->device copy of step i+1 and the device->host
        # read of step i-1 overlap the GEMM of step i (PCIe is full duplex). Every step still moves its own inputs in
        # and its own result out inside the timed region.
        main = torch.cuda.current_stream(dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        nbuf = 1 if kshard or self.h2d + self.d2h > (4 << 30) else 2
        in_flat = [self.dev_in_flat] + [[torch.empty_like(d) for d in self.dev_in_flat] for _ in range(nbuf - 1)]
        in_view = [self.dev_in] + [
            [torch.as_strided(f, v.shape, v.stride(), v.storage_offset()) if f.shape != v.shape or f.stride() != v.stride() else f
             for f, v in zip(in_flat[b], self.dev_in)] for b in range(1, nbuf)]
        bias_d = [self.bias_d] + [None if self.bias_d is None else torch.empty_like(self.bias_d) for _ in range(nbuf - 1)]
        out_d = [self.out_d] + [torch.empty_like(self.out_d) for _ in range(nbuf - 1)]
        ev_in = [torch.cuda.Event() for _ in range(nbuf)]      # inputs of this buffer have landed
        ev_used = [torch.cuda.Event() for _ in range(nbuf)]    # the GEMM that read this buffer is done
        ev_done = [torch.cuda.Event() for _ in range(nbuf)]    # the GEMM that wrote out_d[b] is done
        ev_out = [torch.cuda.Event() for _ in range(nbuf)]     # out_d[b] has been read back
        state = {"i": 0}

        def e2e_step():
            i = state["i"]
            b = i % nbuf
            state["i"] = i + 1
            with torch.cuda.stream(s_in):
                if i >= nbuf:
                    s_in.wait_event(ev_used[b])
                else:
                    s_in.wait_stream(main)
                for h, d in zip(self.host_in, in_flat[b]):
                    d.copy_(h, non_blocking=True)
                if bias_d[b] is not None:
                    bias_d[b].copy_(self.bias_h, non_blocking=True)
                ev_in[b].record(s_in)
            main.wait_event(ev_in[b])
            if i >= nbuf:
                main.wait_event(ev_out[b])
            if kshard and self.name == "c5_kshard_fused":
                res = MG.gemm_k_sharded_fused(in_view[b][0], in_view[b][1], torch.bfloat16, self.slots, layout="nt",
                                              user_kwargs=self._e2e_kwargs)
                result = res.out
            elif kshard:
                res = MG.gemm_k_sharded(in_view[b][0], in_view[b][1], torch.bfloat16, layout="nt", chunks=self.plan_chunks)
                result = res.out
            else:
                gemm_a16w16(in_view[b][0], in_view[b][1], out_d[b], bias=bias_d[b], user_kwargs=self._e2e_kwargs,
                            layout=self._e2e_layout)
                result = out_d[b]
            ev_used[b].record(main)
            ev_done[b].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[b])
                self.out_h.copy_(result, non_blocking=True)
                ev_out[b].record(s_out)

        def e2e_finish():
            main.wait_stream(s_out)
            main.wait_stream(s_in)

        self.e2e_step = e2e_step
        self.e2e_finish = e2e_finish
        self.e2e_buffers = nbuf


def graphed(fn, steps, device):
    """Capture `steps` calls of fn into one CUDA graph (launch-bound loops: the kernels are shorter than the host
    call). Returns a callable that replays all of them, or None if the capture fails."""
    side = torch.cuda.Stream(device)
    try:
        with torch.cuda.stream(side):
            fn(side)
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(steps):
                    fn(side)
        torch.cuda.synchronize(device)
        g.replay()
        torch.cuda.synchronize(device)
        return g.replay
    except Exception:
        return None


def timed(stream, device, fn, steps, world, finish=None):
    import torch.distributed as dist

    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    if finish is not None:
        finish()  # joins the side streams, so the end event covers every copy of the last step
    e1.record(stream)
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


def roofline_entry(workload: str, case, flops_per_launch: float, sec_per_launch: float, peaks: dict, long_run: bool) -> dict:
    """Roofline of one GEMM launch: HBM-bound for the small-M decode shape (c3), tensor-bound otherwise. Runs longer
    than a second are held against the sustained cuBLAS figure, shorter ones against the burst figure."""
    traffic = NCU_TRAFFIC_BYTES.get("c5" if workload in SHARDED else workload)
    if workload == "c3":
        achieved = case.algorithmic_bytes / sec_per_launch / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": traffic, "peak_source": f"{peaks['source']} copy bandwidth"}
    achieved = flops_per_launch / sec_per_launch / 1e12
    sustained = peaks.get("bf16_tflops_sustained")
    peak = sustained if (long_run and sustained) else peaks["bf16_tflops"]
    return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
            "traffic": traffic if workload not in SHARDED else None,
            "peak_source": f"{peaks['source']} cuBLAS bf16 ({'sustained' if long_run and sustained else 'burst'})"}


def sustained_record(w: Workload, ms_per_step: float, stream, device, world, local, peaks, use_graph: bool,
                     seconds: float = 1.2) -> dict:
    """The same step, looped back to back for more than `seconds`, with the SM clock sampled meanwhile."""
    n = max(3, int(math.ceil(seconds * 1e3 / max(ms_per_step, 1e-4))))
    replay, per = None, 1
    if use_graph:
        per = 500
        replay = graphed(w.step, per, device)
    with ClockSampler(physical_gpu_index(local)) as clocks:
        if replay is not None:
            reps = max(1, n // per)
            ms = timed(stream, device, replay, reps, world) / per
            n = reps * per
        else:
            ms = timed(stream, device, w.step, n, world)
    tf = w.total_flops / (ms * 1e-3) / 1e12
    rec = {"steps": n, "seconds": ms * n * 1e-3, "ms_per_step": ms, "value": tf, "unit": "TFLOP/s", "clocks": clocks.summary()}
    per_gpu = w.per_rank_flops / (ms * 1e-3) / 1e12
    if peaks.get("bf16_tflops_sustained"):
        rec["per_gpu_frac_of_sustained_peak"] = per_gpu / peaks["bf16_tflops_sustained"]
    rec["per_gpu_frac_of_burst_peak"] = per_gpu / peaks["bf16_tflops"]
    return rec


def small_config_record(name: str, args, device, stream, local, peaks) -> dict:
    """Device-timed record of one small configuration on this GPU: a short burst (20 calls) and a region of at least
    a quarter of a second with the SM clock sampled, each call on the next of the rotating input sets."""
    from flydsl_examples_b200.gemm_a16w16 import check_status

    saved_policy, args.policy = args.policy, None
    try:
        w = Workload(name, args, 1, 0, device)
    finally:
        args.policy = saved_policy
    case = w.case
    w.step()
    check_status(device)
    for _ in range(20):
        w.step()
    # Device time per call from CUDA-graph replay, like the tuner (and the reference's own benchmark script): configs 1
    # and 3 are shorter than their host-side launch, and for the others back-to-back graph nodes leave no launch gaps.
    per = 500 if name in ("c1", "c3") else 40
    replay = graphed(w.step, per, device)
    use_graph = replay is not None
    if use_graph:
        burst_ms = timed(stream, device, replay, 1, 1) / per
        reps = max(1, int(math.ceil(250.0 / (burst_ms * per))))
        with ClockSampler(physical_gpu_index(local)) as clocks:
            long_ms = timed(stream, device, replay, reps, 1) / per
        calls = reps * per
    else:
        burst_ms = timed(stream, device, w.step, 20, 1)
        calls = max(200, int(math.ceil(250.0 / burst_ms)))
        with ClockSampler(physical_gpu_index(local)) as clocks:
            long_ms = timed(stream, device, w.step, calls, 1)
    check_status(device)
    best = min(burst_ms, long_ms)
    roof = roofline_entry(name, case, float(case.flops), best * 1e-3, peaks, False)
    rec = {
        "workload": workload_label(name, case),
        "us_per_call": best * 1e3,
        "us_per_call_burst": burst_ms * 1e3,
        "us_per_call_long": long_ms * 1e3,
        "long_region": {"calls": calls, "seconds": long_ms * calls * 1e-3, "clocks": clocks.summary()},
        "tflops": case.flops / (best * 1e-3) / 1e12,
        "gbs": case.algorithmic_bytes / (best * 1e-3) / 1e9,
        "roofline": roof,
        "launch": f"CUDA graph of {per} calls" if use_graph else "one host call per GEMM",
        "kernels_per_call": w.launches_per_step,
        "l2": w.rotation,
        "plan": {k: w.plan[k] for k in PLAN_KEYS},
    }
    if roof["bound"] == "tensor" and peaks.get("bf16_tflops_sustained"):
        rec["long_frac_of_sustained_peak"] = case.flops / (long_ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"]
    del w
    gc.collect()
    torch.cuda.empty_cache()
    return rec


def kshard_parity(w: Workload, device, world: int, rank: int, n_rows: int = 64) -> dict | None:
    """Sampled full rows of a K-sharded result against the CPU oracle (fp32 matmul of the up-cast operands, one
    cast), at the benchmark tolerance. Every rank contributes the same number of its own rows; rank 0 gathers them
    together with every rank's K slab of B and checks. Returns the verdict on rank 0, None elsewhere."""
    import torch.distributed as dist

    from oracle import oracle as O

    res, case = w.result, w.case
    per_rank = max(1, n_rows // world)
    g = torch.Generator().manual_seed(1234 + rank)
    local_rows = torch.randint(0, res.out.shape[0], (per_rank,), generator=g)
    block = res.out.shape[0] // len(res.row_ranges)
    global_rows = torch.tensor([res.row_ranges[int(i) // block][0] + int(i) % block for i in local_rows], dtype=torch.int64)
    got = res.out[local_rows.to(device)].contiguous()
    got_all = torch.empty((world,) + tuple(got.shape), dtype=got.dtype, device=device)
    dist.all_gather_into_tensor(got_all, got)
    rows_all = torch.empty((world, per_rank), dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(rows_all, global_rows.to(device))
    verdict = None
    if rank == 0:
        b_full = torch.empty((case.n, case.k), dtype=torch.bfloat16)  # B as stored: [N, K]
    for r in range(world):  # one slab at a time: K/world columns of the stored B from rank r
        slab = w.b_store if r == rank else torch.empty_like(w.b_store)
        dist.broadcast(slab, src=r)
        if rank == 0:
            k0 = r * w.b_store.shape[1]
            b_full[:, k0:k0 + slab.shape[1]] = slab.cpu()
        del slab
    if rank == 0:
        torch.set_num_threads(host_threads())
        rows = rows_all.reshape(-1).cpu()
        ref = O.reference_matmul(w.a_full[rows.to(device)].cpu(), b_full.t(), None, torch.bfloat16)
        cmp = O.compare(got_all.reshape(-1, case.n).cpu(), ref, case.k)
        verdict = {"ok": bool(cmp["ok"]), "rows_checked": int(rows.numel()), "mismatches": cmp["mismatches"],
                   "max_abs": cmp["max_abs"], "rtol": cmp["rtol"], "atol": cmp["atol"],
                   "oracle": "CPU fp32 matmul of the up-cast operands, cast once to bf16"}
    dist.barrier()
    return verdict


def kshard_record(mode: str, args, world, rank, local, device, stream, peaks) -> dict | None:
    """One K-sharded mode of c5 on all ranks: at least five timed steps (max over ranks) and the parity check."""
    import torch.distributed as dist

    from flydsl_examples_b200.gemm_a16w16 import check_status

    saved_policy, args.policy = args.policy, None
    try:
        w = Workload(mode, args, world, rank, device)
    finally:
        args.policy = saved_policy
    w.plan_chunks = args.chunks
    w.step()
    check_status(device)
    parity = kshard_parity(w, device, world, rank)
    for _ in range(2):
        w.step()
    steps = max(5, min(args.steps, 10))
    with ClockSampler(physical_gpu_index(local)) as clocks:
        ms = timed(stream, device, w.step, steps, world)
    check_status(device)
    rec = {
        "workload": workload_label(mode, w.case),
        "partition": w.partition,
        "steps": steps,
        "ms_per_step": ms,
        "value": w.total_flops / (ms * 1e-3) / 1e12,
        "unit": "TFLOP/s",
        "reduce_bytes_per_rank": w.extra["reduce_bytes_per_rank"],
        "nvlink_gbs_per_rank": w.extra["reduce_bytes_per_rank"] / (ms * 1e-3) / 1e9,
        "gemm_launches_per_step": w.gemm_launches_per_step,
        "clocks": clocks.summary(),
        "parity": parity,
    }
    if hasattr(w, "slots"):
        dist.barrier()
        w.slots.close()
    del w
    gc.collect()
    torch.cuda.empty_cache()
    dist.barrier()
    return rec if rank == 0 else None


def run_ours(args) -> dict:
    import torch.distributed as dist

    from flydsl_examples_b200 import _lib
    from flydsl_examples_b200.gemm_a16w16 import check_status

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    _lib.load()  # fail loudly if the CUDA library is missing
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    cpu = None
    if world > 1:
        if rank == 0 and not args.no_cpu_baseline:
            # A short sample, taken while the other ranks wait on the host in the rendezvous below (not at a GPU barrier).
            from oracle import oracle as O

            cpu = cpu_reference_run(O.CONFIGS["c5"], seconds_budget=4.0)
        dist.init_process_group("nccl", device_id=device)
    assert args.gpus == world, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}"

    default_run = args.workload is None and args.policy is None
    workload = args.workload or ("c5" if world == 1 else "c5_nshard")
    peaks = measured_peaks()
    stream = torch.cuda.current_stream(device)
    w = Workload(workload, args, world, rank, device)
    w.plan_chunks = args.chunks
    case = w.case

    # one checked call before anything is timed (a kernel that gave up a wait reports it here)
    w.step()
    check_status(device)

    # ---------------------------------------------------------------- device-timed, inputs resident in HBM
    for _ in range(args.warmup):
        w.step()
    # Launch-bound workloads (one call is shorter than its host-side launch) are timed from a CUDA graph holding all
    # K steps; the graph is replayed once as extra warm-up, then once timed.
    use_graph = args.graph == "on" or (args.graph == "auto" and workload in ("c1", "c3"))
    replay = graphed(w.step, args.steps, device) if use_graph else None
    with ClockSampler(physical_gpu_index(local)) as clocks:
        if replay is not None:
            ms_per_step = timed(stream, device, replay, 1, world) / args.steps
        else:
            ms_per_step = timed(stream, device, w.step, args.steps, world)
    check_status(device)
    value = w.total_flops / (ms_per_step * 1e-3) / 1e12
    sustained = None
    if not args.no_sustained:
        sustained = sustained_record(w, ms_per_step, stream, device, world, local, peaks, replay is not None)
        check_status(device)

    # ---------------------------------------------------------------- end to end: host buffers in, host result out
    w.prepare_e2e()
    # enough steps for the three-stream pipeline to reach its steady state (the first and last step cannot overlap)
    e2e_steps = max(3, min(args.steps, 20 if not workload.startswith("c5") else 10))
    for _ in range(3 if not workload.startswith("c5") else 1):
        w.e2e_step()
    w.e2e_finish()
    ms_e2e = timed(stream, device, w.e2e_step, e2e_steps, world, finish=w.e2e_finish)
    check_status(device)
    e2e = {"value": w.total_flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": w.h2d,
           "d2h_bytes_per_step": w.d2h, "ms_per_step": ms_e2e, "steps": e2e_steps,
           "pipeline": f"{w.e2e_buffers} buffer set(s); copies on their own streams overlap the GEMM of the neighbouring steps"}

    # ---------------------------------------------------------------- roofline of the dominant kernel (the GEMM)
    sec_per_launch = ms_per_step * 1e-3 / w.gemm_launches_per_step
    long_run = ms_per_step * 1e-3 * args.steps > 1.0
    roofline = roofline_entry(workload, case, w.per_rank_flops / w.gemm_launches_per_step, sec_per_launch, peaks, long_run)

    result = {
        "metric": "gemm_tflops",
        "value": value,
        "unit": "TFLOP/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "strong" if workload in SHARDED else "weak",
        "vs_baseline": None,
        "dtype": case.dtype,
        "data": "synthetic",
        "config": {"workload": workload_label(workload, case)},
        "details": {
            "partition": w.partition,
            "l2": w.rotation,
            "launch": "CUDA graph of all timed steps" if replay is not None else "one host call per step",
            "plan": {k: w.plan[k] for k in PLAN_KEYS},
        },
        "roofline": roofline,
        "clocks": clocks.summary(),
        "gpu_launches": w.launches_per_step * args.steps,
        "e2e": e2e,
    }
    if sustained is not None:
        result["sustained"] = sustained
    result.update(w.extra)
    del w, replay
    gc.collect()
    torch.cuda.empty_cache()

    if default_run and world == 1 and not args.no_configs:
        # the small configurations of the benchmark list, one after the other on this GPU
        result["configs"] = {name: small_config_record(name, args, device, stream, local, peaks) for name in SMALL_CONFIGS}
    if default_run and world > 1 and not args.no_kshard:
        for mode, key in (("c5_kshard", "kshard"), ("c5_kshard_fused", "kshard_fused")):
            rec = kshard_record(mode, args, world, rank, local, device, stream, peaks)
            if rank == 0:
                result[key] = rec
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_reference_run(case)
    if cpu is not None:
        result["cpu_baseline"] = {"value": cpu["tflops"], "unit": "TFLOP/s", "cores": cpu["cores"], "kind": "port",
                                  "sample": cpu["sample"], "host_cpu_count": cpu["cpu_count"]}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return result if rank == 0 else None


def run_reference(args) -> dict | None:
    from oracle import oracle as O

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    world = int(os.environ.get("WORLD_SIZE", "1"))
    workload = args.workload or ("c5" if world == 1 else "c5_nshard")
    case = O.CONFIGS["c5" if workload.startswith("c5") else workload]
    # each step is a bounded sample: a slab of rows sized so the whole run stays within a few minutes
    per_step_budget = max(1.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    runs = []
    for i in range(args.warmup + args.steps):
        r = cpu_reference_run(case, seconds_budget=per_step_budget, max_reps=3)
        if i >= args.warmup:
            runs.append(r)
    best = max(runs, key=lambda r: r["tflops"])
    value = statistics.median(r["tflops"] for r in runs)
    return {
        "impl": "reference",
        "metric": "gemm_tflops",
        "value": value,
        "unit": "TFLOP/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": statistics.median(r["full_pass_seconds_est"] for r in runs) * 1e3,
        "higher_is_better": True,
        "scaling": "strong" if workload in SHARDED else "weak",
        "vs_baseline": None,
        "dtype": case.dtype,
        "data": "synthetic",
        "config": {"workload": workload_label(workload, case)},
        "details": {"note": "CPU torch.matmul fp32 (+bias): the ground truth of the reference's own tests; the reference kernel "
                            "itself needs FlyDSL + an AMD gfx950 GPU and cannot run on this machine"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": best["cores"], "kind": "port", "sample": best["sample"],
                         "host_cpu_count": best["cpu_count"]},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--chunks", type=int, default=4)
    ap.add_argument("--policy", default=None, help="JSON dict of user_kwargs overriding the workload's policy")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the records of the small configurations (N = 1)")
    ap.add_argument("--no-kshard", action="store_true", help="skip the K-sharded modes (N > 1)")
    ap.add_argument("--no-sustained", action="store_true", help="skip the loop of more than a second")
    ap.add_argument("--graph", default="auto", choices=("auto", "on", "off"))
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    workload = args.workload or ("c5" if world == 1 else "c5_nshard")
    big = workload.startswith("c5")
    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 3
        args.warmup = args.warmup if args.warmup is not None else 1
        res = run_reference(args)
    else:
        args.steps = args.steps if args.steps is not None else (20 if big else 1000)
        args.warmup = max(3, args.warmup if args.warmup is not None else (3 if big else 50))
        res = run_ours(args)
    if res is not None:
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
