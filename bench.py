#!/usr/bin/env python
"""Benchmark of the attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload H]

Headline workload "H": FlashAttention2 forward + backward, fp16, causal, B=2 N=32 S=8192 D=128
(per GPU; with N GPUs every rank runs its own shard of a batch N times as large -- (batch, head)
slices are independent, so there is no collective in the timed region and scaling is "weak").
One step = one forward + one backward over the shard.  The metric is algorithmic TFLOP/s
(forward 4*B*N*S*S*D/2, backward 2.5x that) summed over ranks, from CUDA-event time, max over ranks.

Prints ONE JSON line.  ``--impl reference`` times the CPU restatement of the reference's
standard-attention path (oracle/attention_ref.py) on a bounded sample instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fa2_fwd_bwd_causal_s8k_d128_tflops"
UNIT = "TFLOP/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="H")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode HBM measurement")
    ap.add_argument("--decode-only", action="store_true",
                    help="run only the decode measurement on a quarter-size cache (B=8; 3 x 1.07 GB), for profiling, "
                         "and print its JSON object")
    ap.add_argument("--decode-group", type=int, default=1,
                    help="with --decode-only: query heads per cache head (N_kv = 32 / group), e.g. 8 for the tensor-core path")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-aux", action="store_true", help="skip the other configurations (2, 3, 4, 5a)")
    return ap.parse_args()


def workload_config(name):
    from acctransformer_b200.workloads import CONFIGS
    c = CONFIGS[name]
    return {"workload": f"{name}: FA2 fwd+bwd {c['dtype']} causal B={c['B']} N={c['N']} S={c['S']} D={c['D']} per GPU",
            "B": c["B"], "N": c["N"], "S": c["S"], "D": c["D"], "mask": "causal (in-kernel triangle)",
            "scale": "D^-1/2", "l2": "inputs_exceed_l2 (q,k,v,dO,O = 671 MB per step vs 126 MB L2)",
            "sharding": "batch x heads, no collective"}


# ----------------------------------------------------------------------------------------------
# CPU baseline (the oracle timed on the host cores) -- also the whole of --impl reference
# ----------------------------------------------------------------------------------------------
def cpu_sample(name, seed=0):
    """One (batch, head) unit of the workload at full sequence length."""
    import numpy as np
    from acctransformer_b200.workloads import CONFIGS
    c = CONFIGS[name]
    rs = np.random.RandomState(seed)
    q, k, v, do = (rs.randn(1, 1, c["S"], c["D"]).astype(np.float16) for _ in range(4))
    return c, q, k, v, do


def cpu_step(c, q, k, v, do):
    import numpy as np
    from oracle import attention_ref as ref
    scale = 1.0 / np.sqrt(c["D"])
    t0 = time.perf_counter()
    o, lse = ref.sa_fwd(q, k, v, causal=True, scale=scale)
    dq, dk, dv = ref.sa_grad(q, k, v, do, causal=True, scale=scale)
    return time.perf_counter() - t0


def cpu_baseline(name, steps=1, warmup=0, min_seconds=0.0):
    """Times the oracle on (batch, head) units at full sequence length: ``steps`` units, and then further units
    until ``min_seconds`` of CPU work have been spent (at most 16 units in all)."""
    from acctransformer_b200.workloads import fwd_bwd_flops
    c, q, k, v, do = cpu_sample(name)
    for _ in range(warmup):
        cpu_step(c, q, k, v, do)
    times = [cpu_step(c, q, k, v, do) for _ in range(steps)]
    while sum(times) < min_seconds and len(times) < 16:
        times.append(cpu_step(c, q, k, v, do))
    sec = sum(times) / len(times)
    flops = fwd_bwd_flops(c, B=1, N=1)
    return {"value": flops / sec / 1e12, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
            "sample": f"{len(times)} of {c['B'] * c['N']} (batch, head) units at full S={c['S']}, one after the other, "
                      f"fp32 NumPy standard attention fwd+grad, {sec:.2f} s per unit ({sum(times):.1f} s of CPU work)"}, sec


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    # torchrun sets OMP_NUM_THREADS=1 for its children; the CPU arm is meant to use every host core, so the BLAS
    # thread count is set back before NumPy is first imported (nothing above imports it)
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[var] = str(os.cpu_count() or 1)
    cb, sec = cpu_baseline(args.workload, steps=max(1, args.steps), warmup=min(args.warmup, 1))
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.workload), "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)
    return 0


# ----------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) every few milliseconds in a
    thread, so that even a timed region of tens of milliseconds gets samples taken under load."""

    def __init__(self, index, period_s=0.004):
        self.rows = []
        self.stop_flag = False
        self.err = None
        self.thread = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.period = period_s
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        except Exception as e:      # no NVML: report that instead of a number
            self.err = f"NVML unavailable: {e}"

    def _run(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.rows.append((time.perf_counter(), mhz, reasons))
            except Exception as e:
                self.err = str(e)
                return
            time.sleep(self.period)

    def stop(self, t0, t1):
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.err or "no samples"]}
        self.stop_flag = True
        self.thread.join(timeout=2)
        nv = self.nv
        rows = [r for r in self.rows if t0 <= r[0] <= t1]
        names = {"hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        seen = set()
        for _, _, bits in rows:
            for name, bit in names.items():
                if bits & bit:
                    seen.add(name)
        mhz = [r[1] for r in rows]
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_min_mhz": min(mhz) if mhz else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(seen), "samples": len(mhz)}


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"tflops": d.get("bf16_tflops_sustained"), "tflops_burst": d.get("bf16_tflops"),
                "hbm_gbs": d.get("hbm_gbs"), "which": "measured"}
    return {"tflops": 1400.0, "tflops_burst": 1590.0, "hbm_gbs": 6650.0, "which": "fallback"}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from acctransformer_b200 import _lib, ops
    from acctransformer_b200.sharding import unit_slice
    from acctransformer_b200.workloads import CONFIGS, fwd_bwd_flops, fwd_flops, make_inputs

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()

    cfg = CONFIGS[args.workload]
    # Weak scaling: the job is a batch `world` times as large; its (batch, head) units are dealt out in contiguous
    # runs (sharding.unit_slice) and every rank draws its own run, seeded by the run's first unit.
    units_per_rank = cfg["B"] * cfg["N"]
    u0, u1 = unit_slice(world * units_per_rank, rank, world)
    assert u1 - u0 == units_per_rank
    inp = make_inputs(args.workload, dev, seed_offset=u0 // units_per_rank)
    q, k, v, do = inp["q"], inp["k"], inp["v"], inp["do"]
    scale = inp["scale"]

    def fwd():
        return ops.fa_forward(q, k, v, causal=True, scale=scale)

    def bwd(o, lse):
        return ops.fa_backward(q, k, v, o, lse, do, causal=True, scale=scale)

    def step():
        o, lse = fwd()
        return bwd(o, lse)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, iters, join=None):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(iters):
            fn()
        if join is not None:
            torch.cuda.current_stream().wait_stream(join)   # the end event also covers work on that stream
        e1.record()
        barrier()
        return e0.elapsed_time(e1) / iters

    for _ in range(max(3, args.warmup)):
        step()
    # clocks are sampled over the timed steps and the two per-kernel legs that follow them (same kernels, same
    # inputs), so that a run of a few tens of milliseconds still yields several samples under load
    sampler = ClockSampler(local_rank) if rank == 0 else None
    t0 = time.perf_counter()
    ms_step = timed(step, args.steps)
    _lib.device_status()

    # per-kernel legs for the roofline (same inputs, same stream)
    ms_fwd = timed(fwd, args.steps)
    o, lse = fwd()
    ms_bwd = timed(lambda: bwd(o, lse), args.steps)
    # the backward KERNEL alone: an event pair recorded by the library directly around its launch in every call
    # (the call also runs a row-sum kernel, a zero-fill and the dQ conversion)
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    for pr in pairs:
        ops.fa_backward(q, k, v, o, lse, do, causal=True, scale=scale, kernel_events=pr)
    barrier()
    ms_bwd_kernel = sum(a.elapsed_time(b) for a, b in pairs) / len(pairs)
    t1 = time.perf_counter()
    clocks = sampler.stop(t0, t1) if sampler else None

    if world > 1:
        t = torch.tensor([ms_step, ms_fwd, ms_bwd, ms_bwd_kernel], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step, ms_fwd, ms_bwd, ms_bwd_kernel = (float(x) for x in t.tolist())

    flops_step = fwd_bwd_flops(cfg)
    value = world * flops_step / (ms_step * 1e-3) / 1e12

    # end to end through the public call with host buffers: H2D of q,k,v,dO and D2H of O,dQ,dK,dV every step
    e2e = None
    if not args.no_e2e:
        host_in = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (q, k, v, do)]
        for h, t in zip(host_in, (q, k, v, do)):
            h.copy_(t)
        host_out = [torch.empty(q.shape, dtype=q.dtype).pin_memory() for _ in range(4)]
        # Three streams: host->device copies into one of two device input sets, the two kernels (current
        # stream), device->host copies of the results.  PCIe is full duplex, so step n's read-back, step n+1's
        # upload and the kernels between them overlap; every step still uploads its inputs from pinned host
        # memory and reads its results back, and the timed region ends when all three streams have drained.
        dev_in = [tuple(torch.empty_like(q) for _ in range(4)) for _ in range(2)]
        # results are written into two preallocated sets (no allocation inside the timed steps): set n & 1 is read
        # back by the copy stream while the kernels of the next step fill the other
        dev_out = [dict(o=torch.empty_like(q), lse=torch.empty(q.shape[:3], dtype=torch.float32, device=dev),
                        g=tuple(torch.empty_like(q) for _ in range(3)),
                        ws=torch.empty(ops.fa_backward_workspace_bytes(q, k), dtype=torch.uint8, device=dev))
                   for _ in range(2)]
        out_free = [None, None]         # event after the read-back that last read each output set
        h2d_stream = torch.cuda.Stream(device=dev)
        d2h_stream = torch.cuda.Stream(device=dev)
        in_free = [None, None]          # event after the kernels that last read each input set
        keep_alive = []
        counter = [0]

        def e2e_step():
            i = counter[0] & 1
            counter[0] += 1
            main = torch.cuda.current_stream()
            with torch.cuda.stream(h2d_stream):
                if in_free[i] is not None:
                    h2d_stream.wait_event(in_free[i])
                for d, h in zip(dev_in[i], host_in):
                    d.copy_(h, non_blocking=True)
                up = torch.cuda.Event()
                up.record()
            main.wait_event(up)
            if out_free[i] is not None:
                main.wait_event(out_free[i])
            dq_, dk_, dv_, do_ = dev_in[i]
            res = dev_out[i]
            o2, lse2 = ops.fa_forward(dq_, dk_, dv_, causal=True, scale=scale, out=res["o"], lse_out=res["lse"])
            g = ops.fa_backward(dq_, dk_, dv_, o2, lse2, do_, causal=True, scale=scale, out=res["g"], workspace=res["ws"])
            done = torch.cuda.Event()
            done.record()
            in_free[i] = done
            outs = (o2,) + tuple(g)
            with torch.cuda.stream(d2h_stream):
                d2h_stream.wait_event(done)
                for h, d in zip(host_out, outs):
                    h.copy_(d, non_blocking=True)
                back = torch.cuda.Event()
                back.record()
            out_free[i] = back
            keep_alive.append(outs)
            if len(keep_alive) > 2:
                keep_alive.pop(0)

        # enough steps for the three-stage pipeline (upload, kernels, read-back) to reach its steady state: its
        # fill and drain (one upload + one read-back, ~2 steps' worth of copying) are inside the timed region
        e2e_iters = max(4, min(args.steps, 40))
        e2e_step()
        ms_e2e = timed(e2e_step, e2e_iters, join=d2h_stream)
        if world > 1:
            t = torch.tensor([ms_e2e], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_e2e = float(t.item())
        nbytes = sum(t.numel() * t.element_size() for t in host_in)

        # What the box's host path allows: the same pinned uploads and read-backs per step on the same two copy
        # streams, all ranks at once, with no kernel in between.
        outs0 = keep_alive[-1]

        def copy_only_step():
            i = counter[0] & 1
            counter[0] += 1
            with torch.cuda.stream(h2d_stream):
                for d, h in zip(dev_in[i], host_in):
                    d.copy_(h, non_blocking=True)
            with torch.cuda.stream(d2h_stream):
                for h, d in zip(host_out, outs0):
                    h.copy_(d, non_blocking=True)

        def join_both():
            torch.cuda.current_stream().wait_stream(h2d_stream)
            return d2h_stream

        copy_only_step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        h2d_stream.wait_event(e0)
        d2h_stream.wait_event(e0)
        for _ in range(e2e_iters):
            copy_only_step()
        torch.cuda.current_stream().wait_stream(h2d_stream)
        torch.cuda.current_stream().wait_stream(d2h_stream)
        e1.record()
        barrier()
        ms_copy = e0.elapsed_time(e1) / e2e_iters
        if world > 1:
            t = torch.tensor([ms_copy], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_copy = float(t.item())
        e2e = {"value": world * flops_step / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": nbytes,
               "d2h_bytes_per_step": nbytes, "ms_per_step": ms_e2e, "steps": e2e_iters,
               # the copies alone, same bytes, same streams, every rank at once: the floor the host path sets
               "copy_ceiling_ms": ms_copy, "frac_of_copy_ceiling": ms_copy / ms_e2e,
               "copy_gbs_per_direction_per_gpu": nbytes / (ms_copy * 1e-3) / 1e9}
        torch.cuda.synchronize()
        del host_in, host_out, dev_in, dev_out, keep_alive

    peaks = measured_peaks()
    bwd_tflops = 2.5 * fwd_flops(cfg) / (ms_bwd_kernel * 1e-3) / 1e12
    fwd_tflops = fwd_flops(cfg) / (ms_fwd * 1e-3) / 1e12
    mhz = (clocks or {}).get("sm_mhz")
    # The kernel is timed alone by an event pair, so the burst figure is the denominator; the sustained one (a
    # seconds-long GEMM loop under the power cap) is given beside it.  kcycles = ms x median SM MHz sampled during
    # the timed legs: runs that the power cap held at different clocks compare on that.
    roofline = {"kernel": "fa_bwd_kernel (CUDA events recorded by the library directly around its launch)",
                "bound": "tensor", "achieved": bwd_tflops, "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
                "frac": bwd_tflops / peaks["tflops_burst"], "peak_source": f"{peaks['which']} bf16_tflops (burst)",
                "frac_of_sustained": bwd_tflops / peaks["tflops"], "peak_sustained": peaks["tflops"],
                "kcycles": ms_bwd_kernel * mhz if mhz else None,
                "ms_whole_backward_call": ms_bwd,   # + row-sum kernel, zero-fill, dQ conversion
                # DRAM read + write bytes of one backward-kernel launch: ncu capture on workload P (203.8 + 89.3 MB,
                # profiles/fa_bwd_kernel_P_ncu_full.md) scaled by the units x sequence ratio of the workload
                "traffic": 293.1e6 * (cfg["B"] * cfg["N"] * cfg["S"]) / (2 * 16 * 4096), "ms": ms_bwd_kernel,
                "fwd": {"kernel": "fa_fwd_kernel", "achieved": fwd_tflops, "frac": fwd_tflops / peaks["tflops_burst"],
                        "frac_of_sustained": fwd_tflops / peaks["tflops"], "ms": ms_fwd,
                        "kcycles": ms_fwd * mhz if mhz else None},
                "step_frac_of_sustained": (flops_step / (ms_step * 1e-3) / 1e12) / peaks["tflops"],
                "step_frac_of_burst": (flops_step / (ms_step * 1e-3) / 1e12) / peaks["tflops_burst"],
                "step_frac_of_datasheet_2250": (flops_step / (ms_step * 1e-3) / 1e12) / 2250.0}

    del q, k, v, do, o, lse, inp
    torch.cuda.empty_cache()

    decode = None
    if not args.no_decode:
        # configuration 5b is ONE job of 1 024 (sequence, head) units: with several GPUs the heads are dealt out
        # (every GPU keeps all 32 sequences, so the ragged lengths load them equally) and no data crosses
        decode = bench_decode(torch, ops, dev, peaks, rank=rank, world=world, dist=dist if world > 1 else None)
        if world == 1 and not args.no_aux:
            # the same step with 4 and 8 query heads per cache head (cache bytes per second; informational)
            decode["grouped_gbs"] = {f"g{g_}": bench_decode(torch, ops, dev, peaks, group=g_)["achieved_gbs"] for g_ in (4, 8)}
    other = None
    if not args.no_aux and rank == 0 and world == 1 and args.workload == "H":
        other = bench_other_configs(torch, ops, dev, peaks)

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp16", "data": "synthetic", "config": workload_config(args.workload),
            "roofline": roofline, "e2e": e2e, "gpu_launches": 4 * args.steps, "clocks": clocks, "decode": decode,
            "other_configs": other}
    if rank == 0:
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"], _ = cpu_baseline(args.workload, min_seconds=12.0)
        print(json.dumps(_rounded(line)), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def _rounded(x):
    """Floats to five significant digits: keeps the one JSON line short enough to be read whole."""
    if isinstance(x, float):
        return float(f"{x:.5g}")
    if isinstance(x, dict):
        return {k: _rounded(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_rounded(v) for v in x]
    return x


def bench_other_configs(torch, ops, dev, peaks):
    """The remaining benchmark configurations at full size, forward and backward, as algorithmic TFLOP/s
    (informational: the headline metric is quoted on workload H)."""
    from acctransformer_b200.workloads import CONFIGS, fwd_flops, make_inputs

    def t(fn, iters):
        for _ in range(2):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    out = {}
    for name in ("cfg2", "cfg3", "cfg4", "cfg5a"):
        inp = make_inputs(name, dev)
        cfg = inp["cfg"]
        q, k, v = inp["q"], inp["k"], inp["v"]
        kw, mask, what = dict(scale=inp["scale"]), None, ""
        if name == "cfg2":
            kw.update(causal=True, alibi=inp["alibi"]); what = "fp16 causal + alibi tensor B=4 N=16 S=2048"
        elif name == "cfg3":
            kw.update(dropout_mask=inp["dropout_mask"], keep_prob=0.9, prev_block_num=4, next_block_num=4)
            what = "bf16 band prev=next=4 + uint8 dropout mask B=2 N=32 S=8192"
        elif name == "cfg4":
            mask = inp["attn_mask"]; kw.update(tri_block=cfg["block_size"], scale=1.0)
            what = "fp16 TriangleAttention block 512, [B,S,S] fp16 mask tensor read, B=8 N=32 S=4096"
        else:
            kw.update(causal=True); what = "fp16 causal prefill B=8 N=32 S=4096 (forward only)"
        fl = fwd_flops(cfg)
        o, lse = ops.fa_forward(q, k, v, mask, **kw)
        ms_f = t(lambda: ops.fa_forward(q, k, v, mask, **kw), 5)
        rec = {"workload": what, "fwd_ms": ms_f, "fwd_tflops": fl / ms_f / 1e9}
        if "do" in inp:
            do = inp["do"]
            ms_b = t(lambda: ops.fa_backward(q, k, v, o, lse, do, mask, **kw), 3)
            rec.update(bwd_ms=ms_b, bwd_tflops=2.5 * fl / ms_b / 1e9, fwd_bwd_tflops=3.5 * fl / (ms_f + ms_b) / 1e9,
                       frac_of_sustained=3.5 * fl / (ms_f + ms_b) / 1e9 / peaks["tflops"])
        out[name] = rec
        if name == "cfg4":
            # what the TriangleAttention cell runs once it has found the mask tensor to be exactly causal
            # (one pass over the mask per tensor, timed here too): in-kernel triangle, no mask read
            ops.mask_is_causal(mask[:1, :128, :128].contiguous())       # (loads the kernel: not part of the figure)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            is_causal = ops.mask_is_causal(mask)
            detect_ms = (time.perf_counter() - t0) * 1e3
            kw4 = dict(scale=1.0, causal=True)
            o4, lse4 = ops.fa_forward(q, k, v, None, **kw4)
            ms_f4 = t(lambda: ops.fa_forward(q, k, v, None, **kw4), 5)
            ms_b4 = t(lambda: ops.fa_backward(q, k, v, o4, lse4, inp["do"], None, **kw4), 3)
            out["cfg4_mask_elided"] = {
                "workload": "the same inputs; the cell detects the causal mask once and the kernels read none",
                "mask_is_causal": bool(is_causal), "detect_once_ms": detect_ms,
                "fwd_ms": ms_f4, "fwd_tflops": fl / ms_f4 / 1e9, "bwd_ms": ms_b4, "bwd_tflops": 2.5 * fl / ms_b4 / 1e9,
                "fwd_bwd_tflops": 3.5 * fl / (ms_f4 + ms_b4) / 1e9,
                "frac_of_sustained": 3.5 * fl / (ms_f4 + ms_b4) / 1e9 / peaks["tflops"]}
            del o4, lse4
            # the mask kept as a tensor (as for a mask that is not causal), with its per-tile summary: the kernels
            # read only the tiles of the mask that are neither all 0 nor all 1 (here the diagonal ones)
            ops.mask_tile_classes(mask[:1, :128, :128].contiguous())    # (loads the kernel: not part of the figure)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            tiles = ops.mask_tile_classes(mask)
            torch.cuda.synchronize()
            classify_ms = (time.perf_counter() - t0) * 1e3
            kw5 = dict(kw, mask_tiles=tiles)
            o5, lse5 = ops.fa_forward(q, k, v, mask, **kw5)
            ms_f5 = t(lambda: ops.fa_forward(q, k, v, mask, **kw5), 5)
            ms_b5 = t(lambda: ops.fa_backward(q, k, v, o5, lse5, inp["do"], mask, **kw5), 3)
            out["cfg4_mask_tiles"] = {
                "workload": "the same inputs, mask tensor kept, with its per-tile summary (made once per mask)",
                "mixed_tile_fraction": float((tiles == 1).float().mean().item()), "classify_once_ms": classify_ms,
                "fwd_ms": ms_f5, "fwd_tflops": fl / ms_f5 / 1e9, "bwd_ms": ms_b5, "bwd_tflops": 2.5 * fl / ms_b5 / 1e9,
                "fwd_bwd_tflops": 3.5 * fl / (ms_f5 + ms_b5) / 1e9,
                "frac_of_sustained": 3.5 * fl / (ms_f5 + ms_b5) / 1e9 / peaks["tflops"]}
            del o5, lse5, tiles
        if name == "cfg3":
            # the same configuration with dropout decided inside the kernels: no 4.3 GB mask tensor is read
            kw2 = dict(kw)
            kw2.pop("dropout_mask")
            kw2.update(dropout_seed=33, dropout_offset=0)
            o2, lse2 = ops.fa_forward(q, k, v, None, **kw2)
            ms_f2 = t(lambda: ops.fa_forward(q, k, v, None, **kw2), 5)
            ms_b2 = t(lambda: ops.fa_backward(q, k, v, o2, lse2, inp["do"], None, **kw2), 3)
            out["cfg3_in_kernel_dropout"] = {
                "workload": "bf16 band prev=next=4, dropout from Philox4x32-10 inside the kernels, B=2 N=32 S=8192",
                "fwd_ms": ms_f2, "fwd_tflops": fl / ms_f2 / 1e9, "bwd_ms": ms_b2, "bwd_tflops": 2.5 * fl / ms_b2 / 1e9,
                "fwd_bwd_tflops": 3.5 * fl / (ms_f2 + ms_b2) / 1e9,
                "frac_of_sustained": 3.5 * fl / (ms_f2 + ms_b2) / 1e9 / peaks["tflops"]}
            del o2, lse2
        del inp, q, k, v, o, lse
        torch.cuda.empty_cache()
    # compact form for the JSON line: algorithmic TFLOP/s (forward + backward, or forward alone for the prefill),
    # fraction of the measured sustained GEMM rate, and the two times
    short = {"legend": "tf = fwd+bwd TFLOP/s (cfg5a: fwd only), frac = of sustained bf16 GEMM, f_ms / b_ms = forward / "
                       "backward call; cfg3 = uint8 dropout tensor, cfg3_in_kernel = Philox in the kernels; cfg4 = mask "
                       "tensor read in full, cfg4_mask_tiles = with its per-tile summary, cfg4_mask_elided = recognised "
                       "as causal"}
    for name, rec in out.items():
        name = name.replace("cfg3_in_kernel_dropout", "cfg3_in_kernel")
        tf = rec.get("fwd_bwd_tflops", rec["fwd_tflops"])
        short[name] = {"tf": round(tf, 1), "frac": round(tf / peaks["tflops"], 3), "f_ms": round(rec["fwd_ms"], 3)}
        if "bwd_ms" in rec:
            short[name]["b_ms"] = round(rec["bwd_ms"], 3)
        for extra in ("detect_once_ms", "classify_once_ms", "mixed_tile_fraction"):
            if extra in rec:
                short[name][extra] = round(rec[extra], 3)
    return short


def bench_decode(torch, ops, dev, peaks, small=False, rank=0, world=1, dist=None, group=1):
    """Decode step of configuration 5b (B=32 N=32 KV<=16384 D=128 fp16, per-sequence lengths): achieved HBM GB/s
    counting only the valid K and V rows.  Three cache sets (25.8 GB) are rotated so that no step finds its
    cache in L2.  ``small``: B=8 (3 x 2.1 GB, still far above L2), few iterations, for a profiler capture.
    With ``world`` > 1 the job's 32 heads are dealt out over the ranks (sharding.unit_slice): every rank streams its
    heads of all sequences, the time is the max over ranks and the figure is the job's bytes over that time."""
    from acctransformer_b200.sharding import unit_slice
    from acctransformer_b200.workloads import CONFIGS
    c = CONFIGS["cfg5b"]
    B, N_job, S, D = (8 if small else c["B"]), c["N"], c["S"], c["D"]
    h0, h1 = unit_slice(N_job, rank, world)
    N = h1 - h0
    # grouped key/value heads (not part of configuration 5b, whose caches have one head per query head): the caches
    # then have N / group heads and every cache row serves `group` query heads
    N_c = max(1, N // group)
    g = torch.Generator(device=dev).manual_seed(6 + 100 * h0)
    sets = []
    for _ in range(3 if group == 1 else min(12, 3 * group)):      # enough sets that no step finds its cache in L2
        kc = torch.empty(B, N_c, S, D, device=dev, dtype=torch.float16)
        vc = torch.empty(B, N_c, S, D, device=dev, dtype=torch.float16)
        kc.normal_(generator=g)
        vc.normal_(generator=g)
        sets.append((kc, vc))
    qd = torch.randn(B, N, 1, D, device=dev, dtype=torch.float16, generator=g)
    gl = torch.Generator(device="cpu").manual_seed(7)
    lens = torch.randint(c["len_lo"], S + 1, (B,), generator=gl, dtype=torch.int32).to(dev)
    ws = ops.DecodeWorkspace(B, N, D, dev)
    y = torch.empty_like(qd)
    ns = len(sets)
    for i in range(3 if small else 6):
        ops.infer_decode(qd, sets[i % ns][0], sets[i % ns][1], lens, workspace=ws, out=y)
    iters = 6 if small else 30
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for i in range(iters):
        ops.infer_decode(qd, sets[i % ns][0], sets[i % ns][1], lens, workspace=ws, out=y)
    e1.record()
    torch.cuda.synchronize()
    ms_rank = e0.elapsed_time(e1) / iters
    ms = ms_rank
    if dist is not None:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    nbytes_rank = float(lens.sum().item()) * N_c * D * 2 * 2
    nbytes = float(lens.sum().item()) * (N_job // group) * D * 2 * 2
    gbps = nbytes / (ms * 1e-3) / 1e9
    return {"workload": f"cfg5b decode B={B} N={N_job} q_len=1 KV<=16384 D=128 fp16, {N} heads per GPU on {world} GPU(s)"
                        + (f", {group} query heads per cache head" if group > 1 else ""),
            "ms": ms, "bytes": nbytes, "achieved_gbs": gbps, "peak_gbs": world * peaks["hbm_gbs"],
            "frac": gbps / (world * peaks["hbm_gbs"]), "per_gpu_gbs_rank0": nbytes_rank / (ms_rank * 1e-3) / 1e9,
            "peak_source": f"{peaks['which']} hbm_gbs x {world}"}


def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.decode_only:
        import torch
        from acctransformer_b200 import ops
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev)
        print(json.dumps({"decode": bench_decode(torch, ops, dev, measured_peaks(), small=True, group=args.decode_group)}),
              flush=True)
        return 0
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
