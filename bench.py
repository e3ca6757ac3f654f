#!/usr/bin/env python
"""Benchmark of the MonarchAttention forward op on B200.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference]

Workload (the configuration the headline metric is quoted on): one bf16 MonarchAttention
call with batch 1, 16 heads, N = 16384 tokens as 128 blocks of 128, head width 64, two
alternating iterations, q/k/v ~ N(0,1)/sqrt(64) from a fixed seed, no mask.  A "step" is
one such call.  With N > 1 GPUs every rank runs the same per-GPU workload on its own
inputs (independent (batch, head) units, no data-path collective): weak scaling.  With
``--scaling strong`` the 16 heads of ONE call are split across the ranks instead (16 / 8 / 4 / 2
heads per GPU), and the per-head checksums of the shards are gathered on rank 0 and compared
with the unsharded call.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(name="op_sweep_bf16_N16384_H16_D64_b128_T2", E=1, H=16, N=16384, D=64, Dv=64, B=128, T=2)
METRIC = "monarch_attention_tokens_per_s"
UNIT = "tokens/s"
N_INPUT_SETS = 4  # rotated between steps so that a step never finds its inputs in L2


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def work_model(w=WORKLOAD, itemsize=2):
    E, H, N, D, Dv, B, T = (w[x] for x in ("E", "H", "N", "D", "Dv", "B", "T"))
    M = -(-N // B)
    flops = E * H * ((T - 1) * 4 * N * D * (B + M) + N * (4 * B * D + 2 * B * Dv + 2 * M * D + 2 * M * Dv))
    nbytes = E * H * N * (2 * D + 2 * Dv) * itemsize
    stage = {  # per launch, in launch order for T = 2
        "right": E * H * 4 * N * B * D,
        "left": E * H * 4 * N * M * D,
        "right_with_v": E * H * (4 * N * B * D + 2 * N * B * Dv),
        "output": E * H * (2 * N * M * D + 2 * N * M * Dv),
    }
    return flops, nbytes, stage


def make_inputs(seed, device=None, w=WORKLOAD, dtype=torch.bfloat16):
    g = torch.Generator(device="cpu").manual_seed(seed)
    shape = (w["E"], w["H"], w["N"], w["D"])
    q, k = (torch.randn(shape, generator=g) / w["D"] ** 0.5 for _ in range(2))
    v = torch.randn((w["E"], w["H"], w["N"], w["Dv"]), generator=g) / w["D"] ** 0.5
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    if device is not None:
        q, k, v = q.to(device), k.to(device), v.to(device)
    return q, k, v


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the GPU is under load."""

    def __init__(self, index, period_s=0.002):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reason_bits = [], 0
        self.window = [None, None]
        self.sm_max = None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self._stop_evt.is_set():
            try:
                t = time.perf_counter()
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((t, mhz, bits))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=2)

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": ["unavailable"]}
        lo, hi = self.window
        inside = [s for s in self.samples if lo is not None and lo <= s[0] <= hi]
        scope = "timed_region"
        if len(inside) < 3:  # very short timed region: fall back to every sample taken under load
            inside, scope = self.samples, "whole_run_under_load"
        bits = 0
        for s in inside:
            bits |= s[2]
        names = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
                 0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}
        reasons = [n for b, n in names.items() if bits & b and n != "gpu_idle"]
        return {"sm_mhz": statistics.median(s[1] for s in inside), "sm_max_mhz": self.sm_max, "reasons": reasons,
                "samples": len(inside), "scope": scope}


def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def max_over_ranks(x, world, device):
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ---------------------------------------------------------------------------------------------
# CPU oracle timing (the reference's algorithm restated on the host; see oracle/)
# ---------------------------------------------------------------------------------------------
def reference_package():
    """The reference's own ``ma`` package from oracle/_ref (placed there by oracle/make_ref.py, git-ignored),
    or None.  Used for timing only, never by the product."""
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "ma")):
        return None
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    try:
        import ma.monarch_attention as mod  # noqa: PLC0415
        return mod
    except Exception:
        return None


def time_oracle(heads, reps, warm):
    """CPU timing of the reference's eager implementation on `heads` heads of the workload: the reference's
    own ma_torch when oracle/_ref holds it (kind "reference"), else the oracle port (kind "port")."""
    w = WORKLOAD
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    q, k, v = make_inputs(0)
    q, k, v = q[:, :heads], k[:, :heads], v[:, :heads]
    mod = reference_package()
    if mod is not None:
        ref = mod.MonarchAttention(w["B"], w["T"], "post", impl="torch")
        fn, kind = (lambda: ref(q, k, v)), "reference"
    else:
        from oracle.monarch_oracle import monarch_attention_oracle
        fn, kind = (lambda: monarch_attention_oracle(q, k, v, None, w["T"], w["B"], False)), "port"
    with torch.no_grad():
        for _ in range(warm):
            fn()
        times = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            times.append(time.perf_counter() - t0)
    return times, cores, kind


def run_reference(args, rank, world):
    """Reference arm: the reference's CPU implementation of the path on the host cores (its own ma_torch
    from oracle/_ref when present, else the oracle port), rank 0 only."""
    if rank != 0:
        return
    w = WORKLOAD
    # probe the cost of one head, then size the per-step sample so the run stays within ~150 s
    probe, cores, kind = time_oracle(1, 1, 1)
    per_head = probe[0]
    seconds_per_step = 150.0 / max(args.steps + args.warmup, 1)
    heads = int(max(1, min(w["H"], seconds_per_step / per_head)))
    times, cores, kind = time_oracle(heads, args.steps, args.warmup)
    total = sum(times)
    # tokens/s of the full 16-head op = E*N / (time for H heads); a sample of `heads` heads scales linearly
    step_s = total / args.steps
    value = w["E"] * w["N"] / (step_s * w["H"] / heads)
    sample = f"{heads} of {w['H']} heads of the workload per step (independent heads, time scaled by {w['H']}/{heads})"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * step_s * w["H"] / heads,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["name"], **{k: w[k] for k in ("E", "H", "N", "D", "B", "T")}},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# Context measurements: the three caller models, the reference's own GPU paths
# ---------------------------------------------------------------------------------------------
def _time_model(model, inputs, steps, warmup):
    with torch.no_grad():
        for _ in range(warmup):
            out = model(*inputs)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            out = model(*inputs)
        e1.record()
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps, bool(torch.isfinite(out.float()).all())


def time_models(device, rank, world, steps=5, warmup=2):
    """Forward throughput of the three caller models (monarch_attention_b200/models.py: plain PyTorch, random
    weights, seeded synthetic inputs) with this library's attention and with dense SDPA, bf16.  The batch of
    each configuration is split across the ranks (64 / 32 / 16 / 8 per GPU ...); the per-rank times are
    gathered on rank 0 with one collective and the slowest rank sets the aggregate rate."""
    from monarch_attention_b200 import MonarchAttention
    from monarch_attention_b200.models import DenseAttention, build_dit_xl2, build_roberta_base, build_vit_b16
    from monarch_attention_b200.sharding import gather_to_rank0, unit_range

    def monarch(B, T, pad):
        def make():
            m = MonarchAttention(B, T, pad)
            m.token_major_output = True
            return m
        return make

    g = torch.Generator(device="cpu").manual_seed(0)

    def vit_inputs(n):
        return (torch.rand(n, 3, 224, 224, generator=g).to(torch.bfloat16).to(device),)

    def roberta_inputs(n):
        ids = torch.randint(3, 50265, (n, 512), generator=g)
        mask = torch.ones(n, 512, dtype=torch.long)
        for e in range(0, n, 4):  # a quarter of the sequences right-padded to a random length in [128, 512]
            ln = int(torch.randint(128, 513, (1,), generator=g))
            mask[e, ln:] = 0
            ids[e, ln:] = 1
        return ids.to(device), mask.to(device)

    def dit_inputs(n):
        return (torch.randn(n, 4, 64, 64, generator=g).to(torch.bfloat16).to(device),
                torch.randint(0, 1000, (n,), generator=g).to(device), torch.randint(0, 1000, (n,), generator=g).to(device))

    configs = [
        ("vit_b16_bf16_batch64_b15_T1", build_vit_b16, vit_inputs, 64, monarch(15, 1, "pre"), "img_per_s"),
        ("roberta_base_bf16_batch32_n512_b32_T1_mask", build_roberta_base, roberta_inputs, 32, monarch(32, 1, "post"), "seq_per_s"),
        ("dit_xl2_bf16_batch64_n1024_d72_b32_T2", build_dit_xl2, dit_inputs, 64, monarch(32, 2, "pre"), "img_per_s"),
    ]
    out = {}
    for name, build, make_in, batch, factory, unit in configs:
        lo, hi = unit_range(batch, rank, world)
        res = {}
        if hi > lo:
            inputs = make_in(hi - lo)
            for label, fac in (("monarch_b200", factory), ("dense_sdpa", DenseAttention)):
                model = build(fac, torch.bfloat16, device)
                ms, finite = _time_model(model, inputs, steps, warmup)
                res[label] = (ms, finite)
                del model
            torch.cuda.empty_cache()
        gathered = gather_to_rank0({"n": hi - lo, "res": res})
        if rank == 0:
            entry = {"batch": batch, "per_rank_batch": [x["n"] for x in gathered]}
            for label in ("monarch_b200", "dense_sdpa"):
                times = [x["res"][label][0] for x in gathered if x["res"]]
                entry[label] = {unit: batch / (max(times) * 1e-3), "ms_per_forward": max(times),
                                "finite": all(x["res"][label][1] for x in gathered if x["res"])}
            out[name] = entry
    return out


def time_reference_gpu(q, k, v, T, B, reps=5):
    """The reference's own module on this GPU: eager PyTorch (impl="torch") and its Triton kernels
    (impl="triton"), from oracle/_ref when that directory travelled with the tree."""
    mod = reference_package()
    if mod is None:
        return {"unavailable": "oracle/_ref is not present (run oracle/make_ref.py where the reference is checked out)"}
    out = {}
    for impl in ("torch", "triton"):
        try:
            m = mod.MonarchAttention(B, T, "post", impl=impl)
            with torch.no_grad():
                for _ in range(2):
                    res = m(q, k, v)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    res = m(q, k, v)
                e1.record()
                torch.cuda.synchronize()
            out[f"reference_{impl}_gpu_ms"] = e0.elapsed_time(e1) / reps
            out[f"reference_{impl}_gpu_finite"] = bool(torch.isfinite(res.float()).all())
        except Exception as exc:  # e.g. the Triton kernels do not compile with the installed Triton
            out[f"reference_{impl}_gpu_ms"] = None
            out[f"reference_{impl}_gpu_unavailable"] = (str(exc).strip().splitlines() or [repr(exc)])[0][:160]
    return out


def fused_kernel_dram_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the fused kernel on the headline workload,
    as recorded in the committed ncu summary (a profiler cannot run inside this script)."""
    import re
    try:
        text = open(os.path.join(ROOT, "profiles", "fused_kernel_c3_n16384_bf16.md")).read()
        m = re.search(r"dram_traffic_bytes_per_launch\s*=\s*([0-9.eE+]+)", text)
        return float(m.group(1)) if m else None
    except OSError:
        return None


def bind_to_gpu_numa_node(local):
    """Run this rank's host threads (and therefore first-touch its pinned staging buffers) on the NUMA node the
    GPU hangs off.  Host placement only; nothing about the GPU is changed."""
    try:
        import pynvml
        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(local)).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        if len(bus.split(":")[0]) == 8:
            bus = bus[4:]
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return {"numa_node": node, "cpus": len(cpus)}
    except Exception:
        pass
    return None


# ---------------------------------------------------------------------------------------------
# Our arm
# ---------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local):
    from monarch_attention_b200 import MonarchAttention, _cabi
    from monarch_attention_b200.monarch_attention import make_problem
    from monarch_attention_b200.sharding import gather_to_rank0, shard_heads

    lib = _cabi.load()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    numa = bind_to_gpu_numa_node(local)
    w = WORKLOAD
    warmup = max(args.warmup, 3)
    strong = args.scaling == "strong"
    mod = MonarchAttention(w["B"], w["T"], "post")
    if strong:
        # ONE call's 16 heads split across the ranks: every rank draws the same full inputs and keeps its slice
        sets = [tuple(t.contiguous() for t in shard_heads(*make_inputs(i, dev), rank, world)) for i in range(N_INPUT_SETS)]
    else:
        sets = [make_inputs(1000 * rank + i, dev) for i in range(N_INPUT_SETS)]
    outs = [torch.empty_like(s[2]) for s in sets]

    def step(i):
        q, k, v = sets[i % N_INPUT_SETS]
        return mod(q, k, v)

    sampler = ClockSampler(local)
    sampler.start()
    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    barrier(world)
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.window[0] = time.perf_counter()
    ev0.record()
    for i in range(args.steps):
        step(i)
    ev1.record()
    torch.cuda.synchronize()
    sampler.window[1] = time.perf_counter()
    barrier(world)
    ms_total = max_over_ranks(ev0.elapsed_time(ev1), world, dev)
    ms_step = ms_total / args.steps
    tokens_per_step = w["E"] * w["N"] * (1 if strong else world)
    value = tokens_per_step / (ms_step * 1e-3)

    shard_check = None
    if strong:
        # per-head checksums of the sharded call, gathered on rank 0 and compared with the unsharded call
        # (integer sums of the 16-bit patterns: exact whatever the order of summation)
        def checksums(t):
            b = t.contiguous().view(torch.int16).to(torch.int64)
            return torch.stack([b.sum(dim=(-1, -2)).flatten(), (b * b).sum(dim=(-1, -2)).flatten()]).cpu()

        parts = gather_to_rank0(checksums(step(0)))
        if rank == 0:
            want = checksums(MonarchAttention(w["B"], w["T"], "post")(*make_inputs(0, dev)))
            got = torch.cat(parts, dim=1)
            shard_check = "bitwise" if torch.equal(got, want) else f"{int((got != want).any(dim=0).sum())} of {want.shape[1]} heads differ"

    # ---- end to end: pinned host inputs -> device -> op -> pinned host result, every step -------------
    e2e_steps = max(3, min(args.steps, 20))
    hq, hk, hv = (t.cpu().pin_memory() for t in sets[0])
    hout = torch.empty(outs[0].shape, dtype=outs[0].dtype).pin_memory()
    from monarch_attention_b200 import monarch_attention_b200_host

    def e2e_step(streamed):
        # the package's host-buffer entry point: chunks of heads, H2D / kernels / D2H on three streams.
        # streamed: the copy-in of a step starts while the kernels and the copy-out of the previous step are
        # still running (every step still copies its own inputs in and its own result out); otherwise the
        # steps do not overlap one another (the caller's stream waits for the last D2H of every step).
        monarch_attention_b200_host(hq, hk, hv, None, w["T"], w["B"], False, out=hout, wait=False, streamed=streamed,
                                    heads_per_chunk=args.e2e_heads_per_chunk)

    def time_e2e(streamed):
        for _ in range(3):
            e2e_step(streamed)
        torch.cuda.synchronize()
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step(streamed)
        e1.record()
        torch.cuda.synchronize()
        barrier(world)
        return max_over_ranks(e0.elapsed_time(e1), world, dev) / e2e_steps

    e2e_serial_ms = time_e2e(False)
    e2e_ms = time_e2e(True)
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv))
    d2h = hout.numel() * hout.element_size()
    sampler.stop()

    # ---- the caller models, batch split across the ranks (one gather per model) ---------------------
    context = {}
    if not args.no_models:
        try:
            models = time_models(dev, rank, world)
            if rank == 0:
                context.update(models)
        except Exception as exc:
            context["models_error"] = str(exc)[:200]

    if rank != 0:
        return

    # ---- per-stage launch durations (CUDA events on the launching stream, inside the library) ------
    # (the headline runs the fused single-launch kernel; the same kernel launched once per stage gives
    # the per-stage breakdown)
    q, k, v = sets[0]
    prob = make_problem(q, k, v, outs[0], None, w["T"], w["B"], False)
    L_auto = _cabi.WorkspaceLayout()
    _cabi.raise_for_status(lib.ma_b200_workspace_layout_of(C.byref(prob), C.byref(L_auto)))
    staged = _cabi.KERNEL_TCGEN05_STAGED if L_auto.kernel == _cabi.KERNEL_TCGEN05 else L_auto.kernel
    prob = make_problem(q, k, v, outs[0], None, w["T"], w["B"], False, staged)
    L = _cabi.WorkspaceLayout()
    _cabi.raise_for_status(lib.ma_b200_workspace_layout_of(C.byref(prob), C.byref(L)))
    ws = torch.empty(L.total, dtype=torch.uint8, device=dev)
    n_stage = 2 * w["T"]
    acc = [0.0] * n_stage
    reps = 20
    buf = (C.c_float * n_stage)()
    stream = torch.cuda.current_stream().cuda_stream
    for r in range(reps + 3):
        qq, kk, vv = sets[r % N_INPUT_SETS]
        prob = make_problem(qq, kk, vv, outs[0], None, w["T"], w["B"], False, staged)
        _cabi.raise_for_status(lib.ma_b200_forward_timed(C.byref(prob), ws.data_ptr(), ws.numel(), stream, buf, n_stage))
        if r >= 3:
            for i in range(n_stage):
                acc[i] += buf[i] / reps
    _cabi.raise_for_status(lib.ma_b200_device_status(ws.data_ptr(), stream))
    _cabi.raise_for_status(lib.ma_b200_poll_device_status(local))
    flops, nbytes, stage_flops = work_model()
    if strong:
        flops, nbytes = flops / world, nbytes / world  # this rank's share; the roofline below is per GPU
    names = ["right", "left", "right_with_v", "output"]
    stages = [{"stage": n, "ms": acc[i], "tflops": stage_flops[n] / (world if strong else 1) / (acc[i] * 1e-3) / 1e12}
              for i, n in enumerate(names)]
    peaks = measured_peaks()
    t_tensor = flops / (peaks["bf16_tflops"] * 1e12)
    t_hbm = nbytes / (peaks["hbm_gbs"] * 1e9)
    achieved_tflops = flops / (ms_step * 1e-3) / 1e12
    fused = L_auto.kernel == _cabi.KERNEL_TCGEN05
    roofline = {
        "bound": "tensor" if t_tensor >= t_hbm else "hbm",
        "achieved": achieved_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
        "frac": achieved_tflops / peaks["bf16_tflops"],
        # per launch of the fused kernel on this workload, from the committed `ncu` summary under profiles/
        "traffic": fused_kernel_dram_traffic() if fused and not strong else None,
        "algorithmic_bytes": nbytes,
        "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
        "scope": "whole op = one fused launch per step; algorithmic FLOPs / ms_per_step; `stages` = the same "
                 "kernel launched once per stage",
        "hbm_floor_frac": t_hbm / (ms_step * 1e-3),
        "stages": stages,
    }

    # ---- context: dense SDPA and the reference's own GPU paths on the same GPU, same q, k, v --------
    try:
        import torch.nn.functional as F
        for _ in range(2):
            F.scaled_dot_product_attention(q, k, v)
        torch.cuda.synchronize()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(5):
            F.scaled_dot_product_attention(q, k, v)
        s1.record()
        torch.cuda.synchronize()
        context["dense_sdpa_ms"] = s0.elapsed_time(s1) / 5
    except Exception as exc:  # context only
        context["dense_sdpa_ms"] = None
        context["dense_sdpa_error"] = str(exc)[:100]
    if not args.no_reference_gpu:
        context.update(time_reference_gpu(q, k, v, w["T"], w["B"]))

    # ---- CPU baseline: the reference's eager path on the host cores, bounded sample -----------------
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        probe, cores, kind = time_oracle(1, 1, 1)
        heads = int(max(1, min(w["H"], 5.0 / probe[0])))
        times, cores, kind = time_oracle(heads, 3, 0)
        step_s = statistics.median(times) * w["H"] / heads
        cpu_baseline = {"value": w["E"] * w["N"] / step_s, "unit": UNIT, "cores": cores, "kind": kind,
                        "sample": f"median of 3 passes over {heads} of {w['H']} heads, scaled by {w['H']}/{heads}",
                        "ms_per_step": 1e3 * step_s}

    heads_per_gpu = w["H"] // world if strong else w["H"]
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if strong else "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["name"], **{k_: w[k_] for k_ in ("E", "H", "N", "D", "B", "T")},
                   "per_gpu_workload": f"{heads_per_gpu} of the 16 heads per rank" if strong else "full (E=1, H=16) on every rank",
                   "l2": f"{N_INPUT_SETS} rotating input sets ({N_INPUT_SETS * 3 * 33.5 / (world if strong else 1):.0f} MB) > 126 MB L2"
                         if not strong or world <= 2 else f"{N_INPUT_SETS} rotating input sets; L2 flushed by nothing else (inputs of a rank are {N_INPUT_SETS * 3 * 33.5 / world:.0f} MB)",
                   "kernel": _cabi.KERNEL_NAMES[L_auto.kernel]},
        "clocks": sampler.summary(),
        "e2e": {"value": tokens_per_step / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps, "host_placement": numa,
                "ms_per_step_without_overlap_between_steps": e2e_serial_ms,
                "api": "monarch_attention_b200_host(streamed=True): pinned host q, k, v in, pinned host result out every "
                       f"step, {args.e2e_heads_per_chunk} heads per chunk; the copy-in of a step overlaps the kernels and "
                       "the copy-out of the step before it"},
        "gpu_launches": args.steps * (1 if fused else n_stage),
        "roofline": roofline,
        "cpu_baseline": cpu_baseline,
        "context": context,
    }
    if strong:
        line["shard_check"] = shard_check
    print(json.dumps(line), flush=True)


def run_layer(args):
    """`--layer E,H,N,D,B,T,pad[,mask]`: kernel-only timing of one attention layer of another configuration
    (ViT: 64,12,197,64,15,1,pre   RoBERTa: 32,12,512,64,32,1,post,mask   DiT: 64,16,1024,72,32,2,post
    N = 65536: 1,16,65536,64,256,2,post), per stage, from CUDA events recorded inside the library.  Not the
    headline line: it exists so that the other kernel families can be timed and profiled with a committed command."""
    import ctypes as C

    from monarch_attention_b200 import _cabi
    from monarch_attention_b200.monarch_attention import make_problem
    f = args.layer.split(",")
    dtype = torch.bfloat16
    if f[-1] in ("f32", "f16", "bf16"):
        dtype = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[f.pop()]
    E, H, N, D, B, T = (int(x) for x in f[:6])
    pre = len(f) > 6 and f[6] == "pre"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(E, H, N, D, generator=g).div(8).to(dtype).to(dev) for _ in range(3))
    mask = (torch.rand(E, N, generator=g) > 0.1).to(torch.uint8).to(dev) if len(f) > 7 and f[7] == "mask" else None
    out = torch.empty_like(v)
    lib = _cabi.load()
    prob = make_problem(q, k, v, out, mask, T, B, pre, _cabi.KERNEL_AUTO)
    L = _cabi.WorkspaceLayout()
    _cabi.raise_for_status(lib.ma_b200_workspace_layout_of(C.byref(prob), C.byref(L)))
    ws = torch.empty(L.total, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    buf = (C.c_float * (2 * T))()
    acc = [0.0] * (2 * T)
    for it in range(args.warmup + args.steps):
        _cabi.raise_for_status(lib.ma_b200_forward_timed(C.byref(prob), ws.data_ptr(), ws.numel(), stream, buf, 2 * T))
        if it >= args.warmup:
            acc = [a + b / args.steps for a, b in zip(acc, buf)]
    print(json.dumps({"layer": args.layer, "kernel": _cabi.KERNEL_NAMES[L.kernel], "stage_ms": acc,
                      "ms_per_layer": sum(acc), "steps": args.steps, "warmup": args.warmup}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-models", action="store_true", help="skip the ViT / RoBERTa / DiT context measurements")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip timing the reference's own GPU paths")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak",
                    help="weak: the full 16-head call on every rank; strong: the 16 heads of one call split across ranks")
    ap.add_argument("--e2e-heads-per-chunk", type=int, default=8,
                    help="heads per pipeline chunk of the end-to-end (host memory) measurement")
    ap.add_argument("--layer", default=None, help="E,H,N,D,B,T,pre|post[,mask][,f32|f16|bf16]: time one layer of that shape instead (bf16 by default)")
    args = ap.parse_args()
    if args.layer:
        run_layer(args)
        return
    if args.impl == "reference":
        rank = int(os.environ.get("RANK", "0"))
        run_reference(args, rank, int(os.environ.get("WORLD_SIZE", "1")))
        return
    rank, world, local = dist_setup(args.gpus)
    try:
        run_ours(args, rank, world, local)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
