#!/usr/bin/env python
"""Benchmark of the MonarchAttention forward op on B200.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference]

Workload (the configuration the headline metric is quoted on): one bf16 MonarchAttention
call with batch 1, 16 heads, N = 16384 tokens as 128 blocks of 128, head width 64, two
alternating iterations, q/k/v ~ N(0,1)/sqrt(64) from a fixed seed, no mask.  A "step" is
one such call.  With N > 1 GPUs every rank runs the same per-GPU workload on its own
inputs (independent (batch, head) units, no data-path collective): weak scaling.

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
def time_oracle(heads, reps, warm):
    from oracle.monarch_oracle import monarch_attention_oracle
    w = WORKLOAD
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    q, k, v = make_inputs(0)
    q, k, v = q[:, :heads], k[:, :heads], v[:, :heads]
    for _ in range(warm):
        monarch_attention_oracle(q, k, v, None, w["T"], w["B"], False)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        monarch_attention_oracle(q, k, v, None, w["T"], w["B"], False)
        times.append(time.perf_counter() - t0)
    return times, cores


def run_reference(args, rank, world):
    """Reference arm: the reference's CPU algorithm (oracle port) on the host cores, rank 0 only."""
    if rank != 0:
        return
    w = WORKLOAD
    # probe the cost of one head, then size the per-step sample so the run stays within ~150 s
    probe, cores = time_oracle(1, 1, 1)
    per_head = probe[0]
    seconds_per_step = 150.0 / max(args.steps + args.warmup, 1)
    heads = int(max(1, min(w["H"], seconds_per_step / per_head)))
    times, cores = time_oracle(heads, args.steps, args.warmup)
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
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# ViT-B/16 forward with MonarchAttention in every layer (second half of the headline metric)
# ---------------------------------------------------------------------------------------------
def build_vit_b(attn_factory, dtype, device):
    """Plain-PyTorch ViT-B/16 (224x224x3 input, 196 patches + CLS, 12 pre-LN layers, hidden 768,
    12 heads of 64, MLP 3072 with GELU), trunc-normal(0.02) random weights.  The attention call site is
    the reference adapter's: q, k, v as permuted (E, H, N, D) views of the projection outputs,
    ``attn_module(q, k, v)``, then ``permute(0, 2, 1, 3)`` back (reference: experiments/vit/model.py:73-103)."""
    import torch.nn as nn

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.ln1, self.ln2 = nn.LayerNorm(768, eps=1e-12), nn.LayerNorm(768, eps=1e-12)
            self.q, self.k, self.v, self.o = (nn.Linear(768, 768) for _ in range(4))
            self.fc1, self.fc2 = nn.Linear(768, 3072), nn.Linear(3072, 768)
            self.attn = attn_factory()

        def forward(self, x):
            E, N, _ = x.shape
            hdn = self.ln1(x)
            q, k, v = (p(hdn).view(E, N, 12, 64).permute(0, 2, 1, 3) for p in (self.q, self.k, self.v))
            ctx = self.attn(q, k, v).permute(0, 2, 1, 3).contiguous().view(E, N, 768)
            x = x + self.o(ctx)
            return x + self.fc2(torch.nn.functional.gelu(self.fc1(self.ln2(x))))

    class ViT(nn.Module):
        def __init__(self):
            super().__init__()
            self.patch = nn.Conv2d(3, 768, 16, 16)
            self.cls = nn.Parameter(torch.zeros(1, 1, 768))
            self.pos = nn.Parameter(torch.zeros(1, 197, 768))
            self.blocks = nn.ModuleList(Block() for _ in range(12))
            self.ln = nn.LayerNorm(768, eps=1e-12)
            self.head = nn.Linear(768, 1000)

        def forward(self, img):
            x = self.patch(img).flatten(2).transpose(1, 2)
            x = torch.cat((self.cls.expand(x.shape[0], -1, -1), x), dim=1) + self.pos
            for b in self.blocks:
                x = b(x)
            return self.head(self.ln(x)[:, 0])

    torch.manual_seed(0)
    model = ViT()
    for p_ in model.parameters():
        if p_.dim() > 1:
            torch.nn.init.trunc_normal_(p_, std=0.02)
    return model.to(device=device, dtype=dtype).eval()


def time_vit(device, steps=10, warmup=3, batch=64):
    """img/s of the ViT-B forward, bf16, batch 64, block size 15, one iteration, front padding; and the
    same model with dense SDPA as context."""
    from monarch_attention_b200 import MonarchAttention

    class Dense(torch.nn.Module):
        def forward(self, q, k, v):
            return torch.nn.functional.scaled_dot_product_attention(q, k, v)

    def monarch():
        m = MonarchAttention(15, 1, "pre")
        m.token_major_output = True
        return m

    g = torch.Generator(device="cpu").manual_seed(0)
    img = torch.rand(batch, 3, 224, 224, generator=g).to(torch.bfloat16).to(device)
    out = {}
    for name, factory in (("monarch_b200", monarch), ("dense_sdpa", Dense)):
        model = build_vit_b(factory, torch.bfloat16, device)
        with torch.no_grad():
            for _ in range(warmup):
                model(img)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                logits = model(img)
            e1.record()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        out[name] = {"img_per_s": batch / (ms * 1e-3), "ms_per_forward": ms, "finite": bool(torch.isfinite(logits).all())}
    return out


# ---------------------------------------------------------------------------------------------
# Our arm
# ---------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local):
    from monarch_attention_b200 import MonarchAttention, _cabi
    from monarch_attention_b200.monarch_attention import make_problem

    lib = _cabi.load()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    w = WORKLOAD
    warmup = max(args.warmup, 3)
    mod = MonarchAttention(w["B"], w["T"], "post")
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
    tokens_per_step = w["E"] * w["N"] * world
    value = tokens_per_step / (ms_step * 1e-3)

    # ---- end to end: pinned host inputs -> device -> op -> pinned host result, every step -------------
    e2e_steps = max(3, min(args.steps, 20))
    hq, hk, hv = (t.cpu().pin_memory() for t in sets[0])
    hout = torch.empty(outs[0].shape, dtype=outs[0].dtype).pin_memory()
    from monarch_attention_b200 import monarch_attention_b200_host

    def e2e_step():
        # the package's host-buffer entry point: chunks of heads, H2D / kernels / D2H on three streams;
        # steps do not overlap one another (the caller's stream waits for the last D2H of every step)
        monarch_attention_b200_host(hq, hk, hv, None, w["T"], w["B"], False, out=hout, wait=False,
                                    heads_per_chunk=args.e2e_heads_per_chunk)

    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    barrier(world)
    e2e_ms = max_over_ranks(e0.elapsed_time(e1), world, dev) / e2e_steps
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv))
    d2h = hout.numel() * hout.element_size()
    sampler.stop()

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
    flops, nbytes, stage_flops = work_model()
    names = ["right", "left", "right_with_v", "output"]
    stages = [{"stage": n, "ms": acc[i], "tflops": stage_flops[n] / (acc[i] * 1e-3) / 1e12} for i, n in enumerate(names)]
    peaks = measured_peaks()
    t_tensor = flops / (peaks["bf16_tflops"] * 1e12)
    t_hbm = nbytes / (peaks["hbm_gbs"] * 1e9)
    achieved_tflops = flops / (ms_step * 1e-3) / 1e12
    roofline = {
        "bound": "tensor" if t_tensor >= t_hbm else "hbm",
        "achieved": achieved_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
        "frac": achieved_tflops / peaks["bf16_tflops"],
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch of the fused kernel on this workload,
        # from an `ncu --set full` capture (profiles/fused_kernel_c3_n16384_bf16.md); not measured live
        "traffic": 245.8e6 if L_auto.kernel == _cabi.KERNEL_TCGEN05 else None,
        "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
        "scope": "whole op = one fused launch per step; algorithmic FLOPs / ms_per_step; `stages` = the same "
                 "kernel launched once per stage",
        "hbm_floor_frac": t_hbm / (ms_step * 1e-3),
        "stages": stages,
    }

    # ---- context: dense SDPA on the same GPU, same q, k, v ------------------------------------------
    context = {}
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

    # ---- second half of the headline metric: ViT-B/16 forward, img/s -----------------------------------
    try:
        context["vit_b16_bf16_batch64_b15_T1"] = time_vit(dev)
    except Exception as exc:
        context["vit_b16_error"] = str(exc)[:200]

    # ---- CPU baseline: the oracle port on the host cores, bounded sample ----------------------------
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        probe, cores = time_oracle(1, 1, 1)
        heads = int(max(1, min(w["H"], 5.0 / probe[0])))
        times, cores = time_oracle(heads, 3, 0)
        step_s = statistics.median(times) * w["H"] / heads
        cpu_baseline = {"value": w["E"] * w["N"] / step_s, "unit": UNIT, "cores": cores, "kind": "port",
                        "sample": f"median of 3 passes over {heads} of {w['H']} heads, scaled by {w['H']}/{heads}",
                        "ms_per_step": 1e3 * step_s}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": w["name"], **{k_: w[k_] for k_ in ("E", "H", "N", "D", "B", "T")},
                   "per_gpu_workload": "full (E=1, H=16) on every rank",
                   "l2": f"{N_INPUT_SETS} rotating input sets ({N_INPUT_SETS * 3 * 33.5:.0f} MB) > 126 MB L2",
                   "kernel": _cabi.KERNEL_NAMES[L_auto.kernel]},
        "clocks": sampler.summary(),
        "e2e": {"value": tokens_per_step / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps,
                "api": "monarch_attention_b200_host: pinned host q, k, v in, pinned host result out, "
                       f"{args.e2e_heads_per_chunk} heads per chunk"},
        "gpu_launches": args.steps * (1 if L_auto.kernel == _cabi.KERNEL_TCGEN05 else n_stage),
        "roofline": roofline,
        "cpu_baseline": cpu_baseline,
        "context": context,
    }
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
    E, H, N, D, B, T = (int(x) for x in f[:6])
    pre = len(f) > 6 and f[6] == "pre"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(E, H, N, D, generator=g).to(torch.bfloat16).to(dev) for _ in range(3))
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
    ap.add_argument("--e2e-heads-per-chunk", type=int, default=8,
                    help="heads per pipeline chunk of the end-to-end (host memory) measurement")
    ap.add_argument("--layer", default=None, help="E,H,N,D,B,T,pre|post[,mask]: time one layer of that shape instead")
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
