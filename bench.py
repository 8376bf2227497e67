"""Benchmark of the Parallax attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--head-dim 128|64]

Workload ("train_dense_causal_B8_H16_L4096_D128"): one step = forward + backward of
the causal training op `parallax_func` on q, r, k, v of shape (8, 16, 4096, D),
bf16, iid N(0,1) from a fixed seed, loss = mean(o.float()^2).  Metric: achieved
algorithmic TFLOP/s, 12 * B * H * D * L * (L + 1) flop per step (4 forward + 8
backward causal matmuls).  With N > 1 GPUs every rank runs the same per-GPU
workload on its own (batch x heads) shard -- there is no collective on the data
path -- and the reported value is the sum over ranks ("weak" scaling).

One JSON line is printed by rank 0:
  value      device-resident throughput (inputs in HBM, CUDA events, max over ranks)
  e2e        the same step through the public API with q, r, k, v copied from pinned
             host memory and the loss read back, every step; with the bare copy time of
             all ranks at once beside it (`h2d_ceiling_ms`)
  roofline   the dominant kernel against the measured bf16 tensor peak (burst and sustained)
  cpu_baseline  the CPU oracle (a PyTorch restatement of the reference's fp32
             implementation) timed on this host's cores on a bounded sample
and, as context (each with an in-line parity number against the CPU oracle):
  cfg1, d64             (N = 1) the small parity configuration and the head_dim-64 variant
  varlen*               (N = 1) packed configurations: 14 sequences, 1024 sequences, one sequence
  decode, roofline_decode  (N = 1) HBM GB/s and microseconds of the decode sweep
  sharded_train_5a      B=16, H=32, L=8192: H/N heads per rank, no collective (strong scaling)
  sharded_decode_5b     B=1, H=32, 524288 keys: T/N keys per rank + exchange of per-head records
  sharded_varlen        the packed 65536-token configuration, 16/N heads per rank

`--impl reference` times that CPU implementation alone (the reference's GPU kernels are Triton
sources; what they do on this GPU is recorded once by baseline/reference_gpu_probe.py and quoted
as `reference_gpu`).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

B, H, L = 8, 16, 4096      # the benchmark workload; --batch / --heads / --seq-len shrink it for profiling runs
SEED = 1002


def train_flops(bsz, heads, length, d):
    return 12.0 * bsz * heads * d * length * (length + 1)


def workload_name(d):
    return f"train_dense_causal_B{B}_H{H}_L{L}_D{d}"


# --------------------------------------------------------------------------- #
# clocks
# --------------------------------------------------------------------------- #
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU every 10 ms on a thread (NVML, read-only)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, gpu_index: int):
        self.gpu, self.thread, self.stop_flag = gpu_index, None, None
        self.sm, self.reasons, self.sm_max, self.power = [], set(), None, []

    def start(self):
        import threading

        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            if visible and not visible.split(",")[self.gpu].strip().isdigit():
                handle = pynvml.nvmlDeviceGetHandleByUUID(visible.split(",")[self.gpu].strip())
            else:
                index = int(visible.split(",")[self.gpu]) if visible else self.gpu
                handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            return
        self.stop_flag = threading.Event()

        def loop():
            while not self.stop_flag.is_set():
                try:
                    self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                    self.power.append(pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0)
                    mask = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                    for bit, name in self.REASONS.items():
                        if mask & bit:
                            self.reasons.add(name)
                except Exception:
                    pass
                time.sleep(0.01)

        self.thread = threading.Thread(target=loop, daemon=True)
        self.thread.start()

    def stop(self):
        if self.thread is None:
            return None
        self.stop_flag.set()
        self.thread.join(timeout=2)
        if not self.sm:
            return None
        return {"sm_mhz": statistics.median(self.sm), "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons),
                "samples": len(self.sm), "power_w_max": max(self.power) if self.power else None}


# --------------------------------------------------------------------------- #
# CPU implementation (oracle) timing -- cpu_baseline and the reference arm
# --------------------------------------------------------------------------- #
def cpu_slice_inputs(d, n_slices):
    g = torch.Generator().manual_seed(SEED)
    mk = lambda: torch.randn(1, n_slices, L, d, generator=g, dtype=torch.float32).to(torch.bfloat16)
    return mk(), mk(), mk(), mk()


def reference_cpu_impl():
    """The reference's own fp32 implementation, `parallax_reference` (parallax/reference.py:15-86 of the
    reference), loaded from the unmodified install under baseline/_ref when that directory is present
    (it is git-ignored but travels with the working tree); None otherwise."""
    path = os.path.join(ROOT, "baseline", "_ref", "parallax", "reference.py")
    if not os.path.exists(path):
        return None
    import importlib.util

    spec = importlib.util.spec_from_file_location("_reference_parallax_reference", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.parallax_reference


def cpu_time_slices(d, n_slices, impl=None):
    """fwd + bwd of `n_slices` (batch, head) slices of the workload on the CPU; returns seconds.  `impl` is
    the reference's `parallax_reference` (forward, autograd backward of mean(o^2)); without it the oracle
    port (closed-form backward) is timed."""
    q, r, k, v = cpu_slice_inputs(d, n_slices)
    if impl is not None:
        leaves = [x.permute(0, 2, 1, 3).float().requires_grad_(True) for x in (q, r, k, v)]      # (B, L, H, D)
        t0 = time.perf_counter()
        o = impl(*leaves, d ** -0.5)
        (o.pow(2).sum() * (1.0 / (o.numel() * (B * H / n_slices)))).backward()
        return time.perf_counter() - t0
    from oracle import parallax_oracle as orc

    t0 = time.perf_counter()
    f = orc.train_forward(q, r, k, v)
    go = orc.mse_loss_grad(f["o"]) * (1.0 / (B * H / n_slices))
    orc.train_backward(q, r, k, v, go)
    return time.perf_counter() - t0


def cpu_kind(impl):
    return ("reference", "the reference's parallax_reference (fp32 PyTorch, autograd backward) from baseline/_ref") if impl is not None \
        else ("port", "fp32 PyTorch restatement of parallax/reference.py with a closed-form backward (oracle/)")


def cpu_baseline(d, budget_s=15.0):
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    impl = reference_cpu_impl()
    kind, what = cpu_kind(impl)
    cpu_time_slices(d, 1, impl)  # warm-up (thread pool, allocator)
    done, spent = 0, 0.0
    while spent < budget_s and done < B * H:
        spent += cpu_time_slices(d, 1, impl)
        done += 1
    return {"value": train_flops(1, done, L, d) / spent / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
            "kind": kind,
            "sample": f"{done} of {B * H} (batch, head) slices of the workload, fwd+bwd, {what}, {spent:.1f} s"}


def run_reference(args):
    """The reference's CPU implementation of the path on the host cores: its own `parallax_reference`
    from baseline/_ref when present, else the oracle port."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    d = args.head_dim
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    impl = reference_cpu_impl()
    kind, what = cpu_kind(impl)
    slices_per_step = 2
    for _ in range(args.warmup):
        cpu_time_slices(d, slices_per_step, impl)
    times = [cpu_time_slices(d, slices_per_step, impl) for _ in range(args.steps)]
    total = sum(times)
    value = train_flops(1, slices_per_step, L, d) * args.steps / total / 1e12
    sample = (f"each step = fwd+bwd of {slices_per_step} of the {B * H} (batch, head) slices of the workload; {what}. "
              "(The reference's GPU kernels are Triton sources; their B200 timings are in BASELINE.md.)")
    print(json.dumps({
        "impl": "reference", "metric": "train_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(d), "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


# --------------------------------------------------------------------------- #
# parity helpers: every context number carries how far it is from the CPU oracle
# --------------------------------------------------------------------------- #
def _err(got, ref):
    from oracle import parallax_oracle as orc

    e = orc.error_metrics(got.float().cpu(), ref)
    return {"rel_l2": float(f"{e['rel_l2']:.3g}"), "max_rel": float(f"{e['max_rel']:.3g}")}


def _worst(errs):
    return {"rel_l2": max(e["rel_l2"] for e in errs.values()), "max_rel": max(e["max_rel"] for e in errs.values()),
            "tensors": sorted(errs)}


def train_slice_parity(q, r, k, v, o, go, grads, b, h):
    """o, dq, dr, dk, dv of (batch b, head h) against the CPU oracle (fp32, same bf16-rounded inputs)."""
    from oracle import parallax_oracle as orc

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    cq, cr, ck, cv = [x[b:b + 1, h:h + 1].cpu() for x in (q, r, k, v)]
    ref_o = orc.train_forward(cq, cr, ck, cv)["o"]
    ref_g = orc.train_backward(cq, cr, ck, cv, go[b:b + 1, h:h + 1].float().cpu())
    errs = {"o": _err(o[b:b + 1, h:h + 1], ref_o)}
    for name, got, ref in zip(("dq", "dr", "dk", "dv"), grads, ref_g):
        errs[name] = _err(got[b:b + 1, h:h + 1], ref)
    return _worst(errs)


# --------------------------------------------------------------------------- #
# one dense training configuration, device-resident, per-kernel events
# --------------------------------------------------------------------------- #
KERNELS = ("fwd", "loss", "bwd_stats", "bwd_dqr", "bwd_dkv")
ALGO_MATMULS = {"fwd": 4, "bwd_dqr": 2, "bwd_dkv": 6}


def timed_train(device, bsz, heads, length, d, steps, warmup, seed, parity_at=None, sync=None, on_timed=None):
    """`steps` timed fwd+bwd steps of (bsz, heads, length, d) after `warmup`; returns the total time of the
    timed region (ms), mean per-kernel ms, the kernel launches counted, and (optionally) the parity of one
    (batch, head) slice against the oracle.  `sync` brackets the timed region (barrier + synchronize)."""
    from parallax_b200 import _cabi, ops

    g = torch.Generator(device=device).manual_seed(seed)
    mk = lambda: torch.randn(bsz, heads, length, d, device=device, generator=g, dtype=torch.float32).to(torch.bfloat16)
    q, r, k, v = mk(), mk(), mk(), mk()
    dq, dr, dk, dv = (torch.empty_like(x) for x in (q, r, k, v))
    scale = d ** -0.5
    n_steps = warmup + steps
    kev = [[torch.cuda.Event(enable_timing=True) for _ in range(6)] for _ in range(n_steps)]
    keep = {}

    def step(i):
        e = kev[i]
        e[0].record()
        o, barv, d1, bart, m = ops.train_fwd(q, r, k, v, scale, -1, ops.BHLD, None)
        e[1].record()
        # loss = mean(o.float()^2) and its gradient 2 o / N, each as ONE pass over o (fp32 accumulation
        # inside the reduction; the bf16 product rounds exactly like autograd's fp32 product cast to bf16)
        loss = torch.linalg.vector_norm(o, dtype=torch.float32).square() / o.numel()
        go = o * (2.0 / o.numel())                                  # d loss / d o
        ws = ops.train_bwd_workspace(q, k, d1, ops.BHLD, None)
        bwd = lambda st: ops.train_bwd_stages(st, q, r, k, v, o, barv, d1, bart, m, go, dq, dr, dk, dv, ws, scale, -1,
                                              ops.BHLD, None)
        e[2].record()
        bwd(ops.BWD_STATS)
        e[3].record()
        bwd(ops.BWD_DQR)
        e[4].record()
        bwd(ops.BWD_DKV)
        e[5].record()
        keep["o"], keep["go"], keep["loss"] = o, go, loss

    for i in range(warmup):
        step(i)
    (sync or torch.cuda.synchronize)()
    if on_timed:
        on_timed(True)
    launches0 = _cabi.launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(warmup, n_steps):
        step(i)
    t1.record()
    (sync or torch.cuda.synchronize)()
    if on_timed:
        on_timed(False)
    out = {"ms_total": t0.elapsed_time(t1), "launches": _cabi.launch_count() - launches0,
           "kernel_ms": {name: statistics.mean(kev[i][j].elapsed_time(kev[i][j + 1]) for i in range(warmup, n_steps))
                         for j, name in enumerate(KERNELS)},
           "input_mb": q.numel() * 2 // 2 ** 20}
    if parity_at is not None:
        out["parity"] = train_slice_parity(q, r, k, v, keep["o"], keep["go"], (dq, dr, dk, dv), *parity_at)
    return out


def kernel_fracs(kernel_ms, flops, peaks):
    """Per tensor kernel: achieved algorithmic TFLOP/s and its fraction of the burst and sustained peaks."""
    unit = flops / 12.0
    out = {}
    for name, n in ALGO_MATMULS.items():
        tf = n * unit / (kernel_ms[name] * 1e-3) / 1e12
        out[name] = {"ms": round(kernel_ms[name], 4), "tflops": round(tf, 1), "frac_burst": round(tf / peaks["burst"], 4),
                     "frac_sustained": round(tf / peaks["sustained"], 4)}
    return out


def train_context_point(device, bsz, heads, length, d, steps, seed, peaks, parity_at=(0, 0)):
    """A training configuration reported as context: ms per step, TFLOP/s, per-kernel fractions, parity."""
    res = timed_train(device, bsz, heads, length, d, steps, 3, seed, parity_at)
    ms = res["ms_total"] / steps
    flops = train_flops(bsz, heads, length, d)
    tf = flops / ms / 1e9
    return {"shape": {"B": bsz, "H": heads, "L": length, "D": d}, "ms_per_step": round(ms, 4), "tflops": round(tf, 1),
            "frac_burst": round(tf / peaks["burst"], 4), "frac_sustained": round(tf / peaks["sustained"], 4),
            "kernels": kernel_fracs(res["kernel_ms"], flops, peaks), "parity_vs_oracle": res.get("parity")}


# --------------------------------------------------------------------------- #
# decode sweep (N = 1)
# --------------------------------------------------------------------------- #
# The reference's published decode table: q50 microseconds of its CuTeDSL kernel on one H200 SXM, H=8,
# D=128, bf16, CUDA-graph replay (README.md:137-153 of the reference), keyed by (B, kv_len).
REFERENCE_H200_US = {(1, 512): 5.79, (1, 1024): 6.48, (1, 4096): 8.61, (1, 16384): 21.53,
                     (32, 512): 24.02, (32, 1024): 39.55, (32, 4096): 279.96, (32, 16384): 1094.37}


def decode_sweep(device):
    """B x kv_len sweep of `parallax_decode` (H=8, D=128, bf16): median microseconds per
    launch and algorithmic HBM GB/s (K and V once).  Timed by CUDA-graph replay of 20
    launches (the reference's method, scripts/bench_decode.py:139-178) that rotate over
    enough distinct K/V sets to exceed the L2, so every launch reads from HBM.  The grid is
    B in {1, 4, 16, 64} x kv_len in {1024, 4096, 32768} plus the sliding-window case, the (B, kv_len)
    cells of the reference's published table (each with its H200 figure beside it, and a second
    timing that replays one K/V set as the reference's protocol does), and two grouped-query shapes.  The largest shape is also checked against the CPU oracle."""
    import parallax_b200 as plx
    from oracle import parallax_oracle as orc

    d, iters = 128, 20
    rows = []
    gen = torch.Generator(device=device).manual_seed(1004)
    mk = lambda *s: torch.randn(*s, device=device, generator=gen, dtype=torch.float32).to(torch.bfloat16)
    grid = [(bsz, t, -1, 8, 8) for bsz in (1, 4, 16, 64) for t in (1024, 4096, 32768)]
    grid.append((64, 32768, 4096, 8, 8))
    grid += [(bsz, t, -1, 8, 8) for bsz in (1, 32) for t in (512, 1024, 4096, 16384) if (bsz, t, -1, 8, 8) not in grid]
    grid += [(16, 8192, -1, 32, 8), (64, 8192, -1, 32, 8)]
    for bsz, kv_len, window, heads_q, heads in grid:
        per_set = 2 * bsz * kv_len * heads * d * 2
        n_sets = 1 if per_set >= 512e6 else min(iters, int(512e6 // per_set) + 1)
        q, r = mk(bsz, 1, heads_q, d), mk(bsz, 1, heads_q, d)
        ks = [mk(bsz, kv_len, heads, d) for _ in range(n_sets)]
        vs = [mk(bsz, kv_len, heads, d) for _ in range(n_sets)]
        out = torch.empty_like(q)

        def replay_us(n_rot):
            side = torch.cuda.Stream(device=device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                for i in range(3):
                    plx.parallax_decode(q, r, ks[i % n_rot], vs[i % n_rot], window_size_left=window, out=out)
            torch.cuda.current_stream(device).wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(iters):
                    plx.parallax_decode(q, r, ks[i % n_rot], vs[i % n_rot], window_size_left=window, out=out)
            times = []
            for _ in range(5):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                graph.replay()
                b.record()
                torch.cuda.synchronize()
                times.append(a.elapsed_time(b) / iters * 1e3)
            return statistics.median(times[1:])

        us = replay_us(n_sets)
        t_eff = kv_len if window < 0 else min(kv_len, window)
        nbytes = 2.0 * bsz * t_eff * heads * d * 2
        row = {"B": bsz, "kv_len": kv_len, "window": window, "heads_q": heads_q, "heads_kv": heads, "us": round(us, 2),
               "hbm_gbs": round(nbytes / us / 1e3, 1), "kv_sets_rotated": n_sets}
        if window < 0 and heads_q == 8 and (bsz, kv_len) in REFERENCE_H200_US:
            row["reference_h200_us"] = REFERENCE_H200_US[(bsz, kv_len)]
            if n_sets > 1:
                # the reference's own protocol replays ONE K/V set (scripts/bench_decode.py:139-178, the default
                # "warm" path), which the L2 then holds for the small shapes: the like-for-like figure
                row["us_same_kv_every_launch"] = round(replay_us(1), 2)
        if (bsz, kv_len, window) == (64, 32768, -1):
            # the last launch of the graph read set (iters - 1) % n_sets: batch row 63, all heads, against the oracle
            j = (iters - 1) % n_sets
            ref = orc.decode(q[63:].cpu(), r[63:].cpu(), ks[j][63:].cpu(), vs[j][63:].cpu())
            row["parity_vs_oracle"] = _err(out[63:], ref)
        rows.append(row)
        del ks, vs
        torch.cuda.empty_cache()
    return rows


def packed_lengths(kind, total=65536):
    """Sequence lengths of the packed benchmark points."""
    if kind == "cfg3":       # uniform on [64, 8192] from seed 0, the last one truncated: 14 sequences
        raw = torch.randint(64, 8193, (64,), generator=torch.Generator().manual_seed(0)).tolist()
        lens, acc = [], 0
        for n in raw:
            n = min(n, total - acc)
            lens.append(n)
            acc += n
            if acc == total:
                break
        return lens
    if kind == "1024_short":  # 1024 sequences of 1..256 tokens, skewed to short (mean 64)
        g = torch.Generator().manual_seed(5)
        lens = (1 + (255 * torch.rand(1024, generator=g) ** 3).long()).tolist()
        excess, i = sum(lens) - total, 0
        while excess != 0:
            step = max(-min(8, 256 - lens[i]), min(lens[i] - 1, excess, 8))
            lens[i] -= step
            excess -= step
            i = (i + 1) % 1024
        return lens
    return [total]            # one sequence


def varlen_point(device, kind="cfg3", heads=16, rank=0, steps=5, parity=True, sync=None):
    """Packed variable-length training (65536 tokens, D=128): fwd+bwd time and algorithmic TFLOP/s
    (12 H D sum len (len + 1)) of `heads` heads, and the shortest sequence (one head) against the oracle."""
    from oracle import parallax_oracle as orc
    from parallax_b200 import ops

    d, total = 128, 65536
    lens = packed_lengths(kind, total)
    cu_list = [0]
    for n in lens:
        cu_list.append(cu_list[-1] + n)
    cu = torch.tensor(cu_list, dtype=torch.int32, device=device)
    gen = torch.Generator(device=device).manual_seed(1003 + 17 * rank)
    mk = lambda h: torch.randn(1, total, h, d, device=device, generator=gen, dtype=torch.float32).to(torch.bfloat16)
    q, r, k, v, go = mk(heads), mk(heads), mk(heads), mk(heads), mk(heads)
    scale = d ** -0.5

    def step():
        f = ops.train_fwd(q, r, k, v, scale, -1, ops.BTHD, cu)
        return f, ops.train_bwd(q, r, k, v, *f, go, scale, -1, ops.BTHD, cu)

    for _ in range(4):
        f, grads = step()      # held across the next call, as in the timed loop: the allocator ends up with both sets of buffers
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    (sync or torch.cuda.synchronize)()
    a.record()
    for _ in range(steps):
        f, grads = step()
    b.record()
    (sync or torch.cuda.synchronize)()
    ms = a.elapsed_time(b) / steps
    flops = 12.0 * heads * d * sum(n * (n + 1) for n in lens)
    out = {"tokens": total, "sequences": len(lens), "heads": heads, "head_dim": d, "ms_fwd_bwd": ms, "flops": flops}
    if parity:
        # a sequence of at most 2048 tokens (the shortest one above 64, else a prefix would not be a sequence)
        torch.set_num_threads(max(1, os.cpu_count() or 1))
        cand = [i for i, n in enumerate(lens) if 64 <= n <= 2048]
        if cand:
            i = min(cand, key=lambda j: lens[j])
            sl = slice(cu_list[i], cu_list[i + 1])
            cq, cr, ck, cv, cg = [x[:, sl, :1].cpu() for x in (q, r, k, v, go)]
            ref_o = orc.varlen_forward(cq, cr, ck, cv, None)["o"]
            ref_g = orc.varlen_backward(cq, cr, ck, cv, cg.float(), None)
            errs = {"o": _err(f[0][:, sl, :1], ref_o)}
            for name, got, ref in zip(("dq", "dr", "dk", "dv"), grads, ref_g):
                errs[name] = _err(got[:, sl, :1], ref)
            out["parity_vs_oracle"] = dict(_worst(errs), sequence_len=lens[i])
        else:      # one long sequence: causality makes its first 1024 tokens a sequence of their own (forward only)
            cq, cr, ck, cv = [x[:, :1024, :1].cpu() for x in (q, r, k, v)]
            out["parity_vs_oracle"] = dict(_err(f[0][:, :1024, :1], orc.varlen_forward(cq, cr, ck, cv, None)["o"]),
                                           tensors=["o"], sequence_len=1024)
    return out


# --------------------------------------------------------------------------- #
# our arm
# --------------------------------------------------------------------------- #
def peaks():
    """Measured denominators: burst and sustained bf16 tensor TFLOP/s and copy GB/s."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"burst": p.get("bf16_tflops", 1629.9), "sustained": p.get("bf16_tflops_sustained", 1391.7),
                "hbm": p.get("hbm_gbs", 6546.2), "source": "measured (MEASURED_PEAKS.json)"}
    return {"burst": 1590.0, "sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


def ncu_traffic(kernel):
    """DRAM bytes per launch of `kernel` at the benchmark size from the committed ncu capture, or None."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.txt")
    if (B, H, L) != (8, 16, 4096) or not os.path.exists(path):
        return None
    with open(path) as fh:
        for line in fh:
            f = line.split()
            if len(f) == 2 and f[0] == kernel:
                return float(f[1])
    return None


def reference_gpu_record():
    """What the reference's own Triton kernels did on a B200 of this pool (measured once by
    baseline/reference_gpu_probe.py and committed), or None."""
    path = os.path.join(ROOT, "baseline", "reference_gpu_measured.json")
    if not os.path.exists(path):
        return None
    with open(path) as fh:
        return json.load(fh)


def sharded_decode(device, rank, world, total_len, sync, max_over_ranks):
    """Long-context decode with the key axis sharded over the ranks (B=1, H=32, D=128, bf16; rank g holds
    keys [g T/n, (g+1) T/n)).  One step = partial sweep of the local shard + exchange of the per-head
    partial records + merge on every rank; the exchange is timed as an NCCL all-gather followed by the
    merge kernel, as ONE kernel over peer memory, and that step captured in a CUDA graph.  Parity: rank 0
    regenerates every shard, runs the single-GPU kernel on the whole cache and the CPU oracle on one head."""
    import torch.distributed as dist

    import parallax_b200 as plx
    from oracle import parallax_oracle as orc
    from parallax_b200.dist import make_decode_exchange, parallax_decode_kv_sharded

    heads, d = 32, 128
    t_local = total_len // world
    gen = torch.Generator(device=device).manual_seed(1005)            # q, r identical on every rank
    mk = lambda g, *s: torch.randn(*s, device=device, generator=g, dtype=torch.float32).to(torch.bfloat16)
    q, r = mk(gen, 1, 1, heads, d), mk(gen, 1, 1, heads, d)
    shard = lambda g: (mk(g, 1, t_local, heads, d), mk(g, 1, t_local, heads, d))
    k, v = shard(torch.Generator(device=device).manual_seed(2000 + rank))
    step = lambda exchange, fused=True: parallax_decode_kv_sharded(q, r, k, v, kv_offset=rank * t_local,
                                                                   total_len=t_local * world, exchange=exchange, fused=fused)

    def timed(fn, iters=20):
        for _ in range(5):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync()
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return max_over_ranks(a.elapsed_time(b) / iters * 1e3)

    us_nccl = timed(lambda: step(None))
    out = step(None)
    exchange = make_decode_exchange(heads, d, device) if world > 1 else None
    us_fused = us_graph = us_one = None
    if exchange is not None:
        us_fused = timed(lambda: step(exchange, False))          # partial sweep, then exchange + merge in one kernel
        same = bool(torch.equal(step(exchange, False), out))
        one_kernel = exchange.fused_step(q, r, k, v, d ** -0.5, -1, rank * t_local, t_local * world, None, None) is not None
        if one_kernel:
            us_one = timed(lambda: step(exchange))               # the whole step as ONE kernel
            same = same and bool(torch.equal(step(exchange), out))
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            step(exchange)
        torch.cuda.current_stream(device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            captured = step(exchange)
        us_graph = timed(graph.replay)
        same = same and bool(torch.equal(captured, out))
        exchange.check()
    elif world == 1:
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            step(None)
        torch.cuda.current_stream(device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step(None)
        us_graph = timed(graph.replay)
    nbytes = 2.0 * t_local * world * heads * d * 2
    best = min(x for x in (us_nccl, us_fused, us_one, us_graph) if x is not None)
    rec = {"shape": {"B": 1, "H": heads, "D": d, "kv_len_total": t_local * world, "kv_len_per_gpu": t_local}, "n_gpus": world,
           "us": round(best, 2), "us_allgather_then_merge": round(us_nccl, 2),
           "us_peer_memory_exchange": None if us_fused is None else round(us_fused, 2),
           "us_sweep_and_exchange_one_kernel": None if us_one is None else round(us_one, 2),
           "us_graph_replay": None if us_graph is None else round(us_graph, 2),
           "hbm_gbs_aggregate": round(nbytes / best / 1e3, 1), "exchange_bytes_per_rank": heads * (2 * d + 4) * 4,
           "scaling": "strong"}
    if exchange is not None:
        rec["peer_exchange_bit_identical_to_allgather"] = same
    if rank == 0:
        # the whole cache on this GPU (8.6 GB at the full size), from the per-rank seeds
        if world > 1:
            del k, v
            parts = [shard(torch.Generator(device=device).manual_seed(2000 + g)) for g in range(world)]
            k = torch.cat([p[0] for p in parts], dim=1)
            v = torch.cat([p[1] for p in parts], dim=1)
            del parts
        single = plx.parallax_decode(q, r, k, v)
        e = (out.float() - single.float()).abs().max().item() / single.float().abs().max().item()
        rec["max_rel_vs_single_gpu"] = float(f"{e:.3g}")
        torch.set_num_threads(max(1, os.cpu_count() or 1))
        h = 7
        ref = orc.decode(q[:, :, h:h + 1].cpu(), r[:, :, h:h + 1].cpu(), k[:, :, h:h + 1].cpu(), v[:, :, h:h + 1].cpu())
        rec["parity_vs_oracle"] = dict(_err(out[:, :, h:h + 1], ref), head=h)
    return rec


def h2d_ceiling_ms(host, device, sync, max_over_ranks, iters=5):
    """Bare host -> device copy of one step's inputs from pinned memory, every rank at once, no kernels."""
    bufs = [torch.empty_like(x, device=device) for x in host]
    for _ in range(2):
        for dst, src in zip(bufs, host):
            dst.copy_(src, non_blocking=True)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    a.record()
    for _ in range(iters):
        for dst, src in zip(bufs, host):
            dst.copy_(src, non_blocking=True)
    b.record()
    sync()
    return max_over_ranks(a.elapsed_time(b) / iters)


def run_ours(args):
    import torch.distributed as dist

    import parallax_b200 as plx
    from parallax_b200 import _cabi

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the library has no CPU path)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    # One JSON line on stdout, nothing else: libraries (NCCL's version banner, for one) print to file
    # descriptor 1 from native code, so descriptor 1 is pointed at stderr for the whole run and the line
    # is written to the saved descriptor at the end.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    d = args.head_dim
    pk = peaks()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    flops = train_flops(B, H, L, d)

    # ---- device-resident step with per-kernel events ---------------------------------------
    sampler = ClockSampler(local)
    clocks_box = {}

    def on_timed(starting):
        if rank != 0:
            return
        if starting:
            sampler.start()
        else:
            clocks_box["clocks"] = sampler.stop()

    res = timed_train(device, B, H, L, d, args.steps, args.warmup, SEED + rank, parity_at=(0, 0) if rank == 0 else None,
                      sync=sync_all, on_timed=on_timed)
    clocks = clocks_box.get("clocks")
    ms_total = max_over_ranks(res["ms_total"])
    value = world * flops * args.steps / (ms_total * 1e-3) / 1e12
    kms = res["kernel_ms"]
    dom = max(ALGO_MATMULS, key=lambda n: kms[n])
    achieved = ALGO_MATMULS[dom] * flops / 12.0 / (kms[dom] * 1e-3) / 1e12
    # Which peak a run is to be held against depends on the clocks it ran at: a short run stays at the
    # burst clock, a long one settles under the power cap.  Both fractions are printed; `peak` / `frac`
    # follow the sampled clocks (burst when the median SM clock stayed within 3 % of the maximum).
    at_burst = bool(clocks and clocks.get("sm_max_mhz") and clocks["sm_mhz"] >= 0.97 * clocks["sm_max_mhz"])
    peak_tf = pk["burst"] if at_burst else pk["sustained"]
    roofline = {"kernel": dom, "bound": "tensor", "achieved": round(achieved, 2), "peak": peak_tf, "unit": "TFLOP/s",
                "frac": round(achieved / peak_tf, 4), "traffic": ncu_traffic(dom),
                "peak_source": pk["source"] + (": burst (median SM clock at maximum)" if at_burst else ": sustained (clock below maximum)"),
                "frac_of_burst_peak": round(achieved / pk["burst"], 4), "frac_of_sustained_peak": round(achieved / pk["sustained"], 4),
                "kernel_ms": {n: round(kms[n], 4) for n in KERNELS}, "algorithmic_matmuls": ALGO_MATMULS,
                "kernels": kernel_fracs(kms, flops, pk)}

    # ---- end to end through the public API, host buffers ------------------------------------
    # Every step copies its own q, r, k, v from pinned host memory and reads its loss back.  As a
    # training loop's data loader does, the copy of step i + 1 runs on a second stream while step i
    # computes; the loss is read back one step late so that the host never stalls the device.
    g = torch.Generator().manual_seed(SEED + rank)
    host = [torch.randn(B, H, L, d, generator=g, dtype=torch.float32).to(torch.bfloat16).pin_memory() for _ in range(4)]
    copy_stream = torch.cuda.Stream(device=device)

    def upload():
        with torch.cuda.stream(copy_stream):
            bufs = [x.to(device, non_blocking=True) for x in host]
            done = torch.cuda.Event()
            done.record(copy_stream)
        return bufs, done

    def e2e_loop(n):
        pending, losses = upload(), []
        prev = None
        for i in range(n):
            bufs, done = pending
            if i + 1 < n:
                pending = upload()
            torch.cuda.current_stream(device).wait_event(done)
            for x in bufs:
                x.record_stream(torch.cuda.current_stream(device))
            leaves = [x.requires_grad_(True) for x in bufs]
            o = plx.parallax_func(*leaves)
            loss = o.float().pow(2).mean()
            loss.backward()
            host_loss = torch.empty((), dtype=torch.float32, pin_memory=True)
            host_loss.copy_(loss.detach(), non_blocking=True)         # device -> host read of the result
            if prev is not None:
                prev[1].synchronize()
                losses.append(float(prev[0]))
            ev = torch.cuda.Event()
            ev.record()
            prev = (host_loss, ev)
        prev[1].synchronize()
        losses.append(float(prev[0]))
        return losses

    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_loop(args.warmup)
    sync_all()
    t0.record()
    e2e_loop(args.steps)
    t1.record()
    sync_all()
    e2e_ms = max_over_ranks(t0.elapsed_time(t1)) / args.steps
    copy_ms = h2d_ceiling_ms(host, device, sync_all, max_over_ranks)
    step_ms = ms_total / args.steps
    e2e = {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in host), "d2h_bytes_per_step": 4,
           "ms_per_step": e2e_ms,
           # what the host can deliver: the bare copy of one step's inputs on all ranks at once, no kernels.
           # The copy of step i + 1 overlaps the compute of step i, so a step cannot beat max(copy, compute).
           "h2d_ceiling_ms": round(copy_ms, 3), "h2d_gbs_per_gpu": round(sum(x.numel() * 2 for x in host) / copy_ms / 1e6, 1),
           "compute_ms": round(step_ms, 3), "frac_of_max_copy_compute": round(max(copy_ms, step_ms) / e2e_ms, 3)}
    del host

    line = {
        "metric": "train_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(d), "per_gpu": {"B": B, "H": H, "L": L, "D": d}, "sharding": "batch x heads, no collective",
                   "l2": "inputs (4 x %d MB) larger than the 126 MB L2" % res["input_mb"]},
        "pct_of_bf16_peak": round(100.0 * value / world / peak_tf, 2),
        "pct_of_bf16_burst_peak": round(100.0 * value / world / pk["burst"], 2),
        "pct_of_bf16_sustained_peak": round(100.0 * value / world / pk["sustained"], 2),
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(res["launches"]), "roofline": roofline,
        "parity_vs_oracle": res.get("parity"),
    }
    ref_gpu = reference_gpu_record()
    if ref_gpu is not None:
        line["reference_gpu"] = ref_gpu
    torch.cuda.empty_cache()

    if not args.no_context and (B, H, L, d) == (8, 16, 4096, 128):
        # ---- the sharded configurations (every N), strong scaling: total work fixed -----------------
        if 32 % world == 0:
            r5 = timed_train(device, 16, 32 // world, 8192, 128, 3, 3, 1005 + rank, parity_at=(15, 0) if rank == 0 else None,
                             sync=sync_all)
            ms5 = max_over_ranks(r5["ms_total"]) / 3
            tf5 = train_flops(16, 32, 8192, 128) / ms5 / 1e9
            line["sharded_train_5a"] = {"shape": {"B": 16, "H": 32, "L": 8192, "D": 128}, "heads_per_gpu": 32 // world,
                                        "n_gpus": world, "ms_per_step": round(ms5, 3), "tflops": round(tf5, 1),
                                        "tflops_per_gpu": round(tf5 / world, 1), "scaling": "strong", "collective": "none",
                                        "kernel_ms_rank0": {n: round(x, 3) for n, x in r5["kernel_ms"].items()},
                                        "parity_vs_oracle": r5.get("parity")}
            torch.cuda.empty_cache()
        if 16 % world == 0:
            vp = varlen_point(device, "cfg3", 16 // world, rank, steps=3, parity=rank == 0, sync=sync_all)
            msv = max_over_ranks(vp["ms_fwd_bwd"])
            tfv = vp["flops"] * world / msv / 1e9
            line["sharded_varlen"] = {"tokens": vp["tokens"], "sequences": vp["sequences"], "heads": 16, "heads_per_gpu": 16 // world,
                                      "n_gpus": world, "ms_fwd_bwd": round(msv, 3), "tflops": round(tfv, 1),
                                      "frac_burst": round(tfv / world / pk["burst"], 4), "scaling": "strong", "collective": "none",
                                      "parity_vs_oracle": vp.get("parity_vs_oracle")}
            torch.cuda.empty_cache()
        line["sharded_decode_5b"] = sharded_decode(device, rank, world, 524288, sync_all, max_over_ranks)
        torch.cuda.empty_cache()

    if world == 1 and not args.no_context:
        line["cfg1"] = train_context_point(device, 2, 8, 1024, 128, 20, 1001, pk)
        if d == 128 and (B, H, L) == (8, 16, 4096):
            line["d64"] = train_context_point(device, 8, 16, 4096, 64, 20, 1002, pk)
        torch.cuda.empty_cache()
        for key, kind in (("varlen", "cfg3"), ("varlen_1024_sequences", "1024_short"), ("varlen_one_sequence", "one")):
            vp = varlen_point(device, kind)
            tf = vp.pop("flops") / vp["ms_fwd_bwd"] / 1e9
            vp.update(ms_fwd_bwd=round(vp["ms_fwd_bwd"], 3), tflops=round(tf, 1), frac_burst=round(tf / pk["burst"], 4),
                      frac_sustained=round(tf / pk["sustained"], 4))
            line[key] = vp
            torch.cuda.empty_cache()
        line["decode"] = decode_sweep(device)
        big = next(x for x in line["decode"] if (x["B"], x["kv_len"], x["window"]) == (64, 32768, -1))
        line["roofline_decode"] = {"kernel": "decode_kernel", "bound": "hbm", "shape": {"B": 64, "kv_len": 32768, "H": 8, "D": 128},
                                   "bytes": 2 * 64 * 32768 * 8 * 128 * 2, "us": big["us"], "achieved": big["hbm_gbs"],
                                   "peak": pk["hbm"], "unit": "GB/s", "frac": round(big["hbm_gbs"] / pk["hbm"], 4),
                                   "frac_of_nominal_8000": round(big["hbm_gbs"] / 8000.0, 4),
                                   "traffic": ncu_traffic("decode_kernel_B64_T32768")}
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(d)
    if world > 1:
        sync_all()          # rank 0 may still have been checking parity on the CPU
        dist.destroy_process_group()
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    os.close(real_stdout)
    if rank == 0:
        print(json.dumps(line), flush=True)


def run_decode_shape(spec):
    """`--decode-shape B,T[,W[,Hq,Hkv]]`: the decode kernel alone on one shape (H=8 unless given, D=128, bf16),
    plain launches on the current stream; prints one small JSON line.  This is the command the ncu captures
    of decode use."""
    import parallax_b200 as plx

    f = [int(x) for x in spec.split(",")]
    bsz, kv_len, window = f[0], f[1], (f[2] if len(f) > 2 else -1)
    heads_q, heads, d = (f[3] if len(f) > 4 else 8), (f[4] if len(f) > 4 else 8), 128
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(1004)
    mk = lambda *s: torch.randn(*s, device=dev, generator=gen, dtype=torch.float32).to(torch.bfloat16)
    q, r, k, v = mk(bsz, 1, heads_q, d), mk(bsz, 1, heads_q, d), mk(bsz, kv_len, heads, d), mk(bsz, kv_len, heads, d)
    out = torch.empty_like(q)
    for _ in range(5):
        plx.parallax_decode(q, r, k, v, window_size_left=window, out=out)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(10):
        plx.parallax_decode(q, r, k, v, window_size_left=window, out=out)
    b.record()
    torch.cuda.synchronize()
    us = a.elapsed_time(b) / 10 * 1e3
    t_eff = kv_len if window < 0 else min(kv_len, window)
    print(json.dumps({"decode_shape": {"B": bsz, "kv_len": kv_len, "window": window, "H": heads_q, "H_kv": heads, "D": d},
                      "us": round(us, 2), "hbm_gbs": round(2.0 * bsz * t_eff * heads * d * 2 / us / 1e3, 1)}), flush=True)


def run_decode_sharded(total_len):
    """`--decode-sharded T` under torchrun: the KV-sharded decode point alone (see sharded_decode)."""
    import torch.distributed as dist

    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    # one JSON line on stdout, nothing else (see main): descriptor 1 points at stderr until the line is written
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    rec = sharded_decode(dev, rank, world, total_len, sync_all, max_over_ranks)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    os.close(real_stdout)
    if rank == 0:
        print(json.dumps({"decode_sharded": rec}), flush=True)


def main():
    global B, H, L
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--head-dim", type=int, default=128, choices=(64, 128))
    ap.add_argument("--batch", type=int, default=B, help="per-GPU batch (profiling runs use a smaller one)")
    ap.add_argument("--heads", type=int, default=H)
    ap.add_argument("--seq-len", type=int, default=L)
    ap.add_argument("--decode-shape", default=None, help="B,T[,W[,Hq,Hkv]]: time only the decode kernel on this shape")
    ap.add_argument("--decode-sharded", type=int, default=0,
                    help="T: time KV-sharded long-context decode over the launched ranks (B=1, H=32, D=128)")
    ap.add_argument("--no-decode", "--no-context", dest="no_context", action="store_true",
                    help="only the headline workload: no cfg1 / d64 / packed / decode / sharded context points")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    B, H, L = args.batch, args.heads, args.seq_len
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.decode_shape:
        run_decode_shape(args.decode_shape)
    elif args.decode_sharded:
        run_decode_sharded(args.decode_sharded)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
