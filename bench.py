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
             host memory and the loss read back, every step
  roofline   the dominant kernel against the measured bf16 tensor peak
  cpu_baseline  the CPU oracle (a PyTorch restatement of the reference's fp32
             implementation) timed on this host's cores on a bounded sample
  varlen     (N = 1 only) fwd+bwd of the packed 65536-token configuration
  decode     (N = 1 only) HBM GB/s and microseconds of the decode sweep

`--impl reference` times that CPU implementation alone (the reference has no
kernel that runs on B200 without its Triton/Helion/CuTeDSL JIT stack).
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


def cpu_time_slices(d, n_slices):
    """fwd + bwd of `n_slices` (batch, head) slices of the workload through the CPU oracle; returns seconds."""
    from oracle import parallax_oracle as orc

    q, r, k, v = cpu_slice_inputs(d, n_slices)
    t0 = time.perf_counter()
    f = orc.train_forward(q, r, k, v)
    go = orc.mse_loss_grad(f["o"]) * (1.0 / (B * H / n_slices))
    orc.train_backward(q, r, k, v, go)
    return time.perf_counter() - t0


def cpu_baseline(d, budget_s=15.0):
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    cpu_time_slices(d, 1)  # warm-up (thread pool, allocator)
    done, spent = 0, 0.0
    while spent < budget_s and done < B * H:
        spent += cpu_time_slices(d, 1)
        done += 1
    return {"value": train_flops(1, done, L, d) / spent / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
            "kind": "port",
            "sample": f"{done} of {B * H} (batch, head) slices of the workload, fwd+bwd, fp32 PyTorch on CPU, "
                      f"{spent:.1f} s"}


def run_reference(args):
    """The reference's CPU implementation of the path (via the oracle port) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    d = args.head_dim
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    slices_per_step = 2
    for _ in range(args.warmup):
        cpu_time_slices(d, slices_per_step)
    times = [cpu_time_slices(d, slices_per_step) for _ in range(args.steps)]
    total = sum(times)
    value = train_flops(1, slices_per_step, L, d) * args.steps / total / 1e12
    sample = (f"each step = fwd+bwd of {slices_per_step} of the {B * H} (batch, head) slices of the workload; "
              "fp32 PyTorch restatement of parallax/reference.py (the reference's Triton/Helion/CuTeDSL kernels "
              "have no build for this box)")
    print(json.dumps({
        "impl": "reference", "metric": "train_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(d), "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


# --------------------------------------------------------------------------- #
# decode sweep (N = 1)
# --------------------------------------------------------------------------- #
def decode_sweep(device):
    """B x kv_len sweep of `parallax_decode` (H=8, D=128, bf16): median microseconds per
    launch and algorithmic HBM GB/s (K and V once).  Timed by CUDA-graph replay of 20
    launches (the reference's method, scripts/bench_decode.py:139-178) that rotate over
    enough distinct K/V sets to exceed the L2, so every launch reads from HBM."""
    import parallax_b200 as plx

    d, iters = 128, 20
    rows = []
    gen = torch.Generator(device=device).manual_seed(1004)
    mk = lambda *s: torch.randn(*s, device=device, generator=gen, dtype=torch.float32).to(torch.bfloat16)
    # (B, kv_len, window, q heads, kv heads): the H=8 grid of the baseline, then two grouped-query shapes
    for bsz, kv_len, window, heads_q, heads in ((1, 1024, -1, 8, 8), (1, 4096, -1, 8, 8), (1, 32768, -1, 8, 8), (4, 4096, -1, 8, 8),
                                                (16, 4096, -1, 8, 8), (16, 32768, -1, 8, 8), (64, 1024, -1, 8, 8),
                                                (64, 4096, -1, 8, 8), (64, 32768, -1, 8, 8), (64, 32768, 4096, 8, 8),
                                                (16, 8192, -1, 32, 8), (64, 8192, -1, 32, 8)):
        per_set = 2 * bsz * kv_len * heads * d * 2
        n_sets = 1 if per_set >= 512e6 else min(iters, int(512e6 // per_set) + 1)
        q, r = mk(bsz, 1, heads_q, d), mk(bsz, 1, heads_q, d)
        ks = [mk(bsz, kv_len, heads, d) for _ in range(n_sets)]
        vs = [mk(bsz, kv_len, heads, d) for _ in range(n_sets)]
        out = torch.empty_like(q)
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for i in range(3):
                plx.parallax_decode(q, r, ks[i % n_sets], vs[i % n_sets], window_size_left=window, out=out)
        torch.cuda.current_stream(device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(iters):
                plx.parallax_decode(q, r, ks[i % n_sets], vs[i % n_sets], window_size_left=window, out=out)
        times = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) / iters * 1e3)
        us = statistics.median(times[1:])
        t_eff = kv_len if window < 0 else min(kv_len, window)
        nbytes = 2.0 * bsz * t_eff * heads * d * 2
        rows.append({"B": bsz, "kv_len": kv_len, "window": window, "heads_q": heads_q, "heads_kv": heads, "us": round(us, 2),
                     "hbm_gbs": round(nbytes / us / 1e3, 1), "kv_sets_rotated": n_sets})
        del graph, ks, vs
        torch.cuda.empty_cache()
    return rows


def varlen_point(device):
    """Packed variable-length training (65536 tokens, H=16, D=128, lengths uniform on [64, 8192] from
    seed 0, the last one truncated): fwd+bwd time and algorithmic TFLOP/s (12 H D sum len (len + 1))."""
    from parallax_b200 import ops

    heads, d, total = 16, 128, 65536
    raw = torch.randint(64, 8193, (64,), generator=torch.Generator().manual_seed(0)).tolist()
    lens, acc = [], 0
    for n in raw:
        n = min(n, total - acc)
        lens.append(n)
        acc += n
        if acc == total:
            break
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=device)
    gen = torch.Generator(device=device).manual_seed(1003)
    mk = lambda h: torch.randn(1, total, h, d, device=device, generator=gen, dtype=torch.float32).to(torch.bfloat16)
    q, r, k, v, go = mk(heads), mk(heads), mk(heads), mk(heads), mk(heads)
    scale = d ** -0.5

    def step():
        f = ops.train_fwd(q, r, k, v, scale, -1, ops.BTHD, cu)
        return ops.train_bwd(q, r, k, v, *f, go, scale, -1, ops.BTHD, cu)

    for _ in range(3):
        step()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(5):
        step()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 5
    flops = 12.0 * heads * d * sum(n * (n + 1) for n in lens)
    return {"tokens": total, "sequences": len(lens), "heads": heads, "head_dim": d, "ms_fwd_bwd": round(ms, 3),
            "tflops": round(flops / ms / 1e9, 1)}


# --------------------------------------------------------------------------- #
# our arm
# --------------------------------------------------------------------------- #
def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return p.get("bf16_tflops_sustained", 1391.7), p.get("hbm_gbs", 6546.2), "measured (sustained, MEASURED_PEAKS.json)"
    return 1400.0, 6650.0, "fallback"


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


def run_ours(args):
    import torch.distributed as dist

    import parallax_b200 as plx
    from parallax_b200 import _cabi, ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the library has no CPU path)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"          # keep NCCL's version banner off stdout (one JSON line only)
        dist.init_process_group("nccl", device_id=device)
    d = args.head_dim

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

    # host inputs (pinned), one per-GPU shard of the weak-scaled job
    g = torch.Generator().manual_seed(SEED + rank)
    host = [torch.randn(B, H, L, d, generator=g, dtype=torch.float32).to(torch.bfloat16).pin_memory() for _ in range(4)]
    dev = [x.to(device, non_blocking=True) for x in host]
    torch.cuda.synchronize()
    scale = d ** -0.5
    flops = train_flops(B, H, L, d)

    # ---- device-resident step with per-kernel events ---------------------------------------
    q, r, k, v = dev
    dq, dr, dk, dv = (torch.empty_like(x) for x in dev)
    n_steps = args.warmup + args.steps
    names = ("fwd", "loss", "bwd_stats", "bwd_dqr", "bwd_dkv")
    kev = [[torch.cuda.Event(enable_timing=True) for _ in range(6)] for _ in range(n_steps)]

    def resident_step(i):
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
        return loss

    for i in range(args.warmup):
        resident_step(i)
    sampler = ClockSampler(local)
    sync_all()
    if rank == 0:
        sampler.start()
    launches0 = _cabi.launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(args.warmup, n_steps):
        resident_step(i)
    t1.record()
    sync_all()
    clocks = sampler.stop() if rank == 0 else None
    launches = _cabi.launch_count() - launches0
    ms_total = max_over_ranks(t0.elapsed_time(t1))
    value = world * flops * args.steps / (ms_total * 1e-3) / 1e12

    # per-kernel mean durations over the timed steps ("loss" = the torch kernels of the loss and its gradient)
    kms = {name: statistics.mean(kev[i][j].elapsed_time(kev[i][j + 1]) for i in range(args.warmup, n_steps))
           for j, name in enumerate(names)}
    unit_flops = flops / 12.0                      # one causal matmul over the whole batch
    algo = {"fwd": 4 * unit_flops, "bwd_dqr": 2 * unit_flops, "bwd_dkv": 6 * unit_flops}
    dom = max(("fwd", "bwd_dqr", "bwd_dkv"), key=lambda n: kms[n])
    peak_tf, peak_hbm, peak_src = peaks()
    achieved = algo[dom] / (kms[dom] * 1e-3) / 1e12
    roofline = {"kernel": dom, "bound": "tensor", "achieved": round(achieved, 2), "peak": peak_tf, "unit": "TFLOP/s",
                "frac": round(achieved / peak_tf, 4), "traffic": ncu_traffic(dom), "peak_source": peak_src,
                "kernel_ms": {n: round(kms[n], 4) for n in names},
                "algorithmic_matmuls": {"fwd": 4, "bwd_dqr": 2, "bwd_dkv": 6}}

    # ---- end to end through the public API, host buffers ------------------------------------
    # Every step copies its own q, r, k, v from pinned host memory and reads its loss back.  As a
    # training loop's data loader does, the copy of step i + 1 runs on a second stream while step i
    # computes; the loss is read back one step late so that the host never stalls the device.
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

    e2e_loop(args.warmup)
    sync_all()
    t0.record()
    e2e_loop(args.steps)
    t1.record()
    sync_all()
    e2e_ms = max_over_ranks(t0.elapsed_time(t1))
    e2e = {"value": world * flops * args.steps / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in host), "d2h_bytes_per_step": 4,
           "ms_per_step": e2e_ms / args.steps}

    line = {
        "metric": "train_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(d), "per_gpu": {"B": B, "H": H, "L": L, "D": d}, "sharding": "batch x heads, no collective",
                   "l2": "inputs (4 x %d MB) larger than the 126 MB L2" % (host[0].numel() * 2 // 2 ** 20)},
        "pct_of_bf16_peak": round(100.0 * value / world / peak_tf, 2),
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline,
    }
    if world == 1:
        del dev, q, r, k, v, dq, dr, dk, dv
        torch.cuda.empty_cache()
        if not args.no_decode:
            line["varlen"] = varlen_point(device)
            line["decode"] = decode_sweep(device)
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(d)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
    """`--decode-sharded T` under torchrun: long-context decode with the key axis sharded over the ranks
    (B=1, H=32, D=128, bf16; rank g holds keys [g T/n, (g+1) T/n)).  One step = partial sweep of the local
    shard + one NCCL all-gather of the per-head partial records + merge on every rank.  Prints one small
    JSON line on rank 0: microseconds per step (max over ranks) and aggregate K/V bytes per second."""
    import torch.distributed as dist

    from parallax_b200.dist import make_decode_exchange, parallax_decode_kv_sharded

    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"          # keep NCCL's version banner off stdout
        dist.init_process_group("nccl", device_id=dev)
    heads, d = 32, 128
    t_local = total_len // world
    gen = torch.Generator(device=dev).manual_seed(1005)            # q, r identical on every rank
    mk = lambda g, *s: torch.randn(*s, device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    q, r = mk(gen, 1, 1, heads, d), mk(gen, 1, 1, heads, d)
    gen_kv = torch.Generator(device=dev).manual_seed(2000 + rank)
    k, v = mk(gen_kv, 1, t_local, heads, d), mk(gen_kv, 1, t_local, heads, d)
    def timed(exchange):
        step = lambda: parallax_decode_kv_sharded(q, r, k, v, kv_offset=rank * t_local, total_len=t_local * world,
                                                  exchange=exchange)
        for _ in range(5):
            step()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a.record()
        for _ in range(20):
            step()
        b.record()
        torch.cuda.synchronize()
        us = torch.tensor([a.elapsed_time(b) / 20 * 1e3], device=dev)
        if world > 1:
            dist.all_reduce(us, op=dist.ReduceOp.MAX)
        return float(us)

    # the exchange of the partial records: NCCL all-gather + merge kernel, and one kernel over peer memory
    us_nccl = timed(None)
    exchange = make_decode_exchange(heads, d, dev) if world > 1 else None
    us_fused = timed(exchange) if exchange is not None else None
    us_graph = None
    if exchange is not None:
        # the same step captured once and replayed (the exchange keeps its step count on the device)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            parallax_decode_kv_sharded(q, r, k, v, kv_offset=rank * t_local, total_len=t_local * world, exchange=exchange)
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            parallax_decode_kv_sharded(q, r, k, v, kv_offset=rank * t_local, total_len=t_local * world, exchange=exchange)
        for _ in range(3):
            graph.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        dist.barrier()
        a.record()
        for _ in range(20):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / 20 * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us_graph = float(t)
    if rank == 0:
        nbytes = 2.0 * t_local * world * heads * d * 2
        best = min(x for x in (us_nccl, us_fused, us_graph) if x is not None)
        print(json.dumps({"decode_sharded": {"B": 1, "H": heads, "D": d, "kv_len_total": t_local * world, "n_gpus": world},
                          "us": round(best, 2), "us_allgather_then_merge": round(us_nccl, 2),
                          "us_peer_memory_exchange": None if us_fused is None else round(us_fused, 2),
                          "us_peer_memory_exchange_graph_replay": None if us_graph is None else round(us_graph, 2),
                          "hbm_gbs_aggregate": round(nbytes / best / 1e3, 1),
                          "exchange_bytes_per_rank": heads * (2 * d + 4) * 4}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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
    ap.add_argument("--no-decode", action="store_true")
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
