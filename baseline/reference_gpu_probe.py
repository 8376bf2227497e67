"""One bounded run of the REFERENCE's own Triton kernels on the GPU of this box.

    python baseline/reference_gpu_probe.py [--budget-s 600] [--full-autotune] [--out FILE]

The reference package (Yifei-Zuo/Parallax, installed unmodified under ``baseline/_ref`` by
``pip install --no-deps --target baseline/_ref``) ships arch-generic Triton kernels:
``parallax.triton.parallax_func`` (fwd + bwd, three autotuned kernels with 36 configurations each,
parallax/triton/parallax_train.py:27-45, 1039-1087) and ``parallax.triton.parallax_decode``
(parallax/triton/parallax_decode.py:100-148).  This script times them with CUDA events on the shapes
the benchmark of this repository uses, so that its numbers have an on-box GPU figure beside them.

Bounds: every case runs in a child process with its own wall-clock limit, cases run in order of cost,
and the script stops between cases once the budget is spent.  Unless ``--full-autotune`` is given the
autotuner's search space is cut to six tile/warp/stage configurations per kernel (named in the output);
the kernels themselves are the reference's, untouched.  Nothing of this repository's library is imported.
"""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

# (row tile, column tile, warps, stages) kept when the autotune space is cut
SHORT_LIST = [(128, 64, 8, 2), (128, 128, 8, 2), (64, 64, 4, 2), (64, 128, 8, 2), (128, 64, 4, 2), (64, 32, 4, 2)]


def _import_reference():
    root = os.path.dirname(HERE)
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") not in (root, HERE)]
    sys.path.insert(0, REF)
    import parallax                       # noqa: F401  (the reference, from baseline/_ref)
    assert os.path.abspath(parallax.__file__).startswith(REF), parallax.__file__
    return parallax


def _cut_autotune(full: bool):
    import parallax.triton.parallax_train as pt

    if full:
        return "all 36"
    for kern in (pt._fwd_kernel, pt._bwd_rq_kernel, pt._bwd_kv_kernel):
        keep = [c for c in kern.configs
                if (c.kwargs["ROW_TILE_SIZE"], c.kwargs["COL_TILE_SIZE"], c.num_warps, c.num_stages) in SHORT_LIST]
        kern.configs = keep or kern.configs[:1]
    pre = pt._bwd_preprocess_kernel
    pre.configs = [c for c in pre.configs if c.num_stages == 2 and c.num_warps == 4][:3] or pre.configs[:1]
    return f"{len(SHORT_LIST)} of 36 per kernel: (row, col, warps, stages) in {SHORT_LIST}"


def _time(fn, iters, warm):
    import torch

    for _ in range(warm):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def case_train(bsz, heads, length, d, full, q):
    import torch

    _import_reference()
    space = _cut_autotune(full)
    import parallax.triton as ptr

    g = torch.Generator(device="cuda").manual_seed(1002)
    mk = lambda: torch.randn(bsz, heads, length, d, device="cuda", generator=g, dtype=torch.float32).to(torch.bfloat16)
    leaves = [mk().requires_grad_(True) for _ in range(4)]
    t0 = time.time()

    def step():
        for x in leaves:
            x.grad = None
        o = ptr.parallax_func(*leaves)
        o.float().pow(2).mean().backward()

    step()                                  # compiles and autotunes
    torch.cuda.synchronize()
    tune_s = time.time() - t0
    ms = _time(step, 10, 2)
    with torch.no_grad():
        fwd_ms = _time(lambda: ptr.parallax_func(*leaves), 10, 2)
    flops = 12.0 * bsz * heads * d * length * (length + 1)
    q.put({"ms_fwd_bwd": round(ms, 3), "ms_fwd": round(fwd_ms, 3), "tflops_fwd_bwd": round(flops / ms / 1e9, 1),
           "autotune_space": space, "first_call_s": round(tune_s, 1)})


def case_decode(bsz, kv_len, heads, d, q):
    import torch

    _import_reference()
    import parallax.triton as ptr

    g = torch.Generator(device="cuda").manual_seed(1004)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g, dtype=torch.float32).to(torch.bfloat16)
    per_set = 2 * bsz * kv_len * heads * d * 2
    n_sets = 1 if per_set >= 512e6 else min(20, int(512e6 // per_set) + 1)
    qq, rr = mk(bsz, 1, heads, d), mk(bsz, 1, heads, d)
    ks = [mk(bsz, kv_len, heads, d) for _ in range(n_sets)]
    vs = [mk(bsz, kv_len, heads, d) for _ in range(n_sets)]
    i = [0]

    def step():
        ptr.parallax_decode(qq, rr, ks[i[0] % n_sets], vs[i[0] % n_sets])
        i[0] += 1

    us = _time(step, 40, 5) * 1e3
    q.put({"us": round(us, 2), "hbm_gbs": round(per_set / us / 1e3, 1), "kv_sets_rotated": n_sets,
           "timing": "plain launches, CUDA events (includes the Python launch overhead of the Triton wrapper)"})


CASES = [
    ("decode_B64_T32768_H8_D128", case_decode, (64, 32768, 8, 128), 120),
    ("decode_B1_T4096_H8_D128", case_decode, (1, 4096, 8, 128), 120),
    ("train_B8_H16_L4096_D128", case_train, (8, 16, 4096, 128), 900),
    ("train_B2_H8_L1024_D128", case_train, (2, 8, 1024, 128), 600),
    ("train_B8_H16_L4096_D64", case_train, (8, 16, 4096, 64), 600),
]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--budget-s", type=float, default=600.0)
    ap.add_argument("--full-autotune", action="store_true")
    ap.add_argument("--out", default=os.path.join(HERE, "reference_gpu_probe_run.json"),
                    help="where the record of this run goes (the committed record is reference_gpu_measured.json)")
    args = ap.parse_args()
    os.environ.setdefault("TRITON_CACHE_DIR", "/tmp/triton_cache_reference_probe")
    mp.set_start_method("spawn")
    t_start, results = time.time(), {}
    for name, fn, shape, limit in CASES:
        left = args.budget_s - (time.time() - t_start)
        if left < 30:
            results[name] = {"skipped": "wall-clock budget spent"}
            continue
        q = mp.Queue()
        extra = (args.full_autotune, q) if fn is case_train else (q,)
        p = mp.Process(target=fn, args=(*shape, *extra))
        t0 = time.time()
        p.start()
        p.join(min(limit, left))
        if p.is_alive():
            p.terminate()                  # this exact child only
            p.join(30)
            results[name] = {"stopped": f"still running after {time.time() - t0:.0f} s (compile / autotune); no number"}
        elif p.exitcode != 0:
            results[name] = {"failed": f"child exited with code {p.exitcode} after {time.time() - t0:.0f} s (see stderr)"}
        else:
            try:
                results[name] = q.get(timeout=5)
            except Exception as exc:       # noqa: BLE001
                results[name] = {"failed": f"no result: {exc!r}"}
        results[name]["wall_s"] = round(time.time() - t0, 1)
        print(name, json.dumps(results[name]), flush=True)
    import torch
    import triton

    doc = {"what": "the reference's Triton kernels, timed on this box", "torch": torch.__version__, "triton": triton.__version__,
           "gpu": torch.cuda.get_device_name(0), "cases": results}
    os.makedirs(os.path.dirname(args.out), exist_ok=True)
    with open(args.out, "w") as fh:
        json.dump(doc, fh, indent=1)
    print(json.dumps(doc))


if __name__ == "__main__":
    main()
