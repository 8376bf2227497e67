"""Generate the golden vectors under ``tests/golden/`` from the REFERENCE itself.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/Parallax

It loads the reference's fp32 implementation (``parallax/reference.py``) straight
from that checkout, runs it (forward, and torch autograd for the gradients) on
small seeded inputs, and stores inputs (raw bf16 bit patterns) and fp32 outputs
in ``tests/golden/*.npz``.  The tests only read the ``.npz`` files, never the
reference checkout.

Case lists follow the reference's own sweeps: MHA / GQA / MQA / sliding window
for training (``scripts/parity_train.py:39-50``), pinned edge lengths for packed
sequences (``scripts/parity_varlen.py:39-45``), and sliding window, left padding
(``cache_start``) and runtime lengths (``seqused_k``) for decode
(``scripts/test_decode_triton.py:75-103``, ``tests/test_decode_parity.py:162-177``).
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root):
    spec = importlib.util.spec_from_file_location("_plx_reference", os.path.join(root, "parallax", "reference.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.parallax_reference


def bf16_randn(shape, gen, mul=1.0):
    return (torch.randn(shape, generator=gen, dtype=torch.float32) * mul).to(torch.bfloat16)


def bits(x):
    return x.view(torch.int16).numpy().copy()


# (name, B, Hq, Hkv, L, D, window_left)
TRAIN_CASES = [
    ("mha_d64", 1, 2, 2, 96, 64, -1),
    ("mha_d128", 1, 2, 2, 80, 128, -1),
    ("gqa_d64", 1, 4, 2, 70, 64, -1),
    ("mqa_d128", 1, 3, 1, 65, 128, -1),
    ("swa_d64", 1, 2, 2, 100, 64, 24),
    ("gqa_swa_d128", 1, 2, 1, 72, 128, 16),
    ("single_row", 1, 1, 1, 1, 64, -1),
]

# (name, lens, Hq, Hkv, D, window_left)
VARLEN_CASES = [
    ("packed_d64", [1, 37, 64, 30], 2, 2, 64, -1),
    ("packed_gqa_d128", [1, 65, 20], 2, 1, 128, -1),
    ("packed_swa_d64", [50, 3, 41], 2, 1, 64, 17),
]

# (name, B, Hq, Hkv, T, D, window_left, cache_start, seqused_k)
DECODE_CASES = [
    ("plain_d64", 2, 4, 4, 200, 64, -1, None, None),
    ("plain_d128", 1, 2, 2, 333, 128, -1, None, None),
    ("swa_gqa_d128", 2, 4, 2, 130, 128, 50, None, None),
    ("window_ge_len", 1, 2, 2, 65, 64, 1024, None, None),
    ("cache_start", 2, 4, 4, 150, 64, -1, [3, 77], None),
    ("cache_start_swa", 2, 4, 2, 150, 128, 40, [0, 120], None),
    ("seqused", 2, 4, 4, 160, 64, -1, None, [100, 160]),
    ("seqused_swa", 2, 2, 2, 160, 128, 33, None, [1, 97]),
]


def gen_train(ref, seed, B, Hq, Hkv, L, D, W):
    g = torch.Generator().manual_seed(seed)
    q, r = bf16_randn((B, Hq, L, D), g), bf16_randn((B, Hq, L, D), g)
    k, v = bf16_randn((B, Hkv, L, D), g), bf16_randn((B, Hkv, L, D), g)
    go = bf16_randn((B, Hq, L, D), g)
    leaves = [x.float().permute(0, 2, 1, 3).contiguous().requires_grad_(True) for x in (q, r, k, v)]
    o = ref(*leaves, D ** -0.5, causal=True, window_size_left=W)
    o.backward(go.float().permute(0, 2, 1, 3))
    back = lambda x: x.detach().permute(0, 2, 1, 3).contiguous().numpy()
    return dict(q=bits(q), r=bits(r), k=bits(k), v=bits(v), go=bits(go), o=back(o),
                dq=back(leaves[0].grad), dr=back(leaves[1].grad), dk=back(leaves[2].grad),
                dv=back(leaves[3].grad), window=np.int64(W))


def gen_varlen(ref, seed, lens, Hq, Hkv, D, W):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    q, r = bf16_randn((1, T, Hq, D), g), bf16_randn((1, T, Hq, D), g)
    k, v = bf16_randn((1, T, Hkv, D), g), bf16_randn((1, T, Hkv, D), g)
    go = bf16_randn((1, T, Hq, D), g)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    outs = {n: np.zeros((1, T, h, D), np.float32) for n, h in
            (("o", Hq), ("dq", Hq), ("dr", Hq), ("dk", Hkv), ("dv", Hkv))}
    for bos, eos in zip(cu[:-1], cu[1:]):
        leaves = [x[:, bos:eos].float().contiguous().requires_grad_(True) for x in (q, r, k, v)]
        o = ref(*leaves, D ** -0.5, causal=True, window_size_left=W)
        o.backward(go[:, bos:eos].float())
        outs["o"][:, bos:eos] = o.detach().numpy()
        for n, leaf in zip(("dq", "dr", "dk", "dv"), leaves):
            outs[n][:, bos:eos] = leaf.grad.numpy()
    return dict(q=bits(q), r=bits(r), k=bits(k), v=bits(v), go=bits(go), cu_seqlens=cu,
                window=np.int64(W), **outs)


def gen_decode(ref, seed, B, Hq, Hkv, T, D, W, cache_start, seqused):
    g = torch.Generator().manual_seed(seed)
    q, r = bf16_randn((B, 1, Hq, D), g), bf16_randn((B, 1, Hq, D), g, 0.5)
    k, v = bf16_randn((B, T, Hkv, D), g), bf16_randn((B, T, Hkv, D), g)
    rows = []
    for b in range(B):
        lo = 0 if cache_start is None else cache_start[b]
        hi = T if seqused is None else seqused[b]
        # left padding / runtime length == the same call on the sliced cache
        # (scripts/test_decode_triton.py:57-66, tests/test_decode_parity.py:162-177)
        rows.append(ref(q[b:b + 1], r[b:b + 1], k[b:b + 1, lo:hi], v[b:b + 1, lo:hi], D ** -0.5,
                        causal=True, window_size_left=W))
    d = dict(q=bits(q), r=bits(r), k=bits(k), v=bits(v), o=torch.cat(rows).numpy(), window=np.int64(W))
    if cache_start is not None:
        d["cache_start"] = np.asarray(cache_start, np.int32)
    if seqused is not None:
        d["seqused_k"] = np.asarray(seqused, np.int32)
    return d


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path to a checkout of the reference (the directory that holds parallax/)>")
    root = sys.argv[1]
    ref = load_reference(root)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    for i, (name, *c) in enumerate(TRAIN_CASES):
        np.savez_compressed(os.path.join(HERE, f"train_{name}.npz"), **gen_train(ref, 100 + i, *c))
    for i, (name, *c) in enumerate(VARLEN_CASES):
        np.savez_compressed(os.path.join(HERE, f"varlen_{name}.npz"), **gen_varlen(ref, 200 + i, *c))
    for i, (name, *c) in enumerate(DECODE_CASES):
        np.savez_compressed(os.path.join(HERE, f"decode_{name}.npz"), **gen_decode(ref, 300 + i, *c))
    total = sum(os.path.getsize(os.path.join(HERE, f)) for f in os.listdir(HERE) if f.endswith(".npz"))
    print(f"wrote {len(TRAIN_CASES) + len(VARLEN_CASES) + len(DECODE_CASES)} fixtures, {total / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
