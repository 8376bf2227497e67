"""Parity of the packed variable-length training op on the GPU."""
import pytest
import torch

import parallax_b200 as plx
from oracle import parallax_oracle as orc
from tests._util import (TRAIN_MAX_REL, TRAIN_REL_L2, assert_close, golden_names, load_golden, seeded_bf16)

pytestmark = pytest.mark.gpu
NAMES = ("o", "dq", "dr", "dk", "dv")


def run_gpu(q, r, k, v, go, cu, window=-1, cu_dtype=torch.int32):
    leaves = [x.cuda().requires_grad_(True) for x in (q, r, k, v)]
    cu_t = None if cu is None else torch.tensor(cu, dtype=cu_dtype, device="cuda")
    o = plx.parallax_varlen_func(*leaves, None, window, cu_t)
    o.backward(go.cuda())
    return [o.detach().float().cpu()] + [x.grad.float().cpu() for x in leaves]


def make(lens, hq, hkv, d, seed, bsz=1):
    total = sum(lens)
    mk = lambda h, s: seeded_bf16((bsz, total, h, d), s)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    return mk(hq, seed), mk(hq, seed + 1), mk(hkv, seed + 2), mk(hkv, seed + 3), mk(hq, seed + 4), cu


@pytest.mark.parametrize("name", golden_names("varlen"))
def test_golden_vectors(name):
    g = load_golden("varlen", name)
    got = run_gpu(g["q"], g["r"], g["k"], g["v"], g["go"], g["cu_seqlens"].tolist(), g["window"])
    for key, x in zip(NAMES, got):
        assert_close(x, g[key], TRAIN_REL_L2, TRAIN_MAX_REL, f"{name} {key}")


def seqlens(nseq, l_max, seed):
    """Random lengths in [1, l_max] with the edge cases pinned (reference: scripts/parity_varlen.py:39-45)."""
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(1, l_max + 1, (nseq,), generator=g).tolist()
    lens[0], lens[-1] = 1, l_max
    return lens


# (Hq, Hkv, L_max, D, window) -- reference: scripts/parity_varlen.py:26-34
@pytest.mark.parametrize("case", [
    (8, 8, 1024, 128, -1), (8, 8, 1024, 64, -1), (16, 4, 512, 128, -1), (32, 1, 512, 64, -1),
    (8, 8, 1024, 128, 256), (8, 2, 512, 128, 128), (16, 4, 512, 128, 64),
])
@pytest.mark.parametrize("cu_dtype", [torch.int32, torch.int64])
def test_packed_against_oracle_and_dense(case, cu_dtype):
    hq, hkv, l_max, d, window = case
    if cu_dtype == torch.int64 and case != (8, 8, 1024, 64, -1):
        pytest.skip("int64 cu_seqlens is covered by one case")
    lens = seqlens(6, l_max, 3)
    q, r, k, v, go, cu = make(lens, hq, hkv, d, 17)
    got = run_gpu(q, r, k, v, go, cu, window, cu_dtype)
    ref_o = orc.varlen_forward(q, r, k, v, cu, None, window)["o"]
    ref_g = orc.varlen_backward(q, r, k, v, go.float(), cu, None, window)
    for name, g, e in zip(NAMES, got, (ref_o, *ref_g)):
        assert_close(g, e, TRAIN_REL_L2, TRAIN_MAX_REL, f"{case} {name}")
    # packed == each sequence run alone through the dense path (reference: scripts/parity_varlen.py:127-130)
    for bos, eos in zip(cu[:-1], cu[1:]):
        alone = run_gpu(q[:, bos:eos], r[:, bos:eos], k[:, bos:eos], v[:, bos:eos], go[:, bos:eos], None, window)
        for name, g, a in zip(NAMES, got, alone):
            assert torch.equal(g[:, bos:eos], a), f"{case} {name} [{bos}:{eos}]"


def test_dense_batch_without_cu_seqlens():
    q, r, k, v, go, _ = make([300], 4, 2, 64, 23, bsz=3)
    got = run_gpu(q, r, k, v, go, None)
    ref_o = orc.varlen_forward(q, r, k, v, None)["o"]
    ref_g = orc.varlen_backward(q, r, k, v, go.float(), None)
    for name, g, e in zip(NAMES, got, (ref_o, *ref_g)):
        assert_close(g, e, TRAIN_REL_L2, TRAIN_MAX_REL, name)


def test_many_short_sequences_and_empty_ones():
    lens = [1, 1, 0, 2, 65, 0, 3, 64, 63, 1]
    q, r, k, v, go, cu = make(lens, 2, 2, 64, 29)
    got = run_gpu(q, r, k, v, go, cu)
    ref_o = orc.varlen_forward(q, r, k, v, cu)["o"]
    ref_g = orc.varlen_backward(q, r, k, v, go.float(), cu)
    for name, g, e in zip(NAMES, got, (ref_o, *ref_g)):
        assert_close(g, e, TRAIN_REL_L2, TRAIN_MAX_REL, name)


def test_benchmark_shape_properties():
    """65536 packed tokens, H=16, D=128, lengths uniform on [64, 8192] from seed 0
    (last one truncated): two heads of two sequences against the oracle, and a
    sequence run alone gives the same bits."""
    g = torch.Generator().manual_seed(0)
    raw = torch.randint(64, 8193, (64,), generator=g).tolist()
    lens, total = [], 0
    for n in raw:
        n = min(n, 65536 - total)
        lens.append(n)
        total += n
        if total == 65536:
            break
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    heads, d = 16, 128
    gen = torch.Generator(device="cuda").manual_seed(1003)
    mk = lambda: torch.randn(1, 65536, heads, d, device="cuda", generator=gen, dtype=torch.float32).to(torch.bfloat16)
    q, r, k, v = mk(), mk(), mk(), mk()
    leaves = [x.clone().requires_grad_(True) for x in (q, r, k, v)]
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    o = plx.parallax_varlen_func(*leaves, cu_seqlens=cu_t)
    go = (o.detach().float() * (2.0 / o.numel())).to(o.dtype)
    o.backward(go)
    grads = [x.grad for x in leaves]
    assert all(torch.isfinite(x.float()).all() for x in [o] + grads)
    shortest = min(range(len(lens)), key=lambda i: lens[i])
    for i in (shortest, 0):
        bos, eos = cu[i], cu[i + 1]
        hs = slice(4, 6)
        sub = [x[:, bos:eos, hs].clone().requires_grad_(True) for x in (q, r, k, v)]
        o_sub = plx.parallax_varlen_func(*sub)
        o_sub.backward(go[:, bos:eos, hs].contiguous())
        assert torch.equal(o_sub.detach(), o.detach()[:, bos:eos, hs])
        for a, b in zip(sub, grads):
            assert torch.equal(a.grad, b[:, bos:eos, hs])
        cq, cr, ck, cv = [x[:, bos:eos, hs].cpu() for x in (q, r, k, v)]
        ref_o = orc.varlen_forward(cq, cr, ck, cv, None)["o"]
        ref_g = orc.varlen_backward(cq, cr, ck, cv, go[:, bos:eos, hs].float().cpu(), None)
        for name, got, e in zip(NAMES, [o.detach()] + grads, (ref_o, *ref_g)):
            assert_close(got[:, bos:eos, hs].float().cpu(), e, TRAIN_REL_L2, TRAIN_MAX_REL, f"seq {i} {name}")


def test_a_thousand_short_sequences():
    """65536 tokens in 1024 sequences of 1..256 tokens (every tile finds its sequence by binary search
    over cu_seqlens; most 128-row tile ids between two sequences are empty): the whole packed result
    against the oracle on a sample of sequences, and packed == the sequence run alone, bit for bit."""
    g = torch.Generator().manual_seed(5)
    lens = (1 + (255 * torch.rand(1024, generator=g) ** 3).long()).tolist()     # skewed to short: mean about 64
    lens[0], lens[1], lens[-1] = 1, 256, 128
    excess, i = sum(lens) - 65536, 2
    while excess != 0:                      # spread the remainder over the sequences, keeping lengths in [1, 256]
        step = max(-min(8, 256 - lens[i]), min(lens[i] - 1, excess, 8))
        lens[i] -= step
        excess -= step
        i = 2 + (i - 1) % 1020
    assert sum(lens) == 65536 and min(lens) >= 1 and max(lens) <= 256
    q, r, k, v, go, cu = make(lens, 2, 1, 128, 37)
    got = run_gpu(q, r, k, v, go, cu)
    assert all(torch.isfinite(x).all() for x in got)
    for s in (0, 1, 2, 511, 777, 1023):
        bos, eos = cu[s], cu[s + 1]
        sl = [x[:, bos:eos] for x in (q, r, k, v, go)]
        alone = run_gpu(*sl, None)
        ref_o = orc.varlen_forward(*sl[:4], None)["o"]
        ref_g = orc.varlen_backward(*sl[:4], sl[4].float(), None)
        for name, gpk, a, e in zip(NAMES, got, alone, (ref_o, *ref_g)):
            assert torch.equal(gpk[:, bos:eos], a), f"seq {s} {name}: packed != alone"
            assert_close(a, e, TRAIN_REL_L2 * (8.0 if eos - bos < 8 else 1.0), TRAIN_MAX_REL * (8.0 if eos - bos < 8 else 1.0),
                         f"seq {s} (len {eos - bos}) {name}")


def test_one_sequence_of_65536_tokens():
    """The other extreme of the packed op: a single 65536-token sequence (513 tile ids, one sequence).
    Causality gives a size-independent check: the first 2048 rows equal, bit for bit, the op run on the
    2048-token prefix alone, and that prefix is checked against the oracle."""
    total, heads, d = 65536, 2, 128
    gen = torch.Generator(device="cuda").manual_seed(41)
    mk = lambda: torch.randn(1, total, heads, d, device="cuda", generator=gen, dtype=torch.float32).to(torch.bfloat16)
    q, r, k, v = mk(), mk(), mk(), mk()
    cu = torch.tensor([0, total], dtype=torch.int32, device="cuda")
    o = plx.parallax_varlen_func(q, r, k, v, cu_seqlens=cu)
    assert torch.isfinite(o.float()).all()
    pre = [x[:, :2048].contiguous() for x in (q, r, k, v)]
    o_pre = plx.parallax_varlen_func(*pre, cu_seqlens=torch.tensor([0, 2048], dtype=torch.int32, device="cuda"))
    assert torch.equal(o_pre, o[:, :2048])
    ref = orc.varlen_forward(*[x.cpu() for x in pre], None)["o"]
    assert_close(o_pre.float().cpu(), ref, TRAIN_REL_L2, TRAIN_MAX_REL, "prefix o")
    # backward over the whole sequence: finite, and deterministic from launch to launch
    leaves = [x.clone().requires_grad_(True) for x in (q, r, k, v)]
    go = (o.float() * (2.0 / o.numel())).to(o.dtype)
    plx.parallax_varlen_func(*leaves, cu_seqlens=cu).backward(go)
    first = [x.grad.clone() for x in leaves]
    assert all(torch.isfinite(x.float()).all() for x in first)
    for x in leaves:
        x.grad = None
    plx.parallax_varlen_func(*leaves, cu_seqlens=cu).backward(go)
    assert all(torch.equal(a, x.grad) for a, x in zip(first, leaves))
