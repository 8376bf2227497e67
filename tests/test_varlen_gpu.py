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
