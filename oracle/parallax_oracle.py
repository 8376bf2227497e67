"""CPU oracle for the Parallax attention hot path.  TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline / reference arm of ``bench.py``
may import it.  The shipped package never routes through it.

It restates, in plain PyTorch on the CPU, the algorithm of the reference's fp32
implementation ``parallax/reference.py:41-86`` (Algorithm 1 of the Parallax
paper), plus the pieces the reference only has inside GPU kernels:

* the saved statistics of the training forward
  (``parallax/triton/parallax_train.py:243-252``: ``barv = O1/d1``,
  ``bart = d2/d1``, un-normalised ``d1``, base-2 row max ``m``),
* the closed-form backward (``parallax/triton/parallax_train.py:561-573`` for
  dq/dr and ``:765-792`` for dk/dv),
* packed variable-length sequences (``parallax/triton/parallax_varlen.py:57-62``),
* single-token decode with ``cache_start`` / ``seqused_k`` / sliding window
  (``parallax/triton/parallax_decode.py:43-97``) and
* the split-KV partial state and its merge
  (``parallax/cute/parallax_decode.py:1089-1136``).

Parity pin: ``tests/golden/make_golden.py`` runs the reference's own
``parallax_reference`` (forward, and autograd for the gradients) on seeded
inputs and stores inputs and outputs under ``tests/golden/``;
``tests/test_oracle_golden.py`` checks every function here against those
vectors.

Everything is computed one (batch, head) slice at a time and in row blocks so
that long sequences fit in host memory (the reference materialises four
``(B, H, Q, L)`` fp32 tensors at once).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

LOG2E = 1.4426950408889634


# --------------------------------------------------------------------------- #
# masks
# --------------------------------------------------------------------------- #
def visible(n_q: int, n_k: int, window_left: int = -1, row0: int = 0, rows: Optional[int] = None):
    """Boolean ``(rows, n_k)`` matrix: which keys each query row may see.

    Causal mask aligned to the END of the key sequence (query ``i`` sits at
    absolute position ``n_k - n_q + i``) and, for ``window_left >= 0``, only the
    ``window_left`` most recent keys ``[pos - W + 1, pos]``
    (``parallax/reference.py:64-73``).
    """
    rows = n_q - row0 if rows is None else rows
    i = torch.arange(row0, row0 + rows).view(-1, 1) + (n_k - n_q)
    j = torch.arange(n_k).view(1, -1)
    ok = j <= i
    if window_left >= 0:
        ok = ok & (j >= i - window_left + 1)
    return ok


# --------------------------------------------------------------------------- #
# one (batch, head) slice
# --------------------------------------------------------------------------- #
def _slice_forward(q, r, k, v, scale, window_left, row_block):
    """q, r: (Lq, D); k, v: (Lk, D), all the working dtype.  Returns
    o, barv (Lq, D) and d1, bart, m2 (Lq,) with m2 the row max in base-2 units."""
    n_q, d = q.shape
    n_k = k.shape[0]
    o = torch.empty_like(q)
    barv = torch.empty_like(q)
    d1 = q.new_empty(n_q)
    bart = q.new_empty(n_q)
    m2 = q.new_empty(n_q)
    for r0 in range(0, n_q, row_block):
        nr = min(row_block, n_q - r0)
        ok = visible(n_q, n_k, window_left, r0, nr)
        s1 = (q[r0:r0 + nr] @ k.T) * scale
        s1 = s1.masked_fill(~ok, float("-inf"))
        s2 = r[r0:r0 + nr] @ k.T
        m = s1.amax(dim=-1, keepdim=True)
        m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        p1 = (s1 - m_safe).exp()
        p2 = p1 * s2
        dd1 = p1.sum(-1, keepdim=True)
        dd2 = p2.sum(-1, keepdim=True)
        inv = torch.where(dd1 > 0, 1.0 / dd1, torch.zeros_like(dd1))
        bv = (p1 @ v) * inv
        bt = dd2 * inv
        o[r0:r0 + nr] = bv + bt * bv - (p2 @ v) * inv
        barv[r0:r0 + nr] = bv
        d1[r0:r0 + nr] = dd1[:, 0]
        bart[r0:r0 + nr] = bt[:, 0]
        m2[r0:r0 + nr] = m[:, 0] * LOG2E
    return o, barv, d1, bart, m2


def _slice_backward(q, r, k, v, go, scale, window_left, row_block, o=None, barv=None):
    """Closed-form gradients of one slice.  ``o`` / ``barv`` may be supplied
    (e.g. the bf16-rounded tensors a kernel saved); otherwise they are
    recomputed exactly."""
    n_q, d = q.shape
    n_k = k.shape[0]
    dq = torch.zeros_like(q)
    dr = torch.zeros_like(q)
    dk = torch.zeros_like(k)
    dv = torch.zeros_like(k)
    for r0 in range(0, n_q, row_block):
        nr = min(row_block, n_q - r0)
        sl = slice(r0, r0 + nr)
        ok = visible(n_q, n_k, window_left, r0, nr)
        s1 = ((q[sl] @ k.T) * scale).masked_fill(~ok, float("-inf"))
        s2 = r[sl] @ k.T
        m = s1.amax(dim=-1, keepdim=True)
        m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        p1 = (s1 - m_safe).exp()
        dd1 = p1.sum(-1, keepdim=True)
        inv = torch.where(dd1 > 0, 1.0 / dd1, torch.zeros_like(dd1))
        p = p1 * inv
        c = (p * s2).sum(-1, keepdim=True)                 # bart
        bv = p @ v if barv is None else barv[sl]
        oo = (bv + c * bv - (p * s2) @ v) if o is None else o[sl]
        a = go[sl] @ v.T
        t = (go[sl] * oo).sum(-1, keepdim=True)
        b = (go[sl] * bv).sum(-1, keepdim=True)
        delta = a - b
        gl = p * (a - t + (c - s2) * delta)
        gu = -p * delta
        w = p * (1.0 + c - s2)
        dq[sl] = (gl @ k) * scale
        dr[sl] = gu @ k
        dk += (gl.T @ q[sl]) * scale + gu.T @ r[sl]
        dv += w.T @ go[sl]
    return dq, dr, dk, dv


# --------------------------------------------------------------------------- #
# dense training op, (B, H, L, D) layout  (parallax_func)
# --------------------------------------------------------------------------- #
def train_forward(q, r, k, v, qk_scale=None, window_size_left=-1, *, dtype=torch.float32,
                  row_block=1024):
    """Forward of ``parallax_func`` (``parallax/triton/parallax_train.py:1039-1087``).

    q, r: (B, Hq, Lq, D); k, v: (B, Hkv, Lk, D).  Returns a dict with ``o``,
    ``barv`` (B, Hq, Lq, D) and ``d1``, ``bart``, ``m`` (B, Hq, Lq)."""
    bsz, hq, n_q, d = q.shape
    hkv = k.shape[1]
    if hq % hkv:
        raise ValueError(f"H_q ({hq}) must be divisible by H_kv ({hkv}) for GQA")
    rep = hq // hkv
    scale = d ** -0.5 if qk_scale is None else float(qk_scale)
    out = {n: torch.empty(bsz, hq, n_q, d, dtype=dtype) for n in ("o", "barv")}
    out.update({n: torch.empty(bsz, hq, n_q, dtype=dtype) for n in ("d1", "bart", "m")})
    for b in range(bsz):
        for h in range(hq):
            res = _slice_forward(q[b, h].to(dtype), r[b, h].to(dtype), k[b, h // rep].to(dtype),
                                 v[b, h // rep].to(dtype), scale, window_size_left, row_block)
            for n, x in zip(("o", "barv", "d1", "bart", "m"), res):
                out[n][b, h] = x
    return out


def train_backward(q, r, k, v, grad_o, qk_scale=None, window_size_left=-1, *,
                   dtype=torch.float32, row_block=1024, o=None, barv=None):
    """Gradients (dq, dr, dk, dv) of ``parallax_func`` w.r.t. its inputs for an
    upstream gradient ``grad_o``; dk/dv are summed over the q heads of a GQA
    group (``parallax/triton/parallax_train.py:998-1005``)."""
    bsz, hq, n_q, d = q.shape
    hkv = k.shape[1]
    rep = hq // hkv
    scale = d ** -0.5 if qk_scale is None else float(qk_scale)
    dq = torch.zeros(bsz, hq, n_q, d, dtype=dtype)
    dr = torch.zeros_like(dq)
    dk = torch.zeros(bsz, hkv, k.shape[2], d, dtype=dtype)
    dv = torch.zeros_like(dk)
    for b in range(bsz):
        for h in range(hq):
            g = _slice_backward(q[b, h].to(dtype), r[b, h].to(dtype), k[b, h // rep].to(dtype),
                                v[b, h // rep].to(dtype), grad_o[b, h].to(dtype), scale,
                                window_size_left, row_block,
                                None if o is None else o[b, h].to(dtype),
                                None if barv is None else barv[b, h].to(dtype))
            dq[b, h] = g[0]
            dr[b, h] = g[1]
            dk[b, h // rep] += g[2]
            dv[b, h // rep] += g[3]
    return dq, dr, dk, dv


def mse_loss_grad(o):
    """Upstream gradient of the loss ``mean(o.float() ** 2)`` used by the
    benchmark configurations: ``2 * o / o.numel()``."""
    return o.float() * (2.0 / o.numel())


# --------------------------------------------------------------------------- #
# packed variable-length training op, (1, T, H, D) layout  (parallax_varlen_func)
# --------------------------------------------------------------------------- #
def _bthd_to_bhld(x):
    return x.permute(0, 2, 1, 3)


def varlen_forward(q, r, k, v, cu_seqlens: Optional[Sequence[int]], qk_scale=None,
                   window_size_left=-1, *, dtype=torch.float32, row_block=1024):
    """Forward of ``parallax_varlen_func`` (``parallax/triton/parallax_varlen.py:738-788``).

    Heads-last layout: q, r (B, T, Hq, D); k, v (B, T, Hkv, D).  With
    ``cu_seqlens`` (length N+1, B must be 1) each sequence
    ``[cu[i], cu[i+1])`` is causal within itself; with ``None`` every batch row
    is one dense causal sequence.  Returns dict like :func:`train_forward`, but
    ``o``/``barv`` are (B, T, Hq, D) and the statistics (B, T, Hq)."""
    bsz, total, hq, d = q.shape
    if cu_seqlens is None:
        bounds = [(0, total)]
    else:
        if bsz != 1:
            raise ValueError("The batch size must be 1 when using cu_seqlens")
        cu = [int(x) for x in cu_seqlens]
        bounds = list(zip(cu[:-1], cu[1:]))
    o = torch.zeros(bsz, total, hq, d, dtype=dtype)
    barv = torch.zeros_like(o)
    stats = {n: torch.zeros(bsz, total, hq, dtype=dtype) for n in ("d1", "bart", "m")}
    for bos, eos in bounds:
        if eos <= bos:
            continue
        f = train_forward(_bthd_to_bhld(q[:, bos:eos]), _bthd_to_bhld(r[:, bos:eos]),
                          _bthd_to_bhld(k[:, bos:eos]), _bthd_to_bhld(v[:, bos:eos]),
                          d ** -0.5 if qk_scale is None else qk_scale, window_size_left,
                          dtype=dtype, row_block=row_block)
        o[:, bos:eos] = f["o"].permute(0, 2, 1, 3)
        barv[:, bos:eos] = f["barv"].permute(0, 2, 1, 3)
        for n in stats:
            stats[n][:, bos:eos] = f[n].permute(0, 2, 1)
    return {"o": o, "barv": barv, **stats}


def varlen_backward(q, r, k, v, grad_o, cu_seqlens: Optional[Sequence[int]], qk_scale=None,
                    window_size_left=-1, *, dtype=torch.float32, row_block=1024):
    """Gradients of ``parallax_varlen_func``; same layout as its inputs."""
    bsz, total, hq, d = q.shape
    if cu_seqlens is None:
        bounds = [(0, total)]
    else:
        cu = [int(x) for x in cu_seqlens]
        bounds = list(zip(cu[:-1], cu[1:]))
    dq = torch.zeros(bsz, total, hq, d, dtype=dtype)
    dr = torch.zeros_like(dq)
    dk = torch.zeros(bsz, total, k.shape[2], d, dtype=dtype)
    dv = torch.zeros_like(dk)
    for bos, eos in bounds:
        if eos <= bos:
            continue
        g = train_backward(_bthd_to_bhld(q[:, bos:eos]), _bthd_to_bhld(r[:, bos:eos]),
                           _bthd_to_bhld(k[:, bos:eos]), _bthd_to_bhld(v[:, bos:eos]),
                           _bthd_to_bhld(grad_o[:, bos:eos]),
                           d ** -0.5 if qk_scale is None else qk_scale, window_size_left,
                           dtype=dtype, row_block=row_block)
        for dst, src in zip((dq, dr, dk, dv), g):
            dst[:, bos:eos] = src.permute(0, 2, 1, 3)
    return dq, dr, dk, dv


# --------------------------------------------------------------------------- #
# single-token decode, heads-last layout  (parallax_decode / parallax_attn_with_kvcache)
# --------------------------------------------------------------------------- #
def decode_key_range(cache_len: int, window_left: int = -1, cache_start: int = 0,
                     seqused: Optional[int] = None):
    """Half-open key range ``[lo, hi)`` one decode query attends to.

    ``hi`` is the active length (``seqused`` clamped to ``[1, cache_len]`` as the
    kernel does, ``parallax/cute/parallax_decode.py:367-369``; the whole cache
    otherwise).  ``lo = max(cache_start, hi - W, 0)``
    (``parallax/triton/parallax_decode.py:48-54``)."""
    hi = cache_len if seqused is None else max(1, min(int(seqused), cache_len))
    lo = max(int(cache_start), 0)
    if window_left >= 0:
        lo = max(lo, hi - window_left)
    return lo, hi


def decode_partial(q, r, k, v, qk_scale, lo: int, hi: int, *, dtype=torch.float32):
    """Un-normalised partial state of one (batch, kv-range) for all heads.

    q, r: (Hq, D); k, v: (T, Hkv, D); keys ``[lo, hi)``.  Returns
    ``m`` (Hq,) natural-log max (``-inf`` when the range is empty), ``d1``,
    ``d2`` (Hq,), ``o1``, ``o2`` (Hq, D) — the five quantities the split-KV
    kernels exchange (``parallax/cute/parallax_decode.py:1368-1385``)."""
    hq, d = q.shape
    hkv = k.shape[1]
    rep = hq // hkv
    m = torch.full((hq,), float("-inf"), dtype=dtype)
    d1 = torch.zeros(hq, dtype=dtype)
    d2 = torch.zeros(hq, dtype=dtype)
    o1 = torch.zeros(hq, d, dtype=dtype)
    o2 = torch.zeros(hq, d, dtype=dtype)
    if hi <= lo:
        return m, d1, d2, o1, o2
    for h in range(hq):
        kk = k[lo:hi, h // rep].to(dtype)
        vv = v[lo:hi, h // rep].to(dtype)
        s1 = (kk @ q[h].to(dtype)) * qk_scale
        s2 = kk @ r[h].to(dtype)
        m[h] = s1.max()
        p1 = (s1 - m[h]).exp()
        p2 = p1 * s2
        d1[h] = p1.sum()
        d2[h] = p2.sum()
        o1[h] = p1 @ vv
        o2[h] = p2 @ vv
    return m, d1, d2, o1, o2


def decode_merge(parts):
    """Combine partial states of disjoint key ranges and finalise.

    ``parts`` is a list of ``(m, d1, d2, o1, o2)`` as returned by
    :func:`decode_partial`.  ``M = max m_s; w_s = exp(m_s - M)``; sums are
    weighted by ``w_s``; ``out = (1 + d2/d1) * O1/d1 - O2/d1``
    (``parallax/cute/parallax_decode.py:1107-1136``); rows without any key give 0."""
    m_all = torch.stack([p[0] for p in parts])                       # (S, Hq)
    big = m_all.max(dim=0).values
    big_safe = torch.where(torch.isinf(big), torch.zeros_like(big), big)
    w = (m_all - big_safe).exp()                                      # exp(-inf) = 0
    d1 = sum(p[1] * w[i] for i, p in enumerate(parts))
    d2 = sum(p[2] * w[i] for i, p in enumerate(parts))
    o1 = sum(p[3] * w[i][:, None] for i, p in enumerate(parts))
    o2 = sum(p[4] * w[i][:, None] for i, p in enumerate(parts))
    inv = torch.where(d1 > 0, 1.0 / d1, torch.zeros_like(d1))[:, None]
    return o1 * inv * (1.0 + d2[:, None] * inv) - o2 * inv


def decode(q, r, k, v, qk_scale=None, *, window_size_left=-1, cache_start=None, seqused_k=None,
           n_splits: int = 1, dtype=torch.float32):
    """Single-token decode.  q, r: (B, 1, Hq, D); k, v: (B, T, Hkv, D).

    ``n_splits > 1`` evaluates the same result through the partial/merge path
    (equal ranges over ``[lo, hi)``), which is what a split-KV or a
    KV-sharded multi-GPU run computes."""
    bsz, sq, hq, d = q.shape
    if sq != 1:
        raise ValueError(f"parallax_decode requires a single query (Sq=1), got Sq={sq}.")
    if hq % k.shape[2]:
        raise ValueError(f"H_q ({hq}) must be divisible by H_kv ({k.shape[2]}) for GQA")
    scale = d ** -0.5 if qk_scale is None else float(qk_scale)
    out = torch.empty(bsz, 1, hq, d, dtype=dtype)
    for b in range(bsz):
        lo, hi = decode_key_range(k.shape[1], window_size_left,
                                  0 if cache_start is None else int(cache_start[b]),
                                  None if seqused_k is None else int(seqused_k[b]))
        step = max(1, math.ceil(max(hi - lo, 1) / n_splits))
        parts = [decode_partial(q[b, 0], r[b, 0], k[b], v[b], scale, a, min(a + step, hi), dtype=dtype)
                 for a in range(lo, max(hi, lo + 1), step)]
        out[b, 0] = decode_merge(parts)
    return out


# --------------------------------------------------------------------------- #
# error metrics shared by tests and the benchmark
# --------------------------------------------------------------------------- #
def error_metrics(got, ref):
    """max-abs, max-abs / max|ref|, relative L2 and the median of |diff| / max|ref|
    (the last is the reference's own gate, ``scripts/parity_train.py:70-81``)."""
    g = got.detach().double().cpu()
    e = ref.detach().double().cpu()
    diff = (g - e).abs()
    ref_max = max(e.abs().max().item(), 1e-12)
    return {
        "max_abs": diff.max().item(),
        "max_rel": diff.max().item() / ref_max,
        "rel_l2": (diff.pow(2).sum().sqrt() / e.pow(2).sum().sqrt().clamp_min(1e-30)).item(),
        "q50": (diff.flatten().median() / ref_max).item(),
    }
