"""Dense causal Parallax training ops (forward + backward through autograd).

Host-side mirror of the reference's ``parallax/triton/parallax_train.py``:
same names, argument meaning and exceptions; the device work is done by
libplx_sm100.so.
"""
from __future__ import annotations

import torch

from . import ops


def _check_dtype(name: str, q: torch.Tensor) -> None:
    if q.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"{name} requires bf16 or fp16 inputs, got q.dtype={q.dtype}")


def _check_cuda(name: str, *tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError(f"{name}: tensors must live on a CUDA device (there is no CPU path)")


def _dense(x: torch.Tensor) -> bool:
    """True if x covers its memory without gaps or overlap in SOME axis order (a permuted view of a
    contiguous tensor), which is what ``torch.empty_like`` reproduces stride for stride."""
    pairs = sorted(((st, n) for st, n in zip(x.stride(), x.shape) if n > 1), reverse=True)
    expect = 1
    for st, n in reversed(pairs):
        if st != expect:
            return False
        expect *= n
    return True


def kernel_ready(x: torch.Tensor, like: torch.Tensor | None = None) -> torch.Tensor:
    """`x` as the kernels can address it WITHOUT a copy when possible.

    The C ABI takes element strides for (batch, head, token) with the head_dim axis contiguous, one
    set for q-like and one for kv-like tensors.  A view is passed through untouched when its last axis
    is contiguous, every other stride is a multiple of 8 elements (16-byte vector and TMA accesses),
    its base is 16-byte aligned, it is dense in some axis order, and -- if `like` is given -- its
    strides equal those of `like` (q with r, k with v share one stride set).  Anything else is copied
    to the layout of `like` (or made contiguous).  A heads-last ``(B, L, H, D)`` buffer viewed as
    ``(B, H, L, D)`` therefore costs nothing; the reference's dense path accepts arbitrary strides too
    (parallax/triton/parallax_train.py:1078-1083, 297-305).
    """
    ok = (x.stride(-1) == 1 and all(s % 8 == 0 for s in x.stride()[:-1]) and x.data_ptr() % 16 == 0 and _dense(x))
    if like is None:
        return x if ok else x.contiguous()
    if ok and x.stride() == like.stride():
        return x
    return torch.empty_like(like).copy_(x)


def parallax_func(q: torch.Tensor, r: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                  qk_scale: float | None = None, window_size_left: int = -1) -> torch.Tensor:
    """Causal Parallax with autograd (reference: ``parallax_func``,
    parallax/triton/parallax_train.py:1039-1087).

    q, r: ``(B, H_q, L_q, D)``; k, v: ``(B, H_kv, L_kv, D)``, bf16 or fp16,
    ``H_q % H_kv == 0``.  ``qk_scale`` defaults to ``D ** -0.5`` and scales
    ``q.k`` only.  ``window_size_left >= 0`` keeps keys ``[i - W + 1, i]``.
    For ``L_q != L_kv`` the causal diagonal is aligned to the END of the keys,
    as in ``parallax/reference.py:64-68``.  Returns ``(B, H_q, L_q, D)``.
    """
    _check_dtype("parallax_func", q)
    bsz, hq, lq, d = q.shape
    hkv = k.shape[1]
    if hq % hkv != 0:
        raise ValueError(f"H_q ({hq}) must be divisible by H_kv ({hkv}) for GQA")
    _check_cuda("parallax_func", q, r, k, v)
    if qk_scale is None:
        qk_scale = d ** -0.5
    q, k = kernel_ready(q), kernel_ready(k)
    o, _, _, _, _ = ops.train_fwd(q, kernel_ready(r, q), k, kernel_ready(v, k),
                                  float(qk_scale), int(window_size_left), ops.BHLD, None)
    return o


def _unfold(x: torch.Tensor, rep: int) -> torch.Tensor:
    """(B * H, L, D) with H = rep heads per kv head -> (B', rep, L, D)."""
    bh, n, d = x.shape
    return x.contiguous().view(bh // rep, rep, n, d)


def parallax_fwd(q, r, k, v, qk_scale, n_rep: int = 1, window_size_left: int = -1):
    """Raw forward with the saved statistics (reference: ``parallax_fwd``,
    parallax/triton/parallax_train.py:255-313).

    q, r: ``(B * H_q, L_q, D)``; k, v: ``(B * H_kv, L_kv, D)``.  Returns
    ``(o, barv, d1, bart, m)``: o, barv like q; d1, bart, m fp32
    ``(B * H_q, L_q, 1)``.
    """
    _check_dtype("parallax_fwd", q)
    assert q.shape[0] % n_rep == 0, f"q batch axis {q.shape[0]} must be divisible by n_rep={n_rep}"
    assert k.shape[0] == q.shape[0] // n_rep, "k batch axis must equal q batch axis // n_rep"
    _check_cuda("parallax_fwd", q, r, k, v)
    o, barv, d1, bart, m = ops.train_fwd(_unfold(q, n_rep), _unfold(r, n_rep), _unfold(k, 1), _unfold(v, 1),
                                         float(qk_scale), int(window_size_left), ops.BHLD, None)
    flat = lambda x: x.reshape(q.shape[0], q.shape[1], -1)
    return flat(o), flat(barv), flat(d1), flat(bart), flat(m)


def parallax_bwd(q, r, k, v, o, barv, d1, bart, m, grad_o, qk_scale, n_rep: int = 1,
                 window_size_left: int = -1):
    """Raw backward (reference: ``parallax_bwd``,
    parallax/triton/parallax_train.py:892-1006).  Returns
    ``(grad_q, grad_r, grad_k, grad_v)`` shaped like q, r, k, v; the kv-head
    gradients are already summed over the ``n_rep`` q heads of each group.
    """
    _check_dtype("parallax_bwd", q)
    assert q.shape[0] % n_rep == 0 and k.shape[0] == q.shape[0] // n_rep
    _check_cuda("parallax_bwd", q, r, k, v, grad_o)
    st = lambda x: x.contiguous().view(q.shape[0] // n_rep, n_rep, q.shape[1])
    dq, dr, dk, dv = ops.train_bwd(_unfold(q, n_rep), _unfold(r, n_rep), _unfold(k, 1), _unfold(v, 1),
                                   _unfold(o, n_rep), _unfold(barv, n_rep), st(d1), st(bart), st(m),
                                   _unfold(grad_o, n_rep), float(qk_scale), int(window_size_left), ops.BHLD, None)
    return dq.view_as(q), dr.view_as(r), dk.view_as(k), dv.view_as(v)
