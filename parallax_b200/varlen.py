"""Packed variable-length causal Parallax training op.

Host-side mirror of the reference's ``parallax/triton/parallax_varlen.py``.
The reference builds a (sequence, tile) table on the device for every call
(``prepare_chunk_indices``, parallax/triton/_kernel_utils.py:37-52), which
needs a device-to-host sync to size the grid.  Here the kernels find their
sequence from ``cu_seqlens`` themselves and the grid is sized from the shapes
alone (``ceil(T / tile) + n_seqs`` tiles), so the call never syncs.
"""
from __future__ import annotations

import torch

from . import ops
from .train import _check_cuda, kernel_ready


def parallax_varlen_func(q: torch.Tensor, r: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                         qk_scale: float | None = None, window_size_left: int = -1,
                         cu_seqlens: torch.Tensor | None = None) -> torch.Tensor:
    """Variable-length (packed) causal Parallax with autograd (reference:
    ``parallax_varlen_func``, parallax/triton/parallax_varlen.py:738-788).

    Heads-last layout: q, r ``(B, T, H_q, D)``; k, v ``(B, T, H_kv, D)``.
    ``cu_seqlens`` (int32 or int64, ``[N + 1]``, starting at 0) packs N
    independent causal sequences along T and requires ``B == 1``; ``None`` runs
    every batch row as one dense causal sequence.  Returns ``(B, T, H_q, D)``.
    """
    if q.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"parallax_varlen_func requires bf16 or fp16 inputs, got q.dtype={q.dtype}")
    if q.shape[2] % k.shape[2] != 0:
        raise ValueError(f"H_q ({q.shape[2]}) must be divisible by H_kv ({k.shape[2]}) for GQA")
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError(
                f"The batch size must be 1 (got {q.shape[0]}) when using cu_seqlens. "
                f"Flatten variable-length inputs into a single packed sequence first.")
        if cu_seqlens.dtype not in (torch.int32, torch.int64):
            raise TypeError(f"cu_seqlens must be int32 or int64, got {cu_seqlens.dtype}")
        cu_seqlens = cu_seqlens.to(device=q.device, dtype=torch.int32).contiguous()
    _check_cuda("parallax_varlen_func", q, r, k, v)
    if qk_scale is None:
        qk_scale = q.shape[-1] ** -0.5
    q, k = kernel_ready(q), kernel_ready(k)
    o, _, _, _, _ = ops.train_fwd(q, kernel_ready(r, q), k, kernel_ready(v, k),
                                  float(qk_scale), int(window_size_left), ops.BTHD, cu_seqlens)
    return o
