"""torch custom ops over the C ABI: ``plx::train_fwd``, ``plx::train_bwd``,
``plx::decode_out``, ``plx::decode_partial``, ``plx::decode_merge``.

The ops only marshal pointers, strides and the current CUDA stream into
libplx_sm100.so; all arithmetic happens in its kernels.  Tensors come in one of
two axis orders, ``BHLD`` = (batch, heads, tokens, head_dim) and ``BTHD`` =
(batch, tokens, heads, head_dim), with any dense strides whose head_dim axis is
contiguous; q-like tensors (q, r, o, barv, grad_o) must share one stride set and
kv-like tensors (k, v) another (the public wrappers take care of that).
"""
from __future__ import annotations

import ctypes as C
import functools
import os
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _cabi

BHLD, BTHD = 0, 1


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return _cabi.PLX_BF16
    if dtype == torch.float16:
        return _cabi.PLX_FP16
    raise TypeError(f"bf16 or fp16 required, got {dtype}")


def _ptr(t: Optional[Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _bht(x: Tensor, layout: int):
    """(batch, head, token) element strides of a 4-d tensor in `layout`."""
    return (x.stride(0), x.stride(1), x.stride(2)) if layout == BHLD else (x.stride(0), x.stride(2), x.stride(1))


def _dims(x: Tensor, layout: int):
    """(batch, heads, tokens, head_dim)"""
    b, a1, a2, d = x.shape
    return (b, a1, a2, d) if layout == BHLD else (b, a2, a1, d)


def _train_problem(q: Tensor, k: Tensor, stats: Tensor, qk_scale: float, window_left: int, layout: int,
                   cu_seqlens: Optional[Tensor]) -> _cabi.TrainProblem:
    bsz, hq, lq, d = _dims(q, layout)
    _, hkv, lk, _ = _dims(k, layout)
    p = _cabi.TrainProblem()
    p.dtype = dtype_code(q.dtype)
    p.batch, p.heads_q, p.heads_kv, p.len_q, p.len_k, p.head_dim = bsz, hq, hkv, lq, lk, d
    p.window_left = int(window_left)
    p.qk_scale = float(qk_scale)
    p.q_stride_b, p.q_stride_h, p.q_stride_t = _bht(q, layout)
    p.kv_stride_b, p.kv_stride_h, p.kv_stride_t = _bht(k, layout)
    if layout == BHLD:
        p.st_stride_b, p.st_stride_h, p.st_stride_t = stats.stride(0), stats.stride(1), stats.stride(2)
    else:
        p.st_stride_b, p.st_stride_h, p.st_stride_t = stats.stride(0), stats.stride(2), stats.stride(1)
    if cu_seqlens is not None:
        p.cu_seqlens = cu_seqlens.data_ptr()
        p.n_seqs = cu_seqlens.numel() - 1
    else:
        p.cu_seqlens = None
        p.n_seqs = 0
    return p


def _stats_shape(q: Tensor, layout: int):
    return q.shape[:3]


# --------------------------------------------------------------------------- #
# training
# --------------------------------------------------------------------------- #
@torch.library.custom_op("plx::train_fwd", mutates_args=(), device_types="cuda")
def train_fwd(q: Tensor, r: Tensor, k: Tensor, v: Tensor, qk_scale: float, window_left: int, layout: int,
              cu_seqlens: Optional[Tensor]) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    o = torch.empty_like(q)
    barv = torch.empty_like(q)
    d1 = torch.empty(_stats_shape(q, layout), device=q.device, dtype=torch.float32)
    bart = torch.empty_like(d1)
    m = torch.empty_like(d1)
    p = _train_problem(q, k, d1, qk_scale, window_left, layout, cu_seqlens)
    with torch.cuda.device(q.device):
        _cabi.raise_if_device_error("plx_train_fwd")
        st = _cabi.lib().plx_train_fwd(C.byref(p), _ptr(q), _ptr(r), _ptr(k), _ptr(v), _ptr(o), _ptr(barv),
                                       _ptr(d1), _ptr(bart), _ptr(m), _stream(q.device))
    _cabi.check(st, "plx_train_fwd")
    return o, barv, d1, bart, m


@train_fwd.register_fake
def _(q, r, k, v, qk_scale, window_left, layout, cu_seqlens):
    stats = q.new_empty(q.shape[:3], dtype=torch.float32)
    return torch.empty_like(q), torch.empty_like(q), stats, torch.empty_like(stats), torch.empty_like(stats)


BWD_STATS, BWD_DQR, BWD_DKV, BWD_ALL = 1, 2, 4, 7


def train_bwd_workspace(q: Tensor, k: Tensor, d1: Tensor, layout: int, cu_seqlens: Optional[Tensor]) -> Tensor:
    """Scratch for the backward row statistics (sized by plx_train_workspace_bytes)."""
    p = _train_problem(q, k, d1, 1.0, -1, layout, cu_seqlens)
    need = C.c_size_t(0)
    _cabi.check(_cabi.lib().plx_train_workspace_bytes(C.byref(p), C.byref(need)), "plx_train_workspace_bytes")
    return torch.empty(max(need.value, 16), device=q.device, dtype=torch.uint8)


def train_bwd_stages(stages: int, q, r, k, v, o, barv, d1, bart, m, grad_o, dq, dr, dk, dv, ws, qk_scale: float,
                     window_left: int, layout: int, cu_seqlens: Optional[Tensor]) -> None:
    """Enqueue the selected backward kernels (mask of BWD_STATS | BWD_DQR | BWD_DKV) into caller-owned outputs."""
    p = _train_problem(q, k, d1, qk_scale, window_left, layout, cu_seqlens)
    with torch.cuda.device(q.device):
        _cabi.raise_if_device_error("plx_train_bwd_stages")
        st = _cabi.lib().plx_train_bwd_stages(C.byref(p), int(stages), _ptr(q), _ptr(r), _ptr(k), _ptr(v), _ptr(o),
                                              _ptr(barv), _ptr(d1), _ptr(bart), _ptr(m), _ptr(grad_o), _ptr(dq),
                                              _ptr(dr), _ptr(dk), _ptr(dv), _ptr(ws), C.c_size_t(ws.numel()),
                                              _stream(q.device))
    _cabi.check(st, "plx_train_bwd_stages")


@torch.library.custom_op("plx::train_bwd", mutates_args=(), device_types="cuda")
def train_bwd(q: Tensor, r: Tensor, k: Tensor, v: Tensor, o: Tensor, barv: Tensor, d1: Tensor, bart: Tensor,
              m: Tensor, grad_o: Tensor, qk_scale: float, window_left: int, layout: int,
              cu_seqlens: Optional[Tensor]) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    dq, dr = torch.empty_like(q), torch.empty_like(q)
    dk, dv = torch.empty_like(k), torch.empty_like(k)
    ws = train_bwd_workspace(q, k, d1, layout, cu_seqlens)
    train_bwd_stages(BWD_ALL, q, r, k, v, o, barv, d1, bart, m, grad_o, dq, dr, dk, dv, ws, qk_scale, window_left,
                     layout, cu_seqlens)
    return dq, dr, dk, dv


@train_bwd.register_fake
def _(q, r, k, v, o, barv, d1, bart, m, grad_o, qk_scale, window_left, layout, cu_seqlens):
    return torch.empty_like(q), torch.empty_like(q), torch.empty_like(k), torch.empty_like(k)


def _setup_ctx(ctx, inputs, output):
    q, r, k, v, qk_scale, window_left, layout, cu_seqlens = inputs
    o, barv, d1, bart, m = output
    ctx.save_for_backward(q, r, k, v, o, barv, d1, bart, m, cu_seqlens)
    ctx.qk_scale, ctx.window_left, ctx.layout = qk_scale, window_left, layout


def _backward(ctx, grad_o, *_unused):
    q, r, k, v, o, barv, d1, bart, m, cu_seqlens = ctx.saved_tensors
    if grad_o.stride() != q.stride():          # one stride set for all q-like tensors: bring grad_o to q's layout
        grad_o = torch.empty_like(q).copy_(grad_o)
    dq, dr, dk, dv = train_bwd(q, r, k, v, o, barv, d1, bart, m, grad_o, ctx.qk_scale, ctx.window_left,
                               ctx.layout, cu_seqlens)
    return dq, dr, dk, dv, None, None, None, None


train_fwd.register_autograd(_backward, setup_context=_setup_ctx)


# --------------------------------------------------------------------------- #
# decode
# --------------------------------------------------------------------------- #
@functools.lru_cache(maxsize=None)
def sm_count(device_index: int) -> int:
    return torch.cuda.get_device_properties(device_index).multi_processor_count


def choose_splits(batch: int, heads_q: int, n_keys: int, device: torch.device, heads_kv: Optional[int] = None) -> int:
    """Split count for the key axis (``PLX_DECODE_SPLITS`` overrides the heuristic)."""
    env = os.environ.get("PLX_DECODE_SPLITS")
    if env:
        return max(1, int(env))
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return int(_cabi.lib().plx_decode_choose_splits_gqa(batch, heads_q, heads_kv or heads_q, n_keys, sm_count(idx)))


def _decode_problem(q: Tensor, k: Tensor, qk_scale: float, window_left: int, n_splits: int, kv_offset: int,
                    total_len: int, page_table: Optional[Tensor] = None) -> _cabi.DecodeProblem:
    p = _cabi.DecodeProblem()
    p.dtype = dtype_code(q.dtype)
    p.batch, p.heads_q, p.head_dim = q.shape[0], q.shape[2], q.shape[3]
    p.cache_len, p.heads_kv = k.shape[1], k.shape[2]
    if page_table is not None:        # k: (num_pages, page_size, heads_kv, head_dim); stride(0) is the page stride
        p.page_table, p.page_size, p.pages_per_seq = page_table.data_ptr(), k.shape[1], page_table.shape[1]
        p.cache_len = page_table.shape[1] * k.shape[1]
    p.window_left, p.n_splits, p.qk_scale = int(window_left), int(n_splits), float(qk_scale)
    p.kv_offset, p.total_len = int(kv_offset), int(total_len)
    p.kv_stride_b, p.kv_stride_t, p.kv_stride_h = k.stride(0), k.stride(1), k.stride(2)
    return p


def decode_workspace_floats(batch: int, heads_q: int, head_dim: int, n_splits: int) -> int:
    bh = batch * heads_q
    groups = (n_splits + 15) // 16 if n_splits > 32 else 0   # PLX_DECODE_GROUPS: first level of the two-level merge
    return bh * (n_splits + groups) * (2 * head_dim + 4) + bh * (1 + groups)


@torch.library.custom_op("plx::decode_out", mutates_args=("out", "workspace"), device_types="cuda")
def decode_out(q: Tensor, r: Tensor, k: Tensor, v: Tensor, out: Tensor, workspace: Tensor, qk_scale: float,
               window_left: int, n_splits: int, seqused_k: Optional[Tensor], cache_start: Optional[Tensor],
               page_table: Optional[Tensor] = None) -> None:
    p = _decode_problem(q, k, qk_scale, window_left, n_splits, 0, 0, page_table)
    with torch.cuda.device(q.device):
        st = _cabi.lib().plx_decode(C.byref(p), _ptr(q), _ptr(r), _ptr(k), _ptr(v), _ptr(out), _ptr(seqused_k),
                                    _ptr(cache_start), _ptr(workspace), C.c_size_t(workspace.numel() * 4),
                                    _stream(q.device))
    _cabi.check(st, "plx_decode")


@torch.library.custom_op("plx::decode_partial", mutates_args=("part", "workspace"), device_types="cuda")
def decode_partial(q: Tensor, r: Tensor, k: Tensor, v: Tensor, part: Tensor, workspace: Tensor, qk_scale: float,
                   window_left: int, n_splits: int, kv_offset: int, total_len: int, seqused_k: Optional[Tensor],
                   cache_start: Optional[Tensor]) -> None:
    p = _decode_problem(q, k, qk_scale, window_left, n_splits, kv_offset, total_len)
    with torch.cuda.device(q.device):
        st = _cabi.lib().plx_decode_partial(C.byref(p), _ptr(q), _ptr(r), _ptr(k), _ptr(v), _ptr(part),
                                            _ptr(seqused_k), _ptr(cache_start), _ptr(workspace),
                                            C.c_size_t(workspace.numel() * 4), _stream(q.device))
    _cabi.check(st, "plx_decode_partial")


@torch.library.custom_op("plx::decode_merge", mutates_args=("out",), device_types="cuda")
def decode_merge(parts: Tensor, out: Tensor) -> None:
    """parts: (n_parts, n_records, 2 * D + 4) fp32; out: (..., D) with n_records rows."""
    n_parts, n_records, rec = parts.shape
    head_dim = (rec - 4) // 2
    with torch.cuda.device(parts.device):
        st = _cabi.lib().plx_decode_merge(_ptr(parts), n_parts, n_records, head_dim, dtype_code(out.dtype), _ptr(out),
                                          _stream(parts.device))
    _cabi.check(st, "plx_decode_merge")


def _exchange_struct(inbox_ptrs, rank: int, n_records: int, head_dim: int, dtype: torch.dtype, status: Optional[Tensor],
                     wait_ms: int) -> _cabi.Exchange:
    x = _cabi.Exchange()
    x.world, x.rank, x.n_records, x.head_dim = len(inbox_ptrs), int(rank), int(n_records), int(head_dim)
    x.dtype = dtype_code(dtype)
    x.wait_ms = int(wait_ms)
    x.status = None if status is None else status.data_ptr()
    for i, ptr in enumerate(inbox_ptrs):
        x.inbox[i] = int(ptr)
    return x


def decode_partial_exchange(q: Tensor, r: Tensor, k: Tensor, v: Tensor, out: Tensor, workspace: Tensor, qk_scale: float,
                            window_left: int, n_splits: int, kv_offset: int, total_len: int, seqused_k: Optional[Tensor],
                            cache_start: Optional[Tensor], inbox_ptrs, rank: int, status: Optional[Tensor] = None,
                            wait_ms: int = 0) -> bool:
    """The KV-sharded step as ONE kernel (sweep of this rank's shard + exchange + merge into `out`).  Returns
    False, having enqueued nothing, when this problem has no fused kernel (grouped-query heads, the
    small-batch arrangement, a single split): the caller then runs decode_partial + decode_exchange_merge."""
    p = _decode_problem(q, k, qk_scale, window_left, n_splits, kv_offset, total_len)
    x = _exchange_struct(inbox_ptrs, rank, q.shape[0] * q.shape[2], q.shape[3], out.dtype, status, wait_ms)
    with torch.cuda.device(q.device):
        _cabi.raise_if_device_error("plx_decode_partial_exchange")
        st = _cabi.lib().plx_decode_partial_exchange(C.byref(p), C.byref(x), _ptr(q), _ptr(r), _ptr(k), _ptr(v), _ptr(out),
                                                     _ptr(seqused_k), _ptr(cache_start), _ptr(workspace),
                                                     C.c_size_t(workspace.numel() * 4), _stream(q.device))
    if st == _cabi.PLX_ERR_UNSUPPORTED:
        return False
    _cabi.check(st, "plx_decode_partial_exchange")
    return True


def decode_exchange_merge(part: Tensor, out: Tensor, inbox_ptrs, rank: int, status: Optional[Tensor] = None,
                          wait_ms: int = 0) -> None:
    """One step of the peer-memory exchange: push `part` (n_records, 2 * D + 4) to every rank's inbox,
    wait (at most `wait_ms` milliseconds, 0 = the library's default) for the others' records of this step,
    write the merged `out` (n_records rows of D).  If a rank never delivers, its bit is set in `status`
    (int32, one element, caller-zeroed) and the affected rows of `out` are NaN."""
    n_records, rec = part.shape
    x = _exchange_struct(inbox_ptrs, rank, n_records, (rec - 4) // 2, out.dtype, status, wait_ms)
    with torch.cuda.device(part.device):
        _cabi.raise_if_device_error("plx_decode_exchange_merge")
        st = _cabi.lib().plx_decode_exchange_merge(C.byref(x), _ptr(part), _ptr(out), _stream(part.device))
    _cabi.check(st, "plx_decode_exchange_merge")
