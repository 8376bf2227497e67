"""Single-token Parallax decode against a KV cache.

Host-side mirror of the reference's two decode front ends: the Triton one
(``parallax/triton/parallax_decode.py:100-148``: ``cache_start``) and the
CuTeDSL one (``parallax/cute/parallax_decode.py``: ``parallax_attn_with_kvcache``
:1554-1662, ``GraphedDecode`` :1665-1815, ``parallax_decode`` :1818-1838:
``seqused_k``, ``out``).  :func:`parallax_decode` accepts the union of their
keyword arguments.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import ops

# split-KV scratch of EAGER calls, one per (device, stream, batch*heads, splits, head_dim): never shared
# by two streams.  A captured launch must not use it (every capture runs on the same capture stream, so
# two graphs of one shape would share an entry and race when replayed on different streams):
# GraphedDecode owns its workspace and passes it in.
_WORKSPACES: dict[tuple, torch.Tensor] = {}


def new_workspace(q: torch.Tensor, n_splits: int) -> torch.Tensor:
    """A zero-filled split-KV workspace for decode calls shaped like `q` with `n_splits` splits."""
    return torch.zeros(ops.decode_workspace_floats(q.shape[0], q.shape[2], q.shape[3], n_splits),
                       device=q.device, dtype=torch.float32)


def _workspace(q: torch.Tensor, n_splits: int) -> torch.Tensor:
    dev = q.device.index if q.device.index is not None else torch.cuda.current_device()
    key = (dev, torch.cuda.current_stream(q.device).cuda_stream, q.shape[0], q.shape[2], q.shape[3], n_splits)
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = new_workspace(q, n_splits)
        _WORKSPACES[key] = ws
    return ws


def _kv_ok(x: torch.Tensor) -> bool:
    return x.stride(3) == 1 and all(s % 8 == 0 for s in x.stride()[:3]) and x.data_ptr() % 16 == 0


def _kv_pair(k: torch.Tensor, v: torch.Tensor):
    """k and v as the kernels can address them: the C ABI carries ONE stride set for both, wants 16-byte
    aligned bases and strides that are multiples of 8 elements.  Views that already satisfy this pass
    through untouched (a slice of a larger cache costs nothing); anything else is made contiguous."""
    if not _kv_ok(k):
        k = k.contiguous()
    if not _kv_ok(v) or v.stride() != k.stride():
        v = v.contiguous()
        if v.stride() != k.stride():
            k = k.contiguous()
    return k, v


def split_count(q: torch.Tensor, k: torch.Tensor, window_size_left: int, cache_len: Optional[int] = None) -> int:
    """Split count of a decode call: chosen from the cache ceiling (and the window), never from the
    runtime lengths, so one captured launch serves every active length."""
    cache_len = k.shape[1] if cache_len is None else cache_len
    n_keys = cache_len if window_size_left < 0 else max(1, min(cache_len, window_size_left))
    return ops.choose_splits(q.shape[0], q.shape[2], n_keys, q.device, k.shape[2])


def _check_page_table(page_table: torch.Tensor, q: torch.Tensor, k: torch.Tensor) -> None:
    if page_table.dtype != torch.int32:
        raise TypeError(f"page_table must be int32, got {page_table.dtype}")
    if page_table.ndim != 2 or page_table.shape[0] != q.shape[0]:
        raise ValueError(f"page_table must have shape (B={q.shape[0]}, max_num_blocks), got {tuple(page_table.shape)}")
    if not page_table.is_cuda or page_table.device != q.device:
        raise ValueError("page_table must live on the same CUDA device as q")
    page_size = k.shape[1]
    if page_size < 1 or page_size & (page_size - 1):
        raise ValueError(f"page size (k_cache.shape[1]) must be a power of two, got {page_size}")


def _decode_core(q, r, k, v, scale: float, *, window_size_left: int = -1, seqused_k=None, cache_start=None,
                 out=None, workspace=None, page_table=None) -> torch.Tensor:
    if q.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"parallax decode requires bf16 or fp16 input, got {q.dtype}")
    if q.ndim != 4 or q.shape[1] != 1:
        raise ValueError(f"parallax_decode requires a single query (Sq=1), got Sq={q.shape[1] if q.ndim == 4 else '?'}.")
    bsz, _, hq, d = q.shape
    if r.shape != q.shape:
        raise ValueError(f"r shape {tuple(r.shape)} != q shape {tuple(q.shape)}")
    if k.ndim != 4 or (page_table is None and k.shape[0] != bsz) or k.shape[3] != d or v.shape != k.shape:
        raise ValueError(f"k/v shape {tuple(k.shape)}/{tuple(v.shape)} incompatible with q {tuple(q.shape)}")
    if page_table is not None:
        _check_page_table(page_table, q, k)
        page_table = page_table.contiguous()
    hkv = k.shape[2]
    if hq % hkv != 0:
        raise ValueError(f"H_q ({hq}) must be divisible by H_kv ({hkv}) for GQA")
    if d not in (64, 128):
        raise NotImplementedError(f"head_dim must be 64 or 128, got {d}")
    if not q.is_cuda:
        raise RuntimeError("parallax decode: tensors must live on a CUDA device (there is no CPU path)")
    if out is not None:
        if tuple(out.shape) != (bsz, 1, hq, d):
            raise ValueError(f"out shape mismatch: expected {(bsz, 1, hq, d)}, got {tuple(out.shape)}")
        if out.dtype != q.dtype:
            raise ValueError(f"out dtype mismatch: expected {q.dtype}, got {out.dtype}")
        if not out.is_contiguous():
            raise ValueError("out must be contiguous")
    else:
        out = torch.empty_like(q, memory_format=torch.contiguous_format)
    q, r = q.contiguous(), r.contiguous()
    k, v = _kv_pair(k, v)
    if cache_start is not None:
        cache_start = cache_start.to(device=q.device, dtype=torch.int32).contiguous()
    cache_len = k.shape[1] if page_table is None else page_table.shape[1] * k.shape[1]
    n_splits = split_count(q, k, window_size_left, cache_len)
    ops.decode_out(q, r, k, v, out, workspace if workspace is not None else _workspace(q, n_splits), float(scale),
                   int(window_size_left), n_splits, seqused_k, cache_start, page_table)
    return out


def parallax_decode(q: torch.Tensor, r: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                    qk_scale: Optional[float] = None, *, window_size_left: int = -1,
                    cache_start: Optional[torch.Tensor] = None, seqused_k: Optional[torch.Tensor] = None,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Single-token decode.  q, r: ``(B, 1, H_q, D)``; k, v: ``(B, L, H_kv, D)``.

    ``window_size_left >= 0`` restricts the query to the most recent W keys;
    ``cache_start`` ``(B,)`` is the first valid key per row (left padding);
    ``seqused_k`` ``(B,)`` int32 the active length per row (clamped to
    ``[1, L]`` in the kernel); ``out`` an optional caller-owned output.
    """
    if q.ndim == 4 and q.shape[1] != 1:
        raise ValueError(f"parallax_decode requires a single query (Sq=1), got Sq={q.shape[1]}.")
    if qk_scale is None:
        qk_scale = q.shape[-1] ** -0.5
    if seqused_k is not None:
        _check_seqused(seqused_k, q, k.shape[1])
    return _decode_core(q, r, k, v, float(qk_scale), window_size_left=window_size_left, seqused_k=seqused_k,
                        cache_start=cache_start, out=out)


def _window_size_to_left(window_size) -> int:
    """FA-style ``window_size`` -> ``window_size_left``
    (parallax/cute/parallax_decode.py:1525-1551): ``None`` / ``(-1, *)`` off, an
    int is the left window, ``(left, right)`` needs ``right <= 0``."""
    if window_size is None:
        return -1
    if isinstance(window_size, int):
        return window_size
    try:
        left, right = window_size
    except (TypeError, ValueError):
        raise ValueError(f"window_size must be None, an int, or a (left, right) pair; got {window_size!r}")
    if right is not None and right > 0:
        raise ValueError(f"parallax decode is single-query causal; window_size right must be <= 0 (got {right}).")
    return int(left)


def _check_seqused(seqused_k: torch.Tensor, q: torch.Tensor, cache_len: int) -> None:
    if seqused_k.dtype != torch.int32:
        raise TypeError(f"seqused_k must be int32, got {seqused_k.dtype}")
    if seqused_k.ndim != 1 or seqused_k.shape[0] != q.shape[0]:
        raise ValueError(f"seqused_k must have shape (B={q.shape[0]},), got {tuple(seqused_k.shape)}")
    if not seqused_k.is_cuda or seqused_k.device != q.device:
        raise ValueError("seqused_k must live on the same CUDA device as q")
    # eager-mode range check; under graph capture the in-kernel clamp enforces it
    if not torch.cuda.is_current_stream_capturing():
        lo, hi = seqused_k.min().item(), seqused_k.max().item()
        if hi > cache_len:
            raise ValueError(f"seqused_k max={hi} exceeds k_cache.shape[1]={cache_len}; values must be in [1, {cache_len}]")
        if lo < 1:
            raise ValueError(f"seqused_k has values < 1; values must be in [1, {cache_len}]")


def parallax_attn_with_kvcache(q: torch.Tensor, r: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *,
                               page_table: Optional[torch.Tensor] = None,
                               seqused_k: Optional[torch.Tensor] = None, window_size=None,
                               scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention against a KV cache with a ``flash_attn_with_kvcache``-like signature
    (reference: parallax/cute/parallax_decode.py:1554-1662).

    ``out=None`` returns a fresh tensor on every call; a given ``out`` is
    written and returned.  Inputs are never modified.  Keys beyond the active
    length are not read, so their contents cannot reach the output.

    Two things the reference's front end names but does not implement
    (parallax/cute/parallax_decode.py:1578-1580, 1627-1632) work here:

    * ``page_table`` ``(B, max_num_blocks)`` int32 -- a paged cache.  ``k_cache`` / ``v_cache`` are then
      ``(num_blocks, page_size, H_kv, D)`` with a power-of-two ``page_size``; key ``j`` of row ``b`` is row
      ``j % page_size`` of block ``page_table[b, j // page_size]``.  The logical cache length is
      ``max_num_blocks * page_size``; pass ``seqused_k`` for the active lengths -- only table entries
      below a row's active length are read, so the rest of the row may hold anything.
    * ``q`` / ``r`` with ``L_q > 1`` rows ``(B, L_q, H, D)`` -- prefill / extend: the ``L_q`` queries are
      the LAST ``L_q`` positions of the sequence (row ``i`` sees keys up to ``L - L_q + i``), as in
      ``flash_attn_with_kvcache``.  This runs the training forward kernel (tensor cores), not the decode
      sweep: one launch for a dense cache whose rows share an active length, one launch per batch row
      for row-dependent ``seqused_k`` and for a paged cache (whose pages are first gathered into a dense
      temporary).  Reading ``seqused_k`` synchronises, so only the single-token form can be captured in
      a CUDA graph.
    """
    if q.ndim == 4 and q.shape[1] > 1:
        return _extend_core(q, r, k_cache, v_cache, page_table=page_table, seqused_k=seqused_k,
                            window_size_left=_window_size_to_left(window_size), scale=scale, out=out)
    if seqused_k is not None:
        ceiling = k_cache.shape[1] if page_table is None else page_table.shape[1] * k_cache.shape[1]
        _check_seqused(seqused_k, q, ceiling)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return _decode_core(q, r, k_cache, v_cache, float(scale), window_size_left=_window_size_to_left(window_size),
                        seqused_k=seqused_k, out=out, page_table=page_table)


def _extend_dense(q, r, k, v, scale, window_size_left):
    """One launch of the training forward kernel for `L_q` query rows against the keys of `k` / `v`
    (B, L, H_kv, D): bottom-right aligned causal mask (parallax/reference.py:64-68)."""
    from .train import kernel_ready

    qk = kernel_ready(q)
    kk = k if (k.stride(-1) == 1 and all(s % 8 == 0 for s in k.stride()[:-1]) and k.data_ptr() % 16 == 0) else k.contiguous()
    vv = v if v.stride() == kk.stride() and v.data_ptr() % 16 == 0 else torch.empty_strided(kk.shape, kk.stride(), dtype=v.dtype, device=v.device).copy_(v)
    return ops.train_fwd(qk, kernel_ready(r, qk), kk, vv, float(scale), int(window_size_left), ops.BTHD, None)[0]


def _extend_core(q, r, k_cache, v_cache, *, page_table, seqused_k, window_size_left, scale, out):
    """L_q > 1 queries against a cache through the training forward kernel.  Rows that share an active
    length (or all rows, without `seqused_k`) of a dense cache run as one launch; row-dependent lengths and
    paged caches run one launch per batch row, a paged row's pages being gathered into a dense temporary
    first.  Reading the lengths synchronises, so this path cannot be captured in a CUDA graph."""
    if q.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"parallax_attn_with_kvcache requires bf16 or fp16 input, got {q.dtype}")
    if r.shape != q.shape:
        raise ValueError(f"r shape {tuple(r.shape)} != q shape {tuple(q.shape)}")
    bsz, lq, hq, d = q.shape
    paged = page_table is not None
    if k_cache.ndim != 4 or (not paged and k_cache.shape[0] != bsz) or k_cache.shape[3] != d or v_cache.shape != k_cache.shape:
        raise ValueError(f"k/v shape {tuple(k_cache.shape)}/{tuple(v_cache.shape)} incompatible with q {tuple(q.shape)}")
    if hq % k_cache.shape[2] != 0:
        raise ValueError(f"H_q ({hq}) must be divisible by H_kv ({k_cache.shape[2]}) for GQA")
    if paged:
        _check_page_table(page_table, q, k_cache)
    if not q.is_cuda:
        raise RuntimeError("parallax_attn_with_kvcache: tensors must live on a CUDA device (there is no CPU path)")
    if out is not None and (tuple(out.shape) != tuple(q.shape) or out.dtype != q.dtype):
        raise ValueError(f"out must be {tuple(q.shape)} {q.dtype}, got {tuple(out.shape)} {out.dtype}")
    page = k_cache.shape[1]
    ceiling = page_table.shape[1] * page if paged else k_cache.shape[1]
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if seqused_k is not None:
        _check_seqused(seqused_k, q, ceiling)
        lens = [int(n) for n in seqused_k.tolist()]          # synchronises: not capturable
    else:
        lens = [ceiling] * bsz
    if min(lens) < lq:
        raise ValueError(f"a row holds {min(lens)} keys but L_q = {lq}: the queries are the last L_q positions")

    if not paged and len(set(lens)) == 1:
        o = _extend_dense(q, r, k_cache[:, :lens[0]], v_cache[:, :lens[0]], scale, window_size_left)
        if out is None:
            return o
        out.copy_(o)
        return out
    res = out if out is not None else torch.empty_like(q, memory_format=torch.contiguous_format)
    for b, n in enumerate(lens):
        if paged:
            pages = page_table[b, :(n + page - 1) // page].long()
            kb = k_cache.index_select(0, pages).reshape(1, -1, k_cache.shape[2], d)[:, :n]
            vb = v_cache.index_select(0, pages).reshape(1, -1, k_cache.shape[2], d)[:, :n]
        else:
            kb, vb = k_cache[b:b + 1, :n], v_cache[b:b + 1, :n]
        res[b:b + 1].copy_(_extend_dense(q[b:b + 1], r[b:b + 1], kb, vb, scale, window_size_left))
    return res


class GraphedDecode:
    """CUDA-graph-captured decode for a fixed launch shape (reference:
    parallax/cute/parallax_decode.py:1665-1815).

    ``max_kv_len`` mode: K/V live in stable buffers of the cache ceiling and the
    captured launch reads the active lengths from ``self.cache_seqlens`` at
    replay.  ``kv_len`` mode: static length, no ``cache_seqlens``."""

    def __init__(self, B: int, H: int, max_kv_len: Optional[int] = None, head_dim: int = 128, *,
                 H_kv: Optional[int] = None, dtype: torch.dtype = torch.bfloat16, window_size=None,
                 scale: Optional[float] = None, device="cuda", warmup: int = 3, kv_len: Optional[int] = None):
        if max_kv_len is None and kv_len is None:
            raise ValueError("GraphedDecode requires max_kv_len (or kv_len for static-length back-compat)")
        if max_kv_len is not None and kv_len is not None:
            raise ValueError("pass exactly one of max_kv_len or kv_len")
        static_mode = max_kv_len is None
        cache_len = kv_len if static_mode else max_kv_len
        H_kv = H if H_kv is None else H_kv
        if H % H_kv != 0:
            raise ValueError(f"H_q={H} must be a multiple of H_kv={H_kv}")
        self.q = torch.zeros(B, 1, H, head_dim, device=device, dtype=dtype)
        self.r = torch.zeros_like(self.q)
        self.k = torch.zeros(B, cache_len, H_kv, head_dim, device=device, dtype=dtype)
        self.v = torch.zeros_like(self.k)
        self.out = torch.empty_like(self.q)
        self._scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
        self._window = window_size
        self.cache_seqlens = None if static_mode else torch.full((B,), cache_len, dtype=torch.int32, device=device)
        self.max_kv_len = cache_len

        # this object's own split-KV workspace, allocated and zeroed BEFORE the capture: the captured
        # launch of one GraphedDecode never shares scratch with another, whatever stream replays it
        window_left = _window_size_to_left(self._window)
        self._workspace = new_workspace(self.q, split_count(self.q, self.k, window_left))

        def call():
            if self.cache_seqlens is not None:
                _check_seqused(self.cache_seqlens, self.q, cache_len)
            _decode_core(self.q, self.r, self.k, self.v, float(self._scale), window_size_left=window_left,
                         seqused_k=self.cache_seqlens, out=self.out, workspace=self._workspace)

        side = torch.cuda.Stream(device=self.q.device)
        side.wait_stream(torch.cuda.current_stream(self.q.device))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                call()
        torch.cuda.current_stream(self.q.device).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            call()

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.out

    def __call__(self, *, q=None, r=None, k=None, v=None, cache_seqlens=None) -> torch.Tensor:
        for dst, src in ((self.q, q), (self.r, r), (self.k, k), (self.v, v)):
            if src is not None:
                dst.copy_(src)
        if cache_seqlens is not None and self.cache_seqlens is not None:
            if isinstance(cache_seqlens, int):
                lo = hi = cache_seqlens
            elif isinstance(cache_seqlens, (list, tuple)):
                lo, hi = min(cache_seqlens), max(cache_seqlens)
            else:
                lo, hi = cache_seqlens.min().item(), cache_seqlens.max().item()
            if lo < 1 or hi > self.max_kv_len:
                raise ValueError(f"cache_seqlens out of range [1, {self.max_kv_len}]: got min={lo}, max={hi}")
            if isinstance(cache_seqlens, int):
                self.cache_seqlens.fill_(cache_seqlens)
            elif isinstance(cache_seqlens, (list, tuple)):
                self.cache_seqlens.copy_(torch.tensor(cache_seqlens, dtype=torch.int32))
            else:
                self.cache_seqlens.copy_(cache_seqlens)
        return self.replay()
