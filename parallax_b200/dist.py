"""Multi-GPU use of the hot path: one process per GPU over ``torch.distributed``.

* Training (dense and packed) shards over (batch x heads) with NO collective:
  every (batch, head) pair is independent, so each rank simply runs the op on
  its slice.  :func:`head_shard` gives the slice that keeps a kv head together
  with the q heads of its group.
* Very long-context decode shards the KEY axis: rank g holds keys
  ``[g * T/n, (g+1) * T/n)``, computes one un-normalised partial state per
  (batch, head) with the split-KV kernel, the partial states (2*D + 4 floats
  per head) are all-gathered, and every rank merges them with the same merge
  kernel the single-GPU path uses
  (merge math: parallax/cute/parallax_decode.py:1107-1136).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def head_shard(heads_q: int, heads_kv: int, rank: int, world: int) -> tuple[slice, slice]:
    """Slices of the q-head and kv-head axes owned by `rank`.  kv heads are dealt
    out in contiguous blocks; a kv head's q heads go with it."""
    if heads_q % heads_kv != 0:
        raise ValueError(f"H_q ({heads_q}) must be divisible by H_kv ({heads_kv}) for GQA")
    if heads_kv % world != 0:
        raise ValueError(f"H_kv ({heads_kv}) must be divisible by the world size ({world})")
    rep, per = heads_q // heads_kv, heads_kv // world
    return slice(rank * per * rep, (rank + 1) * per * rep), slice(rank * per, (rank + 1) * per)


def kv_shard(total_len: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open key range ``[lo, hi)`` of `rank` for a cache of `total_len` keys."""
    per = (total_len + world - 1) // world
    lo = min(rank * per, total_len)
    return lo, min(lo + per, total_len)


class DecodeExchange:
    """Peer-memory exchange of the partial states of a KV-sharded decode (one node, GPUs that can address
    each other): ONE kernel pushes this rank's records into every rank's inbox with NVLink stores, waits
    for the other ranks' records and merges -- instead of an NCCL all-gather followed by a merge kernel.

    The inbox lives in ``torch.distributed``'s symmetric memory.  Every rank must construct the object
    (collectively) and then call it the same number of times.

    The kernel's wait for the peers is bounded by ``wait_ms`` (default: the library's 2000 ms; an NCCL
    all-gather would wait for its own, much longer, watchdog).  Ranks can be skewed by more than that -- a
    first call that loads modules, a graph capture on one rank, a stalled host -- so a time-out is a
    state to handle, not only a bug: the rows of the result whose records never arrived are NaN, the
    bit of the missing rank is set in ``self.status`` (device int32), and the kernel still advances its
    step count, so the next call is in step again.  :meth:`check` turns the status into an exception;
    it synchronises, so call it where the result is consumed on the host anyway.
    """

    def __init__(self, n_records: int, head_dim: int, device: torch.device, group=None, wait_ms: int = 0):
        import torch.distributed._symmetric_memory as symm_mem

        from . import _cabi

        group = group if group is not None else dist.group.WORLD
        world = dist.get_world_size(group)
        if world > _cabi.EXCHANGE_MAX_RANKS:
            raise ValueError(f"at most {_cabi.EXCHANGE_MAX_RANKS} ranks, got {world}")
        nbytes = int(_cabi.lib().plx_decode_exchange_bytes(world, n_records, head_dim))
        self.inbox = symm_mem.empty((nbytes + 3) // 4, dtype=torch.float32, device=device)
        self.inbox.zero_()
        self.handle = symm_mem.rendezvous(self.inbox, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.rank, self.world, self.n_records, self.head_dim = self.handle.rank, world, n_records, head_dim
        self.wait_ms = int(wait_ms)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        self.handle.barrier()        # every inbox is zero before anybody pushes

    def __call__(self, part: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
        from . import ops

        out = torch.empty_like(q)
        ops.decode_exchange_merge(part.contiguous(), out, self.ptrs, self.rank, self.status, self.wait_ms)
        return out

    def fused_step(self, q, r, k_shard, v_shard, scale, window_left, kv_offset, total_len, seqused_k, cache_start):
        """Sweep of this rank's shard, exchange and merge as ONE kernel; ``None`` where the problem has no
        fused kernel (the caller then runs the partial sweep and :meth:`__call__`)."""
        from . import ops
        from .decode import _kv_pair, _workspace

        k, v = _kv_pair(k_shard, v_shard)
        n_splits = ops.choose_splits(q.shape[0], q.shape[2], k.shape[1], q.device, k.shape[2])
        out = torch.empty_like(q, memory_format=torch.contiguous_format)
        done = ops.decode_partial_exchange(q.contiguous(), r.contiguous(), k, v, out, _workspace(q, n_splits), float(scale),
                                           int(window_left), n_splits, int(kv_offset), int(total_len), seqused_k, cache_start,
                                           self.ptrs, self.rank, self.status, self.wait_ms)
        return out if done else None

    def check(self) -> None:
        """Raise if any exchange since the last check timed out (synchronises the device)."""
        missing = int(self.status.item())
        if missing:
            self.status.zero_()
            ranks = [r for r in range(self.world) if missing >> r & 1]
            raise RuntimeError(f"peer-memory exchange: the records of rank(s) {ranks} did not arrive within the "
                               "wait limit; the affected outputs are NaN")


def make_decode_exchange(n_records: int, head_dim: int, device: torch.device, group=None,
                         wait_ms: int = 0) -> Optional[DecodeExchange]:
    """A :class:`DecodeExchange` for `group`, or ``None`` (with a warning that says why) if symmetric
    memory cannot be set up here; the caller then runs the NCCL all-gather + merge path."""
    try:
        return DecodeExchange(n_records, head_dim, device, group, wait_ms)
    except (ImportError, RuntimeError, AttributeError) as exc:
        import warnings

        warnings.warn(f"peer-memory decode exchange unavailable ({type(exc).__name__}: {exc}); "
                      "falling back to NCCL all-gather + merge", RuntimeWarning, stacklevel=2)
        return None


def _cuda_partial(q, r, k, v, scale, window_left, kv_offset, total_len, seqused_k, cache_start):
    from . import ops
    from .decode import _kv_pair, _workspace

    bsz, _, hq, d = q.shape
    k, v = _kv_pair(k, v)            # one stride set for both, 16-byte aligned, strides multiples of 8
    part = torch.empty(bsz * hq, 2 * d + 4, device=q.device, dtype=torch.float32)
    n_splits = ops.choose_splits(bsz, hq, k.shape[1], q.device, k.shape[2])
    ops.decode_partial(q.contiguous(), r.contiguous(), k, v, part, _workspace(q, n_splits), float(scale),
                       int(window_left), n_splits, int(kv_offset), int(total_len), seqused_k, cache_start)
    return part


def _cuda_merge(parts, like):
    from . import ops

    out = torch.empty_like(like, memory_format=torch.contiguous_format)
    ops.decode_merge(parts, out)
    return out


def parallax_decode_kv_sharded(q: torch.Tensor, r: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor,
                               qk_scale: Optional[float] = None, *, kv_offset: int, total_len: int,
                               window_size_left: int = -1, cache_start: Optional[torch.Tensor] = None,
                               seqused_k: Optional[torch.Tensor] = None, group=None,
                               partial_fn: Optional[Callable] = None,
                               merge_fn: Optional[Callable] = None,
                               exchange: Optional[DecodeExchange] = None, fused: bool = True) -> torch.Tensor:
    """Decode with the key axis sharded over the ranks of `group`.

    q, r ``(B, 1, H_q, D)`` are replicated; ``k_shard``/``v_shard``
    ``(B, T_local, H_kv, D)`` hold global keys ``[kv_offset, kv_offset + T_local)``
    of a cache of ``total_len`` keys.  ``window_size_left``, ``cache_start`` and
    ``seqused_k`` are in GLOBAL key positions; a rank whose shard lies outside
    the active range contributes an empty state (m = -inf, d1 = 0).  Every rank
    returns the full ``(B, 1, H_q, D)`` output.

    ``partial_fn`` / ``merge_fn`` replace the CUDA kernels (used by the CPU
    tests of the exchange step, which run over gloo without a GPU).  With an
    ``exchange`` (:func:`make_decode_exchange`) the all-gather and the merge are
    one kernel over peer memory, and -- unless ``fused=False`` or the problem has no
    fused kernel -- that kernel is the sweep itself: one launch per step.
    """
    if qk_scale is None:
        qk_scale = q.shape[-1] ** -0.5
    if exchange is not None and fused and partial_fn is None:
        out = exchange.fused_step(q, r, k_shard, v_shard, qk_scale, window_size_left, kv_offset, total_len, seqused_k,
                                  cache_start)
        if out is not None:
            return out
    partial_fn = partial_fn or _cuda_partial
    merge_fn = merge_fn or _cuda_merge
    part = partial_fn(q, r, k_shard, v_shard, qk_scale, window_size_left, kv_offset, total_len, seqused_k, cache_start)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if exchange is not None:
        return exchange(part, q)
    if world == 1:
        return merge_fn(part.unsqueeze(0), q)
    parts = torch.empty((world * part.shape[0],) + tuple(part.shape[1:]), device=part.device, dtype=part.dtype)
    dist.all_gather_into_tensor(parts, part.contiguous(), group=group)
    return merge_fn(parts.view((world,) + tuple(part.shape)), q)
