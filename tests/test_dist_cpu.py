"""The multi-GPU host logic on CPU ranks (gloo, world_size 2): sharding helpers
and the exchange step of KV-sharded decode, with the oracle's partial / merge
standing in for the CUDA kernels (there is no GPU here)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import parallax_oracle as orc
from parallax_b200 import dist as pdist
from tests._util import seeded_bf16


def test_head_shard_keeps_groups_together():
    for hq, hkv, world in ((32, 32, 8), (16, 4, 2), (8, 2, 2)):
        rep = hq // hkv
        seen_q, seen_k = [], []
        for rank in range(world):
            sq, sk = pdist.head_shard(hq, hkv, rank, world)
            qs, ks = list(range(hq))[sq], list(range(hkv))[sk]
            assert sorted({h // rep for h in qs}) == ks
            seen_q += qs
            seen_k += ks
        assert seen_q == list(range(hq)) and seen_k == list(range(hkv))
    with pytest.raises(ValueError):
        pdist.head_shard(8, 3, 0, 2)
    with pytest.raises(ValueError):
        pdist.head_shard(8, 2, 0, 4)


def test_kv_shard_covers_the_cache():
    for total, world in ((524288, 8), (1000, 3), (5, 8)):
        ranges = [pdist.kv_shard(total, r, world) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))


def _oracle_partial(q, r, k, v, scale, window_left, kv_offset, total_len, seqused_k, cache_start):
    bsz, _, hq, d = q.shape
    recs = torch.zeros(bsz * hq, 2 * d + 4)
    for b in range(bsz):
        lo_g, hi_g = orc.decode_key_range(total_len, window_left, 0 if cache_start is None else int(cache_start[b]),
                                          None if seqused_k is None else int(seqused_k[b]))
        lo = min(max(lo_g - kv_offset, 0), k.shape[1])
        hi = min(max(hi_g - kv_offset, 0), k.shape[1])
        m, d1, d2, o1, o2 = orc.decode_partial(q[b, 0], r[b, 0], k[b], v[b], scale, lo, hi)
        rec = recs[b * hq:(b + 1) * hq]
        rec[:, 0], rec[:, 1], rec[:, 2] = m, d1, d2
        rec[:, 4:4 + d], rec[:, 4 + d:] = o1, o2
    return recs


def _oracle_merge(parts, like):
    n, recs, width = parts.shape
    d = (width - 4) // 2
    states = [(parts[s, :, 0], parts[s, :, 1], parts[s, :, 2], parts[s, :, 4:4 + d], parts[s, :, 4 + d:]) for s in range(n)]
    return orc.decode_merge(states).view(like.shape)


def _worker(rank, world, port, case, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bsz, hq, hkv, total, d, window, cache_start, seqused = case
        q, r = seeded_bf16((bsz, 1, hq, d), 1), seeded_bf16((bsz, 1, hq, d), 2, 0.5)
        k, v = seeded_bf16((bsz, total, hkv, d), 3), seeded_bf16((bsz, total, hkv, d), 4)
        lo, hi = pdist.kv_shard(total, rank, world)
        cs = None if cache_start is None else torch.tensor(cache_start, dtype=torch.int32)
        su = None if seqused is None else torch.tensor(seqused, dtype=torch.int32)
        out = pdist.parallax_decode_kv_sharded(q, r, k[:, lo:hi], v[:, lo:hi], None, kv_offset=lo, total_len=total,
                                               window_size_left=window, cache_start=cs, seqused_k=su,
                                               partial_fn=_oracle_partial, merge_fn=_oracle_merge)
        ref = orc.decode(q, r, k, v, None, window_size_left=window, cache_start=cache_start, seqused_k=seqused)
        ret[rank] = float((out - ref).abs().max())
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("case", [
    (2, 4, 2, 301, 64, -1, None, None),
    (1, 2, 2, 256, 128, 40, None, None),          # window inside the last shard: rank 0 contributes nothing
    (2, 2, 2, 200, 64, 150, [0, 120], [200, 130]),
])
def test_kv_sharded_decode_exchange(case):
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), case, ret), nprocs=world, join=True)
    assert len(ret) == world
    assert max(ret.values()) < 1e-5, dict(ret)
