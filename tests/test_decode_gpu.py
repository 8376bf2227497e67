"""Parity and API contracts of single-token decode on the GPU.  Case lists follow
the reference's decode tests (tests/test_decode_parity.py, tests/test_api_kvcache.py,
tests/test_cuda_graph.py, scripts/test_decode_triton.py of the reference)."""
import pytest
import torch

import parallax_b200 as plx
from oracle import parallax_oracle as orc
from parallax_b200 import ops
from tests._util import DECODE_MAX_REL, DECODE_REL_L2, assert_close, golden_names, load_golden, seeded_bf16

pytestmark = pytest.mark.gpu


def make(bsz, hq, kv_len, d=128, hkv=None, seed=0, dtype=torch.bfloat16):
    hkv = hq if hkv is None else hkv
    q = seeded_bf16((bsz, 1, hq, d), seed).to(dtype)
    r = seeded_bf16((bsz, 1, hq, d), seed + 1, 0.5).to(dtype)
    k = seeded_bf16((bsz, kv_len, hkv, d), seed + 2).to(dtype)
    v = seeded_bf16((bsz, kv_len, hkv, d), seed + 3).to(dtype)
    return q, r, k, v


def cuda(*xs):
    return [x.cuda() for x in xs]


def check(q, r, k, v, window=-1, cache_start=None, seqused=None, what="", **kw):
    cs = None if cache_start is None else torch.tensor(cache_start, dtype=torch.int32, device="cuda")
    su = None if seqused is None else torch.tensor(seqused, dtype=torch.int32, device="cuda")
    out = plx.parallax_decode(*cuda(q, r, k, v), None, window_size_left=window, cache_start=cs, seqused_k=su, **kw)
    ref = orc.decode(q, r, k, v, None, window_size_left=window, cache_start=cache_start, seqused_k=seqused)
    assert out.shape == q.shape and out.dtype == q.dtype
    assert_close(out.float().cpu(), ref, DECODE_REL_L2, DECODE_MAX_REL, what)
    return out


@pytest.mark.parametrize("name", golden_names("decode"))
def test_golden_vectors(name):
    g = load_golden("decode", name)
    cs = g.get("cache_start")
    su = g.get("seqused_k")
    out = plx.parallax_decode(*cuda(g["q"], g["r"], g["k"], g["v"]), None, window_size_left=g["window"],
                              cache_start=None if cs is None else cs.cuda(), seqused_k=None if su is None else su.cuda())
    assert_close(out.float().cpu(), g["o"], DECODE_REL_L2, DECODE_MAX_REL, name)


# (B, H, kv_len, window, D) -- reference: tests/test_decode_parity.py:46-61
FAST = [
    (1, 8, 512, -1, 128), (1, 8, 1024, -1, 128), (1, 8, 4096, -1, 128), (1, 8, 4096, 256, 128), (1, 8, 4096, 64, 128),
    (1, 8, 4096, 100, 128), (1, 8, 1000, 128, 128), (1, 8, 65, 1024, 128), (2, 4, 8192, -1, 128),
    (2, 4, 8192, 1024, 128), (2, 4, 8192, 130, 128), (8, 8, 2048, -1, 128), (32, 8, 1024, -1, 128),
    (1, 8, 1024, -1, 64), (4, 8, 2048, 256, 64), (1, 1, 1, -1, 128), (3, 2, 7, -1, 64), (1, 1, 16384, 333, 128),
    (1, 8, 4096, 33, 128), (1, 8, 4096, 0, 128),
]


@pytest.mark.parametrize("case", FAST)
def test_fast_matrix(case):
    bsz, heads, kv_len, window, d = case
    check(*make(bsz, heads, kv_len, d), window=window, what=str(case))


@pytest.mark.parametrize("splits", [1, 2, 3, 7, 32, 33, 64, 90, 256])   # above 32 the merge has two levels
def test_split_count_does_not_change_the_answer(splits, monkeypatch):
    monkeypatch.setenv("PLX_DECODE_SPLITS", str(splits))
    check(*make(2, 4, 3000, 128, seed=5), what=f"splits={splits}")
    check(*make(2, 4, 3000, 64, seed=6), window=700, what=f"splits={splits} swa")


@pytest.mark.parametrize("case", [(4, 16, 4, 1024, 128, -1), (2, 8, 2, 2048, 128, 256), (1, 32, 1, 4096, 64, -1),
                                  (1, 12, 4, 512, 128, -1), (2, 8, 4, 1024, 64, -1)])
def test_grouped_heads(case):
    bsz, hq, hkv, kv_len, d, window = case
    check(*make(bsz, hq, kv_len, d, hkv=hkv, seed=9), window=window, what=str(case))


# (B, Hq, Hkv, kv_len, D, window, splits or None): the grouped-query kernel packs up to 16 q heads of a kv
# head into one MMA tile -- group sizes 2 .. 40 (three 16-row head groups), ragged last tiles, one- and
# two-level merges, both head dims, fp16
@pytest.mark.parametrize("case", [
    (2, 4, 2, 777, 128, -1, None), (1, 6, 2, 50, 128, -1, None), (3, 32, 2, 1500, 128, -1, None), (1, 40, 1, 900, 64, -1, None),
    (2, 32, 8, 4096, 128, -1, 1), (2, 32, 8, 4096, 128, -1, 7), (1, 32, 8, 8192, 128, -1, 40), (1, 16, 2, 8192, 64, 1000, 100),
    (2, 32, 4, 3000, 128, 257, None), (1, 16, 4, 17, 128, -1, 3), (1, 8, 2, 1, 128, -1, None),
])
def test_grouped_heads_tensor_core_kernel(case, monkeypatch):
    bsz, hq, hkv, kv_len, d, window, splits = case
    if splits:
        monkeypatch.setenv("PLX_DECODE_SPLITS", str(splits))
    check(*make(bsz, hq, kv_len, d, hkv=hkv, seed=21), window=window, what=str(case))
    q, r, k, v = make(bsz, hq, kv_len, d, hkv=hkv, seed=22, dtype=torch.float16)
    check(q, r, k, v, window=window, what=str(case) + " fp16")


@pytest.mark.parametrize("hkv", [8, 2])
@pytest.mark.parametrize("mult", [8.0, 0.05])
def test_peaked_and_flat_logits(hkv, mult):
    """qk_scale far from 1/sqrt(D): the running maximum moves by many powers of two from tile to tile (or not
    at all); both kernels."""
    q, r, k, v = make(2, 8, 3000, 128, hkv=hkv, seed=41)
    scale = mult * 128 ** -0.5
    out = plx.parallax_decode(*cuda(q, r, k, v), scale)
    ref = orc.decode(q, r, k, v, scale)
    assert_close(out.float().cpu(), ref, DECODE_REL_L2, DECODE_MAX_REL, f"hkv={hkv} mult={mult}")


def test_grouped_heads_runtime_lengths_and_left_padding():
    q, r, k, v = make(4, 16, 2048, 128, hkv=4, seed=23)
    check(q, r, k, v, seqused=[1, 100, 2048, 777], what="gqa seqused")
    check(q, r, k, v, cache_start=[0, 5, 1000, 2047], what="gqa cache_start")
    check(q, r, k, v, window=300, cache_start=[0, 5, 1000, 2047], seqused=[600, 2048, 1500, 2048], what="gqa all three")


def test_grouped_heads_repeated_launches_are_bit_identical():
    q, r, k, v = cuda(*make(8, 32, 4096, 128, hkv=8, seed=24))
    first = plx.parallax_decode(q, r, k, v)
    for _ in range(40):
        assert torch.equal(first, plx.parallax_decode(q, r, k, v))


def test_grouped_heads_nan_padding_cannot_leak():
    """Keys outside the active range may hold NaN: they are never multiplied in (ragged last tile, window, left padding)."""
    q, r, k, v = make(2, 8, 1000, 128, hkv=2, seed=25)
    k2, v2 = k.clone(), v.clone()
    k2[:, 700:] = float("nan")
    v2[:, 700:] = float("nan")
    k2[:, :100] = float("nan")
    v2[:, :100] = float("nan")
    su = torch.tensor([700, 700], dtype=torch.int32, device="cuda")
    cs = torch.tensor([100, 100], dtype=torch.int32, device="cuda")
    out = plx.parallax_decode(*cuda(q, r, k2, v2), None, cache_start=cs, seqused_k=su)
    ref = orc.decode(q, r, k, v, None, cache_start=[100, 100], seqused_k=[700, 700])
    assert_close(out.float().cpu(), ref, DECODE_REL_L2, DECODE_MAX_REL, "gqa nan padding")


@pytest.mark.parametrize("case", [
    (2, 8, 8, 1024, -1, [300, 300]), (2, 8, 8, 1024, 128, [300, 300]), (1, 8, 8, 1024, -1, [333]),
    (4, 8, 2, 1024, -1, [0, 256, 512, 700]), (4, 8, 2, 1024, 128, [0, 256, 512, 700]),
])
def test_cache_start_left_padding(case):
    bsz, hq, hkv, kv_len, window, start = case
    check(*make(bsz, hq, kv_len, 128, hkv=hkv, seed=13), window=window, cache_start=start, what=str(case))


@pytest.mark.parametrize("active", [1, 128, 500, 999, 1024])
def test_seqused_k_runtime_length(active):
    q, r, k, v = make(2, 8, 1024, seed=17)
    su = torch.tensor([active, max(1, active // 2)], dtype=torch.int32, device="cuda")
    out = plx.parallax_attn_with_kvcache(*cuda(q, r, k, v), seqused_k=su)
    ref = orc.decode(q, r, k, v, None, seqused_k=su.tolist())
    assert_close(out.float().cpu(), ref, DECODE_REL_L2, DECODE_MAX_REL, f"active={active}")


def test_seqused_k_range_is_checked_in_eager_mode():
    q, r, k, v = cuda(*make(1, 8, 256))
    for bad in (0, 257):
        with pytest.raises(ValueError):
            plx.parallax_attn_with_kvcache(q, r, k, v, seqused_k=torch.tensor([bad], dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_dtypes(dtype):
    q, r, k, v = make(1, 8, 1024, dtype=dtype)
    out = plx.parallax_attn_with_kvcache(*cuda(q, r, k, v))
    assert out.dtype == dtype
    assert_close(out.float().cpu(), orc.decode(q, r, k, v), DECODE_REL_L2, DECODE_MAX_REL, str(dtype))


@pytest.mark.parametrize("kv_len", [65, 100, 1000])
def test_unused_cache_tail_cannot_leak(kv_len):
    """Keys beyond the active length are never read: NaN there must not reach the output."""
    q, r, k, v = cuda(*make(1, 8, 1024))
    k[:, kv_len:] = float("nan")
    v[:, kv_len:] = float("nan")
    su = torch.tensor([kv_len], dtype=torch.int32, device="cuda")
    out = plx.parallax_attn_with_kvcache(q, r, k, v, seqused_k=su)
    assert torch.isfinite(out.float()).all()
    out = plx.parallax_decode(q, r, k[:, :kv_len], v[:, :kv_len])
    assert torch.isfinite(out.float()).all()


def test_nan_in_valid_kv_propagates():
    q, r, k, v = cuda(*make(1, 8, 1024))
    v[0, 10, 0, :] = float("nan")
    assert torch.isnan(plx.parallax_attn_with_kvcache(q, r, k, v)).any()


def test_output_ownership():
    q, r, k, v = cuda(*make(1, 8, 512))
    a = plx.parallax_attn_with_kvcache(q, r, k, v)
    b = plx.parallax_attn_with_kvcache(q * 2, r, k, v)
    assert a.data_ptr() != b.data_ptr() and not torch.equal(a, b)     # no hidden shared buffer
    mine = torch.empty_like(q)
    ret = plx.parallax_attn_with_kvcache(q, r, k, v, out=mine)
    assert ret is mine and torch.equal(mine, a)
    with pytest.raises(ValueError):
        plx.parallax_attn_with_kvcache(q, r, k, v, out=torch.empty(1, 1, 8, 64, device="cuda", dtype=q.dtype))


def test_default_scale_and_window_mapping_are_bit_equal():
    q, r, k, v = cuda(*make(2, 8, 2048))
    base = plx.parallax_attn_with_kvcache(q, r, k, v)
    assert torch.equal(base, plx.parallax_attn_with_kvcache(q, r, k, v, scale=128 ** -0.5))
    assert torch.equal(base, plx.parallax_attn_with_kvcache(q, r, k, v, window_size=(-1, -1)))
    w = plx.parallax_attn_with_kvcache(q, r, k, v, window_size=(256, 0))
    assert torch.equal(w, plx.parallax_attn_with_kvcache(q, r, k, v, window_size=256))
    assert torch.equal(w, plx.parallax_decode(q, r, k, v, window_size_left=256))


def test_repeated_launches_are_bit_identical():
    """60 launches of a split-KV shape (the last-arriver merge must not race)."""
    q, r, k, v = cuda(*make(32, 8, 4096, seed=3))
    first = plx.parallax_decode(q, r, k, v)
    for _ in range(60):
        assert torch.equal(first, plx.parallax_decode(q, r, k, v))


def test_repeated_launches_are_bit_identical_with_a_two_level_merge():
    """Same with enough splits (one batch row, long cache) for the group level of the merge."""
    q, r, k, v = cuda(*make(1, 8, 16384, seed=4))
    first = plx.parallax_decode(q, r, k, v)
    for _ in range(60):
        assert torch.equal(first, plx.parallax_decode(q, r, k, v))


def test_strided_cache_views():
    q, r, k, v = cuda(*make(2, 4, 600, 64))
    big_k = torch.zeros(2, 1000, 4, 64, device="cuda", dtype=k.dtype)
    big_v = torch.zeros_like(big_k)
    big_k[:, :600], big_v[:, :600] = k, v
    assert torch.equal(plx.parallax_decode(q, r, big_k[:, :600], big_v[:, :600]), plx.parallax_decode(q, r, k, v))


@pytest.mark.parametrize("hkv", [8, 2])
def test_cuda_graph_replay_matches_eager_and_tracks_inputs(hkv):
    q, r, k, v = cuda(*make(2, 8, 4096, hkv=hkv, seed=21))
    out = torch.empty_like(q)
    eager = plx.parallax_attn_with_kvcache(q, r, k, v)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        plx.parallax_attn_with_kvcache(q, r, k, v, out=out)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        plx.parallax_attn_with_kvcache(q, r, k, v, out=out)
    out.zero_()
    graph.replay()
    assert torch.equal(out, eager)
    q.mul_(0.5)
    k[:, 100:200].neg_()
    graph.replay()
    assert torch.equal(out, plx.parallax_attn_with_kvcache(q, r, k, v))


def test_graphed_decode_runtime_lengths_and_clamp():
    gd = plx.GraphedDecode(B=2, H=8, max_kv_len=2048, head_dim=128, H_kv=2)
    q, r, k, v = make(2, 8, 2048, hkv=2, seed=25)
    for lens in ([2048, 2048], [1, 700], [1500, 33]):
        out = gd(q=q.cuda(), r=r.cuda(), k=k.cuda(), v=v.cuda(), cache_seqlens=lens)
        assert_close(out.float().cpu(), orc.decode(q, r, k, v, seqused_k=lens), DECODE_REL_L2, DECODE_MAX_REL, str(lens))
    with pytest.raises(ValueError):
        gd(cache_seqlens=[0, 5])
    with pytest.raises(ValueError):
        gd(cache_seqlens=4096)
    # out-of-range values written straight into the buffer are clamped by the kernel to [1, max_kv_len]
    gd.cache_seqlens.copy_(torch.tensor([100000, -5], dtype=torch.int32))
    out = gd.replay()
    assert_close(out.float().cpu(), orc.decode(q, r, k, v, seqused_k=[2048, 1]), DECODE_REL_L2, DECODE_MAX_REL, "clamp")
    static = plx.GraphedDecode(B=1, H=4, kv_len=300, head_dim=64)
    q, r, k, v = make(1, 4, 300, 64, seed=27)
    out = static(q=q.cuda(), r=r.cuda(), k=k.cuda(), v=v.cuda())
    assert static.cache_seqlens is None
    assert_close(out.float().cpu(), orc.decode(q, r, k, v), DECODE_REL_L2, DECODE_MAX_REL, "static")


def test_two_graphed_decodes_of_one_shape_replayed_on_two_streams():
    """Every GraphedDecode owns its split-KV workspace (allocated and zeroed before its capture), so two
    objects of the same launch shape can be replayed at the same time on different streams: the arrival
    counters of one never see the other's warps.  Sixty rounds, as the reference hunts for races in its
    split-K hand-over (scripts/check_decode.py:92-106 of the reference)."""
    a = plx.GraphedDecode(B=4, H=8, max_kv_len=16384, head_dim=128)
    b = plx.GraphedDecode(B=4, H=8, max_kv_len=16384, head_dim=128)
    assert a._workspace.data_ptr() != b._workspace.data_ptr()
    qa, ra, ka, va = make(4, 8, 16384, seed=33)
    qb, rb, kb, vb = make(4, 8, 16384, seed=34)
    want_a = a(q=qa.cuda(), r=ra.cuda(), k=ka.cuda(), v=va.cuda()).clone()
    want_b = b(q=qb.cuda(), r=rb.cuda(), k=kb.cuda(), v=vb.cuda()).clone()
    assert_close(want_a.float().cpu(), orc.decode(qa, ra, ka, va), DECODE_REL_L2, DECODE_MAX_REL, "a")
    assert_close(want_b.float().cpu(), orc.decode(qb, rb, kb, vb), DECODE_REL_L2, DECODE_MAX_REL, "b")
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    for _ in range(60):
        with torch.cuda.stream(s1):
            a.replay()
        with torch.cuda.stream(s2):
            b.replay()
        torch.cuda.synchronize()
        assert torch.equal(a.out, want_a) and torch.equal(b.out, want_b)


def test_partial_states_merge_to_the_direct_answer():
    """The KV-sharded path on one GPU: partial states of two halves of the cache,
    merged by the merge kernel, equal the direct call within rounding."""
    q, r, k, v = cuda(*make(2, 8, 3000, seed=31))
    direct = plx.parallax_decode(q, r, k, v, window_size_left=2500)
    parts = torch.empty(2, 2 * 8, 2 * 128 + 4, device="cuda", dtype=torch.float32)
    for i, (lo, hi) in enumerate(((0, 1400), (1400, 3000))):
        ks, vs = k[:, lo:hi], v[:, lo:hi]
        ws = torch.zeros(ops.decode_workspace_floats(2, 8, 128, 4), device="cuda", dtype=torch.float32)
        ops.decode_partial(q, r, ks, vs, parts[i], ws, 128 ** -0.5, 2500, 4, lo, 3000, None, None)
    merged = torch.empty_like(q)
    ops.decode_merge(parts, merged)
    assert_close(merged.float(), direct.float(), 2e-3, 4e-3, "merge vs direct")
    ref = orc.decode(*[x.cpu() for x in (q, r, k, v)], window_size_left=2500)
    assert_close(merged.float().cpu(), ref, DECODE_REL_L2, DECODE_MAX_REL, "merge vs oracle")


@pytest.mark.parametrize("splits", [1, 4, 40])
def test_partial_states_merge_to_the_direct_answer_with_grouped_heads(splits):
    """Same through the grouped-query kernel (16 q heads on 4 kv heads), with one split, a one-level and a
    two-level merge inside each shard."""
    q, r, k, v = cuda(*make(2, 16, 3000, hkv=4, seed=33))
    direct = plx.parallax_decode(q, r, k, v, window_size_left=2500)
    parts = torch.empty(2, 2 * 16, 2 * 128 + 4, device="cuda", dtype=torch.float32)
    for i, (lo, hi) in enumerate(((0, 1400), (1400, 3000))):
        ks, vs = k[:, lo:hi], v[:, lo:hi]
        ws = torch.zeros(ops.decode_workspace_floats(2, 16, 128, splits), device="cuda", dtype=torch.float32)
        ops.decode_partial(q, r, ks, vs, parts[i], ws, 128 ** -0.5, 2500, splits, lo, 3000, None, None)
    merged = torch.empty_like(q)
    ops.decode_merge(parts, merged)
    # this kernel rounds P to 16 bits relative to each split's own maximum, so two split layouts differ by
    # more than the fp32-P kernel's do: a few output ulps (2^-8 relative) at most
    assert_close(merged.float(), direct.float(), 5e-3, 1e-2, "merge vs direct")
    ref = orc.decode(*[x.cpu() for x in (q, r, k, v)], window_size_left=2500)
    assert_close(merged.float().cpu(), ref, DECODE_REL_L2, DECODE_MAX_REL, "merge vs oracle")


def test_peer_memory_exchange_alone_and_with_a_silent_peer():
    """plx_decode_exchange_merge on one GPU.  World of one: the merge of a single record array equals
    plx_decode_merge.  World of two whose second rank never delivers (its inbox is just a second local
    buffer that nobody stamps): the bounded wait runs out, the kernel returns, the error word says which
    rank was missing, and the context stays usable."""
    from parallax_b200 import _cabi

    q, r, k, v = cuda(*make(2, 8, 1000, seed=51))
    part = torch.empty(16, 2 * 128 + 4, device="cuda", dtype=torch.float32)
    ws = torch.zeros(ops.decode_workspace_floats(2, 8, 128, 4), device="cuda", dtype=torch.float32)
    ops.decode_partial(q, r, k, v, part, ws, 128 ** -0.5, -1, 4, 0, 1000, None, None)
    want = torch.empty_like(q)
    ops.decode_merge(part.unsqueeze(0), want)

    nbytes = _cabi.lib().plx_decode_exchange_bytes(1, 16, 128)
    inbox = torch.zeros(nbytes // 4, device="cuda", dtype=torch.float32)
    for epoch in range(3):
        got = torch.empty_like(q)
        ops.decode_exchange_merge(part, got, [inbox.data_ptr()], 0)
        assert torch.equal(got, want)
    assert _cabi.device_error() == 0

    nbytes = _cabi.lib().plx_decode_exchange_bytes(2, 16, 128)
    mine = torch.zeros(nbytes // 4, device="cuda", dtype=torch.float32)
    silent = torch.zeros(nbytes // 4, device="cuda", dtype=torch.float32)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    got = torch.zeros_like(q)
    ops.decode_exchange_merge(part, got, [mine.data_ptr(), silent.data_ptr()], 0, status=status, wait_ms=200)
    torch.cuda.synchronize()
    assert int(status.item()) == 0b10                      # rank 1 never delivered
    assert torch.isnan(got.float()).all()                  # a result built on a missing record cannot pass for a number
    # the report reaches the host without a synchronising call and is raised by the next launch that looks
    tq = torch.zeros(1, 1, 64, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(_cabi.PlxError, match="rank 1"):
        plx.parallax_func(tq, tq, tq, tq)
    # ... once: it has been acknowledged; a time-out of the exchange does not disable the training kernels
    o = plx.parallax_func(*[x.cuda() for x in make_train_inputs()])
    assert torch.isfinite(o.float()).all() and o.float().abs().max() > 0
    word = _cabi.device_error(clear=True)
    assert word == ((40 + 1) << 8) | 1, hex(word)          # the device word keeps the first error until cleared
    assert torch.equal(plx.parallax_decode(q, r, k, v), plx.parallax_decode(q, r, k, v))   # still usable
    assert _cabi.device_error() == 0
    # the step counter advanced despite the time-out: the next exchange on the one-rank inbox is in step
    got = torch.empty_like(q)
    ops.decode_exchange_merge(part, got, [inbox.data_ptr()], 0)
    assert torch.equal(got, want)


def test_sweep_and_exchange_as_one_kernel_on_one_gpu():
    """plx_decode_partial_exchange with a world of one (the rank's own inbox): the sweep's last stage pushes
    its record, finds nobody to wait for and merges -- the same bits as plx_decode.  Shapes that have no
    fused kernel (grouped-query heads, the small-batch arrangement) are refused before anything is
    enqueued.  With a second, silent rank the bounded wait runs out: NaN rows, the status bit, and the
    step count still advances."""
    from parallax_b200 import _cabi

    q, r, k, v = cuda(*make(2, 8, 3000, seed=61))
    n_records, d, splits = 16, 128, 5
    ws = torch.zeros(ops.decode_workspace_floats(2, 8, d, splits), device="cuda", dtype=torch.float32)
    want = torch.empty_like(q)
    ops.decode_out(q, r, k, v, want, ws, d ** -0.5, 2000, splits, None, None)
    inbox = torch.zeros(_cabi.lib().plx_decode_exchange_bytes(1, n_records, d) // 4, device="cuda", dtype=torch.float32)
    for step in range(3):                       # both inbox parities
        got = torch.zeros_like(q)
        assert ops.decode_partial_exchange(q, r, k, v, got, ws, d ** -0.5, 2000, splits, 0, 3000, None, None,
                                           [inbox.data_ptr()], 0)
        assert torch.equal(got, want), step
    # 44 splits: the two-level merge feeds the exchange
    ws44 = torch.zeros(ops.decode_workspace_floats(2, 8, d, 44), device="cuda", dtype=torch.float32)
    ops.decode_out(q, r, k, v, want, ws44, d ** -0.5, -1, 44, None, None)
    got = torch.zeros_like(q)
    assert ops.decode_partial_exchange(q, r, k, v, got, ws44, d ** -0.5, -1, 44, 0, 3000, None, None, [inbox.data_ptr()], 0)
    assert torch.equal(got, want)
    # no fused kernel: a multiple of 8 splits with few (batch, head) pairs, a single split, grouped-query heads
    before = _cabi.launch_count()
    ws8 = torch.zeros(ops.decode_workspace_floats(2, 8, d, 8), device="cuda", dtype=torch.float32)
    assert not ops.decode_partial_exchange(q, r, k, v, got, ws8, d ** -0.5, -1, 8, 0, 3000, None, None, [inbox.data_ptr()], 0)
    assert not ops.decode_partial_exchange(q, r, k, v, got, ws8, d ** -0.5, -1, 1, 0, 3000, None, None, [inbox.data_ptr()], 0)
    assert not ops.decode_partial_exchange(q, r, k[:, :, :2].contiguous(), v[:, :, :2].contiguous(), got, ws, d ** -0.5, -1,
                                           splits, 0, 3000, None, None, [inbox.data_ptr()], 0)
    assert _cabi.launch_count() == before
    # a silent second rank
    nbytes = _cabi.lib().plx_decode_exchange_bytes(2, n_records, d)
    mine = torch.zeros(nbytes // 4, device="cuda", dtype=torch.float32)
    silent = torch.zeros(nbytes // 4, device="cuda", dtype=torch.float32)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    got = torch.zeros_like(q)
    assert ops.decode_partial_exchange(q, r, k, v, got, ws, d ** -0.5, -1, splits, 0, 3000, None, None,
                                       [mine.data_ptr(), silent.data_ptr()], 0, status=status, wait_ms=100)
    torch.cuda.synchronize()
    assert int(status.item()) == 0b10 and torch.isnan(got.float()).all()
    assert _cabi.device_error(clear=True) == ((40 + 1) << 8) | 1
    # the workspace counters were reset by the launch that timed out: the same workspace serves the next call
    ops.decode_out(q, r, k, v, got, ws, d ** -0.5, 2000, splits, None, None)
    ops.decode_out(q, r, k, v, want, torch.zeros_like(ws), d ** -0.5, 2000, splits, None, None)
    assert torch.equal(got, want) and _cabi.device_error() == 0


def make_train_inputs():
    return [seeded_bf16((1, 2, 200, 64), 300 + i) for i in range(4)]


def test_long_context_key_sharding_at_full_size_on_one_gpu():
    """B=1, H=32, D=128, 524288 keys (8.6 GB of K and V): the key axis cut into 2, 4 and 8 shards as the
    multi-GPU path cuts it -- each shard swept by plx_decode_partial with its global offset, the per-head
    records merged by plx_decode_merge, i.e. exactly the two calls every rank makes around the exchange --
    against the single-launch result and, for two heads, against the CPU oracle.  Also with a window that
    leaves whole shards empty and with a runtime length."""
    from parallax_b200 import dist as pdist

    heads, d, total = 32, 128, 524288
    gen = torch.Generator(device="cuda").manual_seed(1005)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=gen, dtype=torch.float32).to(torch.bfloat16)
    q, r = mk(1, 1, heads, d), mk(1, 1, heads, d)
    k, v = mk(1, total, heads, d), mk(1, total, heads, d)
    for window, used in ((-1, None), (100000, None), (-1, 300001)):
        su = None if used is None else torch.tensor([used], dtype=torch.int32, device="cuda")
        full = plx.parallax_decode(q, r, k, v, window_size_left=window, seqused_k=su)
        assert torch.isfinite(full.float()).all()
        for world in (2, 4, 8):
            parts = []
            for rank in range(world):
                lo, hi = pdist.kv_shard(total, rank, world)
                parts.append(pdist._cuda_partial(q, r, k[:, lo:hi], v[:, lo:hi], d ** -0.5, window, lo, total, su, None))
            out = pdist._cuda_merge(torch.stack(parts), q)
            assert_close(out.float(), full.float(), 5e-3, 1e-2, f"{world} shards, W={window}, used={used}")
        for h in (0, 31):
            hi = total if used is None else used
            ref = orc.decode(q[:, :, h:h + 1].cpu(), r[:, :, h:h + 1].cpu(), k[:, :hi, h:h + 1].cpu(), v[:, :hi, h:h + 1].cpu(),
                             window_size_left=window)
            assert_close(out[:, :, h:h + 1].float().cpu(), ref, DECODE_REL_L2, DECODE_MAX_REL, f"head {h} W={window} used={used}")


def test_largest_benchmark_shape_against_sampled_oracle():
    """B=64, kv_len=32768, H=8, D=128 (8.6 GB of K and V): whole-batch finiteness and
    three batch rows against the oracle; plus the window=4096 variant."""
    bsz, heads, kv_len, d = 64, 8, 32768, 128
    g = torch.Generator(device="cuda").manual_seed(1004)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g, dtype=torch.float32).to(torch.bfloat16)
    q, r = mk(bsz, 1, heads, d), mk(bsz, 1, heads, d)
    k, v = mk(bsz, kv_len, heads, d), mk(bsz, kv_len, heads, d)
    for window in (-1, 4096):
        out = plx.parallax_decode(q, r, k, v, window_size_left=window)
        assert torch.isfinite(out.float()).all()
        for b in (0, 31, 63):
            ref = orc.decode(*[x[b:b + 1].cpu() for x in (q, r, k, v)], window_size_left=window)
            assert_close(out[b:b + 1].float().cpu(), ref, DECODE_REL_L2, DECODE_MAX_REL, f"b={b} W={window}")


# (B, H, kv_len, D, window): few (batch, head) pairs -- the launches that run eight splits per CTA
@pytest.mark.parametrize("case", [(1, 8, 128, 128, -1), (1, 8, 512, 128, -1), (1, 8, 1000, 128, -1), (1, 8, 4096, 128, -1),
                                  (1, 8, 16384, 128, -1), (1, 8, 32768, 128, 4096), (4, 8, 4096, 128, -1), (2, 4, 3000, 64, -1),
                                  (1, 1, 777, 64, 300), (8, 8, 1024, 128, -1), (1, 32, 8192, 128, -1),
                                  (1, 8, 6144, 128, -1), (3, 8, 2560, 128, -1), (1, 4, 5000, 64, -1)])   # clusters beyond 2048 keys
def test_split_group_arrangement_against_oracle(case):
    """Small batches: the heuristic picks a multiple of eight splits of about 16 keys, eight splits share
    a CTA and merge in shared memory, the last CTA merges the CTA records.  Against the oracle, against
    the one-warp-per-split arrangement (a split count that is not a multiple of 8), with runtime
    lengths and left padding, and launch after launch on one workspace (the counters reset themselves)."""
    bsz, heads, kv_len, d, window = case
    q, r, k, v = make(bsz, heads, kv_len, d, seed=400 + kv_len % 97)
    n_keys = kv_len if window < 0 else min(kv_len, window)
    n_splits = ops.choose_splits(bsz, heads, n_keys, torch.device("cuda", 0), heads)
    assert n_splits % 8 == 0 and n_splits >= 8, n_splits            # these shapes are meant to take the new path
    out = check(q, r, k, v, window=window, what=f"{case}")
    for _ in range(5):
        again = plx.parallax_decode(*cuda(q, r, k, v), None, window_size_left=window)
        assert torch.equal(again, out)
    # the other arrangement on the same problem
    cq, cr, ck, cv = cuda(q, r, k, v)
    other = torch.empty_like(cq)
    odd = n_splits - 1
    ws = torch.zeros(ops.decode_workspace_floats(bsz, heads, d, odd), device="cuda", dtype=torch.float32)
    ops.decode_out(cq, cr, ck, cv, other, ws, d ** -0.5, window, odd, None, None)
    assert_close(out.float(), other.float(), 5e-3, 1e-2, f"{case}: two arrangements")
    # runtime lengths and left padding (one captured split count serves every length: short rows leave
    # most of the splits empty)
    used = [max(1, kv_len // (3 + i)) for i in range(bsz)]
    start = [u // 4 for u in used]
    check(q, r, k, v, window=window, seqused=used, cache_start=start, what=f"{case} seqused/cache_start")


def test_split_group_partial_records_for_key_sharding():
    """plx_decode_partial through the split-group arrangement (B=1, H=8, two shards of 2048 keys) merged
    by plx_decode_merge: against the single launch and the oracle."""
    from parallax_b200 import dist as pdist

    q, r, k, v = cuda(*make(1, 8, 4096, 128, seed=77))
    full = plx.parallax_decode(q, r, k, v)
    parts = [pdist._cuda_partial(q, r, k[:, lo:hi], v[:, lo:hi], 128 ** -0.5, -1, lo, 4096, None, None)
             for lo, hi in ((0, 2048), (2048, 4096))]
    out = pdist._cuda_merge(torch.stack(parts), q)
    assert_close(out.float(), full.float(), 5e-3, 1e-2, "sharded vs single")
    ref = orc.decode(*[x.cpu() for x in (q, r, k, v)])
    assert_close(out.float().cpu(), ref, DECODE_REL_L2, DECODE_MAX_REL, "sharded vs oracle")


@pytest.mark.parametrize("case", [(3, 4, 4, 1000, 128, 16), (2, 8, 2, 3000, 64, 64), (1, 8, 8, 5000, 128, 256), (4, 16, 16, 700, 64, 32)])
def test_paged_cache_equals_dense_cache(case):
    """page_table: the same keys scattered over pages of a shared pool, in random order, with garbage in
    the unused table entries.  The kernels only change where a key is fetched from, so the paged result
    equals the dense one bit for bit (same split layout, same arithmetic) and passes the oracle gate.
    (The upstream front end names `page_table` but does not implement it:
    parallax/cute/parallax_decode.py:1627-1632.)"""
    bsz, hq, hkv, kv_len, d, page = case
    q, r, k, v = make(bsz, hq, kv_len, d, hkv=hkv, seed=600 + page)
    per_seq = (kv_len + page - 1) // page
    n_pages = bsz * per_seq + 5
    g = torch.Generator().manual_seed(page)
    perm = torch.randperm(n_pages, generator=g)[:bsz * per_seq].view(bsz, per_seq)
    pool_k = torch.full((n_pages, page, hkv, d), float("nan"), dtype=k.dtype)     # pages nobody owns are poisoned
    pool_v = torch.full((n_pages, page, hkv, d), float("nan"), dtype=v.dtype)
    pad = per_seq * page - kv_len
    kp = torch.nn.functional.pad(k, (0, 0, 0, 0, 0, pad)).view(bsz, per_seq, page, hkv, d)
    vp = torch.nn.functional.pad(v, (0, 0, 0, 0, 0, pad)).view(bsz, per_seq, page, hkv, d)
    for b in range(bsz):
        pool_k[perm[b]] = kp[b]
        pool_v[perm[b]] = vp[b]
    used = [kv_len - 37 * b for b in range(bsz)]
    table = torch.full((bsz, per_seq + 3), -123456, dtype=torch.int32)        # the tail of a row is never read
    table[:, :per_seq] = perm.to(torch.int32)
    for b in range(bsz):                                                      # nor are the pages past the active length
        table[b, (used[b] + page - 1) // page:per_seq] = 10 ** 9
    su = torch.tensor(used, dtype=torch.int32, device="cuda")
    cq, cr = q.cuda(), r.cuda()
    for window in (None, 300):
        paged = plx.parallax_attn_with_kvcache(cq, cr, pool_k.cuda(), pool_v.cuda(), page_table=table.cuda(), seqused_k=su,
                                               window_size=window)
        dense = plx.parallax_attn_with_kvcache(cq, cr, k.cuda(), v.cuda(), seqused_k=su, window_size=window)
        ref = orc.decode(q, r, k, v, None, window_size_left=-1 if window is None else window, seqused_k=used)
        assert_close(paged.float().cpu(), ref, DECODE_REL_L2, DECODE_MAX_REL, f"{case} W={window} vs oracle")
        # the logical ceiling differs (table columns x page size vs the dense length), so the split layout may:
        # compare within the merge tolerance, and bit for bit when the ceilings agree
        assert_close(paged.float(), dense.float(), 5e-3, 1e-2, f"{case} W={window} vs dense")
    table2 = table[:, :per_seq].contiguous()
    if per_seq * page == kv_len:
        a = plx.parallax_attn_with_kvcache(cq, cr, pool_k.cuda(), pool_v.cuda(), page_table=table2.cuda(), seqused_k=su)
        assert torch.equal(a, plx.parallax_attn_with_kvcache(cq, cr, k.cuda(), v.cuda(), seqused_k=su))


@pytest.mark.parametrize("case", [(2, 8, 8, 5, 300, 128, None), (1, 8, 2, 64, 1000, 64, None), (2, 4, 4, 130, 130, 128, None),
                                  (1, 4, 1, 200, 4096, 128, 500), (3, 2, 2, 17, 700, 64, None)])
def test_extend_with_several_query_rows(case):
    """L_q > 1 against a dense cache (prefill / extend): the L_q queries are the last L_q positions.  Runs
    the training forward kernel; checked against the oracle's bottom-right aligned mask
    (parallax/reference.py:64-68), with and without a uniform seqused_k, and the last row against the
    single-token decode."""
    bsz, hq, hkv, lq, kv_len, d, window = case
    q = seeded_bf16((bsz, lq, hq, d), 700)
    r = seeded_bf16((bsz, lq, hq, d), 701, 0.5)
    k = seeded_bf16((bsz, kv_len, hkv, d), 702)
    v = seeded_bf16((bsz, kv_len, hkv, d), 703)
    bhld = lambda x: x.permute(0, 2, 1, 3).contiguous()
    out = plx.parallax_attn_with_kvcache(*cuda(q, r, k, v), window_size=window)
    assert out.shape == q.shape
    ref = orc.train_forward(bhld(q), bhld(r), bhld(k), bhld(v), None, -1 if window is None else window)["o"].permute(0, 2, 1, 3)
    assert_close(out.float().cpu(), ref, 1e-2, 2e-2, f"{case}")
    # the last query row is what single-token decode computes
    one = plx.parallax_decode(*cuda(q[:, -1:], r[:, -1:], k, v), None, window_size_left=-1 if window is None else window)
    assert_close(out[:, -1:].float(), one.float(), 1e-2, 2e-2, f"{case}: last row vs decode")
    # a uniform active length shorter than the cache
    if kv_len - 50 >= lq:
        su = torch.full((bsz,), kv_len - 50, dtype=torch.int32, device="cuda")
        short = plx.parallax_attn_with_kvcache(*cuda(q, r, k, v), seqused_k=su, window_size=window)
        ref = orc.train_forward(bhld(q), bhld(r), bhld(k[:, :kv_len - 50]), bhld(v[:, :kv_len - 50]), None,
                                -1 if window is None else window)["o"].permute(0, 2, 1, 3)
        assert_close(short.float().cpu(), ref, 1e-2, 2e-2, f"{case} seqused")
        if bsz > 1:                 # row-dependent lengths: one launch per row, each row against its own keys
            lens = [kv_len - 50 - 7 * b for b in range(bsz)]
            if min(lens) >= lq:
                su2 = torch.tensor(lens, dtype=torch.int32, device="cuda")
                ragged = plx.parallax_attn_with_kvcache(*cuda(q, r, k, v), seqused_k=su2, window_size=window)
                for b, n in enumerate(lens):
                    ref = orc.train_forward(bhld(q[b:b + 1]), bhld(r[b:b + 1]), bhld(k[b:b + 1, :n]), bhld(v[b:b + 1, :n]), None,
                                            -1 if window is None else window)["o"].permute(0, 2, 1, 3)
                    assert_close(ragged[b:b + 1].float().cpu(), ref, 1e-2, 2e-2, f"{case} row {b} of ragged seqused")
    # the same through a paged cache: the pages of a row are gathered, the answer is the dense one
    page = 64
    n_pages = (kv_len + page - 1) // page
    pool_k = torch.zeros(bsz * n_pages + 3, page, hkv, d, dtype=k.dtype)
    pool_v = torch.zeros_like(pool_k)
    order = torch.randperm(bsz * n_pages + 3, generator=torch.Generator().manual_seed(9))[:bsz * n_pages].reshape(bsz, n_pages)
    kp = torch.zeros(bsz, n_pages * page, hkv, d, dtype=k.dtype)
    vp = torch.zeros_like(kp)
    kp[:, :kv_len], vp[:, :kv_len] = k, v
    for b in range(bsz):
        pool_k[order[b]] = kp[b].reshape(n_pages, page, hkv, d)
        pool_v[order[b]] = vp[b].reshape(n_pages, page, hkv, d)
    su = torch.full((bsz,), kv_len, dtype=torch.int32, device="cuda")
    paged = plx.parallax_attn_with_kvcache(q.cuda(), r.cuda(), pool_k.cuda(), pool_v.cuda(), page_table=order.int().cuda(),
                                           seqused_k=su, window_size=window)
    assert torch.equal(paged, out)
