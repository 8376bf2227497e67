"""plx_decode_static: decode for callers that cannot allocate device memory.

Some users of this library are handed tensors but no allocator: a plugin callback
inside a serving runtime that owns every byte of device memory, or a decode loop
that cannot afford cudaMalloc's device-wide synchronisation.  They cannot supply
the split-KV workspace `plx_decode` asks for, so `plx_decode_static` keeps that
scratch in a fixed 4 MiB array inside the library.  This test drives the entry
point through the C ABI (ctypes), several times in a row with different shapes --
each call finds the previous call's leftovers in the shared array -- and compares
each result with the ordinary `plx_decode` entry point given a caller workspace:
same kernel, same split count, so the two must agree bit for bit.  Covered: the
single-level merge, the two-level merge (more than 32 splits, whose group counters
also live in the region each call clears), the grouped-query kernel, that the
amount of free device memory does not move across calls, and that a refused call
(too large, or a bad pointer) enqueues nothing.

The file sorts last on purpose: if it fails, `pytest -x` has already run every other test.
"""
import ctypes as C

import pytest
import torch

from parallax_b200 import _cabi, ops
from tests._util import DECODE_MAX_REL, DECODE_REL_L2, assert_close, seeded_bf16

pytestmark = pytest.mark.gpu


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _inputs(bsz, hq, hkv, kv_len, d, seed):
    q = seeded_bf16((bsz, 1, hq, d), seed).cuda()
    r = seeded_bf16((bsz, 1, hq, d), seed + 1, 0.5).cuda()
    k = seeded_bf16((bsz, kv_len, hkv, d), seed + 2).cuda()
    v = seeded_bf16((bsz, kv_len, hkv, d), seed + 3).cuda()
    return q, r, k, v


def _both_entry_points(q, r, k, v, n_splits, window, seqused=None):
    lib = _cabi.lib()
    p = ops._decode_problem(q, k, q.shape[-1] ** -0.5, window, n_splits, 0, 0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    su = None if seqused is None else torch.tensor(seqused, dtype=torch.int32, device="cuda")

    # reference: the existing entry point with a caller-owned, zero-filled workspace
    expect = torch.empty_like(q)
    ws = torch.zeros(ops.decode_workspace_floats(q.shape[0], q.shape[2], q.shape[3], n_splits), device="cuda")
    _cabi.check(lib.plx_decode(C.byref(p), _ptr(q), _ptr(r), _ptr(k), _ptr(v), _ptr(expect), _ptr(su), None,
                               _ptr(ws), C.c_size_t(ws.numel() * 4), stream), "plx_decode")

    # under test: no workspace argument at all
    got = torch.full_like(q, float("nan"))
    _cabi.check(lib.plx_decode_static(C.byref(p), _ptr(q), _ptr(r), _ptr(k), _ptr(v), _ptr(got), _ptr(su), None,
                                      stream), "plx_decode_static")
    torch.cuda.synchronize()
    return got, expect


def _same(got, expect, what):
    # the tolerance gate of the other decode tests first (a readable message if something is badly off) ...
    assert_close(got.float(), expect.float(), DECODE_REL_L2, DECODE_MAX_REL, what)
    # ... then the real claim: same kernel, same split layout, same arithmetic -> the same bits
    assert torch.equal(got, expect), what


def test_static_scratch_matches_caller_workspace_on_calls_in_a_row():
    # call 1: 16 (batch, head) pairs x 8 splits, D = 128
    _same(*_both_entry_points(*_inputs(2, 8, 8, 4096, 128, 71), n_splits=8, window=-1), "first call")
    # call 2, straight after, another shape: the counters of this layout sit where call 1 left partial sums
    _same(*_both_entry_points(*_inputs(3, 4, 2, 3000, 64, 75), n_splits=5, window=1000, seqused=[3000, 17, 1500]),
          "second call")
    # and the first shape again
    _same(*_both_entry_points(*_inputs(2, 8, 8, 4096, 128, 79), n_splits=8, window=-1), "third call")


def test_two_level_merge_and_grouped_query_kernel_through_the_static_scratch():
    # 44 splits > 32 (not a multiple of 8, so the one-warp-per-split arrangement): groups of 16, 16 and 12 merge first,
    # then the group records; 8 (batch, head) pairs x
    # (44 + 3) records x 132 floats = 199 KB of the 4 MiB
    _same(*_both_entry_points(*_inputs(1, 8, 8, 5000, 64, 91), n_splits=44, window=-1), "two-level merge")
    # straight after, the grouped-query kernel (8 q heads on 2 kv heads) with 48 splits, two levels as well
    _same(*_both_entry_points(*_inputs(2, 8, 2, 6000, 128, 95), n_splits=48, window=-1, seqused=[6000, 4097]),
          "grouped-query, two-level merge")
    # and back to a single-level layout over the same bytes
    _same(*_both_entry_points(*_inputs(1, 8, 8, 5000, 64, 99), n_splits=7, window=2000), "single level again")


def test_no_device_memory_is_allocated():
    """What the entry point is for: after a first call (which looks up the array's address), further calls
    leave the amount of free device memory exactly where it was."""
    lib = _cabi.lib()
    q, r, k, v = _inputs(2, 8, 8, 4096, 128, 103)
    p = ops._decode_problem(q, k, 128 ** -0.5, -1, 8, 0, 0)
    out = torch.empty_like(q)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    call = lambda: _cabi.check(lib.plx_decode_static(C.byref(p), _ptr(q), _ptr(r), _ptr(k), _ptr(v), _ptr(out), None,
                                                     None, stream), "plx_decode_static")
    call()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        call()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_single_split_needs_no_scratch():
    got, expect = _both_entry_points(*_inputs(1, 2, 2, 300, 64, 83), n_splits=1, window=-1)
    assert_close(got.float(), expect.float(), DECODE_REL_L2, DECODE_MAX_REL, "one split")


def test_problem_larger_than_the_array_is_refused():
    lib = _cabi.lib()
    q, r, k, v = _inputs(8, 8, 8, 64, 128, 87)
    # 64 (batch, head) pairs x 128 splits x 260 floats = 8.5 MB > 4 MiB
    p = ops._decode_problem(q, k, 128 ** -0.5, -1, 128, 0, 0)
    need = C.c_size_t(0)
    assert lib.plx_decode_workspace_bytes(C.byref(p), C.byref(need)) == 0
    assert need.value > _cabi.DECODE_STATIC_SCRATCH_BYTES
    out = torch.zeros_like(q)
    st = lib.plx_decode_static(C.byref(p), _ptr(q), _ptr(r), _ptr(k), _ptr(v), _ptr(out), None, None,
                               C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == _cabi.PLX_ERR_STATIC_SCRATCH
    assert b"built-in" in lib.plx_strerror(st)
    torch.cuda.synchronize()
    assert torch.equal(out, torch.zeros_like(out))      # nothing was launched


def test_a_bad_argument_is_refused_before_anything_is_enqueued():
    """A call that plx_decode would refuse (here: a null v, then a misaligned q) returns the same status
    from the static entry point and leaves the shared array alone: the counters a running call of another
    stream might be using are not cleared under its feet."""
    lib = _cabi.lib()
    q, r, k, v = _inputs(2, 8, 8, 4096, 128, 111)
    p = ops._decode_problem(q, k, 128 ** -0.5, -1, 8, 0, 0)
    out = torch.zeros_like(q)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    before = _cabi.launch_count()
    assert lib.plx_decode_static(C.byref(p), _ptr(q), _ptr(r), _ptr(k), None, _ptr(out), None, None, stream) == -1
    assert lib.plx_decode_static(C.byref(p), C.c_void_p(q.data_ptr() + 2), _ptr(r), _ptr(k), _ptr(v), _ptr(out), None, None,
                                 stream) == -1
    torch.cuda.synchronize()
    assert _cabi.launch_count() == before and torch.equal(out, torch.zeros_like(out))
