"""plx_decode_static: decode for callers that cannot allocate device memory.

Some users of this library are handed tensors but no allocator: a plugin callback
inside a serving runtime that owns every byte of device memory, or a decode loop
that cannot afford cudaMalloc's device-wide synchronisation.  They cannot supply
the split-KV workspace `plx_decode` asks for, so `plx_decode_static` keeps that
scratch in a fixed 4 MiB array inside the library.  This test drives the entry
point through the C ABI (ctypes), twice in a row with different shapes -- the
second call finds the first call's leftovers in the shared array -- and compares
each result with the ordinary `plx_decode` entry point given a caller workspace.
It also checks that a problem too large for the array is refused, not truncated.

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


def test_static_scratch_matches_caller_workspace_on_two_calls_in_a_row():
    # call 1: 16 (batch, head) pairs x 8 splits, D = 128
    got, expect = _both_entry_points(*_inputs(2, 8, 8, 4096, 128, 71), n_splits=8, window=-1)
    assert_close(got.float(), expect.float(), DECODE_REL_L2, DECODE_MAX_REL, "first call")
    # call 2, straight after, another shape: the counters of this layout sit where call 1 left partial sums
    got, expect = _both_entry_points(*_inputs(3, 4, 2, 3000, 64, 75), n_splits=5, window=1000, seqused=[3000, 17, 1500])
    assert_close(got.float(), expect.float(), DECODE_REL_L2, DECODE_MAX_REL, "second call")
    # and the first shape again
    got, expect = _both_entry_points(*_inputs(2, 8, 8, 4096, 128, 79), n_splits=8, window=-1)
    assert_close(got.float(), expect.float(), DECODE_REL_L2, DECODE_MAX_REL, "third call")


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
