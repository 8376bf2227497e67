"""C-ABI checks that need no GPU: the library loads, exports every symbol the
header declares, and validates arguments before touching a device."""
import ctypes as C
import os
import re

import pytest

from parallax_b200 import _cabi
from parallax_b200._paths import INCLUDE, LIB_PATH


def header_symbols():
    text = open(os.path.join(INCLUDE, "plx_abi.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(plx_[a-z_0-9]+)\s*\(", text)))


def test_library_is_built_in_tree():
    assert os.path.exists(LIB_PATH), "run `python -m parallax_b200.build`"


def test_every_declared_symbol_is_exported():
    lib = C.CDLL(LIB_PATH)
    names = header_symbols()
    assert len(names) >= 11
    for name in names:
        assert hasattr(lib, name), f"{name} declared in plx_abi.h but not exported"
    assert set(names) == set(_cabi.SYMBOLS)


def test_version_and_strerror():
    lib = _cabi.lib()
    assert lib.plx_abi_version() == _cabi.ABI_VERSION
    assert lib.plx_strerror(0) == b"ok"
    for code in (-1, -2, -3, -4, -5):
        assert len(lib.plx_strerror(code)) > 3


def _train_problem(**kw):
    p = _cabi.TrainProblem()
    p.dtype, p.batch, p.heads_q, p.heads_kv, p.len_q, p.len_k, p.head_dim = 0, 2, 8, 8, 1024, 1024, 128
    p.window_left, p.qk_scale = -1, 0.088
    p.q_stride_b, p.q_stride_h, p.q_stride_t = 8 * 1024 * 128, 1024 * 128, 128
    p.kv_stride_b, p.kv_stride_h, p.kv_stride_t = 8 * 1024 * 128, 1024 * 128, 128
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def test_train_workspace_and_validation():
    lib = _cabi.lib()
    n = C.c_size_t(0)
    assert lib.plx_train_workspace_bytes(C.byref(_train_problem()), C.byref(n)) == 0
    assert n.value == (2 * 8 * 1024 + 64) * 12 * 4
    bad = [dict(heads_kv=3), dict(batch=0), dict(window_left=-2), dict(q_stride_t=100)]
    for kw in bad:
        assert lib.plx_train_workspace_bytes(C.byref(_train_problem(**kw)), C.byref(n)) == -1, kw
    for kw in (dict(head_dim=96), dict(dtype=7)):
        assert lib.plx_train_workspace_bytes(C.byref(_train_problem(**kw)), C.byref(n)) == -2, kw
    # null pointers are rejected before any device call
    p = _train_problem()
    assert lib.plx_train_fwd(C.byref(p), None, None, None, None, None, None, None, None, None, None) == -1


def test_decode_split_heuristic_and_workspace():
    lib = _cabi.lib()
    assert lib.plx_decode_choose_splits(64, 8, 32768, 148) >= 1
    assert lib.plx_decode_choose_splits(1, 8, 40, 148) == 1           # too few keys to split
    assert lib.plx_decode_choose_splits(4096, 8, 1024, 148) == 1      # enough (batch, head) pairs already
    assert lib.plx_decode_choose_splits(4096, 8, 32768, 148) == 32    # long rows: at most ~1024 keys per warp
    s = lib.plx_decode_choose_splits(1, 8, 32768, 148)
    assert 64 <= s <= 256 and 32768 // s >= 32                        # PLX_DECODE_MAX_SPLITS = 256
    assert lib.plx_decode_choose_splits(16, 8, 4096, 148) == 18                  # 16 * 8 * 18 warps <= 148 SMs * 16
    assert lib.plx_decode_choose_splits_gqa(16, 8, 8, 4096, 148) == 18             # one q head per kv head: same rule
    assert lib.plx_decode_choose_splits_gqa(16, 32, 8, 8192, 148) == 8             # 16 * 8 * 8 warps = 86 % of 148 SMs * 8
    assert lib.plx_decode_choose_splits_gqa(64, 32, 8, 8192, 148) == 2             # 1024 of 1184 resident warps
    assert lib.plx_decode_choose_splits_gqa(1, 32, 8, 256, 148) == 4               # at least 64 keys per split
    # few (batch, head) pairs: groups of eight splits, as a cluster of up to eight CTAs while that is faster
    assert lib.plx_decode_choose_splits(1, 8, 512, 148) == 32                      # at least 16 keys per split
    assert lib.plx_decode_choose_splits(1, 8, 2048, 148) == 64
    assert lib.plx_decode_choose_splits(1, 8, 4096, 148) == 64                     # up to 6144 keys for at most 8 pairs
    assert lib.plx_decode_choose_splits(4, 8, 4096, 148) == 32                     # ... and for 17 to 32 pairs
    assert lib.plx_decode_choose_splits(2, 8, 4096, 148) == 144                    # 16 pairs: every warp resident, through L2
    assert lib.plx_decode_choose_splits(1, 8, 8192, 148) == 256                    # longer rows: the cap of 256 splits
    p = _cabi.DecodeProblem()
    p.dtype, p.batch, p.heads_q, p.heads_kv, p.cache_len, p.head_dim = 0, 4, 8, 8, 4096, 128
    p.window_left, p.n_splits, p.qk_scale = -1, 5, 0.088
    p.kv_stride_b, p.kv_stride_t, p.kv_stride_h = 4096 * 8 * 128, 8 * 128, 128
    n = C.c_size_t(0)
    assert lib.plx_decode_workspace_bytes(C.byref(p), C.byref(n)) == 0
    assert n.value == (4 * 8 * 5 * (2 * 128 + 4) + 4 * 8) * 4      # 5 splits: single-level merge, no group records
    p.n_splits = 70                                                             # two-level merge: 5 groups of 16
    assert lib.plx_decode_workspace_bytes(C.byref(p), C.byref(n)) == 0
    assert n.value == (4 * 8 * (70 + 5) * (2 * 128 + 4) + 4 * 8 * (1 + 5)) * 4
    p.n_splits = 257
    assert lib.plx_decode_workspace_bytes(C.byref(p), C.byref(n)) == -1           # PLX_DECODE_MAX_SPLITS
    p.n_splits = 5
    p.heads_kv = 3
    assert lib.plx_decode_workspace_bytes(C.byref(p), C.byref(n)) == -1
    assert lib.plx_decode_merge(None, 1, 1, 128, 0, None, None) == -1


def test_exchange_sizes_and_argument_checks():
    lib = _cabi.lib()
    rec = 2 * 128 + 4
    assert lib.plx_decode_exchange_bytes(8, 32, 128) == 2 * 8 * 32 * rec * 4 + 2 * 8 * 32 * 4 + 32 * 4   # records + stamps (two parities) + step counters
    assert lib.plx_decode_exchange_bytes(0, 32, 128) == 0 and lib.plx_decode_exchange_bytes(2, 32, 96) == 0
    assert lib.plx_decode_exchange_merge(None, None, None, None) == -1
    x = _cabi.Exchange()
    x.world, x.rank, x.n_records, x.head_dim, x.dtype = 17, 0, 4, 128, 0
    assert lib.plx_decode_exchange_merge(C.byref(x), C.c_void_p(16), C.c_void_p(16), None) == -1   # more than 16 ranks
    x.world, x.rank = 2, 2
    assert lib.plx_decode_exchange_merge(C.byref(x), C.c_void_p(16), C.c_void_p(16), None) == -1   # rank outside the world
    x.rank = 0
    assert lib.plx_decode_exchange_merge(C.byref(x), C.c_void_p(16), C.c_void_p(16), None) == -1   # inbox pointers missing


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setattr(_cabi, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _cabi.lib()
