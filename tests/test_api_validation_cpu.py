"""Argument checks of the public API raise the reference's exception types
before anything is launched (so they can be exercised without a GPU), and the
ops refuse to run on CPU tensors instead of falling back."""
import pytest
import torch

import parallax_b200 as plx
from parallax_b200.decode import _window_size_to_left


def _t(*shape, dtype=torch.bfloat16):
    return torch.zeros(*shape, dtype=dtype)


def test_public_names_match_the_reference_package():
    for name in ("parallax_func", "parallax_varlen_func", "parallax_fwd", "parallax_bwd", "parallax_decode",
                 "parallax_attn_with_kvcache", "GraphedDecode", "cute_decode_available", "__version__"):
        assert hasattr(plx, name)


def test_the_reference_import_name_resolves_to_this_library():
    """`import parallax` is what code written against the reference does (parallax/__init__.py:84-95 and
    parallax/triton/__init__.py of the reference list these names); here it must give the B200 functions."""
    import parallax
    import parallax.cute
    import parallax.triton

    for name in ("parallax_func", "parallax_varlen_func", "parallax_fwd", "parallax_bwd", "parallax_attn_with_kvcache",
                 "parallax_decode", "GraphedDecode", "cute_decode_available", "__version__"):
        assert name in parallax.__all__ and getattr(parallax, name) is getattr(plx, name)
    assert parallax.cute_decode_available is True and parallax.decode_available is True
    for name in ("parallax_func", "parallax_fwd", "parallax_bwd", "parallax_varlen_func", "parallax_decode"):
        assert getattr(parallax.triton, name) is getattr(plx, name)
    for name in ("GraphedDecode", "parallax_attn_with_kvcache", "parallax_decode"):
        assert getattr(parallax.cute, name) is getattr(plx, name)
    # the fp32 CPU implementation is not part of a library without a CPU path, and asking for it says so
    with pytest.raises(AttributeError, match="no CPU path"):
        parallax.parallax_reference


def test_train_dtype_and_gqa_errors():
    with pytest.raises(TypeError, match="bf16 or fp16"):
        plx.parallax_func(_t(1, 2, 8, 64, dtype=torch.float32), _t(1, 2, 8, 64), _t(1, 2, 8, 64), _t(1, 2, 8, 64))
    with pytest.raises(ValueError, match="divisible"):
        plx.parallax_func(_t(1, 4, 8, 64), _t(1, 4, 8, 64), _t(1, 3, 8, 64), _t(1, 3, 8, 64))


def test_no_cpu_fallback():
    with pytest.raises(RuntimeError, match="no CPU path"):
        plx.parallax_func(_t(1, 2, 8, 64), _t(1, 2, 8, 64), _t(1, 2, 8, 64), _t(1, 2, 8, 64))
    with pytest.raises(RuntimeError, match="no CPU path"):
        plx.parallax_varlen_func(_t(1, 8, 2, 64), _t(1, 8, 2, 64), _t(1, 8, 2, 64), _t(1, 8, 2, 64))
    with pytest.raises(RuntimeError, match="no CPU path"):
        plx.parallax_decode(_t(1, 1, 2, 64), _t(1, 1, 2, 64), _t(1, 8, 2, 64), _t(1, 8, 2, 64))


def test_varlen_errors():
    q = _t(2, 8, 2, 64)
    with pytest.raises(TypeError, match="bf16 or fp16"):
        plx.parallax_varlen_func(q.float(), q, q, q)
    with pytest.raises(ValueError, match="divisible"):
        plx.parallax_varlen_func(_t(1, 8, 4, 64), _t(1, 8, 4, 64), _t(1, 8, 3, 64), _t(1, 8, 3, 64))
    with pytest.raises(ValueError, match="batch size must be 1"):
        plx.parallax_varlen_func(q, q, q, q, cu_seqlens=torch.tensor([0, 8], dtype=torch.int32))
    q1 = _t(1, 8, 2, 64)
    with pytest.raises(TypeError, match="int32 or int64"):
        plx.parallax_varlen_func(q1, q1, q1, q1, cu_seqlens=torch.tensor([0., 8.]))


def test_decode_errors():
    q, k = _t(1, 1, 4, 64), _t(1, 16, 4, 64)
    with pytest.raises(ValueError, match="single query"):
        plx.parallax_decode(_t(1, 2, 4, 64), _t(1, 2, 4, 64), k, k)
    with pytest.raises(ValueError, match="divisible"):
        plx.parallax_decode(q, q, _t(1, 16, 3, 64), _t(1, 16, 3, 64))
    # paged cache: the block table is validated like seqused_k (the reference names the argument but
    # raises NotImplementedError for it, parallax/cute/parallax_decode.py:1627-1632; here it is implemented)
    pages = _t(8, 16, 4, 64)
    with pytest.raises(TypeError, match="page_table must be int32"):
        plx.parallax_attn_with_kvcache(q, q, pages, pages, page_table=torch.zeros(1, 4, dtype=torch.int64))
    with pytest.raises(ValueError, match="page_table must have shape"):
        plx.parallax_attn_with_kvcache(q, q, pages, pages, page_table=torch.zeros(2, 4, dtype=torch.int32))
    with pytest.raises(ValueError, match="same CUDA device"):
        plx.parallax_attn_with_kvcache(q, q, pages, pages, page_table=torch.zeros(1, 4, dtype=torch.int32))
    # L_q > 1 (prefill / extend): the same checks, then the same refusal to run on the CPU
    q4 = _t(1, 4, 4, 64)
    with pytest.raises(ValueError, match="same CUDA device"):
        plx.parallax_attn_with_kvcache(q4, q4, pages, pages, page_table=torch.zeros(1, 4, dtype=torch.int32))
    with pytest.raises(TypeError, match="page_table must be int32"):
        plx.parallax_attn_with_kvcache(q4, q4, pages, pages, page_table=torch.zeros(1, 4, dtype=torch.int64))
    with pytest.raises(RuntimeError, match="no CPU path"):
        plx.parallax_attn_with_kvcache(q4, q4, k, k)
    with pytest.raises(TypeError, match="int32"):
        plx.parallax_attn_with_kvcache(q, q, k, k, seqused_k=torch.tensor([4], dtype=torch.int64))
    with pytest.raises(ValueError, match="shape"):
        plx.parallax_attn_with_kvcache(q, q, k, k, seqused_k=torch.tensor([4, 4], dtype=torch.int32))
    with pytest.raises(ValueError, match="same CUDA device"):
        plx.parallax_attn_with_kvcache(q, q, k, k, seqused_k=torch.tensor([4], dtype=torch.int32))
    with pytest.raises(ValueError, match="right must be <= 0"):
        plx.parallax_attn_with_kvcache(q, q, k, k, window_size=(8, 1))
    with pytest.raises(ValueError, match="window_size must be"):
        plx.parallax_attn_with_kvcache(q, q, k, k, window_size=(1, 2, 3))


def test_window_mapping():
    # reference: parallax/cute/parallax_decode.py:1525-1551
    assert _window_size_to_left(None) == -1
    assert _window_size_to_left((-1, -1)) == -1
    assert _window_size_to_left(7) == 7
    assert _window_size_to_left((128, 0)) == 128
    assert _window_size_to_left((128, -1)) == 128


def test_graphed_decode_argument_errors():
    with pytest.raises(ValueError, match="requires max_kv_len"):
        plx.GraphedDecode(1, 8)
    with pytest.raises(ValueError, match="exactly one"):
        plx.GraphedDecode(1, 8, max_kv_len=64, kv_len=64)
