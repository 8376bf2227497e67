"""parallax_b200 -- the Parallax attention hot path as hand-written CUDA for
NVIDIA B200 (sm_100a), behind the reference's Python API.

    import parallax                                        # the reference's import name (alias package)
    o = parallax.parallax_func(q, r, k, v)                 # causal training op, autograd
    o = parallax.parallax_varlen_func(q, r, k, v, cu_seqlens=cu)
    o = parallax.parallax_decode(q, r, k_cache, v_cache)   # one token against a KV cache

Same names and argument meaning as ``parallax/__init__.py:84-95`` of the
reference.  All device work runs in ``lib/libplx_sm100.so`` (build it with
``python -m parallax_b200.build``); there is no Triton, PyTorch or CPU fallback.
"""
from .decode import GraphedDecode, parallax_attn_with_kvcache, parallax_decode
from .train import parallax_bwd, parallax_func, parallax_fwd
from .varlen import parallax_varlen_func

__version__ = "0.1.0"

# The reference sets this flag when its optional decode kernel (parallax_attn_with_kvcache,
# GraphedDecode) can be used (parallax/__init__.py:40-66); callers test it before calling them.
# Here those entry points are always built, so the flag is always true.
cute_decode_available: bool = True
decode_available: bool = True

__all__ = [
    "__version__",
    "parallax_func",
    "parallax_varlen_func",
    "parallax_fwd",
    "parallax_bwd",
    "parallax_attn_with_kvcache",
    "parallax_decode",
    "GraphedDecode",
    "cute_decode_available",
]
