"""``parallax`` -- the import name of the reference package, served by the B200 build.

Code written against the reference (``import parallax`` /
``from parallax import parallax_func``) runs unchanged: every public name of
``parallax/__init__.py:84-95`` of the reference is re-exported here from
:mod:`parallax_b200`, whose device work is hand-written sm_100a CUDA behind a C
ABI.  ``parallax.triton`` and ``parallax.cute`` mirror the reference's
sub-packages for code that imports the decode front ends from there
(``parallax/triton/__init__.py:8``, ``parallax/cute/__init__.py``).

``parallax_reference`` (the fp32 PyTorch implementation, ``parallax/reference.py``
upstream) is deliberately absent: this package has no CPU path, and a name that
silently computed on the CPU would defeat that.  Accessing it raises an
``AttributeError`` that says so.
"""
from parallax_b200 import (
    GraphedDecode,
    __version__,
    cute_decode_available,
    parallax_attn_with_kvcache,
    parallax_bwd,
    parallax_decode,
    parallax_func,
    parallax_fwd,
    parallax_varlen_func,
)

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


def __getattr__(name):
    if name == "decode_available":          # the reference's deprecated alias (parallax/__init__.py:68-81)
        return cute_decode_available
    if name == "parallax_reference":
        raise AttributeError(
            "parallax.parallax_reference is not provided by the B200 build: the library has no CPU path. "
            "Use the upstream package's parallax/reference.py as the fp32 oracle.")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
