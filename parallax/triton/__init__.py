"""Names of the reference's ``parallax.triton`` sub-package (``parallax/triton/__init__.py``),
served by the sm_100a kernels.  ``parallax_decode`` here has the Triton front end's
signature ``(q, r, k, v, qk_scale=None, *, window_size_left=-1, cache_start=None)``
(parallax/triton/parallax_decode.py:100-107); the B200 function accepts it as a subset."""
from parallax_b200 import parallax_bwd, parallax_decode, parallax_func, parallax_fwd, parallax_varlen_func

__all__ = ["parallax_func", "parallax_fwd", "parallax_bwd", "parallax_varlen_func", "parallax_decode"]
