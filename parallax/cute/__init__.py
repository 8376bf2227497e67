"""Names of the reference's ``parallax.cute`` sub-package (the SM90 CuTeDSL decode,
parallax/cute/parallax_decode.py:1554-1838), served by the sm_100a decode kernels."""
from parallax_b200 import GraphedDecode, parallax_attn_with_kvcache, parallax_decode

__all__ = ["GraphedDecode", "parallax_attn_with_kvcache", "parallax_decode"]
