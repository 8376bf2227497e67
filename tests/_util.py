"""Helpers shared by the tests: golden-vector loading and parity gates."""
import glob
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Parity gates against the fp32 oracle for bf16 kernels (inputs iid N(0,1)):
# relative L2 <= 1e-2 and max-abs / max|ref| <= 2e-2 on o, dq, dr, dk, dv;
# decode: both <= 1e-2 (the reference's own gate is max-abs / max|ref| < 1e-2,
# tests/conftest.py:53-66 of the reference).
TRAIN_REL_L2 = 1e-2
TRAIN_MAX_REL = 2e-2
DECODE_REL_L2 = 1e-2
DECODE_MAX_REL = 1e-2


def golden_names(kind):
    return sorted(os.path.basename(p)[len(kind) + 1:-4] for p in glob.glob(os.path.join(GOLDEN, f"{kind}_*.npz")))


def load_golden(kind, name):
    """Returns a dict of tensors; bf16 inputs are restored from their bit patterns."""
    z = np.load(os.path.join(GOLDEN, f"{kind}_{name}.npz"))
    out = {}
    for key in z.files:
        a = z[key]
        if a.dtype == np.int16:
            out[key] = torch.from_numpy(a.copy()).view(torch.bfloat16)
        elif a.ndim == 0:
            out[key] = int(a)
        else:
            out[key] = torch.from_numpy(a.copy())
    return out


def seeded_bf16(shape, seed, mul=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * mul).to(torch.bfloat16)


def assert_close(got, ref, rel_l2, max_rel, what="", atol=1e-4):
    """Gate `got` against `ref`: relative L2 and max-abs / max|ref|.  A tensor whose
    largest absolute error is below `atol` passes outright (gradients that are
    exactly zero in exact arithmetic come out as ~1e-7 noise on both sides)."""
    from oracle.parallax_oracle import error_metrics

    assert torch.isfinite(got.float()).all(), f"{what}: non-finite values"
    e = error_metrics(got, ref)
    if e["max_abs"] <= atol:
        return e
    assert e["rel_l2"] <= rel_l2 and e["max_rel"] <= max_rel, f"{what}: {e}"
    return e
