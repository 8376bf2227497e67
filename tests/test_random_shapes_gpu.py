"""Seeded random shapes of the training and decode ops against the CPU oracle: head_dim, grouped heads,
batch, unequal query / key lengths, sliding windows, both 16-bit dtypes, runtime lengths.  The fixed cases
of the other test files pin known edges; this one walks the space in between."""
import random

import pytest
import torch

import parallax_b200 as plx
from oracle import parallax_oracle as orc
from tests._util import DECODE_MAX_REL, DECODE_REL_L2, TRAIN_MAX_REL, TRAIN_REL_L2, assert_close, seeded_bf16
from tests.test_train_gpu import make, run_gpu
from tests import test_varlen_gpu as tv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", range(6))
def test_training_op_on_random_shapes(seed):
    rng = random.Random(9000 + seed)
    for _ in range(14):
        d = rng.choice([64, 128])
        hkv = rng.choice([1, 2, 4])
        hq = hkv * rng.choice([1, 1, 2, 4])
        bsz = rng.choice([1, 2, 3])
        lq = rng.choice([rng.randint(8, 90), rng.randint(90, 400), rng.randint(400, 900)])
        lk = lq if rng.random() < 0.6 else lq + rng.randint(1, 300)
        window = rng.choice([-1, -1, -1, rng.randint(1, 64), rng.randint(64, 500)])
        dtype = rng.choice([torch.bfloat16, torch.bfloat16, torch.float16])
        q, r, k, v, go = make(bsz, hq, hkv, lq, lk, d, rng.randint(1, 10 ** 6), dtype=dtype)
        got = run_gpu(q, r, k, v, go, window)
        ref_o = orc.train_forward(q, r, k, v, None, window)["o"]
        ref_g = orc.train_backward(q, r, k, v, go.float(), None, window)
        what = f"B={bsz} Hq={hq} Hkv={hkv} Lq={lq} Lk={lk} D={d} W={window} {dtype}"
        for name, g, e in zip(("o", "dq", "dr", "dk", "dv"), got, (ref_o, *ref_g)):
            assert_close(g, e, TRAIN_REL_L2, TRAIN_MAX_REL, f"{what} {name}")


@pytest.mark.parametrize("seed", range(4))
def test_packed_op_on_random_sequence_lists(seed):
    rng = random.Random(9200 + seed)
    for _ in range(6):
        d = rng.choice([64, 128])
        hkv = rng.choice([1, 2, 4])
        hq = hkv * rng.choice([1, 2, 4])
        n_seq = rng.randint(1, 12)
        # lengths around the tile sizes, with empty sequences in between (the reference allows them)
        lens = [rng.choice([0, 1, rng.randint(2, 70), rng.randint(60, 140), rng.randint(120, 420)]) for _ in range(n_seq)]
        if sum(lens) == 0:
            lens[0] = 33
        window = rng.choice([-1, -1, rng.randint(1, 64), rng.randint(64, 300)])
        q, r, k, v, go, cu = tv.make(lens, hq, hkv, d, rng.randint(1, 10 ** 6))
        got = tv.run_gpu(q, r, k, v, go, cu, window)
        ref_o = orc.varlen_forward(q, r, k, v, cu, None, window)["o"]
        ref_g = orc.varlen_backward(q, r, k, v, go.float(), cu, None, window)
        loosen = 8.0 if min(n for n in lens if n > 0) < 8 else 1.0     # as in the dense edge-length test
        for name, g, e in zip(("o", "dq", "dr", "dk", "dv"), got, (ref_o, *ref_g)):
            assert_close(g, e, TRAIN_REL_L2 * loosen, TRAIN_MAX_REL * loosen, f"lens={lens} Hq={hq} Hkv={hkv} D={d} W={window} {name}")


@pytest.mark.parametrize("seed", range(4))
def test_decode_op_on_random_shapes(seed):
    rng = random.Random(9100 + seed)
    for _ in range(20):
        d = rng.choice([64, 128])
        hkv = rng.choice([1, 2, 4, 8])
        hq = hkv * rng.choice([1, 1, 1, 2, 4, 8])
        bsz = rng.choice([1, 1, 2, 3, 5, 8, 17])
        kv_len = rng.choice([rng.randint(1, 200), rng.randint(200, 3000), rng.randint(3000, 9000)])
        window = rng.choice([-1, -1, rng.randint(0, 50), rng.randint(50, 3000)])
        q = seeded_bf16((bsz, 1, hq, d), rng.randint(1, 10 ** 6))
        r = seeded_bf16((bsz, 1, hq, d), rng.randint(1, 10 ** 6), 0.5)
        k = seeded_bf16((bsz, kv_len, hkv, d), rng.randint(1, 10 ** 6))
        v = seeded_bf16((bsz, kv_len, hkv, d), rng.randint(1, 10 ** 6))
        used = [rng.randint(1, kv_len) for _ in range(bsz)] if rng.random() < 0.4 else None
        su = None if used is None else torch.tensor(used, dtype=torch.int32, device="cuda")
        out = plx.parallax_decode(q.cuda(), r.cuda(), k.cuda(), v.cuda(), None, window_size_left=window, seqused_k=su)
        ref = orc.decode(q, r, k, v, window_size_left=window, seqused_k=None if used is None else torch.tensor(used))
        assert_close(out.float().cpu(), ref, DECODE_REL_L2, DECODE_MAX_REL,
                     f"B={bsz} Hq={hq} Hkv={hkv} T={kv_len} D={d} W={window} seqused={used is not None}")
