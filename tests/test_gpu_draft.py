"""draft_sample_rows on the GPU, as the reference's kernel test states it (tests/kernels/test_misc.cpp:357-480): the support
of q exact, its probabilities within 1e-4 relative, the drawn token equal to the race draw from the written q; NaN logits
are never candidates; rows that do not sample or whose chain stopped are left alone; ids go through the vocabulary map."""
import numpy as np
import pytest
import torch

import synth
from gpu_util import dev
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _run(api, x, tks, tps, mps, its, keys, r=1, on=None, ctl=None, vmap=None):
    rows = x.shape[0]
    ctl_all = torch.zeros(rows * 64, dtype=torch.int32, device="cuda") if ctl is None else dev(ctl)
    area = dev(np.arange(rows, dtype=np.int32) * 64)
    qbuf = torch.zeros(rows * 72, dtype=torch.int32, device="cuda")
    i32 = lambda v: dev(np.asarray(v, dtype=np.int32))
    f32 = lambda v: dev(np.asarray(v, dtype=np.float32))
    api.draft_sample_rows(dev(x), ctl_all, area, r, i32(np.ones(rows) if on is None else on), i32(tks), i32(np.arange(rows) * 72),
                          f32(its), f32(tps), f32(mps), dev(np.asarray(keys, dtype=np.uint64).view(np.int64)), qbuf,
                          vmap=None if vmap is None else dev(vmap))
    torch.cuda.synchronize()
    return ctl_all.cpu().numpy().reshape(rows, 64), qbuf.cpu().numpy().reshape(rows, 72)


def _check(oracle, x, tks, tps, mps, its, keys, ctl, q, r=1, vmap=None):
    for b in range(x.shape[0]):
        tok, words = oracle.draft_sample_row(x[b], tks[b], np.float32(its[b]), np.float32(tps[b]), np.float32(mps[b]), int(keys[b]), vmap=vmap)
        n = int(words[0])
        assert q[b, 0] == n, (b, q[b, 0], n)
        assert np.array_equal(q[b, 1:1 + n], words[1:1 + n])
        gp, wp = q[b, 33:33 + n].view(np.float32), words[33:33 + n].view(np.float32)
        np.testing.assert_allclose(gp, wp, rtol=1e-4)
        assert np.isfinite(gp).all()
        got = orc.QDist(n=n)
        for i in range(n):
            got.id[i], got.p[i] = int(q[b, 1 + i]), float(gp[i])
        assert ctl[b, 16 + r] == oracle.spec_sample_race(got, int(keys[b]))  # the draw is the race over the WRITTEN q


def test_reference_kernel_test_shape(oracle):
    from whirl_llm_b200 import api
    n = 248320
    x = synth.normalish(4242, (3, n), 3.0)
    x[1, 100] = x[1, 9000] = 50.0
    x[2, n - 1] = 60.0
    tks, tps, mps, its = [20, 0, 5], [0.95, 0.8, 1.0], [0.0, 0.0, 0.05], [1 / 0.7, 1.0, 1 / 0.6]
    keys = [oracle.race_base(1234, 7), oracle.race_base(42, 0), oracle.race_base(987654321, 100000)]
    ctl, q = _run(api, x, tks, tps, mps, its, keys)
    _check(oracle, x, tks, tps, mps, its, keys, ctl, q)


def test_nan_logits_skips_and_map(oracle):
    from whirl_llm_b200 import api
    n = 50000
    x = synth.normalish(77, (4, n), 3.0)
    am = int(np.argmax(x[0]))
    nan_at = [am, (am + 17) % n, (am + 1001) % n]
    x[0, nan_at] = np.nan
    tks, tps, mps, its = [20, 20, 20, 3], [0.95, 0.95, 0.95, 1.0], [0.0, 0.0, 0.0, 0.0], [1 / 0.7] * 4
    keys = [oracle.race_base(77, 3 + i) for i in range(4)]
    ctl0 = np.zeros((4, 64), dtype=np.int32)
    ctl0[:, 17] = -5            # the greedy draft already there
    ctl0[2, 48], ctl0[2, 49] = 1, 1  # row 2: chain stopped at r = 1
    perm = (100000 + 3 * np.arange(n)).astype(np.int32)
    ctl, q = _run(api, x, tks, tps, mps, its, keys, on=[1, 0, 1, 1], ctl=ctl0.reshape(-1), vmap=perm)
    # row 0: NaNs are never candidates, q is finite
    ids0 = q[0, 1:1 + q[0, 0]]
    assert not set(perm[nan_at].tolist()) & set(ids0.tolist())
    _check(oracle, x[[0, 3]], [tks[0], tks[3]], [tps[0], tps[3]], [mps[0], mps[3]], [its[0], its[3]], [keys[0], keys[3]],
           ctl[[0, 3]], q[[0, 3]], vmap=perm)
    # rows 1 (on = 0) and 2 (stopped chain) are untouched
    assert ctl[1, 17] == -5 and ctl[2, 17] == -5 and q[1, 0] == 0 and q[2, 0] == 0
