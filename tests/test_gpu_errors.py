"""Device-side error reporting of the single-pass sampler.  Every wait inside the kernel has a budget; when one runs out
the kernel records which, leaves the rows it could not answer "pending", and returns.  The multi-pass kernel then redoes
those rows, the batch counters say what happened and whirl_check / whirl_sample_rows_host return WHIRL_ERR_TIMEOUT.

The wait is made to run out on the host's request: the library's testing aid shortens the budget and makes the first
CTA's producer leave one bulk copy out, so the stage never fills.  Nothing faults, traps or spins without a limit."""
import numpy as np
import pytest
import torch

import synth
from gpu_util import compare_rows, dev, row_params

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    from whirl_llm_b200 import api
    return api


def case(R=300, V=36868):
    x = synth.normalish(401, (R, V), 2.0)
    f = lambda v, dt=np.float32: np.full(R, v, dtype=dt)
    prm = dict(inv_t=f(1 / 0.8), top_k=f(50, np.uint32), top_p=f(0.9, np.float64), min_p=f(0.05, np.float64))
    u = synth.hash_u01(402, R, 0)
    return x, prm, u


def test_wait_that_runs_out_is_reported_and_rows_are_redone(api, oracle):
    x, prm, u = case()
    R, V = x.shape
    want = oracle.sample_rows(x, kept_cap=8, u=u, threads=4, **prm)
    ws = api.workspace(R, V, "cuda")
    xd = dev(x)
    api.test_waits(20000, True)  # 20 ms per wait; CTA 0 loses a copy of its first row
    try:
        res = api.sample_rows(xd, row_params(prm, u=u), kept_cap=8, ws=ws)
        where = api.check(ws, R)
    finally:
        api.test_waits(0, False)
    cnt = res.counters.cpu().numpy()
    assert where in (1, 3, 4, 5, 11), where
    assert cnt[api.CNT_TIMEOUT] == 1
    # the first CTA's rows (every gridDim-th from row 0) were left pending and done again by the multi-pass kernel
    assert cnt[api.CNT_REDO] >= 2 and cnt[api.CNT_UNRESOLVED] == 0 and cnt[api.CNT_NAN_ROWS] == 0
    compare_rows(res, want, u=u)
    # the next call on the same workspace, with the defaults back, reports nothing
    res = api.sample_rows(xd, row_params(prm, u=u), kept_cap=8, ws=ws)
    assert api.check(ws, R) == 0
    cnt = res.counters.cpu().numpy()
    assert cnt[api.CNT_TIMEOUT] == 0 and cnt[api.CNT_REDO] == 0
    compare_rows(res, want, u=u)


def test_host_call_returns_timeout(api, oracle):
    x, prm, u = case(R=200)
    R, V = x.shape
    want = oracle.sample_rows(x, kept_cap=8, u=u, threads=4, **prm)
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
    hp = dict(inv_t=pin(prm["inv_t"]), top_k=pin(prm["top_k"].astype(np.int32)), top_p=pin(prm["top_p"]), min_p=pin(prm["min_p"]), u=pin(u))
    out = dict(token=torch.full((R,), -1, dtype=torch.int32).pin_memory(), counters=torch.zeros(api.CNT_WORDS, dtype=torch.int32))
    api.test_waits(20000, True)
    try:
        with pytest.raises(api.WhirlError) as ei:
            api.sample_rows_host(pin(x), hp, R, V, api.F32, out)
    finally:
        api.test_waits(0, False)
    assert ei.value.status == api.ERR_TIMEOUT
    assert out["counters"][api.CNT_TIMEOUT] == 1 and out["counters"][api.CNT_UNRESOLVED] == 0
    assert np.array_equal(out["token"].numpy(), want["token"].astype(np.int32))  # (the outputs were written all the same)
    out["token"].fill_(-1)
    api.sample_rows_host(pin(x), hp, R, V, api.F32, out)
    assert np.array_equal(out["token"].numpy(), want["token"].astype(np.int32))


def test_nan_rows_are_counted(api, oracle):
    x, prm, u = case(R=160)
    x[5, 1000] = np.nan
    x[77, :4] = np.nan
    R, V = x.shape
    want = oracle.sample_rows(x, kept_cap=8, u=u, threads=4, **prm)
    res = api.sample_rows(dev(x), row_params(prm, u=u), kept_cap=8)
    cnt = res.counters.cpu().numpy()
    assert cnt[api.CNT_NAN_ROWS] == 2 and cnt[api.CNT_REDO] >= 2 and cnt[api.CNT_TIMEOUT] == 0
    keep = np.ones(R, dtype=bool)
    keep[[5, 77]] = False
    tok = res.token.cpu().numpy()
    assert np.array_equal(tok[keep], want["token"][keep].astype(np.int32))
    assert (res.status.cpu().numpy()[keep] == api.ROW_DONE).all()


def test_history_length_is_clamped_to_the_history_row(api, oracle):
    """hist_len above hist_stride (or above the library's 4096) reads min(hist_len, hist_stride, 4096) ids, in the
    single-pass kernel and in the multi-pass one (rows with a large top_k, rows kept past 256 candidates) alike."""
    R, V, H = 96, 36868, 64
    x = synth.normalish(411, (R, V), 2.0)
    f = lambda v, dt=np.float32: np.full(R, v, dtype=dt)
    prm = dict(inv_t=f(1 / 0.8), top_k=f(50, np.uint32), top_p=f(0.9, np.float64), min_p=f(0.0, np.float64))
    prm["top_k"][1::3] = 2000            # multi-pass kernel
    prm["top_k"][2::3] = 0
    prm["top_p"][2::3] = 0.999           # second candidate level
    u = synth.hash_u01(412, R, 0)
    hist = synth.zipf_history(413, R, H, V, 1.1)
    hist_len = np.array([0, 10, 64, 100, 5000, 2 ** 31 - 1], dtype=np.int64)[np.arange(R) % 6].astype(np.int32)
    pen = dict(hist=hist, rep=f(1.3), pres=f(0.7), freq=f(0.4))
    want = oracle.sample_rows(x, kept_cap=8, u=u, threads=4, hist_len=np.minimum(hist_len, H).astype(np.uint32), **prm, **pen)
    res = api.sample_rows(dev(x), row_params(prm, u=u, hist_len=hist_len, **pen), kept_cap=8)
    compare_rows(res, want, u=u)


def test_rows_redone_by_the_multi_pass_kernel_still_reach_the_second_level(api, oracle):
    """A rising row overflows the single-pass kernel's candidate log and is redone by the multi-pass kernel at the first
    level; with flat logits and a top-p close to one its kept set reaches past 256 candidates, so the redo has to go on
    to the second level (16384 candidates) instead of leaving the row unanswered."""
    R, V = 24, 36868
    x = synth.normalish(421, (R, V), 0.3)
    x[::2] = np.sort(x[::2], axis=1)
    f = lambda v, dt=np.float32: np.full(R, v, dtype=dt)
    prm = dict(inv_t=f(1.0), top_k=f(0, np.uint32), top_p=f(0.5, np.float64), min_p=f(0.0, np.float64))
    u = synth.hash_u01(422, R, 0)
    want = oracle.sample_rows(x, kept_cap=8, u=u, threads=4, **prm)
    assert (want["n"] > 256).all() and (want["n"] <= 16384).all()
    res = api.sample_rows(dev(x), row_params(prm, u=u), kept_cap=8)
    compare_rows(res, want, u=u)
    cnt = res.counters.cpu().numpy()
    assert cnt[api.CNT_REDO] >= R // 2 and cnt[api.CNT_ESCALATED] == R and cnt[api.CNT_UNRESOLVED] == 0


def test_large_top_k_on_adversarial_rows(api, oracle):
    """Rows keeping more than 64 candidates take their first threshold from a guess made on the first 8192 logits.
    Falling rows (the guess is far too high: fewer than top_k candidates get logged), rising rows (every logit beats the
    threshold so far: the log overflows), constant rows and rows with few distinct values must all come back right: the
    single-pass kernel hands what it cannot finish to the multi-pass kernel."""
    R, V = 64, 65536
    x = synth.normalish(431, (R, V), 2.0)
    x[0::8] = np.sort(x[0::8], axis=1)
    x[1::8] = -np.sort(-x[1::8], axis=1)
    x[2::8] = 0.75
    x[3::8] = np.round(x[3::8])
    x[4::8, :8192] -= 6.0                                  # a first iteration that says nothing about the rest
    x[5::8, :8192] += 6.0
    f = lambda v, dt=np.float32: np.full(R, v, dtype=dt)
    prm = dict(inv_t=f(1.0), top_k=f(300, np.uint32), top_p=f(0.95, np.float64), min_p=f(0.0, np.float64))
    prm["top_k"][R // 2:] = 1000
    u = synth.hash_u01(432, R, 0)
    want = oracle.sample_rows(x, kept_cap=1024, u=u, threads=4, **prm)
    res = api.sample_rows(dev(x), row_params(prm, u=u), kept_cap=1024)
    compare_rows(res, want, u=u)
    cnt = res.counters.cpu().numpy()
    assert cnt[api.CNT_REDO] >= R // 4 and cnt[api.CNT_UNRESOLVED] == 0
    # the candidates entry point on the same rows
    ids, vals, stats = api.topk_rows(dev(x), 1000, inv_t=1.0)
    wi, wv, ws = oracle.topk_rows(x, 1000, 1.0)
    assert np.array_equal(ids.cpu().numpy(), wi) and np.array_equal(vals.cpu().numpy(), wv)
    assert np.array_equal(stats.cpu().numpy()[:, 0], ws[:, 0])
    np.testing.assert_allclose(stats.cpu().numpy()[:, 1], ws[:, 1], rtol=1e-5)
