"""Parity at the benchmark's own sizes.  The logits are drawn on the device (a seeded torch generator) and copied to the
host for the oracle, so both sides read the same bits.

  - the penalised-sampling configuration: 64 x 151,936 f32, histories of 4096 Zipf(1.1) ids, with statistics and kept sets;
  - the headline: 1024 x 262,144 f32 with the same settings, tokens only (the call the benchmark times), all rows
    against the oracle, plus two properties that need no oracle: the call is idempotent, and greedy rows equal the
    argmax kernel's picks;
  - the continuous-batching mix: 1024 x 262,144 bf16, 1 % of the entries + 10, per-row greedy / temperature / top-k up to
    1024 / top-p.
A draw within 1e-6 of a cumulative boundary may pick the neighbour (counted; none is expected at these sizes)."""
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


def device_normal(seed, shape, sigma):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return torch.empty(shape, dtype=torch.float32, device="cuda").normal_(0.0, sigma, generator=g)


def penalised_case(rows, vocab, seed):
    f = lambda v, dt=np.float32: np.full(rows, v, dtype=dt)
    prm = dict(inv_t=f(1 / 0.8), top_k=f(50, np.uint32), top_p=f(0.9, np.float64), min_p=f(0.05, np.float64))
    pen = dict(hist=synth.zipf_history(seed, rows, 4096, vocab, 1.1), hist_len=f(4096, np.int32), rep=f(1.1), pres=f(0.5), freq=f(0.3))
    u = synth.hash_u01(seed + 1, rows, 0)
    return prm, pen, u


def oracle_pen(pen):
    return {k: (v.astype(np.uint32) if k == "hist_len" else v) for k, v in pen.items()}


def test_penalised_sampling_64_x_151936(api, oracle):
    rows, vocab = 64, 151936
    xd = device_normal(11, (rows, vocab), 2.5)
    prm, pen, u = penalised_case(rows, vocab, 12)
    want = oracle.sample_rows(xd.cpu().numpy(), kept_cap=64, u=u, threads=8, **prm, **oracle_pen(pen))
    res = api.sample_rows(xd, row_params(prm, u=u, **pen), kept_cap=64)
    compare_rows(res, want, u=u)
    assert int(res.counters[api.CNT_UNRESOLVED].item()) == 0


def test_headline_1024_x_262144_tokens_only(api, oracle):
    rows, vocab = 1024, 262144
    xd = device_normal(21, (rows, vocab), 2.5)
    prm, pen, u = penalised_case(rows, vocab, 22)
    want = oracle.sample_rows(xd.cpu().numpy(), kept_cap=0, u=u, threads=16, **prm, **oracle_pen(pen))
    rp = row_params(prm, u=u, **pen)
    res = api.sample_rows(xd, rp, want_stats=False)
    tok = res.token.cpu().numpy()
    assert (res.status.cpu().numpy() == api.ROW_DONE).all()
    diff = np.nonzero(tok != want["token"].astype(np.int32))[0]
    assert len(diff) == 0, (diff[:8], tok[diff[:8]], want["token"][diff[:8]])
    assert np.array_equal(res.n_kept.cpu().numpy(), want["n"])
    cnt = res.counters.cpu().numpy()
    assert cnt[api.CNT_UNRESOLVED] == 0 and cnt[api.CNT_TIMEOUT] == 0
    # idempotence: the same call again, into the same result
    again = api.sample_rows(xd, rp, want_stats=False)
    assert torch.equal(again.token, res.token)
    # greedy rows through the sampler == the argmax kernel == the oracle's first maximum (on the raw logits: no history)
    greedy = api.sample_rows(xd, row_params(dict(greedy=np.ones(rows, dtype=np.uint8))), want_stats=False)
    am = api.argmax_rows(xd)
    assert torch.equal(greedy.token, am)
    xh = xd[:64].cpu().numpy()
    assert np.array_equal(am[:64].cpu().numpy(), np.array([oracle.first_max(xh[r]) for r in range(64)], dtype=np.int32))


def test_continuous_batching_mix_1024_x_262144_bf16(api, oracle):
    rows, vocab = 1024, 262144
    g = torch.Generator(device="cuda")
    g.manual_seed(31)
    x = torch.empty((rows, vocab), dtype=torch.float32, device="cuda").normal_(0.0, 3.0, generator=g)
    x += 10.0 * (torch.rand((rows, vocab), generator=g, device="cuda") < 0.01)
    xb = x.to(torch.bfloat16)
    del x
    r = np.random.default_rng(32).random((4, rows))
    prm = dict(inv_t=(1.0 / (0.5 + 0.7 * r[0])).astype(np.float32), top_k=(1 + np.floor(r[1] * 1024)).clip(1, 1024).astype(np.uint32),
               top_p=0.8 + 0.2 * r[2], greedy=(r[3] < 0.25).astype(np.uint8))
    u = synth.hash_u01(33, rows, 0)
    bits = xb.view(torch.int16).cpu().numpy().view(np.uint16)
    want = oracle.sample_rows(bits, kept_cap=16, u=u, threads=16, **prm)
    res = api.sample_rows(xb, row_params(prm, u=u), kept_cap=16)
    compare_rows(res, want, u=u)
    cnt = res.counters.cpu().numpy()
    assert cnt[api.CNT_UNRESOLVED] == 0 and cnt[api.CNT_TIMEOUT] == 0
