"""whirl_sample_rows_host: the fused sampler on HOST buffers (it copies the logits up in blocks of rows on two streams
and the tokens back).  Same tokens as the oracle, across several of its row blocks, with penalties and without."""
import numpy as np
import pytest
import torch

import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    from whirl_llm_b200 import api
    return api


def test_host_buffers_match_oracle(api, oracle):
    R, V, H = 1100, 36868, 256  # 147 KB per row: three 64 MiB blocks of rows
    x = synth.normalish(31, (R, V), 2.0)
    f = lambda v, dt=np.float32: np.full(R, v, dtype=dt)
    prm = dict(inv_t=f(1 / 0.8), top_k=f(50, np.uint32), top_p=f(0.9, np.float64), min_p=f(0.05, np.float64))
    prm["top_k"][3::7] = 1
    u = synth.hash_u01(32, R, 0)
    hist = synth.zipf_history(33, R, H, V, 1.1)
    hist_len = np.full(R, H, dtype=np.int32)
    hist_len[::9] = 0
    pen = dict(hist=hist, hist_len=hist_len, rep=f(1.1), pres=f(0.5), freq=f(0.3))
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
    for with_pen in (False, True):
        extra = pen if with_pen else {}
        want = oracle.sample_rows(x, kept_cap=8, u=u, threads=4, **prm, **{k: (v.astype(np.uint32) if k == "hist_len" else v) for k, v in extra.items()})
        hp = dict(inv_t=pin(prm["inv_t"]), top_k=pin(prm["top_k"].astype(np.int32)), top_p=pin(prm["top_p"]), min_p=pin(prm["min_p"]), u=pin(u))
        if with_pen:
            hp.update(hist=pin(hist), hist_len=pin(hist_len), rep=pin(pen["rep"]), pres=pin(pen["pres"]), freq=pin(pen["freq"]))
        out = dict(token=torch.full((R,), -1, dtype=torch.int32).pin_memory())
        api.sample_rows_host(pin(x), hp, R, V, api.F32, out)
        got = out["token"].numpy()
        diff = np.nonzero(got != want["token"].astype(np.int32))[0]
        assert len(diff) == 0, f"penalties={with_pen}: rows {diff[:8]} got {got[diff[:8]]} want {want['token'][diff[:8]]}"
