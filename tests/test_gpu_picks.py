"""Greedy picks on the GPU against the oracle (first maximum; probabilities of the top token; draft pick chain).
Mirrors the reference's kernel test (tests/kernels/test_misc.cpp:153-300)."""
import numpy as np
import pytest
import torch

import synth
from gpu_util import bf16_tensor, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    from whirl_llm_b200 import api
    return api


def _rows_like_reference(n, rows=5):
    x = synth.normalish(4242, (rows, n), 3.0)
    if n > 9000:
        x[1, 100] = x[1, 9000] = 50.0  # tie: first index must win
    x[2, n - 1] = 60.0                 # last element
    return x


@pytest.mark.parametrize("n", [1, 2, 3, 5, 31, 33, 255, 1000, 4097, 248320, 151936, 262144])
def test_argmax_rows(api, oracle, n):
    x = _rows_like_reference(n)
    want = np.array([oracle.first_max(r) for r in x])
    got = api.argmax_rows(dev(x)).cpu().numpy()
    assert np.array_equal(got, want)
    # unaligned rows: odd row length handled above (n = 3, 5, 31 ...); unaligned base pointer here
    if n > 8:
        xd = dev(np.concatenate([[0.0], x.reshape(-1)]).astype(np.float32))[1:].view(x.shape[0], n)
        assert np.array_equal(api.argmax_rows(xd).cpu().numpy(), want)


def test_argmax_single_and_scatter(api, oracle):
    n = 248320
    x = _rows_like_reference(n)
    want = np.array([oracle.first_max(r) for r in x])
    xd = dev(x)
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    ids = torch.zeros(1, dtype=torch.int32, device="cuda")
    pos = torch.tensor([41], dtype=torch.int32, device="cuda")
    api.argmax(xd[1], out=out, ids=ids, pos=pos, advance=1)
    assert (out.item(), ids.item(), pos.item()) == (want[1], want[1], 42)
    o2 = torch.full((64,), -1, dtype=torch.int32, device="cuda")
    dst = dev(np.array([10 + 3 * r for r in range(5)], dtype=np.int32))
    api.argmax_rows_to(xd, o2, dst)
    o2 = o2.cpu().numpy()
    assert all(o2[10 + 3 * r] == want[r] for r in range(5)) and (o2 == -1).sum() == 59


def test_argmax_many_rows_and_special_values(api, oracle):
    x = synth.grid_logits(5, (700, 1537), 2.0)  # heavy ties
    x[3] = -np.inf
    x[4, 5] = np.nan
    x[4, 9] = 7.0
    x[5] = 0.0
    x[5, 100] = -0.0
    x[6, 0] = np.nan   # a NaN in the first place is skipped like any other (kernels/shared/block_argmax.h:1-8 starts from -inf)
    x[7, :3] = np.nan
    x[8] = np.nan      # nothing above -inf: index 0
    want = np.array([oracle.first_max(r) for r in x])
    assert want[6] != 0 and want[7] >= 3 and want[8] == 0
    assert np.array_equal(api.argmax_rows(dev(x)).cpu().numpy(), want)


def test_argmax_bf16(api, oracle):
    x = synth.normalish(6, (37, 262144), 3.0)
    bits = synth.to_bf16_bits(x)
    wide = oracle.bf16_to_f32(bits)
    want = np.array([oracle.first_max(r) for r in wide])
    assert np.array_equal(api.argmax_rows(bf16_tensor(bits)).cpu().numpy(), want)


def test_argmax_prob(api, oracle):
    x = _rows_like_reference(248320)
    tok, prob = api.argmax_prob(dev(x))
    want_t = np.array([oracle.first_max(r) for r in x])
    want_p = np.array([oracle.softmax_top(r) for r in x])
    assert np.array_equal(tok.cpu().numpy(), want_t)
    np.testing.assert_allclose(prob.cpu().numpy(), want_p, rtol=1e-4)  # the reference test's tolerance


def test_draft_pick_chain(api, oracle):
    n = 248320
    lg = synth.normalish(8, (3, n), 1.0)
    lg[0, 5] = 30.0   # r = 0: confident
    lg[1, 7] = 4.0    # r = 1: unconfident -> the chain stops (n_min = 1)
    lg[2, 9] = 30.0   # r = 2: skipped
    d = dev(lg)
    tok = torch.full((16,), 0x7f7f7f7f, dtype=torch.int32, device="cuda")
    prob = torch.zeros(16, dtype=torch.float32, device="cuda")
    ctl = torch.zeros(2, dtype=torch.int32, device="cuda")
    wt = np.full(16, 0x7f7f7f7f, dtype=np.int32)
    wp = np.zeros(16, dtype=np.float32)
    wc = np.zeros(2, dtype=np.int32)
    for r in range(3):
        api.draft_pick(d[r], tok, prob, ctl, r, 1, 0.5)
        oracle.draft_pick(lg[r], wt, wp, wc, r, 1, 0.5)
    assert np.array_equal(tok.cpu().numpy(), wt) and np.array_equal(ctl.cpu().numpy(), wc)
    assert wt[0] == 5 and wt[2] == 0x7f7f7f7f and list(wc) == [1, 1]
    np.testing.assert_allclose(prob.cpu().numpy()[:2], wp[:2], rtol=1e-4)
    # rows variant: two sequences' control areas, and a vocabulary map
    ctl_all = torch.zeros(2 * 64, dtype=torch.int32, device="cuda")
    area = dev(np.array([0, 64], dtype=np.int32))
    api.draft_pick_rows(d[:2], ctl_all, area, 0, 1, 0.5)
    ca = ctl_all.cpu().numpy()
    assert ca[16] == wt[0] and ca[64 + 16] == oracle.first_max(lg[1]) and ca[48] == 1 and ca[64 + 48] == 1
    perm = (100000 + 3 * np.arange(n)).astype(np.int32)
    cm = torch.zeros(2 * 64, dtype=torch.int32, device="cuda")
    api.draft_pick_rows(d[:2], cm, area, 0, 0, 0.0, vmap=dev(perm))
    cm = cm.cpu().numpy()
    assert cm[16] == perm[wt[0]] and cm[64 + 16] == perm[oracle.first_max(lg[1])]
