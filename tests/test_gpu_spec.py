"""Speculative acceptance on the GPU.
accept_tokens: the accept loop of Acceptor::sample (exact rules) against a direct restatement.
spec_accept_residual (BASELINE config 3, parity unpinned: the reference removed this rule): against the oracle; a sequence
whose acceptance ratio or residual draw lies within 1e-6 of a boundary may differ and is counted."""
import numpy as np
import pytest
import torch

import synth
from gpu_util import dev

pytestmark = pytest.mark.gpu


def test_accept_tokens():
    from whirl_llm_b200 import api
    rng = np.random.default_rng(5)
    seqs, D = 40, 15
    nd = rng.integers(0, 9, seqs).astype(np.int32)
    row0 = np.zeros(seqs, dtype=np.int32)
    row0[1:] = np.cumsum(nd[:-1] + 1)
    rows = int(row0[-1] + nd[-1] + 1)
    tokens = rng.integers(0, 50, rows).astype(np.int32)
    dr = rng.integers(0, 50, (seqs, D)).astype(np.int32)
    for s in range(seqs):  # make most drafts match for a while
        k = int(rng.integers(0, nd[s] + 1))
        dr[s, :k] = tokens[row0[s]: row0[s] + k]
    acc, chosen = api.accept_tokens(dev(tokens), dev(dr), dev(nd), dev(row0))
    acc, chosen = acc.cpu().numpy(), chosen.cpu().numpy()
    for s in range(seqs):
        a = 0
        while a < nd[s] and tokens[row0[s] + a] == dr[s, a]:
            a += 1
        assert acc[s] == a and chosen[s] == tokens[row0[s] + a]
    assert acc.sum() > 0 and (acc < nd).any()


@pytest.mark.parametrize("B,L,V", [(6, 3, 5000), (16, 8, 151936)])
def test_accept_residual_config3(oracle, B, L, V):
    from whirl_llm_b200 import api
    target = synth.normalish(300 + V, (B, L + 1, V), 3.0)
    draft = (target[:, :L] + synth.normalish(301 + V, (B, L, V), 0.5)).astype(np.float32)
    # draft tokens sampled from the draft softmax (temperature 1) by inverse CDF with hashed uniforms
    ud = synth.hash_u01(302, B * L, 1).reshape(B, L)
    tok = np.zeros((B, L), dtype=np.int32)
    for b in range(B):
        for j in range(L):
            q = np.exp(draft[b, j].astype(np.float64) - draft[b, j].max())
            tok[b, j] = min(int(np.searchsorted(np.cumsum(q / q.sum()), ud[b, j])), V - 1)
    u_acc = synth.hash_u01(303, B * L, 2).reshape(B, L)
    u_res = synth.hash_u01(304, B * (L + 1), 3).reshape(B, L + 1)
    n_acc, nxt = api.spec_accept_residual(dev(target), dev(draft), dev(tok), None, dev(u_acc), dev(u_res))
    n_acc, nxt = n_acc.cpu().numpy(), nxt.cpu().numpy()
    differ = 0
    for b in range(B):
        wa, wt = oracle.spec_accept_residual(target[b], draft[b], tok[b], 1.0, u_acc[b], u_res[b])
        if (n_acc[b], nxt[b]) != (wa, wt):
            differ += 1
    # sums over 150k terms in another (blocked) order: a draw within ~1e-12 of a boundary may flip; none expected
    assert differ == 0, differ
    assert 0 < n_acc.sum() < B * L  # both outcomes occur
