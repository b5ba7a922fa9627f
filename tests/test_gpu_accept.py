"""whirl_accept_rows: the accept step of sampling::Acceptor with the relaxed rules, on the device.

(1) The reference's 33 recorded acceptance cases (tests/golden/accept_cases.*, made from the reference's own code) and
    the 400 random cases of the oracle-vs-reference test go through the device entry.  Those cases run the sampler at
    candidate levels 4 / 16 (a 64-token vocabulary), which the GPU sampler does not offer, so each verify row's
    sampler outputs (token, kept set, max / sum) come from the oracle at those levels and the device decides on them.
(2) The whole device pipeline - whirl_sample_rows / whirl_argmax_rows / whirl_topk_rows, then whirl_accept_rows, all in
    one batch of sequences - against oracle.accept_sample / accept_greedy at the library's own levels (256 / 16384),
    with whirl_accept_tokens checked against the same oracle results for the exact rules."""
import numpy as np
import pytest
import torch

import synth
from gpu_util import dev, row_params
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    from whirl_llm_b200 import api
    return api


def bits(d):
    return int(np.float64(d).view(np.uint64))


RP = dict(k=4, alpha=0.1, eps=0.09, delta=0.3)


def kept_result(api, res):
    """An oracle sample_rows result as the device arrays whirl_sample_rows would have written."""
    return api.SampleResult(token=dev(res["token"].astype(np.int32)), status=None, n_kept=dev(res["n"].astype(np.int32)),
                            closed=dev(res["closed"].astype(np.int32)), stats=dev(np.stack([res["m"], res["sum"]], axis=1).astype(np.float32)),
                            kept_ids=dev(res["kept_ids"].astype(np.int32)), kept_p=dev(res["kept_p"]), counters=None)


def device_accept_sample(api, oracle, rows, c, dr, hist, ks, kb):
    """One sequence of a sampling case: per-row sampler outputs from the oracle at levels ks / kb, decision on the device."""
    n_rows, V = rows.shape
    pos = np.array([c["n_gen"] + max(r - c["row0"], 0) for r in range(n_rows)], dtype=np.uint64)
    f = lambda v, dt: np.full(n_rows, v, dtype=dt)
    res = oracle.sample_rows(rows, kept_cap=V, inv_t=f(np.float32(1.0 / c["temp"]), np.float32), top_k=f(c["top_k"], np.uint32),
                             top_p=f(c["top_p"], np.float64), min_p=f(c["min_p"], np.float64), race=f(int(c["race"]), np.uint8),
                             seed=f(c["seed"], np.uint64), pos_idx=pos, ks=ks, kb=kb)
    kept = kept_result(api, res)
    out = api.accept_rows(kept.token, dev(dr.astype(np.int32)[None, :]), dev(np.array([c["nd"]], dtype=np.int32)),
                          dev(np.array([c["row0"]], dtype=np.int32)), api.RelaxParams(**RP),
                          relax_on=dev(np.array([int(c["relax"])], dtype=np.uint8)), next_tok=dev(np.array([c["next"]], dtype=np.int32)),
                          hist=dev(hist.astype(np.int32)[None, :]), hist_len=dev(np.array([len(hist)], dtype=np.int32)), kept=kept,
                          x=dev(rows), inv_t=dev(f(np.float32(1.0 / c["temp"]), np.float32)))
    return [int(t.cpu()[0]) for t in out[:3]] + [float(out[3].cpu()[0]), int(out[4].cpu()[0])]


def test_recorded_cases_through_the_device_entry(api, oracle, golden):
    meta, arr = golden.json("accept_cases"), golden.npz("accept_cases")
    assert len(meta) == 33
    for i, c in enumerate(meta):
        rows, dr, am, rh, hist = (arr[f"{i}_{k}"] for k in ("rows", "dr", "argmax", "relax_host", "hist"))
        if c["greedy"]:
            mr, rk = c["max_rows"], 4
            tokens = np.zeros(mr + 16, dtype=np.int32)
            tokens[c["row0"]: c["row0"] + len(am)] = am  # the slot's control area holds argmax[acc]; the batch holds rows
            ids = rh[: mr * rk * 4].view(np.int32).reshape(mr, rk)
            vals = rh[mr * rk * 4: mr * rk * 8].view(np.float32).reshape(mr, rk)
            st = rh[mr * rk * 8:].view(np.float32).reshape(mr, 2)
            out = api.accept_rows(dev(tokens), dev(dr.astype(np.int32)[None, :]), dev(np.array([c["nd"]], dtype=np.int32)),
                                  dev(np.array([c["row0"]], dtype=np.int32)), api.RelaxParams(**RP),
                                  greedy=dev(np.ones(1, dtype=np.uint8)), relax_on=dev(np.array([int(c["relax"])], dtype=np.uint8)),
                                  next_tok=dev(np.array([c["next"]], dtype=np.int32)), hist=dev(hist.astype(np.int32)[None, :]),
                                  hist_len=dev(np.array([len(hist)], dtype=np.int32)), rk_ids=dev(ids), rk_vals=dev(vals), rk_stats=dev(st))
            got = (int(out[0].cpu()[0]), int(out[1].cpu()[0]), int(out[2].cpu()[0]), bits(float(out[3].cpu()[0])))
            assert got == (c["acc"], c["chosen"], c["relaxed"], c["gap_bits"]), (c["name"], got)
        else:
            acc, chosen, relaxed, _, flags = device_accept_sample(api, oracle, rows, c, dr, hist, 4, 16)
            assert (acc, chosen, relaxed, flags) == (c["acc"], c["chosen"], c["relaxed"], 0), (c["name"], acc, chosen, relaxed)


def test_random_cases_through_the_device_entry(api, oracle):
    """The 400 random cases on which the oracle is compared with the reference (same generator, same seeds)."""
    rng = np.random.default_rng(7)
    n_acc = n_relaxed = 0
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
        rp = orc.Relax(on=int(typ), **RP)
        hist = np.array([1, 2, 3, 4, 5, 6, 7, 8], dtype=np.uint32)
        sm = orc.Sampler(inv_t=np.float32(1.0 / temp), top_k=top_k, top_p=top_p, min_p=min_p, seed=seed, race=int(race))
        a = oracle.accept_sample(rows, sm, dr, nd, row0, typ, n_gen, rp, hist, 7)
        c = dict(n_gen=n_gen, row0=row0, nd=nd, temp=temp, top_k=top_k, top_p=top_p, min_p=min_p, race=race, seed=seed, relax=typ, next=7)
        acc, chosen, relaxed, _, flags = device_accept_sample(api, oracle, rows, c, dr, hist, 4, 16)
        assert (acc, chosen, relaxed, flags) == (a.acc, a.chosen, a.relaxed, 0), (it, acc, chosen, relaxed, a.acc, a.chosen, a.relaxed)
        n_acc += acc
        n_relaxed += relaxed
    assert n_acc > 100 and n_relaxed > 30


def test_pipeline_on_the_device(api, oracle):
    """Sampler and acceptance both on the device, a batch of sequences per call, against the oracle's accept loops."""
    rng = np.random.default_rng(11)
    V, H, D = 1000, 64, 8
    rp = orc.Relax(on=1, **RP)
    for race in (False, True):
        seqs = 48
        nd = rng.integers(0, 6, seqs).astype(np.int32)
        row0 = np.zeros(seqs, dtype=np.int32)
        row0[1:] = np.cumsum(nd[:-1] + 1)
        R = int(row0[-1] + nd[-1] + 1)
        x = synth.normalish(500 + race, (R, V), 2.5)
        relax_on = rng.integers(0, 2, seqs).astype(np.uint8)
        seq_of = np.repeat(np.arange(seqs), nd + 1)
        temp = np.array([0.5, 0.8, 1.0, 1.6])[rng.integers(0, 4, seqs)]
        top_k = np.array([0, 0, 5, 20, 400])[rng.integers(0, 5, seqs)].astype(np.uint32)
        top_p = np.array([1, 1, 0.9, 0.97])[rng.integers(0, 4, seqs)]
        min_p = np.array([0, 0, 0.05])[rng.integers(0, 3, seqs)]
        seed = rng.integers(0, 2 ** 32, seqs).astype(np.uint64)
        n_gen = rng.integers(0, 1000, seqs)
        nxt = rng.integers(0, V, seqs).astype(np.int32)
        hist = rng.integers(0, 6, (seqs, H)).astype(np.int32)      # few distinct tokens: repeated 6-grams do occur
        hist_len = rng.integers(0, H + 1, seqs).astype(np.int32)
        dr = np.zeros((seqs, D), dtype=np.int32)
        for s in range(seqs):
            for j in range(nd[s]):
                order = np.lexsort((np.arange(V), -x[row0[s] + j].astype(np.float64)))
                dr[s, j] = order[int(rng.integers(0, 3))]
        pos = np.array([n_gen[seq_of[r]] + (r - row0[seq_of[r]]) for r in range(R)], dtype=np.uint64)
        prm = dict(inv_t=(1.0 / temp[seq_of]).astype(np.float32), top_k=top_k[seq_of], top_p=top_p[seq_of].astype(np.float64),
                   min_p=min_p[seq_of].astype(np.float64))
        u = np.array([oracle.uniform(int(seed[seq_of[r]]), int(pos[r]), 0) for r in range(R)])
        rk = np.array([oracle.race_base(int(seed[seq_of[r]]), int(pos[r])) for r in range(R)], dtype=np.uint64) if race else None
        xd = dev(x)
        res = api.sample_rows(xd, row_params(prm, u=u, race_key=rk), kept_cap=V)
        acc, chosen, relaxed, _, flags = api.accept_rows(res.token, dev(dr), dev(nd), dev(row0), api.RelaxParams(**RP), relax_on=dev(relax_on),
                                                        next_tok=dev(nxt), hist=dev(hist), hist_len=dev(hist_len), kept=res, x=xd,
                                                        inv_t=dev(prm["inv_t"]))
        acc, chosen, relaxed, flags = (t.cpu().numpy() for t in (acc, chosen, relaxed, flags))
        acc_t, chosen_t = (t.cpu().numpy() for t in api.accept_tokens(res.token, dev(dr), dev(nd), dev(row0)))
        n_rel = 0
        for s in range(seqs):
            sm = orc.Sampler(inv_t=np.float32(1.0 / temp[s]), top_k=int(top_k[s]), top_p=float(top_p[s]), min_p=float(min_p[s]), seed=int(seed[s]),
                             race=int(race))
            a = oracle.accept_sample(x, sm, dr[s].astype(np.uint32), int(nd[s]), int(row0[s]), bool(relax_on[s]), int(n_gen[s]), rp,
                                     hist[s, : hist_len[s]].astype(np.uint32), int(nxt[s]), ks=256, kb=16384)
            assert (acc[s], chosen[s], relaxed[s], flags[s]) == (a.acc, a.chosen, a.relaxed, 0), (race, s, acc[s], chosen[s], relaxed[s], a.acc, a.chosen, a.relaxed)
            n_rel += a.relaxed
            if not relax_on[s]:
                assert (acc_t[s], chosen_t[s]) == (a.acc, a.chosen)
        assert n_rel > 5 and acc.sum() > n_rel
    # ---- greedy sequences: argmax and the 4 best logits of every verify row from the device
    seqs = 64
    nd = rng.integers(0, 6, seqs).astype(np.int32)
    row0 = np.zeros(seqs, dtype=np.int32)
    row0[1:] = np.cumsum(nd[:-1] + 1)
    R = int(row0[-1] + nd[-1] + 1)
    x = synth.normalish(510, (R, V), 1.0)
    relax_on = rng.integers(0, 2, seqs).astype(np.uint8)
    nxt = rng.integers(0, V, seqs).astype(np.int32)
    hist = rng.integers(0, 6, (seqs, H)).astype(np.int32)
    hist_len = rng.integers(0, H + 1, seqs).astype(np.int32)
    dr = np.zeros((seqs, D), dtype=np.int32)
    for s in range(seqs):
        for j in range(nd[s]):
            order = np.lexsort((np.arange(V), -x[row0[s] + j].astype(np.float64)))
            dr[s, j] = order[int(rng.choice([0, 0, 0, 1, 2, 3, 5]))]
    xd = dev(x)
    am = api.argmax_rows(xd)
    ids, vals, st = api.topk_rows(xd, 4)
    acc, chosen, relaxed, gap, _ = api.accept_rows(am, dev(dr), dev(nd), dev(row0), api.RelaxParams(**RP), greedy=dev(np.ones(seqs, dtype=np.uint8)),
                                                   relax_on=dev(relax_on), next_tok=dev(nxt), hist=dev(hist), hist_len=dev(hist_len),
                                                   rk_ids=ids, rk_vals=vals, rk_stats=st)
    acc, chosen, relaxed, gap = (t.cpu().numpy() for t in (acc, chosen, relaxed, gap))
    oi, ov, os_ = oracle.topk_rows(x, 4, 1.0)
    relax_host = np.concatenate([oi.astype(np.int32).view(np.uint8).ravel(), ov.view(np.uint8).ravel(), os_.view(np.uint8).ravel()])
    amx = np.array([oracle.first_max(x[r]) for r in range(R)], dtype=np.int32)
    n_rel = 0
    for s in range(seqs):
        a = oracle.accept_greedy(amx[row0[s]: row0[s] + nd[s] + 1], dr[s].astype(np.uint32), int(nd[s]), int(row0[s]), bool(relax_on[s]), rp,
                                 relax_host, R, hist[s, : hist_len[s]].astype(np.uint32), int(nxt[s]))
        assert (acc[s], chosen[s], relaxed[s], bits(gap[s])) == (a.acc, a.chosen, a.relaxed, bits(a.relax_gap)), (s, acc[s], a.acc)
        n_rel += a.relaxed
    assert n_rel > 5
