"""The CPU oracle (oracle/whirl_oracle.c) against the fixtures generated from the reference's own code
(tests/golden/make_golden.py).  Runs anywhere; no GPU, no reference checkout."""
import numpy as np

import synth
from golden import make_golden as mg
from oracle import oracle as orc


def bits(d):
    return int(np.float64(d).view(np.uint64))


def test_uniform_and_race_keys(oracle, golden):
    kat = golden.json("uniform_kat")
    toks = kat["tokens"]
    for r in kat["records"]:
        s, p = r["seed"], r["pos"]
        assert bits(oracle.uniform(s, p, 0)) == r["u0"] == r["sampler_u"]
        assert bits(oracle.uniform(s, p, 1)) == r["u1"]
        base = oracle.race_base(s, p)
        assert base == r["base"]
        assert [bits(oracle.race_e(base, t)) for t in toks] == r["race_e"]


def test_uniform_formula_kat(oracle):
    # the reference's own known-answer statement (tests/unit/spec_sample_tests.cpp:247-256)
    seed, pos = 987654321, 41
    m = (1 << 64) - 1
    z = (seed + (pos + 1) * 0x9E3779B97F4A7C15) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    z ^= z >> 31
    assert oracle.uniform(seed, pos, 0) == (z >> 11) * (1.0 / 9007199254740992.0)
    assert oracle.uniform(seed, pos, 1) != oracle.uniform(seed, pos, 0)


def test_filter_cases(oracle, golden):
    g = golden.npz("filter_cases")
    for i, (count, spread, inv_t, top_k, top_p, min_p, complete, tail) in enumerate(mg.FILTER_SETS):
        lg = synth.grid_logits(1000 + i, (count,), spread) if i % 2 else synth.normalish(1000 + i, (count,), spread)
        ids = (np.arange(count, dtype=np.uint32) * 7 + 3).astype(np.uint32)
        m, s = g[f"{i}_ms"][0], g[f"{i}_ms"][1]
        r = oracle.filter_cands(ids, lg, inv_t=inv_t, top_k=top_k, top_p=top_p, min_p=min_p, m=m, sum_=s, complete=complete)
        ok, n, closed = g[f"{i}_res"]
        assert (r["ok"], r["n"], r["closed"]) == (bool(ok), n, bool(closed)), i
        assert np.array_equal(r["ids"], g[f"{i}_ids"]), i
        assert np.array_equal(r["p"], g[f"{i}_p"]), i  # same libm, same order: bit-equal
        assert (r["m"], r["sum"]) == (g[f"{i}_ms"][2], g[f"{i}_ms"][3])


def test_sampler_boundary_rules(oracle):
    # the reference's testSampler statements (tests/sampling/sampling_unit.inc:8-61)
    logits = [1, 5, 3, 3, 0, -1, 2, 4]
    z = float(np.float32(sum(np.exp(np.float64(l) - 5) for l in logits)))
    r = oracle.filter_cands(range(8), logits, top_k=3, m=5, sum_=z)
    assert r["ok"] and r["n"] == 3 and r["closed"] and list(r["ids"][:3]) == [1, 7, 2]
    assert abs(r["p"][:3].sum() - 1.0) < 1e-9
    assert not oracle.filter_cands(range(8), logits, top_k=20, m=5, sum_=z)["ok"]  # open: escalate
    r = oracle.filter_cands(range(8), logits, top_k=8, m=5, sum_=z)  # top_k == count closes with every candidate
    assert r["ok"] and r["n"] == 8 and r["closed"]
    r = oracle.filter_cands(range(4), [5, 5, 3, 1], min_p=1.0, complete=True)  # min-p keeps equality
    assert r["ok"] and r["n"] == 2 and r["closed"]


def _check_rows(res, g, what):
    for k in ("token", "n", "closed", "big_used", "full_used"):
        assert np.array_equal(res[k], g[k]), (what, k, np.nonzero(res[k] != g[k]))
    assert np.array_equal(res["m"], g["m"]), what
    np.testing.assert_allclose(res["sum"], g["sum"], rtol=1e-6)  # f64 sums in index vs sorted order, cast to f32
    for r in range(len(res["n"])):
        n = min(int(res["n"][r]), res["kept_ids"].shape[1])
        assert np.array_equal(res["kept_ids"][r, :n], g["kept_ids"][r, :n]), (what, r)
        np.testing.assert_allclose(res["kept_p"][r, :n], g["kept_p"][r, :n], rtol=1e-12, atol=0)


def test_rows_small(oracle, golden):
    R, V = mg.SMALL_ROWS["rows"], mg.SMALL_ROWS["V"]
    x = np.where(np.arange(R)[:, None] % 3 == 0, synth.grid_logits(77, (R, V), 2.0), synth.normalish(78, (R, V), 1.5))
    res = oracle.sample_rows(x.astype(np.float32), kept_cap=V, ks=4, kb=16, **mg.row_params(R, 79, 24))
    _check_rows(res, golden.npz("rows_small"), "small")


def test_rows_engine(oracle, golden):
    R, V = mg.ENGINE_ROWS["rows"], mg.ENGINE_ROWS["V"]
    x = synth.normalish(80, (R, V), 3.0)
    x[::5] = synth.grid_logits(81, (R, V), 3.0)[::5]
    x[3] = 0.0
    res = oracle.sample_rows(x, kept_cap=1024, threads=4, **mg.row_params(R, 82, 600))
    g = golden.npz("rows_engine")
    assert g["big_used"].sum() > 0 and g["full_used"].sum() > 0  # the fixture reaches both escalation levels
    _check_rows(res, g, "engine")


def test_accept_cases(oracle, golden):
    meta, arr = golden.json("accept_cases"), golden.npz("accept_cases")
    rules = set()
    for i, c in enumerate(meta):
        rp = orc.Relax(on=int(c["relax"]), k=4, alpha=0.1, eps=0.09, delta=0.3)
        rows, dr, am, rh, hist = (arr[f"{i}_{k}"] for k in ("rows", "dr", "argmax", "relax_host", "hist"))
        if c["greedy"]:
            a = oracle.accept_greedy(am, dr, c["nd"], c["row0"], c["relax"], rp, rh, c["max_rows"], hist, c["next"])
        else:
            sm = orc.Sampler(inv_t=np.float32(1.0 / c["temp"]), top_k=c["top_k"], top_p=c["top_p"], min_p=c["min_p"],
                             seed=c["seed"], race=int(c["race"]))
            a = oracle.accept_sample(rows, sm, dr, c["nd"], c["row0"], c["relax"], c["n_gen"], rp, hist, c["next"])
        got = (a.acc, a.chosen, a.relaxed, bits(a.relax_gap), a.pos_idx, a.full_used, a.big_used)
        want = tuple(c[k] for k in ("acc", "chosen", "relaxed", "gap_bits", "pos_idx", "full_used", "big_used"))
        assert got == want, (c["name"], got, want)
        for j in range(c["acc"] + 1):
            assert bits(oracle.uniform(c["seed"], c["n_gen"] + j, 0)) == c["draws"][j]
        rules.add((c["greedy"], c["relax"], c["race"]))
    assert len(meta) == 33 and len(rules) >= 5


def test_draft_dist(oracle, golden):
    g = golden.npz("draft_dist")
    i = 0
    while f"{i}_in" in g:
        top_k, K = (int(v) for v in g[f"{i}_in"])
        top_p, min_p, inv_t, m, s = (float(v) for v in g[f"{i}_f"])
        lg = synth.grid_logits(300 + i, (K,), 3.0) if i % 2 else synth.normalish(300 + i, (K,), 3.0)
        ids = ((np.arange(K, dtype=np.uint32) * 2654435761) % 248320).astype(np.uint32)
        q = oracle.draft_dist(ids, lg, m, s, inv_t, top_k, top_p, min_p)
        n, tok = (int(v) for v in g[f"{i}_n"])
        assert q.n == n
        assert list(q.id[:n]) == list(g[f"{i}_id"][:n])
        assert np.array_equal(np.array(q.p[:n], dtype=np.float32), g[f"{i}_p"][:n])
        assert oracle.spec_sample_race(q, int(g[f"{i}_key"][0])) == tok
        i += 1
    assert i == 7


def test_draft_dist_reference_statements(oracle):
    # tests/unit/spec_sample_tests.cpp:258-282
    ids, lg, m = [7, 3, 9, 1], [1.0, 3.0, 2.0, 2.0], 3.0
    s = np.float32(0)
    for v in lg:
        s = np.float32(s + np.exp(np.float32(v - m)))
    s = float(np.float32(s + np.float32(0.5)))
    a = oracle.draft_dist(ids, lg, m, s, 1.0, 0, 1.0, 0.0)
    assert a.n == 4 and list(a.id[:4]) == [3, 1, 9, 7] and abs(sum(a.p[:4]) - 1) < 1e-6
    b = oracle.draft_dist(ids, lg, m, s, 1.0, 2, 1.0, 0.0)
    assert b.n == 2 and list(b.id[:2]) == [3, 1]
    c = oracle.draft_dist(ids, lg, m, s, 1.0, 0, 1.0, 0.5)
    assert c.n == 1 and c.id[0] == 3 and c.p[0] == 1.0


def test_relax_rules(oracle):
    # tests/unit/accept_policy_tests.cpp:46-71
    p = orc.Relax(on=1, k=2, alpha=0.5, eps=0.09, delta=0.3)
    ids, lg = [7, 3, 9], [1.0, 2.0, 2.0 - 0.6]
    assert oracle.relax_accept_greedy(p, ids, lg, 2.0, 3) and oracle.relax_accept_greedy(p, ids, lg, 2.0, 9)
    assert not oracle.relax_accept_greedy(p, ids, lg, 2.0, 7) and not oracle.relax_accept_greedy(p, ids, lg, 2.0, 42)
    p.alpha = 0.6
    assert not oracle.relax_accept_greedy(p, ids, lg, 2.0, 9)
    p.alpha, p.k = 0.5, 1
    assert not oracle.relax_accept_greedy(p, ids, lg, 2.0, 9) and oracle.relax_accept_greedy(p, ids, lg, 2.0, 3)
    assert not oracle.relax_accept_greedy(p, [5, 4], [1.0, 1.0], 1.0, 5) and oracle.relax_accept_greedy(p, [5, 4], [1.0, 1.0], 1.0, 4)
    h = [1, 2, 3, 4, 5, 6, 9, 1]
    assert oracle.relax_extends_repeat(h, [2, 3, 4, 5, 6]) and not oracle.relax_extends_repeat(h, [2, 3, 4, 5, 7])
    assert oracle.relax_accept_typical(p, 0.1, 0.0) and not oracle.relax_accept_typical(p, 0.08, 0.0)
    assert oracle.relax_accept_typical(p, 0.3 * np.exp(-3.0) + 1e-9, 3.0) and not oracle.relax_accept_typical(p, 0.01, 3.0)


def test_philox_known_answers(oracle):
    # Random123 kat_vectors, philox4x32 with 10 rounds
    assert list(oracle.philox4x32_10([0, 0, 0, 0], [0, 0])) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert list(oracle.philox4x32_10([0xffffffff] * 4, [0xffffffff] * 2)) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert list(oracle.philox4x32_10([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0])) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]
    u = [oracle.philox_uniform(1234, i, 0) for i in range(1000)]
    assert all(0 <= v < 1 for v in u) and 0.45 < np.mean(u) < 0.55


def test_penalties_and_bf16(oracle):
    x = np.array([2.0, -1.0, 0.5, 3.0, 0.0], dtype=np.float32)
    y, skipped = oracle.apply_penalties(x, [0, 1, 1, 3, 3, 3, 9, -1], 1.1, 0.5, 0.3)
    f = np.float32
    want = [f(f(2.0) / f(1.1)) - f(f(0.5) + f(f(0.3) * f(1))), f(f(-1.0) * f(1.1)) - f(f(0.5) + f(f(0.3) * f(2))), 0.5,
            f(f(3.0) / f(1.1)) - f(f(0.5) + f(f(0.3) * f(3))), 0.0]
    assert skipped == 2 and np.array_equal(y, np.array(want, dtype=np.float32))
    b = synth.to_bf16_bits(synth.normalish(5, (64,), 3.0))
    w = oracle.bf16_to_f32(b)
    assert np.array_equal(w.view(np.uint32), b.astype(np.uint32) << 16)


def test_first_max_and_topk(oracle):
    x = synth.normalish(9, (3, 5000), 3.0)
    x[1, 100] = x[1, 4000] = 50.0
    x[2, 4999] = 60.0
    assert [oracle.first_max(r) for r in x] == [int(np.argmax(x[0])), 100, 4999]
    ids, vals, stats = oracle.topk_rows(x, 40, 1 / 0.7)
    for r in range(3):
        order = np.lexsort((np.arange(5000), -x[r].astype(np.float64)))[:40]
        assert np.array_equal(ids[r], order) and np.array_equal(vals[r], x[r][order])
        assert stats[r, 0] == x[r].max()
        ref_sum = np.exp((x[r].astype(np.float64) - x[r].max()) * np.float32(1 / 0.7)).sum()
        assert abs(stats[r, 1] - ref_sum) <= 1e-6 * ref_sum
