"""Generates the fixtures in this directory from the REFERENCE's own sampling code (oracle/_ref, built from a
reference checkout by oracle/Makefile).  Run where the reference is present:

    python tests/golden/make_golden.py            # rewrites tests/golden/*.npz / *.json

The fixtures are what travels: the tests check the oracle (and, on a GPU, the CUDA path) against them on machines
that have no reference checkout.  Inputs are regenerated in the tests from the recorded seeds (tests/synth.py), so
the files hold seeds, parameters and the reference's outputs only.

EXPECTED_ACCEPT below is the table the reference's own test pins (tests/sampling/sampling_unit.inc:149-186,
acceptExpected(): acc, chosen, relaxed, gap bits, pos_idx, full_used, big_used, uniform bits per output index);
the generator asserts that the reference code run here reproduces it before writing anything.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import synth  # noqa: E402
from oracle import oracle as orc  # noqa: E402

# name, acc, chosen, relaxed, gap_bits, pos_idx, full_used, big_used, draws (uniform bit patterns)
EXPECTED_ACCEPT = [
    ("greedy_all_match", 3, 28, 0, 0x0, 0, 0, 0, [0x3fd95fbb374f2c4e, 0x3fe85a64dc00ab7b, 0x3fe0c43407fc177b, 0x3fe1c3eeaab30755]),
    ("greedy_reject_1", 1, 16, 0, 0x0, 0, 0, 0, [0x3fd95fbb374f2c4e, 0x3fe85a64dc00ab7b]),
    ("greedy_reject_0", 0, 6, 0, 0x0, 0, 0, 0, [0x3fd95fbb374f2c4e]),
    ("greedy_no_drafts", 0, 54, 0, 0x0, 0, 0, 0, [0x3fd95fbb374f2c4e]),
    ("relax_greedy_rank1", 3, 41, 2, 0x3fc0e56080000000, 0, 0, 0, [0x3fd95fbb374f2c4e, 0x3fe85a64dc00ab7b, 0x3fe0c43407fc177b, 0x3fe1c3eeaab30755]),
    ("relax_greedy_rank3", 4, 23, 3, 0x3fa9581100000000, 0, 0, 0, [0x3fd95fbb374f2c4e, 0x3fe85a64dc00ab7b, 0x3fe0c43407fc177b, 0x3fe1c3eeaab30755, 0x3fe6a9c1e2c01989]),
    ("relax_greedy_far", 1, 57, 1, 0x3fa6872800000000, 0, 0, 0, [0x3fd95fbb374f2c4e, 0x3fe85a64dc00ab7b]),
    ("relax_greedy_repeat", 1, 2, 1, 0x3f7eb85000000000, 0, 0, 0, [0x3fd95fbb374f2c4e, 0x3fe85a64dc00ab7b]),
    ("sample_closed_topk", 1, 11, 0, 0x0, 21, 0, 2, [0x3fbd67c34f6a2a30, 0x3fef99504bda8630]),
    ("sample_topp", 0, 30, 0, 0x0, 21, 1, 1, [0x3fe545e33bf7f406]),
    ("sample_minp", 0, 39, 0, 0x0, 22, 1, 1, [0x3fd60b59c5ea4748]),
    ("sample_open_tail", 0, 24, 0, 0x0, 23, 1, 0, [0x3fd9b75720072950]),
    ("sample_open_tail_b", 0, 43, 0, 0x0, 0, 1, 0, [0x3fe5d5ea5fd7ce0c]),
    ("sample_escalate_topk", 0, 16, 0, 0x0, 24, 0, 1, [0x3fed89574c81bac9]),
    ("specsample_closed", 2, 46, 0, 0x0, 27, 0, 3, [0x3fedc97a524aca41, 0x3feb8329339ad37b, 0x3fe7ef828545b800]),
    ("specsample_topp", 0, 12, 0, 0x0, 26, 1, 1, [0x3fdae54e1f7ab804]),
    ("specsample_open", 0, 15, 0, 0x0, 27, 1, 0, [0x3fd3c1ac84edb6c2]),
    ("specsample_open_b", 0, 60, 0, 0x0, 28, 1, 0, [0x3fedb9ea18198051]),
    ("specsample_minp", 0, 22, 0, 0x0, 29, 1, 1, [0x3fc040b9dc918150]),
    ("specsample_no_drafts", 0, 37, 0, 0x0, 30, 1, 0, [0x3fe388eea59b03bf]),
    ("typical_closed", 4, 50, 4, 0x0, 35, 0, 5, [0x3fd82adf0b38cce2, 0x3fd0439ace23450a, 0x3fe2b35fc9016eca, 0x3fec05399b7ae104, 0x3fe080aaac70a7c6]),
    ("typical_topp", 4, 59, 4, 0x0, 36, 5, 5, [0x3fdc66b2091fcfb8, 0x3fdc84cfae5a6fea, 0x3fe55ca8c2e34d42, 0x3fed6973a34de399, 0x3fef0ffd3e892faa]),
    ("typical_open_F2_02", 0, 46, 0, 0x0, 33, 1, 0, [0x3fe7e0b9b7ce6965]),
    ("typical_open_race", 0, 55, 0, 0x0, 34, 1, 0, [0x3feb38b858a7a633]),
    ("typical_far", 0, 47, 0, 0x0, 35, 0, 1, [0x3fdadc7f85086cd0]),
    ("sample_t_match", 4, 28, 0, 0x0, 44, 5, 5, [0x3fd17a564ed562d2, 0x3fee8ccbaf14db13, 0x3fe36a629689298b, 0x3fd4319b0f01ee66, 0x3feaea97a9fe5082]),
    ("sample_t_open", 2, 9, 0, 0x0, 43, 2, 0, [0x3fa609756bcb6960, 0x3fd6415f9ea5af10, 0x3fcc85d0b63575ec]),
    ("specsample_t_match", 4, 37, 0, 0x0, 46, 0, 5, [0x3f95efb74bfb9100, 0x3fd544e98de425b0, 0x3fe9362924b58baa, 0x3fcb38348ed71918, 0x3fe0fc5c865248c3]),
    ("specsample_t_open", 3, 51, 0, 0x0, 46, 2, 0, [0x3fa0196f8d4ab2b0, 0x3fed3c3f6655cd41, 0x3fcb8e0f91f6b85c, 0x3fa37ce8f0abbb10]),
    ("specsample_t_minp", 3, 7, 0, 0x0, 47, 4, 4, [0x3f8314663cf52f80, 0x3fe172766f5d8333, 0x3fe922decdf99f29, 0x3fe84a3b7aa47f8b]),
    ("typical_t_open", 1, 41, 0, 0x0, 46, 2, 0, [0x3fc414499d119280, 0x3fe570836d21e63e]),
    ("typical_t_race", 4, 18, 4, 0x0, 50, 5, 5, [0x3fcd6b1d03f31e98, 0x3fedb9a47cb51293, 0x3fd69d0c84003ab0, 0x3fe742df9f54dd12, 0x3fb432ff66d751e8]),
    ("typical_repeat", 1, 44, 1, 0x0, 37, 0, 2, [0x3fecd9bb06f00448, 0x3fe5ac3e22af6700]),
]


def bits(d: float) -> int:
    return int(np.float64(d).view(np.uint64))


def run_case(ref, c):
    rp = orc.Relax(on=int(c["relax"]), k=4, alpha=0.1, eps=0.09, delta=0.3)
    if c["greedy"]:
        a = ref.accept_greedy(c["argmax"], c["dr"], c["nd"], c["row0"], c["relax"], rp, c["relax_host"], c["max_rows"],
                              c["hist"], c["next"])
    else:
        sm = orc.Sampler(inv_t=np.float32(1.0 / c["temp"]) if c["temp"] > 0 else 1.0, top_k=c["top_k"], top_p=c["top_p"],
                         min_p=c["min_p"], seed=c["seed"], race=int(c["race"]))
        a = ref.accept_sample(c["rows"], sm, c["dr"], c["nd"], c["row0"], c["relax"], c["n_gen"], rp, c["hist"], c["next"])
    return a


def accept_cases(ref):
    cases = ref.cases()
    assert len(cases) == len(EXPECTED_ACCEPT)
    meta, arrays = [], {}
    for i, (c, e) in enumerate(zip(cases, EXPECTED_ACCEPT)):
        name, acc, chosen, relaxed, gap_bits, pos_idx, full_used, big_used, draws = e
        assert c["name"] == name
        a = run_case(ref, c)
        got = (a.acc, a.chosen, a.relaxed, bits(a.relax_gap), a.pos_idx, a.full_used, a.big_used)
        assert got == (acc, chosen, relaxed, gap_bits, pos_idx, full_used, big_used), (name, got, e)
        for j in range(acc + 1):
            assert bits(ref.sampler_uniform(c["seed"], c["n_gen"] + j)) == draws[j], name
        meta.append({k: (v if not isinstance(v, (np.integer, np.floating)) else v.item())
                     for k, v in c.items() if not isinstance(v, np.ndarray)}
                    | dict(acc=acc, chosen=chosen, relaxed=relaxed, gap_bits=gap_bits, pos_idx=pos_idx, full_used=full_used,
                           big_used=big_used, draws=draws))
        for k in ("rows", "dr", "argmax", "relax_host", "hist"):
            arrays[f"{i}_{k}"] = c[k]
    np.savez_compressed(os.path.join(HERE, "accept_cases.npz"), **arrays)
    with open(os.path.join(HERE, "accept_cases.json"), "w") as f:
        json.dump(meta, f, indent=1)
    print(f"accept_cases: {len(cases)} cases reproduce the reference's recorded table")


def scalar_kats(ref):
    rng = np.random.default_rng(20261125)
    seeds = [0, 1, 7, 1234, 987654321, 2**63 + 12345, 2**64 - 1] + [int(x) for x in rng.integers(0, 2**63, 9)]
    poss = [0, 1, 3, 41, 999, 100000, 2**40 + 5]
    toks = [0, 1, 31, 151935, 248319, 262143]
    rec = []
    for s in seeds:
        for p in poss:
            base = ref.race_base(s, p)
            rec.append(dict(seed=s, pos=p, u0=bits(ref.uniform(s, p, 0)), u1=bits(ref.uniform(s, p, 1)),
                            sampler_u=bits(ref.sampler_uniform(s, p)), base=base,
                            race_e=[bits(ref.race_e(base, t)) for t in toks]))
    with open(os.path.join(HERE, "uniform_kat.json"), "w") as f:
        json.dump(dict(tokens=toks, records=rec), f)
    print(f"uniform_kat: {len(rec)} records")


FILTER_SETS = [  # (count, spread, inv_t, top_k, top_p, min_p, complete, tail_mass)
    (8, 2.0, 1.0, 3, 1.0, 0.0, False, 0.0), (8, 2.0, 1.0, 20, 1.0, 0.0, False, 0.0), (8, 2.0, 1.0, 8, 1.0, 0.0, False, 0.0),
    (4, 2.0, 1.0, 0, 1.0, 1.0, True, 0.0), (256, 3.0, 1.0 / 0.7, 40, 0.95, 0.0, False, 0.3),
    (256, 2.5, 1.25, 50, 0.9, 0.05, False, 0.5), (256, 3.0, 1.0, 0, 0.9, 0.0, False, 0.1), (256, 3.0, 1.0, 0, 0.9, 0.0, False, 5.0),
    (256, 1.0, 1.0, 0, 1.0, 0.1, False, 1.0), (256, 1.0, 1.0, 0, 1.0, 1e-9, False, 1.0), (256, 3.0, 2.0, 0, 1.0, 0.0, False, 2.0),
    (1024, 3.0, 1.0, 1024, 0.8, 0.0, False, 0.2), (1024, 3.0, 1.1, 777, 0.99, 0.01, False, 0.2), (1, 1.0, 1.0, 1, 0.5, 0.5, False, 0.0),
    (64, 0.3, 1.0, 0, 0.9, 0.0, True, 0.0), (64, 4.0, 0.5, 5, 0.5, 0.2, True, 0.0), (300, 0.01, 1.0, 100, 0.5, 0.0, False, 0.0),
]


def filter_cases(ref):
    out = {}
    for i, (count, spread, inv_t, top_k, top_p, min_p, complete, tail) in enumerate(FILTER_SETS):
        lg = synth.grid_logits(1000 + i, (count,), spread) if i % 2 else synth.normalish(1000 + i, (count,), spread)
        ids = (np.arange(count, dtype=np.uint32) * 7 + 3).astype(np.uint32)
        m = float(lg.max())
        s = float(np.float32(np.exp((lg.astype(np.float64) - m) * np.float32(inv_t)).sum() + tail))
        r = ref.filter_cands(ids, lg, inv_t=inv_t, top_k=top_k, top_p=top_p, min_p=min_p, m=m, sum_=s, complete=complete)
        out[f"{i}_ids"] = r["ids"]
        out[f"{i}_p"] = r["p"]
        out[f"{i}_res"] = np.array([r["ok"], r["n"], r["closed"]], dtype=np.int64)
        out[f"{i}_ms"] = np.array([m, s, r["m"], r["sum"]], dtype=np.float32)
    np.savez_compressed(os.path.join(HERE, "filter_cases.npz"), **out)
    print(f"filter_cases: {len(FILTER_SETS)} sets")


SMALL_ROWS = dict(rows=96, V=200)
ENGINE_ROWS = dict(rows=40, V=20000)


def row_params(rows, seed, kmax):
    """A mix of sampler settings, one per row, reproducible from the seed."""
    u = synth.hash_u01(seed, rows * 8, 3).reshape(rows, 8)
    kind = (u[:, 0] * 6).astype(int)
    inv_t = (1.0 / (0.5 + 1.1 * u[:, 1])).astype(np.float32)
    top_k = np.where(kind == 0, 0, 1 + (u[:, 2] * kmax).astype(np.uint32)).astype(np.uint32)
    top_p = np.where(kind == 1, 1.0, 0.5 + 0.5 * u[:, 3])
    min_p = np.where(kind == 2, 0.02 + 0.2 * u[:, 4], 0.0)
    top_k = np.where(kind == 3, 0, top_k).astype(np.uint32)
    top_p = np.where(kind == 3, 1.0, top_p)  # kind 3: no filter at all (open set, tail walk)
    min_p = np.where(kind == 3, 0.0, min_p)
    greedy = (kind == 4).astype(np.uint8)
    race = ((kind == 5) | (u[:, 5] < 0.2)).astype(np.uint8)
    seedv = (synth.hash_u01(seed, rows, 4) * 2**53).astype(np.uint64)
    pos = (synth.hash_u01(seed, rows, 5) * 5000).astype(np.uint64)
    return dict(inv_t=inv_t, top_k=top_k, top_p=top_p, min_p=min_p, greedy=greedy, race=race, seed=seedv, pos_idx=pos)


def rows_cases(ref):
    # small vocabulary, the reference test's hostPrepare (escalation 4 -> 16 -> V)
    R, V = SMALL_ROWS["rows"], SMALL_ROWS["V"]
    x = np.where(np.arange(R)[:, None] % 3 == 0, synth.grid_logits(77, (R, V), 2.0), synth.normalish(78, (R, V), 1.5))
    x = x.astype(np.float32)
    prm = row_params(R, 79, 24)
    r = ref.sample_rows_small(x, kept_cap=V, **prm)
    np.savez_compressed(os.path.join(HERE, "rows_small.npz"), **{k: v for k, v in r.items()})
    # engine path: the real SampleBuffers (k_small 256, k_big 16384) over FakeServerModel::topkRows
    R, V = ENGINE_ROWS["rows"], ENGINE_ROWS["V"]
    x = synth.normalish(80, (R, V), 3.0)
    x[::5] = synth.grid_logits(81, (R, V), 3.0)[::5]
    x[3] = 0.0  # a flat row: everything ties
    prm = row_params(R, 82, 600)
    r = ref.sample_rows(x, kept_cap=1024, threads=4, **prm)
    np.savez_compressed(os.path.join(HERE, "rows_engine.npz"), **{k: v for k, v in r.items()})
    print(f"rows: small {SMALL_ROWS}, engine {ENGINE_ROWS}; escalations big={int(r['big_used'].sum())} full={int(r['full_used'].sum())}")


def draft_cases(ref):
    out = {}
    sets = [(20, 0.95, 0.0, 1 / 0.7), (0, 0.8, 0.0, 1.0), (5, 1.0, 0.05, 1 / 0.6), (0, 1.0, 0.0, 1.0), (32, 0.5, 0.3, 2.0),
            (1, 1.0, 0.0, 1.0), (40, 0.99, 0.0, 0.8)]
    for i, (top_k, top_p, min_p, inv_t) in enumerate(sets):
        K = ref._draft_cands(top_k)
        lg = synth.grid_logits(300 + i, (K,), 3.0) if i % 2 else synth.normalish(300 + i, (K,), 3.0)
        ids = ((np.arange(K, dtype=np.uint32) * 2654435761) % 248320).astype(np.uint32)
        m = float(lg.max())
        s = float(np.float32(np.exp((lg.astype(np.float64) - m) * np.float32(inv_t)).sum() + 0.7))
        q = ref.draft_dist(ids, lg, m, s, inv_t, top_k, top_p, min_p)
        key = ref.race_base(1234 + i, 7 * i)
        out[f"{i}_in"] = np.array([top_k, K], dtype=np.int64)
        out[f"{i}_f"] = np.array([top_p, min_p, inv_t, m, s], dtype=np.float32)
        out[f"{i}_n"] = np.array([q.n, ref.spec_sample_race(q, key)], dtype=np.int64)
        out[f"{i}_key"] = np.array([key], dtype=np.uint64)
        out[f"{i}_id"] = np.array(q.id[:], dtype=np.uint32)
        out[f"{i}_p"] = np.array(q.p[:], dtype=np.float32)
    np.savez_compressed(os.path.join(HERE, "draft_dist.npz"), **out)
    print(f"draft_dist: {len(sets)} sets")


def main():
    path = orc.build_reference()
    if not path:
        raise SystemExit("no reference checkout: cannot generate fixtures")
    ref = orc.Reference(path)
    accept_cases(ref)
    scalar_kats(ref)
    filter_cases(ref)
    rows_cases(ref)
    draft_cases(ref)


if __name__ == "__main__":
    main()
