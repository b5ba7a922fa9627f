"""The fused sampler on the GPU against the oracle and against the fixtures generated from the reference's own code.
Tokens, kept-set sizes and kept ids must match exactly (a draw within 1e-6 of a cumulative boundary may pick the
neighbour; such rows are counted); probabilities within 1e-5 relative; the row maximum exactly; the softmax normaliser
within 1e-5 relative."""
import numpy as np
import pytest
import torch

import synth
from golden import make_golden as mg
from gpu_util import bf16_tensor, compare_rows, dev, row_params

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    from whirl_llm_b200 import api
    return api


def uniforms(oracle, prm):
    return np.array([oracle.uniform(int(s), int(p), 0) for s, p in zip(prm["seed"], prm["pos_idx"])])


def race_keys(oracle, prm):
    return np.array([oracle.race_base(int(s), int(p)) for s, p in zip(prm["seed"], prm["pos_idx"])], dtype=np.uint64)


def run_split(api, oracle, x, prm, kept_cap, **pen):
    """GPU sample_rows takes one draw rule per call (race key array or not): run race and non-race rows separately."""
    u = uniforms(oracle, prm)
    rk = race_keys(oracle, prm)
    race = prm.get("race")
    race = np.zeros(len(u), dtype=np.uint8) if race is None else race
    out = []
    for flag in (0, 1):
        sel = np.nonzero(race == flag)[0]
        if len(sel) == 0:
            continue
        sub = {k: (None if v is None else np.asarray(v)[sel]) for k, v in prm.items()}
        pp = {k: (None if v is None else np.asarray(v)[sel]) for k, v in pen.items()}
        res = api.sample_rows(dev(np.ascontiguousarray(x[sel])), row_params(sub, u=u[sel], race_key=rk[sel] if flag else None, **pp),
                              kept_cap=kept_cap)
        out.append((sel, res))
    return out, u


def subset(want, sel):
    return {k: (None if v is None else v[sel]) for k, v in want.items()}


def test_small_vocab_mix(api, oracle):
    R, V = 300, 777
    x = np.where(np.arange(R)[:, None] % 3 == 0, synth.grid_logits(31, (R, V), 2.0), synth.normalish(32, (R, V), 1.5)).astype(np.float32)
    prm = mg.row_params(R, 33, 64)
    # rows with no filter at all are open sets: 256 sorted candidates, then the rest of the row in id order
    want = oracle.sample_rows(x, kept_cap=V, **prm)
    assert (want["closed"] == 0).sum() > 10 and want["full_used"][want["closed"] == 0].sum() > 0  # some draws walk the row
    assert want["full_used"][want["closed"] != 0].sum() == 0
    runs, u = run_split(api, oracle, x, prm, V)
    for sel, res in runs:
        compare_rows(res, subset(want, sel), u=u[sel])


def test_golden_engine_rows(api, oracle, golden):
    """The fixture made by the reference's real SampleBuffers / filterCands / sampleRow (V = 20000)."""
    R, V = mg.ENGINE_ROWS["rows"], mg.ENGINE_ROWS["V"]
    x = synth.normalish(80, (R, V), 3.0)
    x[::5] = synth.grid_logits(81, (R, V), 3.0)[::5]
    x[3] = 0.0
    prm = mg.row_params(R, 82, 600)
    g = golden.npz("rows_engine")
    want = {k: g[k] for k in g.files}
    # the fixture holds rows closed at 256 candidates, rows closed at 16384, and open rows whose draw walks the row; all of
    # them must come back answered and equal
    runs, u = run_split(api, oracle, x, prm, 1024)
    for sel, res in runs:
        compare_rows(res, subset(want, sel), u=u[sel])


def test_third_level_rows(api, oracle):
    """Rows whose kept set reaches past 16384 candidates: flat logits and a top-p close to one, so the whole row is
    sorted (the reference's last escalation step); inverse-CDF and race draws, with and without penalties."""
    R, V = 12, 65536
    x = synth.normalish(91, (R, V), 0.4)
    f = lambda v, dt=np.float32: np.full(R, v, dtype=dt)
    prm = dict(inv_t=f(1.0), top_k=f(0, np.uint32), top_p=f(0.9995, np.float64), min_p=f(0.0, np.float64))
    prm["top_p"][1::3] = 0.97
    prm["min_p"][2::3] = 1e-3
    prm["top_k"][5] = 40000
    u = synth.hash_u01(92, R, 0)
    want = oracle.sample_rows(x, kept_cap=512, u=u, threads=4, **prm)
    assert (want["n"] > 16384).sum() >= R // 2 and (want["closed"] != 0).all()
    res = api.sample_rows(dev(x), row_params(prm, u=u), kept_cap=512)
    compare_rows(res, want, u=u)
    assert int(res.counters[api.CNT_UNRESOLVED].item()) == 0
    # the same rows with a token history and penalties
    hist = synth.zipf_history(93, R, 1024, V, 1.1)
    pen = dict(hist=hist, hist_len=np.full(R, 1024, dtype=np.int32), rep=f(1.2), pres=f(0.4), freq=f(0.2))
    want = oracle.sample_rows(x, kept_cap=512, u=u, threads=4, **prm, **{k: (v.astype(np.uint32) if k == "hist_len" else v) for k, v in pen.items()})
    res = api.sample_rows(dev(x), row_params(prm, u=u, **pen), kept_cap=512)
    compare_rows(res, want, u=u)


def test_adversarial_and_special_rows(api, oracle):
    """Element orders and values that stress the single-pass kernel: rising rows (every logit beats the threshold so far,
    the candidate log overflows and the row is redone by the multi-pass kernel), falling rows, constant rows (all ties:
    the lower id wins), rows with +-inf entries, a row length that is no multiple of the stage size, and more rows than
    SMs so that CTAs take several rows; then the same with a token history and penalties."""
    R, V = 320, 36868  # 9 stages and a 4-logit remainder
    x = synth.normalish(71, (R, V), 2.0)
    x[0::8] = np.sort(x[0::8], axis=1)                    # rising
    x[1::8] = -np.sort(-x[1::8], axis=1)                  # falling
    x[2::8] = 1.25                                        # constant
    x[3::8, ::97] = -np.inf
    x[4::8, 5::1013] = np.inf                             # several +inf: ties at the top
    x[5::8] = np.round(x[5::8] * 2) / 2                   # heavy ties
    f = lambda v, dt=np.float32: np.full(R, v, dtype=dt)
    prm = dict(inv_t=f(1 / 0.9), top_k=f(40, np.uint32), top_p=f(0.92, np.float64), min_p=f(0.01, np.float64))
    prm["top_k"][6::8] = 256
    prm["top_k"][7::8] = 1
    u = synth.hash_u01(72, R, 0)
    want = oracle.sample_rows(x, kept_cap=256, u=u, threads=4, **prm)
    res = api.sample_rows(dev(x), row_params(prm, u=u), kept_cap=256)
    compare_rows(res, want, u=u)
    assert int(res.counters[api.CNT_UNRESOLVED].item()) == 0
    hist = synth.zipf_history(73, R, 512, V, 1.1)
    hist_len = np.full(R, 512, dtype=np.int32)
    hist_len[::5] = 17
    pen = dict(hist=hist, hist_len=hist_len, rep=f(1.3), pres=f(0.2), freq=f(0.1))
    want = oracle.sample_rows(x, kept_cap=256, u=u, threads=4, **prm, **{k: (v.astype(np.uint32) if k == "hist_len" else v) for k, v in pen.items()})
    res = api.sample_rows(dev(x), row_params(prm, u=u, **pen), kept_cap=256)
    compare_rows(res, want, u=u)


def test_open_rows_large_vocab(api, oracle):
    """Pure temperature sampling (no filter): the single-pass kernel hands rows whose draw falls past the 256 candidates to
    the multi-pass kernel, which walks the row in id order."""
    R, V = 24, 151936
    x = synth.normalish(61, (R, V), 1.0)  # flat rows: the candidates hold little mass, most draws walk
    f = lambda v, dt=np.float32: np.full(R, v, dtype=dt)
    prm = dict(inv_t=f(1.0), top_k=f(0, np.uint32), top_p=f(1.0, np.float64), min_p=f(0.0, np.float64))
    u = synth.hash_u01(62, R, 0)
    want = oracle.sample_rows(x, kept_cap=256, u=u, threads=4, **prm)
    assert want["full_used"].sum() >= R // 2
    res = api.sample_rows(dev(x), row_params(prm, u=u), kept_cap=256)
    compare_rows(res, want, u=None)  # u only matters for the boundary allowance inside the candidates
    assert int(res.counters[api.CNT_OPEN_TAIL].item()) == int(want["full_used"].sum())


def test_config2_penalised(api, oracle):
    """BASELINE config 2 (reduced batch): V 151936, N(0, 2.5^2), 4096-id Zipf history, rep 1.1 / pres 0.5 / freq 0.3,
    T 0.8, top-k 50, top-p 0.9, min-p 0.05."""
    R, V, H = 16, 151936, 4096
    x = synth.normalish(21, (R, V), 2.5)
    hist = synth.zipf_history(22, R, H, V)
    hist_len = np.full(R, H, dtype=np.int32)
    hist_len[1] = 100
    hist_len[2] = 0
    f = lambda v, dt=np.float32: np.full(R, v, dtype=dt)
    prm = dict(inv_t=f(1 / 0.8), top_k=f(50, np.uint32), top_p=f(0.9, np.float64), min_p=f(0.05, np.float64))
    u = np.array([oracle.philox_uniform(1234, 0, r) for r in range(R)])
    pen = dict(hist=hist, hist_len=hist_len, rep=f(1.1), pres=f(0.5), freq=f(0.3))
    want = oracle.sample_rows(x, kept_cap=50, u=u, threads=4, **prm, **{k: (v.astype(np.uint32) if k == "hist_len" else v) for k, v in pen.items()})
    res = api.sample_rows(dev(x), row_params(prm, u=u, **pen), kept_cap=50)
    compare_rows(res, want, u=u)
    # without the row statistics the kernel normalises over the candidates only: same tokens, kept sets, probabilities
    res = api.sample_rows(dev(x), row_params(prm, u=u, **pen), kept_cap=50, want_stats=False)
    compare_rows(res, want, u=u)
    # the penalties changed something: the unpenalised run differs in at least one kept set
    plain = oracle.sample_rows(x, kept_cap=50, u=u, threads=4, **prm)
    assert any(not np.array_equal(plain["kept_ids"][r], want["kept_ids"][r]) for r in range(R))


def test_config1_draws(api, oracle):
    """BASELINE config 1: one row, V 151936, 20 boosted ids, greedy + T 0.7 / top-k 40 / top-p 0.95, successive draws."""
    V, draws = 151936, 200
    x = synth.normalish(1234, (1, V), 3.0)
    x[0, (np.arange(20) * 7573 + 11) % V] += 15.0
    xs = np.repeat(x, draws, axis=0)
    f = lambda v, dt=np.float32: np.full(draws, v, dtype=dt)
    prm = dict(inv_t=f(1 / 0.7), top_k=f(40, np.uint32), top_p=f(0.95, np.float64))
    for src in ("splitmix", "philox"):
        u = np.array([oracle.uniform(1234, i, 0) if src == "splitmix" else oracle.philox_uniform(1234, i, 0) for i in range(draws)])
        want = oracle.sample_rows(xs, kept_cap=40, u=u, threads=4, **prm)
        res = api.sample_rows(dev(xs), row_params(prm, u=u), kept_cap=40)
        compare_rows(res, want, u=u)
        res = api.sample_rows(dev(xs), row_params(prm, u=u), kept_cap=40, want_stats=False)
        compare_rows(res, want, u=u)
    g = api.sample_rows(dev(x), row_params(dict(greedy=np.ones(1, dtype=np.uint8))))
    assert g.token.item() == oracle.first_max(x[0])


def test_config4_bf16_mix(api, oracle):
    """BASELINE config 4 (reduced batch): bf16, V 262144, 1% of entries +10, 25% greedy, T U[0.5,1.2], top-k U{1..1024},
    top-p U[0.8,1]."""
    R, V = 24, 262144
    x = synth.normalish(41, (R, V), 3.0)
    x[synth.hash_u01(42, R * V, 1).reshape(R, V) < 0.01] += 10.0
    bits = synth.to_bf16_bits(x)
    u8 = synth.hash_u01(43, R * 4, 2).reshape(R, 4)
    prm = dict(inv_t=(1.0 / (0.5 + 0.7 * u8[:, 0])).astype(np.float32), top_k=(1 + (u8[:, 1] * 1024).astype(np.uint32)).astype(np.uint32),
               top_p=0.8 + 0.2 * u8[:, 2], greedy=(u8[:, 3] < 0.25).astype(np.uint8))
    u = synth.hash_u01(44, R, 3)
    want = oracle.sample_rows(bits, kept_cap=1024, u=u, threads=4, **prm)
    res = api.sample_rows(bf16_tensor(bits), row_params(prm, u=u), kept_cap=1024)
    compare_rows(res, want, u=u)
    res = api.sample_rows(bf16_tensor(bits), row_params(prm, u=u), kept_cap=1024, want_stats=False)
    compare_rows(res, want, u=u)


def test_large_kept_sets_with_ties_and_penalties(api, oracle):
    """Rows keeping 65 .. 1024 candidates out of logits with few distinct values (many equal keys for the histogram that
    ranks them), half of the rows penalised with a history that holds their best tokens, one row whose cumulative
    probabilities meet top_p exactly (285 of 300 equal candidates against 0.95: the division-free cuts must hand it to
    the dividing form).  Tokens and kept-set sizes only, so that the single-pass kernel takes its quick tail; f32 and
    bf16."""
    R, V, H = 48, 65536, 512
    x = np.round(synth.normalish(611, (R, V), 2.0) * 8.0).astype(np.float32) / 8.0
    x[5] = -50.0
    x[5, 1000:1300] = 3.0
    ks = np.array([65, 128, 256, 257, 300, 300, 512, 1000, 1024, 96, 640, 200], dtype=np.uint32)
    u8 = synth.hash_u01(612, R * 2, 1).reshape(R, 2)
    prm = dict(inv_t=np.full(R, 1.0, dtype=np.float32), top_k=np.tile(ks, R // len(ks)),
               top_p=np.array([0.7, 0.9, 0.95, 1.0])[(u8[:, 0] * 4).astype(int)], min_p=np.where(u8[:, 1] < 0.5, 0.0, 0.01))
    prm["top_p"][5] = 0.95
    prm["min_p"][5] = 0.0
    order = np.argsort(-x, axis=1, kind="stable")[:, :H].astype(np.int32)
    hist = np.ascontiguousarray(order[:, ::-1])                       # the best 512 tokens of every row, some of them twice
    hist[:, ::7] = hist[:, 3:4]
    hist_len = np.where(np.arange(R) % 2 == 0, H, 0).astype(np.int32)  # (odd rows: no penalties)
    f = lambda v: np.full(R, v, dtype=np.float32)
    pen = dict(hist=hist, hist_len=hist_len, rep=f(1.2), pres=f(0.3), freq=f(0.1))
    u = synth.hash_u01(613, R, 2)
    open_pen = {k: (v.astype(np.uint32) if k == "hist_len" else v) for k, v in pen.items()}
    want = oracle.sample_rows(x, kept_cap=1024, u=u, threads=4, **prm, **open_pen)
    res = api.sample_rows(dev(x), row_params(prm, u=u, **pen), kept_cap=0, want_stats=False)
    compare_rows(res, want, u=u)
    assert int(want["n"][5]) in (285, 286)
    bits = synth.to_bf16_bits(x)
    want = oracle.sample_rows(bits, kept_cap=1024, u=u, threads=4, **prm, **open_pen)
    res = api.sample_rows(bf16_tensor(bits), row_params(prm, u=u, **pen), kept_cap=0, want_stats=False)
    compare_rows(res, want, u=u)


def test_argument_errors(api):
    x = torch.zeros((2, 64), device="cuda")
    with pytest.raises(api.WhirlError) as e:
        api.sample_rows(x, api.RowParams(), ws=torch.zeros(16, dtype=torch.uint8, device="cuda"))
    assert e.value.status == 3
    with pytest.raises(ValueError):
        api.sample_rows(torch.zeros((2, 64)), api.RowParams())
