"""The library's draw generators through the C ABI: the host functions against the fixture made from the reference's
own Sampler::uniform / spec::uniform / spec::raceBase and against the published Philox4x32-10 known answers (no GPU),
and the device fill kernel against the host functions (GPU)."""
import numpy as np
import pytest


@pytest.fixture(scope="module")
def api():
    from whirl_llm_b200 import api
    return api


def bits(d):
    return int(np.float64(d).view(np.uint64))


def test_splitmix_uniform_and_race_base_match_the_reference_fixture(api, golden, oracle):
    kat = golden.json("uniform_kat")
    for r in kat["records"]:
        s, p = r["seed"], r["pos"]
        assert bits(api.uniform_splitmix(s, p, 0)) == r["u0"] == r["sampler_u"]
        assert bits(api.uniform_splitmix(s, p, 1)) == r["u1"]
        assert api.race_base(s, p) == r["base"]
    # the reference's own known-answer statement (tests/unit/spec_sample_tests.cpp:247-256)
    seed, pos, m = 987654321, 41, (1 << 64) - 1
    z = (seed + (pos + 1) * 0x9E3779B97F4A7C15) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    z ^= z >> 31
    assert api.uniform_splitmix(seed, pos, 0) == (z >> 11) * (1.0 / 9007199254740992.0)
    rng = np.random.default_rng(5)
    for s, p, st in zip(rng.integers(0, 2 ** 63, 200), rng.integers(0, 2 ** 40, 200), rng.integers(0, 4, 200)):
        assert api.uniform_splitmix(int(s), int(p), int(st)) == oracle.uniform(int(s), int(p), int(st))
        assert api.race_base(int(s), int(p)) == oracle.race_base(int(s), int(p))


def test_philox_known_answers(api, oracle):
    # Random123 kat_vectors, philox4x32 with 10 rounds
    assert api.philox4x32_10([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert api.philox4x32_10([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert api.philox4x32_10([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]
    for i in range(100):
        assert api.uniform_philox4x32(1234 + (i << 40), i * 7919, i, i & 3) == oracle.philox_uniform(1234 + (i << 40), i * 7919, i, i & 3)


@pytest.mark.gpu
def test_device_fill_matches_the_host_functions(api):
    import torch
    rng = np.random.default_rng(9)
    R = 1500
    seed = rng.integers(0, 2 ** 64, R, dtype=np.uint64)
    pos = rng.integers(0, 2 ** 48, R, dtype=np.uint64)
    sd, pd = torch.from_numpy(seed.view(np.int64)).cuda(), torch.from_numpy(pos.view(np.int64)).cuda()
    for gen in (api.GEN_SPLITMIX, api.GEN_PHILOX):
        for sid in (0, 1, 3):
            u, rk = api.fill_draws(sd, pd, gen, sid)
            u, rk = u.cpu().numpy(), rk.cpu().numpy().view(np.uint64)
            for r in range(0, R, 7):
                s, p = int(seed[r]), int(pos[r])
                want = api.uniform_philox4x32(s, p, r, sid) if gen == api.GEN_PHILOX else api.uniform_splitmix(s, p, sid)
                assert u[r] == want and int(rk[r]) == api.race_base(s, p)
    u, rk = api.fill_draws(sd, pd, want_race_key=False)
    assert rk is None and 0.45 < float(u.mean()) < 0.55
