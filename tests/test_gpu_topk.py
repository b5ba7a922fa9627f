"""topk_rows on the GPU against the oracle: the candidate set with the (logit desc, id asc) tie rule, exact; the row
maximum exact; the softmax normaliser to 1e-5 (the reference's kernel test allows 1e-4, tests/kernels/test_misc.cpp:353)."""
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


def _check(api, oracle, x, K, inv_t, xd=None):
    ids, vals, stats = api.topk_rows(dev(x) if xd is None else xd, K, inv_t)
    wi, wv, ws = oracle.topk_rows(x, K, inv_t)
    kk = min(K, x.shape[1])
    assert np.array_equal(ids.cpu().numpy()[:, :kk], wi[:, :kk])
    assert np.array_equal(vals.cpu().numpy()[:, :kk].view(np.uint32), wv[:, :kk].view(np.uint32))
    st = stats.cpu().numpy()
    assert np.array_equal(st[:, 0], ws[:, 0])
    np.testing.assert_allclose(st[:, 1], ws[:, 1], rtol=1e-5)


@pytest.mark.parametrize("n,K", [(1, 1), (2, 1), (5, 5), (5, 9), (33, 7), (255, 40), (256, 256), (257, 256), (1000, 16),
                                 (4097, 40), (4097, 1024), (20000, 16384), (248320, 40), (151936, 256), (262144, 1024)])
def test_topk_random(api, oracle, n, K):
    _check(api, oracle, synth.normalish(100 + n + K, (3, n), 3.0), K, 1 / 0.7)


@pytest.mark.parametrize("n,K", [(257, 16), (4097, 300), (70000, 256), (70000, 2000)])
def test_topk_heavy_ties(api, oracle, n, K):
    x = synth.grid_logits(200 + n, (4, n), 0.02)  # ~40 distinct values: the K-th logit has many ties
    x[1] = 1.5                                    # everything ties
    x[2, ::2] = -0.0
    x[2, 1::2] = 0.0                              # -0 == +0: order by id alone
    _check(api, oracle, x, K, 1.0)


def test_topk_k_big_and_reference_shape(api, oracle):
    # the reference kernel test's shape (5 rows x 248320, K = 40, T = 0.7) and the engine's escalation size
    x = synth.normalish(4242, (5, 248320), 3.0)
    x[1, 100] = x[1, 9000] = 50.0
    x[2, 248319] = 60.0
    _check(api, oracle, x, 40, 1 / 0.7)
    _check(api, oracle, x[:2], 16384, 1.0)


def test_topk_bf16_and_unaligned(api, oracle):
    x = synth.normalish(11, (4, 50001), 3.0)
    bits = synth.to_bf16_bits(x)
    _check(api, oracle, oracle.bf16_to_f32(bits), 64, 1.0, xd=bf16_tensor(bits))
    flat = dev(np.concatenate([[0.0], x.reshape(-1)]).astype(np.float32))[1:].view(4, 50001)
    _check(api, oracle, x, 64, 1.3, xd=flat)


def test_topk_argument_errors(api):
    x = torch.zeros((2, 64), device="cuda")
    with pytest.raises(api.WhirlError) as e:
        api.topk_rows(x, 0)
    assert e.value.status == 1
    with pytest.raises(api.WhirlError) as e:
        api.topk_rows(x, 20000)
    assert e.value.status == 4
