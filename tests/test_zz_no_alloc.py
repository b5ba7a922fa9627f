"""The allocation-free greedy pick (whirl_argmax_rows_static) against the workspace variant, through the C ABI.

Some hosts cannot allocate device memory when they sample (a serving engine with a memory plan fixed at start-up, a call
site with no workspace to pass), so this entry point keeps its scratch in a fixed array inside the library.  The picks are
integers: the two entry points must agree exactly, on two calls in a row (the second call finds the first one's leftovers
in the shared scratch).  This file sorts last on purpose, so a run that stops at the first failure has run everything else.
"""
import numpy as np
import pytest
import torch

import synth
from gpu_util import dev

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_workspace_variant_twice(oracle):
    from whirl_llm_b200 import api
    n = 248320
    for call, (rows, seed) in enumerate([(5, 11), (37, 12)]):
        x = synth.normalish(seed, (rows, n), 3.0)
        x[1, 100] = x[1, 9000] = 50.0  # tie: the first index wins
        x[2, n - 1] = 60.0
        xd = dev(x)
        want = api.argmax_rows(xd)                  # caller workspace
        out = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
        got = api.argmax_rows_static(xd, out=out)   # the library's fixed scratch
        torch.cuda.synchronize()
        assert torch.equal(got, want), (call, got.tolist(), want.tolist())
        assert got.cpu().tolist() == [oracle.first_max(r) for r in x]   # and both agree with the CPU checker
        assert got[1].item() == 100 and got[2].item() == n - 1


def test_static_scratch_limit_is_refused():
    from whirl_llm_b200 import api
    x = torch.zeros((api.STATIC_MAX_ROWS + 1, 64), device="cuda")
    with pytest.raises(api.WhirlError) as e:
        api.argmax_rows_static(x)
    assert e.value.status == 4 and "WHIRL_STATIC_MAX_ROWS" in str(e.value)
