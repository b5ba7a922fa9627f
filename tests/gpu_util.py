"""Helpers of the GPU parity tests: numpy <-> device tensors, and one comparison of a GPU result with the oracle's."""
import numpy as np
import torch

from whirl_llm_b200 import api


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def bf16_tensor(bits: np.ndarray) -> torch.Tensor:
    """uint16 bf16 bit patterns -> a CUDA bfloat16 tensor with those bits."""
    return torch.from_numpy(bits.astype(np.int16)).cuda().view(torch.bfloat16)


def row_params(prm: dict, u=None, race_key=None, hist=None, hist_len=None, rep=None, pres=None, freq=None) -> api.RowParams:
    g = lambda k, dt: None if prm.get(k) is None else dev(np.asarray(prm[k]).astype(dt))
    return api.RowParams(
        inv_t=g("inv_t", np.float32), top_k=g("top_k", np.int32), top_p=g("top_p", np.float64), min_p=g("min_p", np.float64),
        greedy=g("greedy", np.uint8), u=None if u is None else dev(np.asarray(u, dtype=np.float64)),
        race_key=None if race_key is None else dev(np.asarray(race_key, dtype=np.uint64).view(np.int64)),
        hist=None if hist is None else dev(np.asarray(hist, dtype=np.int32)),
        hist_len=None if hist_len is None else dev(np.asarray(hist_len, dtype=np.int32)),
        rep=None if rep is None else dev(np.asarray(rep, dtype=np.float32)),
        pres=None if pres is None else dev(np.asarray(pres, dtype=np.float32)),
        freq=None if freq is None else dev(np.asarray(freq, dtype=np.float32)))


def compare_rows(res: api.SampleResult, want: dict, *, p_rtol=1e-5, sum_rtol=1e-5, u=None, allow_boundary=0):
    """GPU result vs oracle rows: tokens, kept-set sizes and ids exact; probabilities and the normaliser to tolerance.
    Rows whose draw lies within 1e-6 of a cumulative boundary may differ in the token; they are counted and returned."""
    torch.cuda.synchronize()
    tok = res.token.cpu().numpy().astype(np.int64)
    st = res.status.cpu().numpy()
    n = res.n_kept.cpu().numpy()
    closed = res.closed.cpu().numpy()
    stats = None if res.stats is None else res.stats.cpu().numpy()
    assert (st == api.ROW_DONE).all(), f"rows not resolved: {np.nonzero(st != api.ROW_DONE)[0][:10]} status {st[st != 0][:10]}"
    assert np.array_equal(n, want["n"]), (np.nonzero(n != want["n"])[0][:10], n[n != want["n"]][:10], want["n"][n != want["n"]][:10])
    assert np.array_equal(closed != 0, want["closed"] != 0)
    if stats is not None:
        assert np.array_equal(stats[:, 0], want["m"])
        nz = want["sum"] != 0
        np.testing.assert_allclose(stats[nz, 1], want["sum"][nz], rtol=sum_rtol)
    if res.kept_ids is not None:
        kid = res.kept_ids.cpu().numpy()
        kp = res.kept_p.cpu().numpy()
        cap = kid.shape[1]
        for r in range(len(n)):
            k = min(int(n[r]), cap, want["kept_ids"].shape[1])
            assert np.array_equal(kid[r, :k], want["kept_ids"][r, :k].astype(np.int64)), (r, kid[r, :k][:8], want["kept_ids"][r, :k][:8])
            np.testing.assert_allclose(kp[r, :k], want["kept_p"][r, :k], rtol=p_rtol, atol=0, err_msg=f"row {r}")
    diff = np.nonzero(tok != want["token"].astype(np.int64))[0]
    boundary = 0
    for r in diff:
        ok = False
        if u is not None and res.kept_ids is not None:
            k = min(int(n[r]), want["kept_p"].shape[1])
            cum = np.cumsum(want["kept_p"][r, :k])
            ok = bool((np.abs(cum - u[r]) < 1e-6).any())
        assert ok, f"row {r}: token {tok[r]} != {want['token'][r]} and the draw is not within 1e-6 of a boundary"
        boundary += 1
    assert boundary <= allow_boundary, f"{boundary} boundary draws"
    return boundary
