"""Vocab-sharded sampling on the GPU: per-slice candidates with global ids, merge, sample.  On one GPU the slices are
computed one after the other and stacked (what the all-gather would deliver); with two or more GPUs the real NCCL
exchange runs in child processes."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

import synth
from gpu_util import compare_rows, dev, row_params

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _case(oracle, rows=12, n_total=32768, shards=8, ks=256):
    x = synth.normalish(55, (rows, n_total), 3.0)
    x[1] = synth.grid_logits(56, (n_total,), 3.0)  # ties across slices
    f = lambda v, dt=np.float32: np.full(rows, v, dtype=dt)
    prm = dict(inv_t=f(1.25), top_k=f(ks, np.uint32), top_p=f(0.9, np.float64))
    prm["top_k"][2] = 40
    prm["greedy"] = f(0, np.uint8)
    prm["greedy"][3] = 1
    u = np.array([oracle.uniform(99, r, 0) for r in range(rows)])
    want = oracle.sample_rows(x, kept_cap=ks, u=u, threads=2, kb=16384, **prm)
    return x, prm, u, want


def test_merge_single_gpu(oracle):
    from whirl_llm_b200 import api
    rows, n_total, shards, ks = 12, 32768, 8, 256
    x, prm, u, want = _case(oracle, rows, n_total, shards, ks)
    w = n_total // shards
    parts = [api.topk_rows_shard(dev(np.ascontiguousarray(x[:, s * w:(s + 1) * w])), ks, s * w, inv_t=1.25) for s in range(shards)]
    ids = torch.stack([p[0] for p in parts]).contiguous()
    vals = torch.stack([p[1] for p in parts]).contiguous()
    stats = torch.stack([p[2] for p in parts]).contiguous()
    assert int(ids.min()) >= 0 and int(ids.max()) < n_total
    res = api.merge_sample_rows(ids, vals, stats, n_total, row_params(prm, u=u), kept_cap=ks)
    compare_rows(res, want, u=u, sum_rtol=2e-5)


def test_packed_blocks_at_full_size(oracle):
    """256 rows x 262,144 tokens in 8 slices, 1024 candidates per slice, global top-p 0.9: every slice's selection writes
    straight into its packed block of the gathered buffer (the layout one all-gather leaves), and the merge reads the
    blocks in place."""
    from whirl_llm_b200 import api
    rows, n_total, shards, ks = 256, 262144, 8, 1024
    x = synth.normalish(57, (rows, n_total), 3.0)
    x[1] = synth.grid_logits(58, (n_total,), 3.0)
    f = lambda v, dt=np.float32: np.full(rows, v, dtype=dt)
    prm = dict(inv_t=f(1.0), top_k=f(ks, np.uint32), top_p=f(0.9, np.float64))
    prm["top_k"][2::5] = 50
    u = synth.hash_u01(59, rows, 0)
    want = oracle.sample_rows(x, kept_cap=ks, u=u, threads=8, kb=16384, **prm)
    w = n_total // shards
    words = api.lib.whirl_shard_block_words(rows, ks)
    assert words == rows * (2 * ks + 2)
    gathered = torch.empty(shards * words, dtype=torch.int32, device="cuda")
    for s in range(shards):
        views = api.shard_block_views(gathered[s * words:(s + 1) * words], rows, ks)
        api.topk_rows_shard(dev(np.ascontiguousarray(x[:, s * w:(s + 1) * w])), ks, s * w, inv_t=1.0, out=views)
    res = api.merge_sample_rows_packed(gathered, shards, rows, ks, n_total, row_params(prm, u=u), kept_cap=ks)
    compare_rows(res, want, u=u, sum_rtol=2e-5)


def _nccl_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from oracle import oracle as orc
        from whirl_llm_b200 import sharded
        o = orc.Oracle()
        rows, n_total, ks = 12, 32768, 256
        x, prm, u, want = _case(o, rows, n_total, world, ks)
        b, e = sharded.slice_bounds(n_total, world, rank)
        res = sharded.sample_vocab_sharded(dev(np.ascontiguousarray(x[:, b:e])), n_total, row_params(prm, u=u), k_s=ks, inv_t=1.25,
                                           kept_cap=ks)
        compare_rows(res, want, u=u, sum_rtol=2e-5)
        # the stated size: 256 rows x 262,144 tokens, 1024 candidates per slice, top-p 0.9; buffers kept across steps
        rows, n_total, ks = 256, 262144, 1024
        x = synth.normalish(57, (rows, n_total), 3.0)
        f = lambda v, dt=np.float32: np.full(rows, v, dtype=dt)
        prm = dict(inv_t=f(1.0), top_k=f(ks, np.uint32), top_p=f(0.9, np.float64))
        u = synth.hash_u01(59, rows, 0)
        want = o.sample_rows(x, kept_cap=8, u=u, threads=8, kb=16384, **prm)
        vs = sharded.VocabShardedSampler(rows, n_total, ks, torch.device("cuda", rank))
        xl = dev(np.ascontiguousarray(x[:, vs.begin:vs.end]))
        for _ in range(2):
            res = vs.sample(xl, row_params(prm, u=u), kept_cap=8)
        compare_rows(res, want, u=u, sum_rtol=2e-5)
        q.put((rank, "ok"))
    except Exception as ex:
        q.put((rank, repr(ex)))
    finally:
        dist.destroy_process_group()


def test_merge_nccl_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ps = [ctx.Process(target=_nccl_worker, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = [q.get(timeout=300) for _ in range(world)]
    for p in ps:
        p.join(timeout=60)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res
