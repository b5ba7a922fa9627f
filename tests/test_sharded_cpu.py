"""The multi-rank host logic on CPU: two gloo ranks exchange their candidates / tokens; the merged result equals the
oracle's on the unsharded rows.  (Kernels need a GPU; here each rank's slice candidates come from the oracle.)"""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import synth
        from oracle import oracle as orc
        from whirl_llm_b200 import sharded
        o = orc.Oracle()
        rows, n_total, ks, inv_t = 6, 4096, 64, 1.25
        x = synth.normalish(321, (rows, n_total), 3.0)  # every rank regenerates the same rows and keeps its slice
        b, e = sharded.slice_bounds(n_total, world, rank)
        ids, vals, stats = o.topk_rows(x[:, b:e], ks, inv_t)
        ids = ids + b
        g_ids, g_vals, g_stats = sharded.exchange_candidates(torch.from_numpy(ids), torch.from_numpy(vals), torch.from_numpy(stats))
        assert g_ids.shape == (world, rows, ks) and g_stats.shape == (world, rows, 2)
        # the gathered block of this rank is what it sent
        assert torch.equal(g_ids[rank], torch.from_numpy(ids)) and torch.equal(g_vals[rank], torch.from_numpy(vals))
        # the packed form: the block of every rank arrives whole and in rank order, and its views alias it
        block = torch.empty(sharded.block_words(rows, ks), dtype=torch.int32)
        b_ids, b_vals, b_stats = sharded.block_views(block, rows, ks)
        b_ids.copy_(torch.from_numpy(ids)), b_vals.copy_(torch.from_numpy(vals)), b_stats.copy_(torch.from_numpy(stats))
        assert b_ids.data_ptr() == block.data_ptr() and b_stats.data_ptr() == block.data_ptr() + 8 * rows * ks
        flat = sharded.exchange_blocks(block)
        assert flat.numel() == world * block.numel() and torch.equal(flat[rank * block.numel():(rank + 1) * block.numel()], block)
        for r in range(world):
            gi, gv, gs = sharded.block_views(flat[r * block.numel():(r + 1) * block.numel()], rows, ks)
            assert torch.equal(gi, g_ids[r]) and torch.equal(gv, g_vals[r]) and torch.equal(gs, g_stats[r])
        # merged candidates == the unsharded row's candidates
        wi, wv, ws = o.topk_rows(x, ks, inv_t)
        for r in range(rows):
            mi, mv, ms = o.merge_shards(g_ids[:, r].numpy(), g_vals[:, r].numpy(), g_stats[:, r].numpy(), ks, inv_t)
            assert np.array_equal(mi, wi[r]) and np.array_equal(mv, wv[r])
            assert ms[0] == ws[r, 0] and abs(ms[1] - ws[r, 1]) <= 1e-6 * ws[r, 1]
        # row-sharded mode: blocks cover the rows once, tokens come back in row order
        blocks = [sharded.row_block(11, world, r) for r in range(world)]
        assert blocks[0][0] == 0 and blocks[-1][1] == 11 and all(blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
        lb, le = sharded.row_block(11, world, rank)
        toks = sharded.gather_tokens(torch.arange(lb, le, dtype=torch.int32) * 7, 11)
        assert torch.equal(toks, torch.arange(11, dtype=torch.int32) * 7)
        q.put((rank, "ok"))
    except Exception as ex:  # report instead of hanging the other rank
        q.put((rank, repr(ex)))
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in ps:
        p.join(timeout=60)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res
