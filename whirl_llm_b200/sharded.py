"""Multi-GPU host logic of the sampling path (one process per GPU, torch.distributed).

Row-sharded mode: rows are independent, so a batch splits into contiguous blocks of rows, one per rank, with no
data-path collective; only the 4-byte tokens are gathered.
Vocab-sharded mode: each rank holds a slice of every row (the output of a tensor-parallel lm_head); ranks exchange their
per-slice candidates with ONE all-gather (NCCL over NVLink on GPUs) and every rank merges and samples.
The reference has no multi-GPU path (include/whirl/gpu_select.h:23-25); this module is new.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def row_block(rows: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of the rows rank `rank` samples: contiguous blocks, sizes differ by at most one."""
    base, extra = divmod(rows, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def gather_tokens(local_tokens: torch.Tensor, rows: int, group=None) -> torch.Tensor:
    """All ranks' tokens in row order (row-sharded mode).  local_tokens: this rank's block, int32."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    sizes = [row_block(rows, world, r)[1] - row_block(rows, world, r)[0] for r in range(world)]
    assert local_tokens.numel() == sizes[rank]
    pad = max(sizes)
    buf = torch.zeros(pad, dtype=local_tokens.dtype, device=local_tokens.device)
    buf[: sizes[rank]] = local_tokens
    out = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(out, buf, group=group)
    return torch.cat([o[:s] for o, s in zip(out, sizes)])


def slice_bounds(n_total: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of the token ids rank `rank` owns in vocab-sharded mode (equal slices, n_total % world == 0)."""
    if n_total % world:
        raise ValueError("vocab-sharded mode wants a vocabulary divisible by the number of ranks")
    w = n_total // world
    return rank * w, (rank + 1) * w


def exchange_candidates(ids: torch.Tensor, vals: torch.Tensor, stats: torch.Tensor, group=None):
    """One all-gather of every rank's [rows, K_s] ids / vals and [rows, 2] stats -> [world, rows, K_s] / [world, rows, 2].

    The three arrays travel as one buffer (ids and vals are 4-byte words; 2 * K_s + 2 words per row), so the exchange
    is a single collective: 2 MiB per rank at 256 rows x 1024 candidates."""
    world = dist.get_world_size(group)
    rows, ks = ids.shape
    packed = torch.cat([ids.view(torch.int32), vals.view(torch.int32), stats.view(torch.int32)], dim=1).contiguous()
    flat = torch.empty((world * rows, 2 * ks + 2), dtype=torch.int32, device=ids.device)
    dist.all_gather_into_tensor(flat, packed, group=group)
    out = flat.view(world, rows, 2 * ks + 2)
    g_ids = out[:, :, :ks].contiguous()
    g_vals = out[:, :, ks: 2 * ks].contiguous().view(torch.float32)
    g_stats = out[:, :, 2 * ks:].contiguous().view(torch.float32)
    return g_ids, g_vals, g_stats


def sample_vocab_sharded(x_local: torch.Tensor, n_total: int, params, k_s: int = 1024, inv_t: float = 1.0,
                         inv_t_rows: Optional[torch.Tensor] = None, kept_cap: int = 0, group=None):
    """x_local: this rank's [rows, n_total / world] slice of the logits on its GPU.  Returns the SampleResult (the same
    on every rank).  inv_t / inv_t_rows: the temperature the slice statistics are taken at (must match params.inv_t)."""
    from . import api
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    begin, end = slice_bounds(n_total, world, rank)
    assert x_local.shape[1] == end - begin
    ids, vals, stats = api.topk_rows_shard(x_local, k_s, begin, inv_t=inv_t, inv_t_rows=inv_t_rows)
    g_ids, g_vals, g_stats = exchange_candidates(ids, vals, stats, group)
    return api.merge_sample_rows(g_ids, g_vals, g_stats, n_total, params, kept_cap=kept_cap)
