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


def block_words(rows: int, ks: int) -> int:
    """4-byte words of one rank's packed block: ids [rows][ks] | vals [rows][ks] | stats [rows][2]
    (whirl_shard_block_words)."""
    return rows * (2 * ks + 2)


def block_views(block: torch.Tensor, rows: int, ks: int):
    """ids (int32), vals (float32), stats (float32) views of one packed block; no copy."""
    assert block.dtype == torch.int32 and block.is_contiguous() and block.numel() == block_words(rows, ks)
    ids = block[: rows * ks].view(rows, ks)
    vals = block[rows * ks: 2 * rows * ks].view(torch.float32).view(rows, ks)
    stats = block[2 * rows * ks:].view(torch.float32).view(rows, 2)
    return ids, vals, stats


def exchange_blocks(block: torch.Tensor, out: Optional[torch.Tensor] = None, group=None) -> torch.Tensor:
    """ONE all-gather of every rank's packed block -> [world * block_words] int32 (rank r's block at r * block_words).
    Nothing is repacked on either side: the selection kernel wrote into `block`, the merge kernel reads `out` in
    place.  2 MiB per rank at 256 rows x 1024 candidates."""
    world = dist.get_world_size(group)
    if out is None:
        out = torch.empty(world * block.numel(), dtype=torch.int32, device=block.device)
    dist.all_gather_into_tensor(out, block, group=group)
    return out


def exchange_candidates(ids: torch.Tensor, vals: torch.Tensor, stats: torch.Tensor, group=None):
    """Three separate arrays -> [world, rows, K_s] ids / vals and [world, rows, 2] stats (views of the gathered blocks).
    For callers that hold the arrays apart; it packs them first (one copy), which sample_vocab_sharded avoids by
    letting the kernel write into the block."""
    world = dist.get_world_size(group)
    rows, ks = ids.shape
    block = torch.empty(block_words(rows, ks), dtype=torch.int32, device=ids.device)
    b_ids, b_vals, b_stats = block_views(block, rows, ks)
    b_ids.copy_(ids), b_vals.copy_(vals), b_stats.copy_(stats)
    flat = exchange_blocks(block, group=group).view(world, block_words(rows, ks))
    g_ids = flat[:, : rows * ks].view(world, rows, ks)
    g_vals = flat[:, rows * ks: 2 * rows * ks].view(torch.float32).view(world, rows, ks)
    g_stats = flat[:, 2 * rows * ks:].view(torch.float32).view(world, rows, 2)
    return g_ids, g_vals, g_stats


class VocabShardedSampler:
    """Vocab-sharded sampling with its buffers kept across steps: this rank's packed block and the gathered blocks."""

    def __init__(self, rows: int, n_total: int, k_s: int = 1024, device=None, group=None):
        self.rows, self.n_total, self.k_s, self.group = rows, n_total, k_s, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.begin, self.end = slice_bounds(n_total, self.world, self.rank)
        self.block = torch.empty(block_words(rows, k_s), dtype=torch.int32, device=device)
        self.gathered = torch.empty(self.world * self.block.numel(), dtype=torch.int32, device=device)
        self.views = block_views(self.block, rows, k_s)

    def select(self, x_local: torch.Tensor, inv_t: float = 1.0, inv_t_rows: Optional[torch.Tensor] = None):
        from . import api
        assert x_local.shape == (self.rows, self.end - self.begin)
        api.topk_rows_shard(x_local, self.k_s, self.begin, inv_t=inv_t, inv_t_rows=inv_t_rows, out=self.views)

    def exchange(self):
        exchange_blocks(self.block, self.gathered, self.group)

    def merge(self, params, kept_cap: int = 0):
        from . import api
        return api.merge_sample_rows_packed(self.gathered, self.world, self.rows, self.k_s, self.n_total, params, kept_cap=kept_cap)

    def sample(self, x_local: torch.Tensor, params, inv_t: float = 1.0, inv_t_rows: Optional[torch.Tensor] = None, kept_cap: int = 0):
        self.select(x_local, inv_t, inv_t_rows)
        self.exchange()
        return self.merge(params, kept_cap)


def sample_vocab_sharded(x_local: torch.Tensor, n_total: int, params, k_s: int = 1024, inv_t: float = 1.0,
                         inv_t_rows: Optional[torch.Tensor] = None, kept_cap: int = 0, group=None):
    """x_local: this rank's [rows, n_total / world] slice of the logits on its GPU.  Returns the SampleResult (the same
    on every rank).  inv_t / inv_t_rows: the temperature the slice statistics are taken at (must match params.inv_t)."""
    s = VocabShardedSampler(x_local.shape[0], n_total, k_s, x_local.device, group)
    return s.sample(x_local, params, inv_t, inv_t_rows, kept_cap)
