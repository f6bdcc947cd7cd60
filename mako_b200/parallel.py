"""Host logic of the two multi-GPU modes (one process per GPU, torch.distributed).

Row-sharded: rows are independent, every rank samples its own contiguous block of rows; no collective.
Vocab-parallel: every rank holds a contiguous block of columns of every row; one exchange step — an all-gather of
the per-row shard records — between the local kernel and the merge kernel. The reference has neither (it runs on
one device, one row at a time); the single-device sampler defines the expected result.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist


def row_shard(batch: int, rank: int, world: int) -> Tuple[int, int]:
    """Rows [lo, hi) of rank `rank`: contiguous blocks, the first batch % world ranks hold one row more."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("rank/world out of range")
    base, extra = divmod(batch, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def vocab_shard(n_vocab: int, rank: int, world: int) -> Tuple[int, int]:
    """Columns [lo, hi) of rank `rank`. Shard boundaries fall on multiples of 32 columns so that a packed
    allowed-token mask can be sliced by words, and of 4 columns so that rows stay 16-byte aligned."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("rank/world out of range")
    words = (n_vocab + 31) // 32
    base, extra = divmod(words, world)
    lo_w = rank * base + min(rank, extra)
    hi_w = lo_w + base + (1 if rank < extra else 0)
    return min(lo_w * 32, n_vocab), min(hi_w * 32, n_vocab)


def shard_width(n_vocab: int, world: int) -> int:
    """Width of the widest shard; the merge kernel maps a token id to its shard with this (equal-width shards)."""
    return max(vocab_shard(n_vocab, r, world)[1] - vocab_shard(n_vocab, r, world)[0] for r in range(world))


def gather_records(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather of the per-row shard records: local [batch, record_bytes] uint8 -> [world, batch, record_bytes],
    shard r at index r (the layout mk_sampler_vp_merge expects)."""
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    if local.device.type == "cpu":  # gloo has no all_gather_into_tensor for every dtype: gather a list
        parts = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(parts, local.contiguous(), group=group)
        for r, p in enumerate(parts):
            out[r].copy_(p)
    else:
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
    return out


def vocab_parallel_sample(sampler, shard_logits: torch.Tensor, params, u: torch.Tensor, n_vocab_total: int, k: int = 64,
                          *, history=None, mask=None, bias=None, group=None):
    """Local step, all-gather, merge. `shard_logits` holds this rank's columns of every row."""
    from ._lib import lib
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    lo, hi = vocab_shard(n_vocab_total, rank, world)
    assert shard_logits.shape[1] == hi - lo, "shard width does not match vocab_shard()"
    batch = shard_logits.shape[0]
    rb = lib.mk_vp_record_bytes(k)
    records = torch.empty((batch, rb), dtype=torch.uint8, device=shard_logits.device)
    sampler.vp_local(shard_logits, params, k, records, id_offset=lo, history=history, mask=mask, bias=bias)
    gathered = gather_records(records, group)
    return sampler.vp_merge(gathered, world, batch, k, n_vocab_total, params, u)
