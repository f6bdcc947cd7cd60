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
    """Width of the widest shard (the first one): what a buffer that must hold any rank's columns is sized for."""
    return max(vocab_shard(n_vocab, r, world)[1] - vocab_shard(n_vocab, r, world)[0] for r in range(world))


def _world(group=None) -> int:
    """Ranks of the group; 1 in a process that never joined one (a single GPU is a group of one)."""
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _rank(group=None) -> int:
    return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


def _all_gather(local: torch.Tensor, group=None) -> torch.Tensor:
    """local [...] -> [world, ...], rank r at index r. NCCL gathers into one tensor; gloo (CPU tests) into a list."""
    world = _world(group)
    if world == 1:
        return local.contiguous().unsqueeze(0).clone()
    out = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    if local.device.type == "cpu":
        parts = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(parts, local.contiguous(), group=group)
        for r, p in enumerate(parts):
            out[r].copy_(p)
    else:
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
    return out


def gather_records(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather of the per-row shard records: local [batch, record_bytes] uint8 -> [world, batch, record_bytes],
    shard r at index r (the layout mk_sampler_vp_merge expects)."""
    return _all_gather(local, group)


def shard_widths(n_vocab: int, world: int, unit: int = 1):
    """Width of every rank's shard, in columns (unit 1) or in words of a packed mask (unit 32)."""
    out = []
    for r in range(world):
        lo, hi = vocab_shard(n_vocab, r, world)
        out.append((hi + unit - 1) // unit - lo // unit)
    return out


def gather_columns(shard: torch.Tensor, widths, group=None) -> torch.Tensor:
    """Whole rows from their column shards: shard [rows, widths[rank]] -> [rows, sum(widths)] on every rank. Shards
    may differ in width: each is padded to the widest for the collective and trimmed when the rows are put together."""
    world = _world(group)
    assert len(widths) == world and shard.shape[1] == widths[_rank(group)]
    rows, wmax = shard.shape[0], max(widths)
    padded = torch.zeros((rows, wmax), dtype=shard.dtype, device=shard.device)
    padded[:, : shard.shape[1]] = shard
    parts = _all_gather(padded, group)
    out = torch.empty((rows, sum(widths)), dtype=shard.dtype, device=shard.device)
    at = 0
    for r in range(world):
        out[:, at:at + widths[r]] = parts[r][:, : widths[r]]
        at += widths[r]
    return out


def truncated_rows(flags: torch.Tensor) -> torch.Tensor:
    """Indices of the rows whose merge reported MK_FLAG_VP_TRUNCATED (a host synchronisation: the count decides what
    is exchanged next)."""
    from ._lib import FLAG_VP_TRUNCATED
    return torch.nonzero((flags.to(torch.int64) & FLAG_VP_TRUNCATED) != 0).flatten()


def vocab_parallel_sample(sampler, shard_logits: torch.Tensor, params, u: torch.Tensor, n_vocab_total: int, k: int = 64,
                          *, history=None, mask=None, bias=None, group=None, exact: bool = True, whole_sampler=None):
    """Local step, all-gather, merge. `shard_logits` holds this rank's columns of every row; `history` and `bias` are
    whole (ids outside the shard are ignored locally), `mask` holds the shard's words.

    A row whose nucleus reaches past some shard's k-entry list comes back from the merge with MK_FLAG_VP_TRUNCATED:
    its token may differ from the single-device one. With `exact` (the default) such rows take a second round: their
    columns are all-gathered into whole rows on every rank and sampled by the single-device kernel, so every row
    returns the token the reference returns; the flag is cleared on those rows. The second round costs a host
    synchronisation (the flags are read) and 4 * n_vocab_total bytes per truncated row and rank. `whole_sampler`
    (default: `sampler`) is the handle that samples the whole rows: it must have been created for n_vocab_total
    columns; rows are taken in chunks of its max_batch.
    """
    from ._lib import FLAG_VP_TRUNCATED, lib
    rank, world = _rank(group), _world(group)
    lo, hi = vocab_shard(n_vocab_total, rank, world)
    assert shard_logits.shape[1] == hi - lo, "shard width does not match vocab_shard()"
    batch = shard_logits.shape[0]
    rb = lib.mk_vp_record_bytes(k)
    records = torch.empty((batch, rb), dtype=torch.uint8, device=shard_logits.device)
    sampler.vp_local(shard_logits, params, k, records, id_offset=lo, history=history, mask=mask, bias=bias)
    gathered = gather_records(records, group)
    res = sampler.vp_merge(gathered, world, batch, k, n_vocab_total, params, u)
    if not exact:
        return res
    idx = truncated_rows(res.flags)       # the merge is deterministic: every rank sees the same rows
    if idx.numel() == 0:
        return res
    keep = {name: getattr(res, name).clone() for name in ("token", "prob", "flags", "n_cand")}
    rows = gather_columns(shard_logits.index_select(0, idx), shard_widths(n_vocab_total, world), group)
    kw = {}
    if history is not None:
        kw["history"] = history.index_select(0, idx).contiguous()
    if mask is not None:
        mw = shard_widths(n_vocab_total, world, 32)
        kw["mask"] = gather_columns(mask.index_select(0, idx)[:, : mw[rank]].contiguous(), mw, group)
    if bias is not None:
        kw["bias"] = bias.index_select(0, idx).contiguous()
    ws = whole_sampler if whole_sampler is not None else sampler
    assert ws.n_vocab >= n_vocab_total, "the handle that samples whole rows must cover the whole vocabulary"
    u_rows = u.index_select(0, idx).contiguous()
    for c0 in range(0, idx.numel(), ws.max_batch):
        c1 = min(c0 + ws.max_batch, idx.numel())
        whole = ws.sample(rows[c0:c1], params, u_rows[c0:c1], **{n: t[c0:c1] for n, t in kw.items()})
        for name in keep:
            keep[name][idx[c0:c1]] = getattr(whole, name)[: c1 - c0]
    for name in keep:                      # back into the sampler's output tensors, which `res` views
        getattr(res, name).copy_(keep[name])
    return res
