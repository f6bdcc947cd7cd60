"""Host logic of the multi-GPU modes on CPU: shard arithmetic, and the record exchange with two gloo ranks."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mako_b200.parallel import gather_columns, gather_records, row_shard, shard_width, shard_widths, vocab_shard


def test_row_shards_partition_the_batch():
    for batch, world in [(1024, 8), (256, 3), (5, 8), (0, 2), (1000, 7)]:
        spans = [row_shard(batch, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == batch
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [hi - lo for lo, hi in spans]
        assert max(sizes) - min(sizes) <= 1


def test_vocab_shards_are_word_aligned_and_cover_the_vocabulary():
    for v, world in [(151552, 8), (129280, 8), (129280, 3), (1000, 4), (33, 2)]:
        spans = [vocab_shard(v, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == v
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(lo % 32 == 0 for lo, _ in spans)
    assert vocab_shard(151552, 3, 8) == (3 * 18944, 4 * 18944) and shard_width(151552, 8) == 18944
    with pytest.raises(ValueError):
        vocab_shard(100, 2, 2)


def test_uneven_vocab_shards():
    # 151936 columns are 4748 words: 8 ranks get 594 or 593 words each, the wider ones first
    spans = [vocab_shard(151936, r, 8) for r in range(8)]
    assert [hi - lo for lo, hi in spans] == [19008] * 4 + [18976] * 4
    assert shard_widths(151936, 8) == [19008] * 4 + [18976] * 4
    assert shard_widths(151936, 8, 32) == [594] * 4 + [593] * 4
    assert shard_width(151936, 8) == 19008
    # a vocabulary that ends inside a word: the last shard is the ragged one, its mask still a whole word
    assert shard_widths(1000, 3) == [352, 352, 296] and shard_widths(1000, 3, 32) == [11, 11, 10]
    assert sum(shard_widths(129280, 3)) == 129280


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        batch, rb = 6, 528
        local = torch.full((batch, rb), rank + 1, dtype=torch.uint8)
        local[:, 0] = torch.arange(batch, dtype=torch.uint8)
        g = gather_records(local)
        ok = g.shape == (world, batch, rb)
        for r in range(world):
            ok = ok and bool((g[r, :, 1:] == r + 1).all()) and bool((g[r, :, 0] == torch.arange(batch)).all())
        lo, hi = row_shard(10, rank, world)
        t = torch.tensor([hi - lo])
        dist.all_reduce(t)
        ok = ok and int(t.item()) == 10
        # whole rows from uneven column shards (1000 columns over two ranks: 512 + 488)
        full = torch.arange(3 * 1000, dtype=torch.float32).reshape(3, 1000)
        clo, chi = vocab_shard(1000, rank, world)
        rows = gather_columns(full[:, clo:chi].contiguous(), shard_widths(1000, world))
        ok = ok and bool(torch.equal(rows, full))
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_record_exchange_with_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, True), (1, True)]
