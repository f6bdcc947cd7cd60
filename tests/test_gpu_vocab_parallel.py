"""Vocab-parallel sampling on one GPU: the shards of a row are processed as separate launches of the local step,
their records laid out as an all-gather would leave them, and the merge must reproduce the single-device result
whenever no shard's top-k list is exhausted (which the merge reports otherwise)."""
import numpy as np
import pytest

from helpers import Inputs
from mako_b200 import lib
from mako_b200.sampler import SamplingParams

pytestmark = pytest.mark.gpu


PARAMS = [
    SamplingParams(temperature=0.8, top_p=0.9, repetition_penalty=1.1, presence_penalty=0.5, frequency_penalty=0.3),
    SamplingParams(temperature=0.8, top_p=0.9, min_p=0.05, repetition_penalty=1.1, presence_penalty=0.5,
                   frequency_penalty=0.3),
    SamplingParams(temperature=0.7, top_k=40, top_p=0.95),
    SamplingParams(temperature=0.0),
]


# (vocabulary, shards): even splits, and splits where the ranks' widths differ (151936 columns over 8 ranks are
# 19008 x 4 + 18976 x 4; three ranks never split these vocabularies evenly)
@pytest.mark.parametrize("v,n_shards", [(151552, 2), (151552, 8), (151936, 8), (151552, 3), (40003, 3)])
@pytest.mark.parametrize("params", PARAMS, ids=["topp", "minp", "topk", "greedy"])
def test_vocab_parallel_equals_single_device(gpu_sampler_factory, ref, v, n_shards, params):
    import torch
    from mako_b200.parallel import vocab_shard
    b, k = 12, 64
    inp = Inputs(141, b, v, n_history=4096)
    s = gpu_sampler_factory(151936, b, 128)
    rb = lib.mk_vp_record_bytes(k)
    gathered = torch.zeros((n_shards, b, rb), dtype=torch.uint8, device="cuda")
    full = torch.from_numpy(inp.logits).cuda()
    hist = torch.from_numpy(inp.history).cuda()
    for g in range(n_shards):
        lo, hi = vocab_shard(v, g, n_shards)
        shard = full[:, lo:hi].contiguous()
        s.vp_local(shard, params, k, gathered[g], id_offset=lo, history=hist)
    res = s.vp_merge(gathered, n_shards, b, k, v, params, torch.from_numpy(inp.u).cuda())
    torch.cuda.synchronize()
    tok, flags, ncand = res.token.cpu().numpy(), res.flags.cpu().numpy(), res.n_cand.cpu().numpy()
    ids = res.cand_ids.cpu().numpy()
    exact, truncated, banded = 0, 0, 0
    for i in range(b):
        w = ref.sample(params, inp.logits[i], inp.u[i], cap=128, history=inp.history[i])
        if flags[i] & 0x20:
            # reported: the nucleus may reach past a shard's list — only legitimate when some shard holds at least
            # as many members of it as its list is long
            lens = [int(((w["cand_ids"] >= vocab_shard(v, g, n_shards)[0]) &
                         (w["cand_ids"] < vocab_shard(v, g, n_shards)[1])).sum()) for g in range(n_shards)]
            assert w["n_cand"] > 128 or max(lens) >= k // 2, f"row {i} flagged with a nucleus of {w['n_cand']} ({lens})"
            truncated += 1
            continue
        if flags[i] & 0x2:
            banded += 1
            continue  # a decision sat in the guard band of the rescaled partial sums
        assert tok[i] == w["token"], f"row {i}"
        assert ncand[i] == w["n_cand"]
        assert np.array_equal(ids[i, :ncand[i]], w["cand_ids"][:ncand[i]])
        exact += 1
    # the comparison must not be empty: flagged rows are the exception (top_p alone flags the few flat rows)
    assert banded <= 1 and truncated <= 3 and exact >= b - 3, (exact, truncated, banded)
    if params.min_p > 0 or params.top_k > 0 or params.temperature <= 0:
        assert exact == b, (exact, truncated, banded)


def test_uneven_shards_count_a_boundary_id_for_its_own_shard(gpu_sampler_factory, ref):
    """151936 columns over 8 ranks are 19008 x 4 + 18976 x 4 wide, so shard 0 ends at column 19008 while equal-width
    arithmetic (ceil(V / 8) = 18992) would put columns 18992..19007 into shard 1. Row 0 has 70 heavy columns at the
    end of shard 0, 16 of them past 18992: shard 0's 64-entry list is exhausted by the candidates, and the merge must
    say so — which it only can if it counts each candidate for the shard it came from. Row 1 spreads its heavy
    columns over the shards: nothing is exhausted, no flag, and the token is the single-device one."""
    import torch
    from mako_b200.parallel import vocab_shard
    v, n_shards, k, b = 151936, 8, 64, 2
    spans = [vocab_shard(v, g, n_shards) for g in range(n_shards)]
    assert spans[0] == (0, 19008) and spans[4][1] - spans[4][0] == 18976
    # a spread-out background far below the heavy columns (identical values would all tie for a shard's list)
    logits = np.random.default_rng(5).uniform(-1000.0, -30.0, size=(b, v)).astype(np.float32)
    logits[0, 19008 - 70:19008] = 10.0 - 0.001 * np.arange(70, dtype=np.float32)
    cols = np.concatenate([np.arange(lo + 5, lo + 15) for lo, _ in spans[:7]])
    logits[1, cols] = 10.0 - 0.001 * np.arange(70, dtype=np.float32)
    u = np.array([0.5, 0.5], dtype=np.float32)
    params = SamplingParams(temperature=1.0, min_p=0.01)
    s = gpu_sampler_factory(151936, 12, 128)
    rb = lib.mk_vp_record_bytes(k)
    gathered = torch.zeros((n_shards, b, rb), dtype=torch.uint8, device="cuda")
    full = torch.from_numpy(logits).cuda()
    for g, (lo, hi) in enumerate(spans):
        s.vp_local(full[:, lo:hi].contiguous(), params, k, gathered[g], id_offset=lo)
    res = s.vp_merge(gathered, n_shards, b, k, v, params, torch.from_numpy(u).cuda())
    torch.cuda.synchronize()
    flags, tok, ncand = res.flags.cpu().numpy(), res.token.cpu().numpy(), res.n_cand.cpu().numpy()
    assert flags[0] & 0x20, "shard 0's list is exhausted by the candidates: the row must be reported"
    assert not (flags[1] & 0x20), "no shard's list is exhausted"
    w = ref.sample(params, logits[1], u[1])
    assert tok[1] == w["token"] and ncand[1] == w["n_cand"] == 70
