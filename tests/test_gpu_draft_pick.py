"""The drafter pick (ds_markov + ds_draft_pick, src/kernels/dsv41.metal:664-742) as one fused step: score = logits +
head . embed[prev], argmax with the lowest id on ties, confidence = sigmoid([x, embed[prev]] . w). The reference for
this path is Metal shader code (not runnable here): the checker below restates its arithmetic in numpy; parity is
pinned to that restatement. Scores are floating-point dot products summed in another order than the shader's, so the
argmax is compared where the two best scores are further apart than the summation error, and on constructed ties."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def draft_pick_cpu(logits, head, embed, x, w, prev):
    drafts, confs, gaps = [], [], []
    dim = x.shape[1]
    for b in range(logits.shape[0]):
        e = embed[prev[b]].astype(np.float64)
        score = logits[b].astype(np.float64) + head.astype(np.float64) @ e        # dsv41.metal:667-684
        best = int(np.argmax(score))                                               # first maximum = lowest id
        srt = np.partition(score, -2)[-2:]
        drafts.append(best)
        gaps.append(float(srt[1] - srt[0]))
        s = float(w[:dim].astype(np.float64) @ x[b].astype(np.float64) + w[dim:].astype(np.float64) @ e)
        confs.append(1.0 / (1.0 + np.exp(-s)))                                     # dsv41.metal:739
    return drafts, confs, gaps


def test_draft_pick_chain_matches_restatement(gpu_sampler_factory):
    import torch
    v, rank, dim, n_seq, steps, n_embed = 40003, 256, 512, 5, 3, 40003
    rng = np.random.default_rng(11)
    head = (rng.normal(0, 0.05, size=(v, rank))).astype(np.float32)
    embed = (rng.normal(0, 1.0, size=(n_embed, rank))).astype(np.float32)
    w = (rng.normal(0, 0.05, size=dim + rank)).astype(np.float32)
    logits = rng.normal(0, 2.0, size=(steps, n_seq, v)).astype(np.float32)
    x = rng.normal(0, 1.0, size=(steps, n_seq, dim)).astype(np.float32)
    s = gpu_sampler_factory(v, 8, 0)
    d_head, d_embed, d_w = (torch.from_numpy(t).cuda() for t in (head, embed, w))
    prev = rng.integers(0, v, size=n_seq).astype(np.int32)      # the last sampled token of each sequence
    d_prev = torch.from_numpy(prev).cuda()
    checked = 0
    for k in range(steps):                                       # the chain: a step's draft is the next step's prev
        draft, conf = s.draft_pick(torch.from_numpy(logits[k]).cuda(), d_head, d_embed, torch.from_numpy(x[k]).cuda(),
                                   d_w, d_prev)
        torch.cuda.synchronize()
        wd, wc, gaps = draft_pick_cpu(logits[k], head, embed, x[k], w, prev)
        got = draft.cpu().numpy()
        for b in range(n_seq):
            if gaps[b] > 1e-4:                                   # summation-order error is ~1e-6 at these magnitudes
                assert got[b] == wd[b], f"step {k} seq {b}"
                checked += 1
        assert np.allclose(conf.cpu().numpy(), wc, rtol=2e-6, atol=2e-7)
        prev = got.astype(np.int32)
        d_prev = draft
    assert checked >= steps * n_seq - 2


def test_draft_pick_ties_and_non_finite(gpu_sampler_factory):
    """Zero head: the score is the logit itself, exact — ties break toward the lower id, NaN and -inf never win, a
    row with nothing above -inf picks id 0 (the shader's `s > bv` from bv = -inf, bi = 0)."""
    import torch
    v, rank, dim = 5003, 64, 8
    s = gpu_sampler_factory(v, 8, 0)
    logits = np.zeros((4, v), dtype=np.float32)
    logits[0, [4000, 70, 2999]] = 3.5            # three equal maxima: 70
    logits[1, :] = -np.inf
    logits[1, 17] = np.nan                       # nothing comparable: 0
    logits[2, 9] = np.nan
    logits[2, 4500] = 1.0                        # NaN ignored: 4500
    logits[3, 5002] = np.inf                     # the last column
    z = lambda *shape: torch.zeros(shape, dtype=torch.float32, device="cuda")
    prev = torch.tensor([1, 2, 3, 4], dtype=torch.int32, device="cuda")
    draft, conf = s.draft_pick(torch.from_numpy(logits).cuda(), z(v, rank), z(10, rank), z(4, dim), z(dim + rank), prev)
    torch.cuda.synchronize()
    assert draft.cpu().tolist() == [70, 0, 4500, 5002]
    assert conf.cpu().tolist() == [0.5, 0.5, 0.5, 0.5]


def test_draft_pick_plain(gpu_sampler_factory):
    """hy4_draft_pick (src/kernels/hy4f.metal:352-397): the largest logit with the lowest index on ties, confidence =
    sigmoid(conf_w . h + bias); the argmax is exact, the confidence a float dot product (tolerance)."""
    import torch
    v, width, n = 129283, 4096, 6
    rng = np.random.default_rng(3)
    logits = rng.normal(0, 2, size=(n, v)).astype(np.float32)
    logits[1, [90000, 17, 4000]] = 50.0          # ties: 17
    logits[2, :] = -np.inf                       # nothing above -inf: 0
    logits[3, 5] = np.nan
    logits[4, v - 1] = 60.0                      # the last column
    h = rng.normal(0, 1, size=(n, width)).astype(np.float32)
    w = rng.normal(0, 0.02, size=width).astype(np.float32)
    s = gpu_sampler_factory(v, 8, 0)
    nxt = torch.full((n,), -1, dtype=torch.int32, device="cuda")
    logits = np.ascontiguousarray(logits)        # row stride v floats: only row 0 is 16-byte aligned
    draft, conf = s.draft_pick_plain(torch.from_numpy(logits).cuda(), torch.from_numpy(h).cuda(),
                                     torch.from_numpy(w).cuda(), 0.25, next_prev=nxt)
    torch.cuda.synchronize()
    want = []
    for b in range(n):
        row = np.where(np.isnan(logits[b]), -np.inf, logits[b])
        want.append(int(np.argmax(row)) if np.isfinite(row).any() or (row == np.inf).any() else 0)
    assert draft.cpu().tolist() == want
    assert nxt.cpu().tolist() == want
    wc = 1.0 / (1.0 + np.exp(-(h.astype(np.float64) @ w.astype(np.float64) + 0.25)))
    assert np.allclose(conf.cpu().numpy(), wc, rtol=2e-6, atol=2e-7)
