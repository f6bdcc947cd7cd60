"""Whole speculative rounds on the device against the reference's sequential loop (src/gen/session.cpp:451-506).

For every sequence the CPU side walks the round as Session::run does: position by position, the forced token first,
else Sampler::verify on that position's logits with the history grown by every draft kept so far, stopping at the
first rejection, and Sampler::sample on the bonus row when every draft was kept; uniforms are taken from the
sequence's stream in the order the reference's generator would hand them out. The GPU does all positions of all
sequences in one launch (mk_sampler_spec_round) and keeps the history on the device between rounds (mk_spec_commit)."""
import numpy as np
import pytest

from mako_b200 import synth
from mako_b200.sampler import SamplingParams

pytestmark = pytest.mark.gpu


def _cpu_round(ref, p, logits, drafts, forced, u, hist):
    """Returns (n_kept, next_token) for one sequence; logits [n_pos, V], drafts [n_pos - 1], forced [n_pos] or None."""
    n_pos = logits.shape[0]
    hist = list(hist)
    drawn = 0
    for j in range(n_pos - 1):
        f = -1 if forced is None else int(forced[j])
        if f >= 0:
            tok, acc = f, f == int(drafts[j])
        elif p.temperature <= 0:
            tok, acc = ref.verify(p, logits[j], int(drafts[j]), 0.0, 0.0, history=hist)
        else:
            tok, acc = ref.verify(p, logits[j], int(drafts[j]), u[drawn], u[drawn + 1], history=hist)
            drawn += 1
        if not acc:
            return j, tok
        hist.append(int(drafts[j]))
    f = -1 if forced is None else int(forced[n_pos - 1])
    if f >= 0:
        return n_pos - 1, f
    return n_pos - 1, ref.sample(p, logits[n_pos - 1], u[drawn], history=hist)["token"]


@pytest.mark.parametrize("params,with_forced", [
    (SamplingParams(temperature=0.8, top_p=0.9, min_p=0.05, repetition_penalty=1.1, presence_penalty=0.5,
                    frequency_penalty=0.3), False),
    (SamplingParams(temperature=0.7, top_k=40, top_p=0.95, repetition_penalty=1.3), True),
    (SamplingParams(temperature=0.0), True),
], ids=["penalised", "nucleus+forced", "greedy+forced"])
@pytest.mark.parametrize("v,n_seq", [(40003, 64), (129280, 24)], ids=["ragged_rows", "aligned_rows"])
def test_rounds_of_four_drafts_and_a_bonus_row(gpu_sampler_factory, ref, params, with_forced, v, n_seq):
    """Rows of 40003 columns are not 16-byte aligned and take the kernel's plain-load path, rows of 129280 columns
    the bulk-copy path: the round's bookkeeping is the same on both."""
    import torch
    n_drafts, cap, rounds = 4, 256, 3
    n_pos = n_drafts + 1
    s = gpu_sampler_factory(v, n_seq * n_pos)
    rng = np.random.default_rng(77)
    hist0 = synth.history_zipf(77, n_seq, v, 40)
    hist_dev = torch.zeros((n_seq, cap), dtype=torch.int32, device="cuda")
    hist_dev[:, :40] = torch.from_numpy(hist0).cuda()
    hlen_dev = torch.full((n_seq,), 40, dtype=torch.int32, device="cuda")
    cpu_hist = [list(hist0[i]) for i in range(n_seq)]
    kept_total = 0
    for rnd in range(rounds):
        logits, spikes = synth.logits(500 + rnd, n_seq * n_pos, v)
        # drafts: mostly the row's strongest tokens (often kept), sometimes a random one (rejected), sometimes a repeat
        drafts = np.empty((n_seq, n_drafts), dtype=np.int32)
        for i in range(n_seq):
            for j in range(n_drafts):
                r = rng.random()
                row = logits[i * n_pos + j]
                drafts[i, j] = int(np.argmax(row)) if r < 0.6 else (int(spikes[i * n_pos + j, 1]) if r < 0.85
                                                                   else int(rng.integers(0, v)))
        forced = None
        if with_forced:
            forced = np.full((n_seq, n_pos), -1, dtype=np.int32)
            pick = rng.random((n_seq, n_pos)) < 0.15
            forced[pick] = np.where(rng.random(pick.sum()) < 0.5, drafts[:, [0]].repeat(n_pos, 1)[pick], 17)
            # where a draft exists, make half of the forced tokens agree with that position's draft
            for i, j in zip(*np.nonzero(pick)):
                if j < n_drafts and rng.random() < 0.5:
                    forced[i, j] = drafts[i, j]
        u = rng.random((n_seq, n_pos + 1), dtype=np.float32)
        kept, nxt, res = s.spec_round(torch.from_numpy(logits).cuda(), params, torch.from_numpy(drafts).cuda(),
                                      torch.from_numpy(u).cuda(), history=hist_dev, history_len=hlen_dev,
                                      forced=None if forced is None else torch.from_numpy(forced).cuda())
        d_drafts = torch.from_numpy(drafts).cuda()
        s.spec_commit(d_drafts, kept, nxt, hist_dev, hlen_dev)
        torch.cuda.synchronize()
        kept, nxt = kept.cpu().numpy(), nxt.cpu().numpy()
        flags = res.flags.cpu().numpy().reshape(n_seq, n_pos)
        assert not (flags & 0x50).any()
        for i in range(n_seq):
            wk, wt = _cpu_round(ref, params, logits[i * n_pos:(i + 1) * n_pos], drafts[i],
                                None if forced is None else forced[i], u[i], cpu_hist[i])
            if (flags[i, : wk + 1] & 0x2).any():
                cpu_hist[i] += [int(t) for t in drafts[i, :kept[i]]] + [int(nxt[i])]  # follow the device past a flagged decision
                continue
            assert (kept[i], nxt[i]) == (wk, wt), f"round {rnd} sequence {i}"
            cpu_hist[i] += [int(t) for t in drafts[i, :wk]] + [wt]
            kept_total += wk
        # the device kept the same histories
        hl = hlen_dev.cpu().numpy()
        hd = hist_dev.cpu().numpy()
        for i in range(n_seq):
            assert hl[i] == len(cpu_hist[i]) and hd[i, : hl[i]].tolist() == [int(t) for t in cpu_hist[i]]
    assert 0 < kept_total < rounds * n_seq * n_drafts
