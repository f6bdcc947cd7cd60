"""Shared pieces of the parity tests: seeded inputs, the GPU call, the per-row oracle call, the comparison."""
from __future__ import annotations

import numpy as np

from mako_b200 import synth
from mako_b200.sampler import SamplingParams, pack_bias


class Inputs:
    def __init__(self, seed, batch, n_vocab, *, n_history=0, with_mask=False, n_bias=0, zipf_s=1.1, ld=None,
                 sigma=2.0, n_spikes=8, mask_fraction=0.02):
        self.seed, self.batch, self.n_vocab = seed, batch, n_vocab
        self.logits, self.spikes = synth.logits(seed, batch, n_vocab, ld=ld, sigma=sigma, n_spikes=n_spikes)
        self.history = synth.history_zipf(seed, batch, n_vocab, n_history, s=zipf_s) if n_history else None
        self.mask = synth.mask(seed, batch, n_vocab, fraction=mask_fraction,
                               spike_ids=self.spikes if n_spikes else None) if with_mask else None
        if n_bias:
            self.bias_ids, self.bias_vals = synth.bias(seed, batch, n_vocab, n_bias)
        else:
            self.bias_ids = self.bias_vals = None
        self.u = synth.uniforms(seed, batch, purpose=0)
        self.u2 = synth.uniforms(seed, batch, purpose=1)
        self.u3 = synth.uniforms(seed, batch, purpose=2)

    def row_kwargs(self, b):
        kw = {}
        if self.history is not None:
            kw["history"] = self.history[b]
        if self.mask is not None:
            kw["mask"] = self.mask[b]
        if self.bias_ids is not None:
            kw["bias_ids"], kw["bias_vals"] = self.bias_ids[b], self.bias_vals[b]
        return kw

    def to_gpu(self):
        import torch
        d = {"logits": torch.from_numpy(self.logits).cuda()}
        kw = {}
        if self.history is not None:
            kw["history"] = torch.from_numpy(self.history).cuda()
        if self.mask is not None:
            kw["mask"] = torch.from_numpy(self.mask.view(np.int32)).cuda()
        if self.bias_ids is not None:
            kw["bias"] = torch.from_numpy(pack_bias(self.bias_ids, self.bias_vals)).cuda()
        d["kw"] = kw
        d["u"] = torch.from_numpy(self.u).cuda()
        d["u2"] = torch.from_numpy(self.u2).cuda()
        d["u3"] = torch.from_numpy(self.u3).cuda()
        return d


def oracle_sample_rows(oracle, params: SamplingParams, inp: Inputs, cap=0):
    out = []
    for b in range(inp.batch):
        out.append(oracle.sample(params, inp.logits[b, : inp.n_vocab], inp.u[b], cap=cap, **inp.row_kwargs(b)))
    return out


def compare_sample(res, want, cap=0, prob_rtol=1e-5):
    """res: SampleResult (GPU), want: list of oracle dicts. Token ids and candidate sets bit-exact, q bit-exact,
    probabilities within prob_rtol relative. Returns the number of rows whose draw was flagged near a CDF boundary."""
    tok = res.token.cpu().numpy()
    prob = res.prob.cpu().numpy()
    ncand = res.n_cand.cpu().numpy()
    flags = res.flags.cpu().numpy()
    ids = res.cand_ids.cpu().numpy() if res.cand_ids is not None else None
    qs = res.cand_q.cpu().numpy() if res.cand_q is not None else None
    near = 0
    for b, w in enumerate(want):
        assert not (flags[b] & (0x10 | 0x40)), f"row {b}: flags {flags[b]:#x}"
        assert ncand[b] == w["n_cand"], f"row {b}: n_cand {ncand[b]} != {w['n_cand']}"
        if cap and ids is not None:
            k = min(w["n_cand"], cap)
            assert np.array_equal(ids[b, :k], w["cand_ids"][:k]), f"row {b}: candidate ids differ"
            assert np.array_equal(qs[b, :k].view(np.uint32), w["cand_q"][:k].view(np.uint32)), f"row {b}: q differ"
        assert tok[b] == w["token"], f"row {b}: token {tok[b]} != {w['token']} (flags {flags[b]:#x})"
        assert abs(prob[b] - w["prob"]) <= prob_rtol * abs(w["prob"]), f"row {b}: prob {prob[b]} vs {w['prob']}"
        assert bool(flags[b] & 1) == bool(w["near_boundary"]), f"row {b}: near-boundary flag differs"
        near += int(flags[b] & 1)
    return near
