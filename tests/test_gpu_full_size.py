"""The benchmark configurations at their full sizes, GPU tokens against the CPU reference on identical inputs:
1000 independent single-row steps (V=151552, top_k 40 / top_p 0.95), 128 masked + biased rows (draw and greedy),
320 positions of p/q verification, and the 1024-row scale-out batch (top_p alone over penalised rows). The CPU side
runs the reference sampler on all host threads. Every token must be the reference's; rows whose decision the kernel
itself reports as inside a numeric guard band are left out of the comparison, counted, and must stay rare."""
import os

import numpy as np
import pytest

from mako_b200 import synth
from mako_b200.sampler import SamplingParams, pack_bias

pytestmark = pytest.mark.gpu

THREADS = os.cpu_count() or 1


def _gpu_tokens(factory, v, logits, params, u, chunk, **kw):
    """Tokens and flags of the batched kernel over all rows, `chunk` rows per launch."""
    import torch
    s = factory(v, chunk)
    toks, flags = [], []
    for lo in range(0, logits.shape[0], chunk):
        hi = min(lo + chunk, logits.shape[0])
        dk = {}
        if kw.get("history") is not None:
            dk["history"] = torch.from_numpy(kw["history"][lo:hi]).cuda()
        if kw.get("mask") is not None:
            dk["mask"] = torch.from_numpy(kw["mask"][lo:hi].view(np.int32)).cuda()
        if kw.get("bias_ids") is not None:
            dk["bias"] = torch.from_numpy(pack_bias(kw["bias_ids"][lo:hi], kw["bias_vals"][lo:hi])).cuda()
        res = s.sample(torch.from_numpy(logits[lo:hi]).cuda(), params, torch.from_numpy(u[lo:hi]).cuda(), **dk)
        torch.cuda.synchronize()
        toks.append(res.token.cpu().numpy().copy())
        flags.append(res.flags.cpu().numpy().copy())
    return np.concatenate(toks), np.concatenate(flags)


def _check(tok, flags, want, max_banded):
    assert not (flags & 0x50).any(), "a row overflowed or timed out"
    sure = (flags & 0x2) == 0
    assert int((~sure).sum()) <= max_banded, f"{int((~sure).sum())} rows in a guard band"
    bad = np.nonzero(tok[sure] != want[sure])[0]
    assert bad.size == 0, f"{bad.size} token mismatches, first at row {np.nonzero(sure)[0][bad[0]]}"
    assert int(sure.sum()) >= tok.size - max_banded


def test_config0_thousand_single_row_steps(gpu_sampler_factory, ref):
    """1000 independent steps, fresh logits and one uniform each (the reference-runnable case). The rows go through
    the kernel 250 at a time — rows are independent, so that is 1000 steps — and the first 16 once more one row per
    launch, as a decode loop issues them."""
    import torch
    v, n = 151552, 1000
    p = SamplingParams(temperature=0.7, top_k=40, top_p=0.95)
    logits, _ = synth.logits(5000, n, v)
    u = synth.uniforms(5000, n)
    _, want = ref.time_sample_batch(p, logits, u, n_threads=THREADS)
    tok, flags = _gpu_tokens(gpu_sampler_factory, v, logits, p, u, 250)
    _check(tok, flags, want, max_banded=2)
    one = gpu_sampler_factory(v, 250)
    for i in range(16):
        res = one.sample(torch.from_numpy(logits[i:i + 1]).cuda(), p, torch.from_numpy(u[i:i + 1]).cuda())
        torch.cuda.synchronize()
        assert int(res.token.cpu()[0]) == want[i] or int(res.flags.cpu()[0]) & 0x2


@pytest.mark.parametrize("params", [SamplingParams(temperature=1.0, top_p=1.0), SamplingParams(temperature=0.0)],
                         ids=["draw", "greedy"])
def test_config2_masked_biased_128_rows(gpu_sampler_factory, ref, params):
    v, b, nb = 151552, 128, 64
    logits, spikes = synth.logits(5002, b, v)
    u = synth.uniforms(5002, b)
    mask = synth.mask(5002, b, v, spike_ids=spikes)
    bias_ids, bias_vals = synth.bias(5002, b, v, nb)
    _, want = ref.time_sample_batch(params, logits, u, mask=mask, bias_ids=bias_ids, bias_vals=bias_vals,
                                    n_threads=THREADS)
    tok, flags = _gpu_tokens(gpu_sampler_factory, v, logits, params, u, b, mask=mask, bias_ids=bias_ids,
                             bias_vals=bias_vals)
    _check(tok, flags, want, max_banded=0)


def test_config3_pq_verification_320_positions(gpu_sampler_factory, ref):
    """64 sequences x (4 drafted + 1 bonus) positions: drafter logits = target + N(0,1) noise, T 0.6 / top_p 0.95 on
    both; draft token, acceptance and returned token must all be the restatement's (no reference counterpart: the
    checker builds general p/q rejection from two calls of the reference's distribution())."""
    import torch
    v, b = 129280, 320
    p = SamplingParams(temperature=0.6, top_p=0.95)
    target, _ = synth.logits(5003, b, v)
    drafter = synth.add_noise(5003, target, v)
    u1, u2, u3 = (synth.uniforms(5003, b, purpose=k) for k in range(3))
    s = gpu_sampler_factory(v, b)
    res = s.verify_pq(torch.from_numpy(target).cuda(), torch.from_numpy(drafter).cuda(), p,
                      torch.from_numpy(u1).cuda(), torch.from_numpy(u2).cuda(), torch.from_numpy(u3).cuda())
    torch.cuda.synchronize()
    d, acc, tok = res.draft_token.cpu().numpy(), res.accepted.cpu().numpy(), res.token.cpu().numpy()
    flags = res.flags.cpu().numpy()
    assert not (flags & 0x50).any()
    n_acc = banded = 0
    for i in range(b):
        if flags[i] & 0x2:
            banded += 1
            continue
        wd, wa, wt = ref.verify_pq(p, target[i], drafter[i], u1[i], u2[i], u3[i])
        assert (d[i], bool(acc[i]), tok[i]) == (wd, wa, wt), f"position {i}"
        n_acc += wa
    assert banded <= 3 and 0 < n_acc < b


def test_config4_1024_rows_top_p_alone(gpu_sampler_factory, ref):
    v, b, h = 151552, 1024, 4096
    p = SamplingParams(temperature=0.8, top_p=0.9, repetition_penalty=1.1, presence_penalty=0.5, frequency_penalty=0.3)
    logits, _ = synth.logits(5004, b, v)
    u = synth.uniforms(5004, b)
    hist = synth.history_zipf(5004, b, v, h)
    _, want = ref.time_sample_batch(p, logits, u, history=hist, n_threads=THREADS)
    tok, flags = _gpu_tokens(gpu_sampler_factory, v, logits, p, u, 256, history=hist)
    _check(tok, flags, want, max_banded=6)
