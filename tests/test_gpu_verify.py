"""GPU parity of speculative verification: the deterministic-draft form (Sampler::verify, sampler.cpp:86-107), the
general p/q form built on it, the acceptance loop of a speculative round, and the stateful one-row object with
the reference's generator."""
import numpy as np
import pytest

from helpers import Inputs
from mako_b200 import synth
from mako_b200.sampler import Sampler, SamplingParams

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("params", [
    SamplingParams(temperature=0.6, top_p=0.95),
    SamplingParams(temperature=0.7, top_k=40, top_p=0.95),
    SamplingParams(temperature=0.8, top_p=0.9, min_p=0.05, repetition_penalty=1.1, presence_penalty=0.5,
                   frequency_penalty=0.3),
    SamplingParams(temperature=0.0),
], ids=["topp", "topk", "penalised", "greedy"])
def test_verify_deterministic_draft(gpu_sampler_factory, ref, params):
    import torch
    v, b = 129280, 40
    inp = Inputs(51, b, v, n_history=512)
    g = inp.to_gpu()
    # drafts: the most likely token for most rows (often accepted), a spike or a random id for others
    draft = np.zeros(b, dtype=np.int32)
    for i in range(b):
        top = ref.sample(params, inp.logits[i], 0.0, cap=4, **inp.row_kwargs(i))
        draft[i] = top["cand_ids"][0] if i % 3 else (inp.spikes[i, 1] if i % 2 else (i * 977) % v)
    s = gpu_sampler_factory(v, b, 16)
    res = s.verify(g["logits"], params, torch.from_numpy(draft).cuda(), g["u"], g["u2"], **g["kw"])
    torch.cuda.synchronize()
    tok, acc = res.token.cpu().numpy(), res.accepted.cpu().numpy()
    n_acc = 0
    for i in range(b):
        wt, wa = ref.verify(params, inp.logits[i], int(draft[i]), inp.u[i], inp.u2[i], **inp.row_kwargs(i))
        assert (tok[i], bool(acc[i])) == (wt, wa), f"row {i}"
        n_acc += wa
    assert 0 < n_acc < b


def test_verify_pq_with_lists_of_thousands(gpu_sampler_factory, ref):
    """Rows without spikes: the target keeps thousands of candidates, so a rejected position's resample runs over long
    lists (ranked through bitmaps instead of sorted); draft token, acceptance and returned token against the
    restatement, and some positions must be rejected."""
    import torch
    v, b = 129280, 12
    params = SamplingParams(temperature=0.55, top_p=0.9)      # 1300 to 2500 target candidates, up to 300 drafter's
    inp = Inputs(4242, b, v, n_spikes=0, sigma=2.0)
    lq = synth.add_noise(4242, inp.logits, v, sigma=1.0)
    g = inp.to_gpu()
    s = gpu_sampler_factory(v, b, 16)
    res = s.verify_pq(g["logits"], torch.from_numpy(lq).cuda(), params, g["u"], g["u2"], g["u3"])
    torch.cuda.synchronize()
    d, acc, tok = res.draft_token.cpu().numpy(), res.accepted.cpu().numpy(), res.token.cpu().numpy()
    flags = res.flags.cpu().numpy()
    n_rej = 0
    for i in range(b):
        wd, wa, wt = ref.verify_pq(params, inp.logits[i], lq[i], inp.u[i], inp.u2[i], inp.u3[i])
        assert not (flags[i] & 0x50), f"row {i} flags {flags[i]:#x}"
        if flags[i] & 0x2:
            continue
        assert (d[i], bool(acc[i]), tok[i]) == (wd, wa, wt), f"row {i}"
        n_rej += not wa
    assert n_rej >= 3


def test_verify_pq_config3(gpu_sampler_factory, ref):
    """64 sequences x 5 positions in the benchmark; here 24 positions with the same distributions."""
    import torch
    v, b = 129280, 24
    params = SamplingParams(temperature=0.6, top_p=0.95)
    inp = Inputs(61, b, v)
    lq = synth.add_noise(61, inp.logits, v, sigma=1.0)
    g = inp.to_gpu()
    s = gpu_sampler_factory(v, b, 16)
    res = s.verify_pq(g["logits"], torch.from_numpy(lq).cuda(), params, g["u"], g["u2"], g["u3"])
    torch.cuda.synchronize()
    d, acc, tok = res.draft_token.cpu().numpy(), res.accepted.cpu().numpy(), res.token.cpu().numpy()
    flags = res.flags.cpu().numpy()
    n_acc = 0
    for i in range(b):
        wd, wa, wt = ref.verify_pq(params, inp.logits[i], lq[i], inp.u[i], inp.u2[i], inp.u3[i])
        assert not (flags[i] & 0x50), f"row {i} flags {flags[i]:#x}"
        assert (d[i], bool(acc[i]), tok[i]) == (wd, wa, wt), f"row {i}"
        n_acc += wa
    assert 0 < n_acc < b


def test_spec_resolve_acceptance_loop(gpu_sampler_factory):
    import torch
    s = gpu_sampler_factory(1024, 8)
    acc = torch.tensor([[1, 1, 1, 1, 0], [1, 0, 1, 1, 0], [0, 0, 0, 0, 0], [1, 1, 1, 0, 0]], dtype=torch.int32).cuda()
    tok = torch.arange(20, dtype=torch.int32).reshape(4, 5).cuda()
    kept, nxt = s.spec_resolve(acc, tok)
    torch.cuda.synchronize()
    assert kept.cpu().tolist() == [4, 1, 0, 3]
    assert nxt.cpu().tolist() == [4, 6, 10, 18]


def test_row_sampler_reproduces_reference_token_stream(ref):
    """Same seed, same logits: the stateful object draws the reference's tokens (own mt19937_64, accept() history)."""
    import torch
    if ref.kind != "reference":
        pytest.skip("needs the reference build for its generator path")
    v = 151552
    lg, _ = synth.logits(71, 2, v)
    for b, p in enumerate([SamplingParams(temperature=0.7, top_k=40, top_p=0.95),
                           SamplingParams(temperature=0.8, top_p=0.9, min_p=0.05)]):
        want = ref.sample_rng(p, lg[b], 4242 + b, 25)
        smp = Sampler(p, v, 4242 + b)
        dev_row = torch.from_numpy(lg[b]).cuda()
        got = [smp.sample(lg[b] if i % 2 else dev_row) for i in range(25)]  # host and device rows alike
        assert got == want.tolist()


def test_row_sampler_accept_and_verify(ref):
    v = 40000
    lg, sp = synth.logits(81, 1, v)
    p = SamplingParams(temperature=0.9, top_p=0.9, repetition_penalty=1.2, presence_penalty=0.4, frequency_penalty=0.2)
    smp = Sampler(p, v, 99)
    hist = [int(sp[0, 0]), int(sp[0, 0]), int(sp[0, 1]), 5, 5, 5]
    for t in hist:
        smp.accept(t)
    us = ref.uniforms(99, 8)
    # verify consumes u[0] (+u[1] after a rejection), then sample consumes the next one
    d = int(sp[0, 2])
    tok, acc = smp.verify(lg[0], d)
    wt, wa = ref.verify(p, lg[0], d, us[0], us[1], history=hist)
    assert (tok, acc) == (wt, wa)
    nxt = 1 if acc else 2
    assert smp.sample(lg[0]) == ref.sample(p, lg[0], us[nxt], history=hist)["token"]
    g = Sampler(SamplingParams(temperature=0.0), v, 1)
    assert g.greedy() and g.sample(lg[0]) == int(np.argmax(lg[0]))
    assert g.verify(lg[0], int(np.argmax(lg[0]))) == (int(np.argmax(lg[0])), True)
