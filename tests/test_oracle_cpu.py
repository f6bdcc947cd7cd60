"""CPU tests of the checkers themselves: the restatement ("port") against the known answers of the reference's own
test (tests/sampler_test.cpp) re-expressed as exact checks, and — where the reference build is present — against
the reference's unmodified sampler.cpp call for call."""
import numpy as np
import pytest

from mako_b200 import synth
from mako_b200.sampler import SamplingParams
from oracle.oracle import Oracle, have_reference

L8 = np.array([2.0, 1.5, 0.3, -0.5, 1.9, -2.0, 0.0, 1.0], dtype=np.float32)  # tests/sampler_test.cpp:56


def kinds():
    return ["port", "reference"] if have_reference() else ["port"]


@pytest.fixture(params=kinds())
def orc(request):
    from oracle.oracle import build
    build()
    return Oracle(request.param)


def test_greedy_picks_largest_and_verifies(orc):
    p = SamplingParams(temperature=0.0)
    assert orc.sample(p, L8, 0.3)["token"] == 0                       # sampler_test.cpp:63
    assert orc.verify(p, L8, 4, 0.1, 0.2) == (0, False)               # :65
    assert orc.verify(p, L8, 0, 0.1, 0.2) == (0, True)                # :66


def test_top_k_keeps_0_4_1(orc):
    r = orc.sample(SamplingParams(temperature=1.0, top_k=3), L8, 0.5, cap=8)
    assert sorted(r["cand_ids"].tolist()) == [0, 1, 4]                # :92-96
    # a draft outside the top 3 is never accepted (:97-102)
    for u in np.linspace(0, 0.999, 50):
        tok, acc = orc.verify(SamplingParams(temperature=1.0, top_k=3), L8, 7, float(u), 0.5)
        assert not acc and tok in (0, 1, 4)


def test_top_p_keeps_0_4_1(orc):
    r = orc.sample(SamplingParams(temperature=1.0, top_p=0.7), L8, 0.5, cap=8)
    assert r["cand_ids"].tolist() == [0, 4, 1]                        # :105-109, sorted by weight


def test_min_p_keeps_0_1_4_7(orc):
    r = orc.sample(SamplingParams(temperature=1.0, min_p=0.3), L8, 0.5, cap=8)
    assert r["cand_ids"].tolist() == [0, 1, 4, 7]                     # :112-116, ascending id


def test_penalty_arithmetic(orc):
    # presence + frequency * count subtracted once (:118-125); repetition divides positive, multiplies others (:126-133)
    p = SamplingParams(temperature=1.0, presence_penalty=0.5, frequency_penalty=0.25)
    r = orc.sample(p, L8, 0.5, history=[0, 0], cap=8)
    pen = L8.copy()
    pen[0] -= np.float32(0.5) + np.float32(0.25) * np.float32(2)
    q = np.exp((pen - pen.max()).astype(np.float32)).astype(np.float32)
    assert np.allclose(r["cand_q"], q, rtol=1e-6)
    p = SamplingParams(temperature=1.0, repetition_penalty=2.0)
    r = orc.sample(p, L8, 0.5, history=[0, 5], cap=8)
    rp = L8.copy()
    rp[0] /= 2.0
    rp[5] *= 2.0
    q = np.exp((rp - rp.max()).astype(np.float32)).astype(np.float32)
    assert np.allclose(r["cand_q"], q, rtol=1e-6)


def test_vanishing_temperature_and_zero_repetition(orc):
    assert orc.sample(SamplingParams(temperature=1e-40), L8, 0.7)["token"] == 0            # :137-138
    t = orc.sample(SamplingParams(temperature=1.0, repetition_penalty=0.0), L8, 0.3, history=[0, 4])["token"]
    assert 0 <= t < 8                                                                       # :139-143


def test_verify_acceptance_rate_is_p_draft(orc):
    # acceptance = P(u * total < q_draft) = p(draft) for uniform u (:76-89), checked on a grid instead of Monte Carlo
    p = SamplingParams(temperature=0.7)
    q = np.exp(((L8 - L8.max()) / np.float32(0.7)).astype(np.float64))
    prob = q / q.sum()
    us = (np.arange(20000) + 0.5) / 20000
    for draft in (0, 4, 5):
        acc = sum(orc.verify(p, L8, draft, float(u), 0.5)[1] for u in us)
        assert abs(acc / us.size - prob[draft]) < 1e-3


def test_empty_vocabulary_is_an_error(orc):
    with pytest.raises(ValueError):
        orc.sample(SamplingParams(), np.zeros(0, dtype=np.float32), 0.5)


def test_all_masked_and_nonfinite_rows(orc):
    l = np.full(16, -np.inf, dtype=np.float32)
    assert orc.sample(SamplingParams(temperature=1.0), l, 0.5)["token"] == 0
    l = np.array([1.0, np.nan, 3.0, np.inf, 2.0], dtype=np.float32)
    assert orc.sample(SamplingParams(temperature=1.0), l, 0.5)["token"] == 3
    l = np.array([np.nan, 5.0, 3.0], dtype=np.float32)
    assert orc.sample(SamplingParams(temperature=1.0), l, 0.5)["token"] == 0


@pytest.mark.skipif(not have_reference(), reason="reference build not present")
def test_own_generator_path_equals_uniform_driven_path():
    """Sampler::sample with its own mt19937_64 equals the u-driven draw with the mirrored uniforms."""
    ref = Oracle("reference")
    lg, _ = synth.logits(77, 3, 151552)
    for b, p in enumerate([SamplingParams(temperature=0.7, top_k=40, top_p=0.95), SamplingParams(temperature=1.0),
                           SamplingParams(temperature=0.8, top_p=0.9, min_p=0.05)]):
        n = 40 if p.top_k or p.min_p else 12
        toks = ref.sample_rng(p, lg[b], 1234 + b, n)
        us = ref.uniforms(1234 + b, n)
        mine = [ref.sample(p, lg[b], float(u))["token"] for u in us]
        assert toks.tolist() == mine


@pytest.mark.skipif(not have_reference(), reason="reference build not present")
@pytest.mark.parametrize("params", [
    SamplingParams(temperature=0.7, top_k=40, top_p=0.95),
    SamplingParams(temperature=0.8, top_p=0.9, min_p=0.05, repetition_penalty=1.1, presence_penalty=0.5,
                   frequency_penalty=0.3),
    SamplingParams(temperature=1.0),
    SamplingParams(temperature=0.6, top_p=0.95),
    SamplingParams(temperature=1.3, top_k=17),
    SamplingParams(temperature=1.3, top_k=200, min_p=0.3),   # fewer candidates than top_k: nothing is reordered
    SamplingParams(temperature=0.0),
])
def test_port_equals_reference(params):
    ref, port = Oracle("reference"), Oracle("port")
    v = 20011
    lg, sp = synth.logits(5, 12, v)
    h = synth.history_zipf(5, 12, v, 300)
    m = synth.mask(5, 12, v, fraction=0.2, spike_ids=sp)
    bi, bv = synth.bias(5, 12, v, 16)
    u = synth.uniforms(5, 12)
    u2 = synth.uniforms(5, 12, purpose=1)
    u3 = synth.uniforms(5, 12, purpose=2)
    lq = synth.add_noise(5, lg, v)
    for b in range(12):
        kw = dict(history=h[b]) if b % 2 else {}
        if b % 3 == 0:
            kw.update(mask=m[b], bias_ids=bi[b], bias_vals=bv[b])
        a = ref.sample(params, lg[b], u[b], cap=v, **kw)
        c = port.sample(params, lg[b], u[b], cap=v, **kw)
        assert a["token"] == c["token"] and a["n_cand"] == c["n_cand"] and a["prob"] == c["prob"]
        assert np.array_equal(a["cand_ids"], c["cand_ids"]) and np.array_equal(a["cand_q"], c["cand_q"])
        d = int(a["cand_ids"][min(1, a["n_cand"] - 1)])
        assert ref.verify(params, lg[b], d, u[b], u2[b], **kw) == port.verify(params, lg[b], d, u[b], u2[b], **kw)
        assert ref.verify_pq(params, lg[b], lq[b], u[b], u2[b], u3[b], **kw) == \
            port.verify_pq(params, lg[b], lq[b], u[b], u2[b], u3[b], **kw)


def test_one_hot_drafter_reduces_to_verify(orc):
    """max(0, p - q) with a one-hot q is the reference's verify (sampler.cpp:86-107)."""
    v = 5003
    lg, _ = synth.logits(9, 6, v)
    p = SamplingParams(temperature=0.9, top_p=0.9)
    u1, u2 = synth.uniforms(9, 6, purpose=1), synth.uniforms(9, 6, purpose=2)
    for b in range(6):
        d = int(orc.sample(p, lg[b], 0.6, cap=4)["cand_ids"][0])
        onehot = np.full(v, -np.inf, dtype=np.float32)
        onehot[d] = 0.0
        dd, acc, tok = orc.verify_pq(p, lg[b], onehot, 0.5, u1[b], u2[b])
        tok2, acc2 = orc.verify(p, lg[b], d, u1[b], u2[b])
        assert dd == d and acc == acc2
        if acc:
            assert tok == tok2 == d


@pytest.mark.skipif(not have_reference(), reason="reference build not present")
def test_top_k_that_does_not_truncate_leaves_ascending_ids():
    """top_k without top_p: the checker sorts the list only when top_k truncated it (the reference's own order there
    is nth_element's); with no more candidates than top_k, and with exactly top_k, the list stays in ascending id as
    the reference leaves it (sampler.cpp:30-43), and the draw walks it in that order."""
    ref = Oracle("reference")
    v = 5003
    lg = np.full(v, -30.0, dtype=np.float32)
    ids = np.array([4000, 17, 2500, 900, 3100], dtype=np.int64)
    lg[ids] = np.array([1.0, 2.0, 3.0, 2.5, 0.5], dtype=np.float32)
    for top_k, expect in ((9, sorted(ids.tolist())), (5, sorted(ids.tolist())), (3, [2500, 900, 17])):
        p = SamplingParams(temperature=1.0, top_k=top_k, min_p=0.01)
        r = ref.sample(p, lg, 0.999, cap=16)
        assert r["cand_ids"].tolist() == expect, (top_k, r["cand_ids"])
        assert r["token"] == expect[-1]       # u close to 1 lands on the last candidate of the walk
