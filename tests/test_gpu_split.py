"""Small batches under a top_k: every row split over many CTAs and merged (three launches) must give what one CTA per
row gives, and both what the CPU reference gives: token ids, candidate lists and weights bit for bit. Covers ragged
vocabulary sizes, penalised histories, masks and biases, and a row whose best entries all sit in one column shard,
which the merge must report and the follow-up launch must run again as one CTA."""
import numpy as np
import pytest

from helpers import Inputs, compare_sample, oracle_sample_rows
from mako_b200.sampler import SamplingParams

pytestmark = pytest.mark.gpu

TOPK = SamplingParams(temperature=0.7, top_k=40, top_p=0.95)
TOPK_PEN = SamplingParams(temperature=0.8, top_k=50, top_p=0.9, min_p=0.01, repetition_penalty=1.1,
                          presence_penalty=0.5, frequency_penalty=0.3)
TOPK_ONLY = SamplingParams(temperature=1.3, top_k=64)


def _both(factory, ref, params, inp, cap=64):
    """Runs the split path and the one-CTA-per-row path on the same inputs; checks both against the reference."""
    import torch
    s = factory(inp.n_vocab, 8, cap)
    g = inp.to_gpu()
    logits = g["logits"][:, : inp.n_vocab] if g["logits"].shape[1] != inp.n_vocab else g["logits"]
    want = oracle_sample_rows(ref, params, inp, cap=cap)
    out = []
    for on in (True, False):
        s.set_split(on)
        res = s.sample(logits, params, g["u"], **g["kw"])
        torch.cuda.synchronize()
        compare_sample(res, want, cap=cap)
        out.append(res)
    s.set_split(True)
    a, b = out
    assert np.array_equal(a.token.cpu().numpy(), b.token.cpu().numpy())
    assert np.array_equal(a.n_cand.cpu().numpy(), b.n_cand.cpu().numpy())
    return a


@pytest.mark.parametrize("batch", [1, 3, 8])
@pytest.mark.parametrize("n_vocab,ld", [(151552, None), (129280, None), (50001, 50004), (16385, 16388)])
def test_split_rows_match_the_reference(gpu_sampler_factory, ref, batch, n_vocab, ld):
    inp = Inputs(7100 + batch, batch, n_vocab, ld=ld)
    _both(gpu_sampler_factory, ref, TOPK, inp)


@pytest.mark.parametrize("params", [TOPK_PEN, TOPK_ONLY], ids=["penalised", "top_k_alone"])
def test_split_rows_with_history_mask_and_bias(gpu_sampler_factory, ref, params):
    inp = Inputs(7200, 4, 151552, n_history=4096, with_mask=True, n_bias=64, mask_fraction=0.3)
    _both(gpu_sampler_factory, ref, params, inp)
    inp = Inputs(7201, 8, 129280, n_history=512)
    _both(gpu_sampler_factory, ref, params, inp)


def test_a_shard_that_holds_the_whole_top_k_is_run_again(gpu_sampler_factory, ref):
    """All of a row's high logits inside one tile: that shard's list ends inside the deciding set, so the merge
    cannot know what lies below it. The row comes back with the plain path's result and without the truncation flag;
    the other rows of the call are untouched by the follow-up."""
    n_vocab = 151552
    inp = Inputs(7300, 4, n_vocab)
    rng = np.random.default_rng(7300)
    cols = 8192 + rng.choice(4096, size=120, replace=False)
    inp.logits[2, cols] = rng.uniform(9.0, 11.0, size=120).astype(np.float32)
    res = _both(gpu_sampler_factory, ref, TOPK, inp)
    assert not (res.flags.cpu().numpy() & 0x20).any()


def test_split_path_repeats_itself(gpu_sampler_factory):
    """Two calls in a row on the same handle and inputs give identical outputs (the records and the flags buffer of
    the handle are rewritten, nothing is carried over)."""
    import torch
    inp = Inputs(7400, 2, 151552, n_history=1024)
    s = gpu_sampler_factory(151552, 8, 64)
    g = inp.to_gpu()
    r1 = s.sample(g["logits"], TOPK_PEN, g["u"], **g["kw"])
    torch.cuda.synchronize()
    t1, q1 = r1.token.cpu().numpy().copy(), r1.cand_q.cpu().numpy().copy()
    r2 = s.sample(g["logits"], TOPK_PEN, g["u"], **g["kw"])
    torch.cuda.synchronize()
    assert np.array_equal(t1, r2.token.cpu().numpy())
    assert np.array_equal(q1.view(np.uint32), r2.cand_q.cpu().numpy().view(np.uint32))
