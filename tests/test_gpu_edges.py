"""GPU edge cases the reference's semantics define: non-finite rows, ties, all-masked rows, per-row parameters,
long histories, unaligned rows, the host-buffer entry point."""
import numpy as np
import pytest

from helpers import Inputs, compare_sample, oracle_sample_rows
from mako_b200 import synth
from mako_b200.sampler import SamplingParams, pack_params

pytestmark = pytest.mark.gpu


def gpu_rows(factory, logits, params, u, cap=32, **kw):
    import torch
    s = factory(logits.shape[1], logits.shape[0], cap)
    tkw = {}
    if "history" in kw:
        tkw["history"] = torch.from_numpy(kw["history"]).cuda()
    if "mask" in kw:
        tkw["mask"] = torch.from_numpy(kw["mask"].view(np.int32)).cuda()
    res = s.sample(torch.from_numpy(logits).cuda(), params, torch.from_numpy(u).cuda(), **tkw)
    torch.cuda.synchronize()
    return res


def test_nonfinite_rows(gpu_sampler_factory, ref):
    v = 5000
    rows = np.zeros((8, v), dtype=np.float32)
    rng = np.random.default_rng(3)
    rows[:] = rng.normal(0, 2, size=rows.shape).astype(np.float32)
    rows[0, :] = -np.inf                      # nothing finite: token 0
    rows[1, 100] = np.inf                     # an infinite maximum: first +inf
    rows[1, 4000] = np.inf
    rows[2, 0] = np.nan                       # NaN in front: max_element keeps it -> token 0
    rows[3, 17] = np.nan                      # NaN elsewhere is never a candidate
    rows[4, :] = 1.5                          # all equal: every token a candidate
    rows[5, 7] = rows[5, 4321] = 30.0         # tied maxima -> lower id for greedy
    rows[6, :] = -np.inf
    rows[6, 4999] = -3.0                      # single finite token, last column
    rows[7, 1:] = -1e30
    u = synth.uniforms(1, 8)
    for params in [SamplingParams(temperature=1.0), SamplingParams(temperature=0.0),
                   SamplingParams(temperature=0.5, top_k=3), SamplingParams(temperature=1e-40),
                   SamplingParams(temperature=1.0, repetition_penalty=0.0)]:
        hist = np.tile(np.array([[7, 4321, 0, 17]], dtype=np.int32), (8, 1))
        res = gpu_rows(gpu_sampler_factory, rows, params, u, cap=5000, history=hist)
        want = [ref.sample(params, rows[b], u[b], cap=5000, history=hist[b]) for b in range(8)]
        compare_sample(res, want, cap=5000)


def test_weight_ties_break_toward_lower_id(gpu_sampler_factory, ref):
    """Distinct logits that round to the same weight q tie; top_k keeps the lower ids (sampler.cpp:39-43). With the
    tied logits well inside a bin of the top_k histogram (3.2) nothing below the collected bound can tie with them:
    every row must be decided, unflagged. With the tied logits exactly on a bin edge (3.0) a value just below the
    bound would round to the same weight, so the kernel may report the row instead — but never cut it silently."""
    v = 9000
    compared = 0
    for base in (np.float32(3.2), np.float32(3.0)):
        rows = np.full((2, v), -20.0, dtype=np.float32)
        ups = [base, np.nextafter(base, np.float32(4)), np.nextafter(np.nextafter(base, np.float32(4)), np.float32(4))]
        for j, i in enumerate([8000, 6000, 4000, 2000, 100]):
            rows[0, i] = ups[j % 3]
            rows[1, i] = base
        rows[:, 50] = 10.0
        u = synth.uniforms(2, 2)
        for k in (2, 3, 4):
            p = SamplingParams(temperature=2.0, top_k=k)
            res = gpu_rows(gpu_sampler_factory, rows, p, u, cap=16)
            want = [ref.sample(p, rows[b], u[b], cap=16) for b in range(2)]
            # the case is what it claims to be: in row 1 the k-th weight is shared by candidates the cut leaves out
            assert k == 2 or len(set(want[1]["cand_q"].tolist())) < k
            ids = res.cand_ids.cpu().numpy()
            flags = res.flags.cpu().numpy()
            for b in range(2):
                if flags[b] & 0x2:
                    assert base == np.float32(3.0), "a tie inside a histogram bin must be decided, not reported"
                    continue
                assert sorted(ids[b, :k].tolist()) == sorted(want[b]["cand_ids"].tolist())
                compared += 1
    assert compared >= 6, "the tie cases were all skipped"


def test_all_masked_row_reports_flag(gpu_sampler_factory, ref):
    inp = Inputs(91, 4, 3000, with_mask=True, mask_fraction=0.1)
    inp.mask[1, :] = 0
    res = gpu_rows(gpu_sampler_factory, inp.logits, SamplingParams(temperature=1.0), inp.u, cap=512, mask=inp.mask)
    want = [ref.sample(SamplingParams(temperature=1.0), inp.logits[b], inp.u[b], cap=512, mask=inp.mask[b])
            for b in range(4)]
    compare_sample(res, want, cap=512)
    assert res.flags.cpu().numpy()[1] & 0x8 and res.token.cpu().numpy()[1] == 0


def test_per_row_parameters(gpu_sampler_factory, ref):
    import torch
    v, b = 33000, 6
    inp = Inputs(101, b, v, n_history=200)
    ps = [SamplingParams(temperature=0.0), SamplingParams(temperature=0.7, top_k=40, top_p=0.95),
          SamplingParams(temperature=1.0, min_p=0.02), SamplingParams(temperature=0.8, top_p=0.9),
          SamplingParams(temperature=1.2, top_k=5, repetition_penalty=1.5),
          SamplingParams(temperature=0.9, presence_penalty=1.0, frequency_penalty=0.5, min_p=0.01)]
    s = gpu_sampler_factory(v, b, 256)
    g = inp.to_gpu()
    res = s.sample(g["logits"], torch.from_numpy(pack_params(ps)).cuda(), g["u"], **g["kw"])
    torch.cuda.synchronize()
    want = [ref.sample(ps[i], inp.logits[i], inp.u[i], cap=256, **inp.row_kwargs(i)) for i in range(b)]
    compare_sample(res, want, cap=256)


def test_long_history_and_heavy_repeats(gpu_sampler_factory, ref):
    """More history entries than the shared-memory bucket holds, and one id repeated thousands of times."""
    v, b = 20000, 3
    inp = Inputs(111, b, v)
    h = synth.history_zipf(111, b, v, 6000, s=1.3)
    h[1, :5000] = 77
    p = SamplingParams(temperature=1.0, min_p=0.001, repetition_penalty=1.1, presence_penalty=0.1,
                       frequency_penalty=0.001)
    res = gpu_rows(gpu_sampler_factory, inp.logits, p, inp.u, cap=1024, history=h)
    want = [ref.sample(p, inp.logits[i], inp.u[i], cap=1024, history=h[i]) for i in range(b)]
    compare_sample(res, want, cap=1024)


def test_unaligned_rows_take_the_plain_load_path(gpu_sampler_factory, ref):
    import torch
    v, b = 10001, 5
    inp = Inputs(121, b, v, ld=v + 2)            # ld % 4 != 0: rows are not 16-byte aligned
    s = gpu_sampler_factory(v, b, 64)
    t = torch.from_numpy(inp.logits).cuda()
    p = SamplingParams(temperature=0.8, top_k=20, top_p=0.9)
    res = s.sample(t[:, :v], p, torch.from_numpy(inp.u).cuda())
    torch.cuda.synchronize()
    compare_sample(res, oracle_sample_rows(ref, p, inp, cap=64), cap=64)


def test_host_buffer_entry_point(gpu_sampler_factory, ref):
    v, b = 129280, 6
    inp = Inputs(131, b, v, n_history=1000)
    p = SamplingParams(temperature=0.8, top_p=0.9, min_p=0.05, repetition_penalty=1.1, presence_penalty=0.5,
                       frequency_penalty=0.3)
    s = gpu_sampler_factory(v, b, 0)
    tok, prob, flags = s.sample_host(inp.logits, p, inp.u, history=inp.history)
    want = oracle_sample_rows(ref, p, inp)
    assert tok.tolist() == [w["token"] for w in want]
    assert np.allclose(prob, [w["prob"] for w in want], rtol=1e-5)


@pytest.mark.parametrize("params", [
    SamplingParams(temperature=1.0, top_p=0.9),                         # top_p alone: the total covers every column
    SamplingParams(temperature=1.3, top_p=0.95, min_p=1e-6),            # tens of thousands pass min_p
    SamplingParams(temperature=1.0, top_k=30000, top_p=0.8),            # a very large top_k, then top_p
    SamplingParams(temperature=1.0, top_k=20000),                       # top_k alone, longer than the on-chip sort
], ids=["topp", "minp_topp", "topk_topp", "topk"])
def test_flat_rows_keep_long_sorted_lists(gpu_sampler_factory, ref, params):
    """Near-flat rows keep more candidates than the on-chip sort holds; the list is sorted in device memory and
    must still be the reference's, element for element (sampler.cpp:39-61), for the draw and for verify."""
    import torch
    v, b, cap = 60013, 6, 60016
    rng = np.random.default_rng(17)
    rows = rng.normal(0, 0.4, size=(b, v)).astype(np.float32)
    rows[1] = np.round(rows[1] * 8) / 8          # many exact ties in weight: order by id inside a tie
    rows[2, 1234] = 9.0                          # one spike over a flat floor
    rows[3] = 0.25                               # all equal
    u = synth.uniforms(23, b)
    u2 = synth.uniforms(23, b, purpose=1)
    res = gpu_rows(gpu_sampler_factory, rows, params, u, cap=cap)
    want = [ref.sample(params, rows[i], u[i], cap=cap) for i in range(b)]
    assert max(w["n_cand"] for w in want) > 8192
    compare_sample(res, want, cap=cap)
    draft = np.array([w["cand_ids"][min(i, w["n_cand"] - 1)] for i, w in enumerate(want)], dtype=np.int32)
    s = gpu_sampler_factory(v, b, cap)
    vr = s.verify(torch.from_numpy(rows).cuda(), params, torch.from_numpy(draft).cuda(), torch.from_numpy(u).cuda(),
                  torch.from_numpy(u2).cuda())
    torch.cuda.synchronize()
    tok, acc = vr.token.cpu().numpy(), vr.accepted.cpu().numpy()
    for i in range(b):
        assert (tok[i], bool(acc[i])) == ref.verify(params, rows[i], int(draft[i]), u[i], u2[i]), f"row {i}"


@pytest.mark.parametrize("params", [
    SamplingParams(temperature=1.0, top_p=0.4),
    SamplingParams(temperature=1.0, top_k=10000),
    SamplingParams(temperature=1.0, top_k=11000, top_p=0.999),
], ids=["topp", "topk", "topk_topp"])
def test_lists_a_little_longer_than_the_on_chip_sort(gpu_sampler_factory, ref, params):
    """A little over 8192 candidates: the list is merge-sorted through the row's scratch and still fits shared memory
    for the sequential chains, which read it from there (longer lists stay in device memory): flat rows, one of them
    with many exact ties in weight, element for element against the reference."""
    v, b, cap = 40000, 4, 12000
    rng = np.random.default_rng(19)
    rows = rng.normal(0, 0.4, size=(b, v)).astype(np.float32)
    rows[1] = np.round(rows[1] * 16) / 16        # exact ties in weight: order by id inside a tie
    rows[2, 777] = 3.0
    u = synth.uniforms(29, b)
    res = gpu_rows(gpu_sampler_factory, rows, params, u, cap=cap)
    want = [ref.sample(params, rows[i], u[i], cap=cap) for i in range(b)]
    n_c = [w["n_cand"] for w in want]
    assert max(n_c) > 8192 and min(n_c) < 11500, n_c
    compare_sample(res, want, cap=cap)


def test_second_pass_only_for_rows_that_ask(gpu_sampler_factory, ref):
    """top_p alone: the first launch keeps the 24 largest elements per row; rows whose nucleus is longer stream a
    second time. Flat and peaked rows share a batch, with histories and a mask, and the same handle is then used for
    a batch in which no row asks for the second pass: marks left by one call must not leak into the next."""
    v, b, cap = 50021, 8, 4096
    inp = Inputs(171, b, v, n_history=300, with_mask=True, mask_fraction=0.6)
    rng = np.random.default_rng(5)
    for i in (1, 4, 6):                          # flat rows: nuclei of thousands
        inp.logits[i, :v] = rng.normal(0, 0.5, size=v).astype(np.float32)
    p = SamplingParams(temperature=0.9, top_p=0.92, repetition_penalty=1.2, presence_penalty=0.2)
    g = inp.to_gpu()
    s = gpu_sampler_factory(v, b, cap)
    for _ in range(2):
        res = s.sample(g["logits"], p, g["u"], **g["kw"])
        want = oracle_sample_rows(ref, p, inp, cap=cap)
        compare_sample(res, want, cap=cap)
    n = [w["n_cand"] for w in want]
    assert max(n) > 256 and min(n) <= 256        # both kinds of row are present
    inp2 = Inputs(172, b, v, n_history=300)
    g2 = inp2.to_gpu()
    res = s.sample(g2["logits"], p, g2["u"], **g2["kw"])
    compare_sample(res, oracle_sample_rows(ref, p, inp2, cap=cap), cap=cap)


def test_overlap_modes_give_the_same_tokens(gpu_sampler_factory, ref):
    """Back-to-back launches behind one another with programmatic dependent launch, with and without the history
    tables built ahead of the wait, replayed from a CUDA graph as well: the tokens are those of plain stream order
    and of the CPU reference. The same handle (and so the same scratch) serves consecutive launches."""
    import torch
    from mako_b200 import BatchSampler
    v, b, h = 40003, 24, 700
    p = SamplingParams(temperature=0.8, top_p=0.9, min_p=0.05, repetition_penalty=1.1, presence_penalty=0.5,
                       frequency_penalty=0.3)
    sets = [Inputs(300 + k, b, v, n_history=h) for k in range(3)]
    gs = [i.to_gpu() for i in sets]
    want = [[ref.sample(p, i.logits[r], i.u[r], history=i.history[r])["token"] for r in range(b)] for i in sets]
    s = BatchSampler(v, b, 0)
    outs = [torch.empty(b, dtype=torch.int32, device="cuda") for _ in sets]
    for mode in (0, 1, 2):
        s.set_overlap(mode)
        for k, g in enumerate(gs):                      # three launches in a row on the current stream
            outs[k].copy_(s.sample(g["logits"], p, g["u"], **g["kw"]).token)
        torch.cuda.synchronize()
        for k in range(3):
            assert outs[k].cpu().tolist() == want[k], f"overlap mode {mode}, launch {k}"
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for k, g in enumerate(gs):
                outs[k].copy_(s.sample(g["logits"], p, g["u"], **g["kw"]).token)
    torch.cuda.current_stream().wait_stream(side)
    for o in outs:
        o.zero_()
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    for k in range(3):
        assert outs[k].cpu().tolist() == want[k], f"graph replay, launch {k}"
    s.set_overlap(0)


@pytest.mark.parametrize("with_history", [True, False], ids=["fix-up warps wait", "readers wait"])
def test_a_wait_that_runs_out_ends_the_row_in_good_order(ref, with_history):
    """Every wait in the kernel is bounded. With the test hook that never requests one tile's copy, the waits for
    that tile run out after a few milliseconds: each row returns token -1 with MK_FLAG_TIMEOUT, nothing traps or
    hangs, and the same handle samples correctly right afterwards."""
    import torch
    from mako_b200 import BatchSampler, lib
    v, b = 40003, 6
    inp = Inputs(411, b, v, n_history=600 if with_history else 0)
    p = SamplingParams(temperature=0.8, top_p=0.9, min_p=0.05, repetition_penalty=1.1, presence_penalty=0.5,
                       frequency_penalty=0.3)
    g = inp.to_gpu()
    s = BatchSampler(v, b, 0)
    assert lib.mk_debug_withhold_tile(s._h, 7, 100) == 0          # tile 7 of 10 never arrives; 100 probes of <= 20 us
    res = s.sample(g["logits"], p, g["u"], **g["kw"])
    torch.cuda.synchronize()
    assert res.token.cpu().tolist() == [-1] * b
    assert all(f == 0x40 for f in res.flags.cpu().tolist())
    assert lib.mk_debug_withhold_tile(s._h, -1, 0) == 0
    res = s.sample(g["logits"], p, g["u"], **g["kw"])
    torch.cuda.synchronize()
    want = [ref.sample(p, inp.logits[r], inp.u[r], **inp.row_kwargs(r))["token"] for r in range(b)]
    assert res.token.cpu().tolist() == want


def test_top_k_alone_keeps_the_reference_candidate_set(gpu_sampler_factory, ref):
    """top_k without top_p is the one case where the draw ORDER is not the reference's (it walks whatever order
    std::nth_element left, sampler.cpp:41, 64-73; here and in the checker the list is sorted). What must still be
    identical is the candidate set with its weights: ids and weights are compared as sets, order ignored."""
    v, b = 50257, 6
    inp = Inputs(515, b, v, n_history=300)
    for p in (SamplingParams(temperature=1.0, top_k=50), SamplingParams(temperature=0.7, top_k=5, min_p=0.001,
                                                                       repetition_penalty=1.2)):
        res = gpu_rows(gpu_sampler_factory, inp.logits, p, inp.u, cap=64, history=inp.history)
        ids, qs, n = res.cand_ids.cpu().numpy(), res.cand_q.cpu().numpy(), res.n_cand.cpu().numpy()
        flags = res.flags.cpu().numpy()
        for r in range(b):
            w = ref.sample(p, inp.logits[r], inp.u[r], cap=64, history=inp.history[r])
            assert not (flags[r] & 0x52) and n[r] == w["n_cand"] == p.top_k
            got = sorted(zip(ids[r, :n[r]].tolist(), qs[r, :n[r]].view(np.uint32).tolist()))
            want = sorted(zip(w["cand_ids"].tolist(), w["cand_q"].view(np.uint32).tolist()))
            assert got == want, f"row {r}"


@pytest.mark.parametrize("params", [
    SamplingParams(temperature=1.0, top_k=50),
    SamplingParams(temperature=0.9, top_k=45, top_p=0.98),
    SamplingParams(temperature=1.2, top_k=33, min_p=0.001, repetition_penalty=1.2, presence_penalty=0.3,
                   frequency_penalty=0.1),
    SamplingParams(temperature=1.5, min_p=0.3),
], ids=["top_k50", "top_k45_top_p", "top_k33_penalised", "min_p_about_50"])
def test_rows_with_33_to_64_candidates(gpu_sampler_factory, ref, params):
    """Between 33 and 64 candidates a row is finished by one warp with two candidates a lane: token, probability,
    candidate list and weights against the reference for sampling, token and acceptance for verification (drafts that
    are the likeliest token, a token in the second half of the list, and a token outside it)."""
    import torch
    from helpers import Inputs, compare_sample, oracle_sample_rows
    v, b = 129280, 48
    # no spikes: the largest logits of a row lie close together, so min_p 0.3 at T 1.5 keeps some tens of them
    inp = Inputs(8100, b, v, n_history=256, n_spikes=0)
    g = inp.to_gpu()
    s = gpu_sampler_factory(v, b, 64)
    s.set_split(False)
    res = s.sample(g["logits"], params, g["u"], **g["kw"])
    torch.cuda.synchronize()
    want = oracle_sample_rows(ref, params, inp, cap=64)
    compare_sample(res, want, cap=64)
    n_c = np.array([w["n_cand"] for w in want])
    if params.top_p >= 1.0: # what is left after top_p says nothing about how many candidates went in
        assert ((n_c > 32) & (n_c <= 64)).sum() >= 4, "the inputs must land in the two-per-lane finish"
    draft = np.zeros(b, dtype=np.int32)
    for i in range(b):
        ids = want[i]["cand_ids"]
        draft[i] = ids[0] if i % 3 == 0 else (ids[min(len(ids) - 1, 40)] if i % 3 == 1 else (i * 977) % v)
    res = s.verify(g["logits"], params, torch.from_numpy(draft).cuda(), g["u"], g["u2"], **g["kw"])
    torch.cuda.synchronize()
    tok, acc = res.token.cpu().numpy(), res.accepted.cpu().numpy()
    for i in range(b):
        wt, wa = ref.verify(params, inp.logits[i], int(draft[i]), inp.u[i], inp.u2[i], **inp.row_kwargs(i))
        assert (tok[i], bool(acc[i])) == (wt, wa), f"row {i}"
    s.set_split(True)
