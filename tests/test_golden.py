"""Committed golden vectors (tests/golden/sampler_golden.npz, produced by tests/golden/make_golden.py from the
reference's own sampler.cpp): the CPU restatement must reproduce them without the reference being present, and so
must the GPU kernels through the C ABI."""
import os

import numpy as np
import pytest

from mako_b200.sampler import SamplingParams, pack_bias

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sampler_golden.npz"))
B, V, CAP = int(G["B"]), int(G["V"]), 2048


def params_of(ci):
    a = G[f"params{ci}"]
    return SamplingParams(float(np.float32(a[0])), int(a[1]), float(np.float32(a[2])), float(np.float32(a[3])),
                          float(np.float32(a[4])), float(np.float32(a[5])), float(np.float32(a[6])))


def row_kwargs(b):
    kw = dict(history=G["history"][b])
    if b % 2 == 0:
        kw.update(mask=G["mask"][b], bias_ids=G["bias_ids"][b], bias_vals=G["bias_vals"][b])
    return kw


@pytest.mark.parametrize("ci", range(int(G["n_cases"])))
def test_port_reproduces_reference_golden(port, ci):
    p = params_of(ci)
    for b in range(B):
        r = port.sample(p, G["logits"][b], G["u0"][b], cap=CAP, **row_kwargs(b))
        n = int(G[f"ncand{ci}"][b])
        assert r["token"] == G[f"token{ci}"][b] and r["n_cand"] == n
        assert np.array_equal(r["cand_ids"], G[f"ids{ci}"][b, :n])
        assert np.array_equal(r["cand_q"].view(np.uint32), G[f"q{ci}"][b, :n].view(np.uint32))
        assert port.verify(p, G["logits"][b], int(G[f"draft{ci}"][b]), G["u1"][b], G["u2"][b], **row_kwargs(b)) == \
            (int(G[f"vtoken{ci}"][b]), bool(G[f"vacc{ci}"][b]))
        d, acc, tok = port.verify_pq(p, G["logits"][b], G["drafter"][b], G["u0"][b], G["u1"][b], G["u2"][b],
                                     **row_kwargs(b))
        assert [d, int(acc), tok] == G[f"pq{ci}"][b].tolist()


@pytest.mark.gpu
@pytest.mark.parametrize("ci", range(int(G["n_cases"])))
def test_gpu_reproduces_reference_golden(gpu_sampler_factory, ci):
    import torch
    p = params_of(ci)
    s = gpu_sampler_factory(V, B, CAP)
    for group in (0, 1):                       # even rows carry mask + bias, odd rows do not
        rows = list(range(group, B, 2))
        lg = torch.from_numpy(np.ascontiguousarray(G["logits"][rows])).cuda()
        hist = torch.from_numpy(np.ascontiguousarray(G["history"][rows])).cuda()
        kw = dict(history=hist)
        if group == 0:
            kw["mask"] = torch.from_numpy(np.ascontiguousarray(G["mask"][rows]).view(np.int32)).cuda()
            kw["bias"] = torch.from_numpy(pack_bias(G["bias_ids"][rows], G["bias_vals"][rows])).cuda()
        u = [torch.from_numpy(np.ascontiguousarray(G[f"u{k}"][rows])).cuda() for k in range(3)]
        res = s.sample(lg, p, u[0], **kw)
        torch.cuda.synchronize()
        tok, nc = res.token.cpu().numpy(), res.n_cand.cpu().numpy()
        ids, qs = res.cand_ids.cpu().numpy(), res.cand_q.cpu().numpy()
        for i, b in enumerate(rows):
            n = int(G[f"ncand{ci}"][b])
            assert tok[i] == G[f"token{ci}"][b] and nc[i] == n
            assert np.array_equal(ids[i, :n], G[f"ids{ci}"][b, :n])
            assert np.array_equal(qs[i, :n].view(np.uint32), G[f"q{ci}"][b, :n].view(np.uint32))
        draft = torch.from_numpy(np.ascontiguousarray(G[f"draft{ci}"][rows])).cuda()
        res = s.verify(lg, p, draft, u[1], u[2], **kw)
        torch.cuda.synchronize()
        assert res.token.cpu().numpy().tolist() == G[f"vtoken{ci}"][rows].tolist()
        assert res.accepted.cpu().numpy().tolist() == G[f"vacc{ci}"][rows].tolist()
        lq = torch.from_numpy(np.ascontiguousarray(G["drafter"][rows])).cuda()
        res = s.verify_pq(lg, lq, p, u[0], u[1], u[2], **kw)
        torch.cuda.synchronize()
        got = np.stack([res.draft_token.cpu().numpy(), res.accepted.cpu().numpy(), res.token.cpu().numpy()], axis=1)
        assert got.tolist() == G[f"pq{ci}"][rows].tolist()
