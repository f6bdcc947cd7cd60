"""The allocation-free entry point, mk_sample_rows_static, against the handle-based mk_sampler_sample_batch.

Some users of this library cannot call cudaMalloc where they sample: their process hands out all device memory at
start-up, or they are a plugin inside a runtime whose allocator they must not touch, so they cannot create a sampler
handle (its scratch is allocated). For them the library keeps a fixed scratch array of its own. This test calls that
entry point through the C ABI several times in a row (the array keeps the previous call's contents) and expects the
very same tokens, probabilities, candidate counts and flags as the ordinary entry point, and the tokens of the CPU
reference. One of the cases is top_p alone, where the kernel is launched a second time for the rows that marked
themselves in the scratch array: the mark sits behind the candidate area, whose size differs between the library's
array and a handle's buffer. It is collected last so that a run that stops at the first failure has already run
everything else; it passes alone as well as after the others."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call_static(lib, rows_c, u, out_tensors, cand_cap=0):
    from mako_b200._lib import SampleOutC
    import torch
    o = SampleOutC()
    o.token = out_tensors["token"].data_ptr()
    o.prob = out_tensors["prob"].data_ptr()
    o.flags = out_tensors["flags"].data_ptr()
    o.n_cand = out_tensors["n_cand"].data_ptr()
    rc = lib.mk_sample_rows_static(0, C.byref(rows_c), u.data_ptr(), C.byref(o),
                                   torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.mk_last_error().decode()


def test_static_scratch_entry_point_matches_handle_entry_point(ref):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from mako_b200 import BatchSampler, SamplingParams, lib, synth
    v, b, h = 129280, 8, 4096
    handle = BatchSampler(v, b, 0)
    cases = [
        SamplingParams(temperature=0.8, top_p=0.9, min_p=0.05, repetition_penalty=1.1, presence_penalty=0.5,
                       frequency_penalty=0.3),
        SamplingParams(temperature=0.7, top_k=40, top_p=0.95),
        # top_p alone: rows that the first launch cannot settle are streamed again by a second launch
        SamplingParams(temperature=0.6, top_p=0.95),
        SamplingParams(temperature=0.8, top_p=0.9, repetition_penalty=1.1, presence_penalty=0.5, frequency_penalty=0.3),
    ]
    second_pass_rows = 0
    for call, params in enumerate(cases):          # calls in a row share the library's scratch array
        logits, _ = synth.logits(900 + call, b, v)
        hist = synth.history_zipf(900 + call, b, v, h)
        u = synth.uniforms(900 + call, b)
        d_logits = torch.from_numpy(logits).cuda()
        d_hist = torch.from_numpy(hist).cuda()
        d_u = torch.from_numpy(u).cuda()
        want = handle.sample(d_logits, params, d_u, history=d_hist)
        torch.cuda.synchronize()
        want = {k: getattr(want, k).cpu().numpy().copy() for k in ("token", "prob", "flags", "n_cand")}

        got = {"token": torch.full((b,), -7, dtype=torch.int32, device="cuda"),
               "prob": torch.zeros(b, dtype=torch.float32, device="cuda"),
               "flags": torch.zeros(b, dtype=torch.int32, device="cuda"),
               "n_cand": torch.zeros(b, dtype=torch.int32, device="cuda")}
        rows_c = handle._rows(d_logits, params, d_hist)
        _call_static(lib, rows_c, d_u, got)
        torch.cuda.synchronize()
        for k in want:
            a = got[k].cpu().numpy()
            assert np.array_equal(a.view(np.uint32), want[k].view(np.uint32)), f"call {call}: {k} differs"
        # and against the CPU reference, row by row
        tok, flags, ncand = (got[k].cpu().numpy() for k in ("token", "flags", "n_cand"))
        assert not (flags & 0x50).any()
        for i in range(b):
            w = ref.sample(params, logits[i], u[i], history=hist[i])
            if flags[i] & 0x2:
                continue
            assert tok[i] == w["token"] and ncand[i] == w["n_cand"], f"call {call} row {i}"
        if params.min_p == 0 and params.top_k == 0:
            second_pass_rows += int((ncand > 256).sum())   # a nucleus beyond the first launch's 256 kept elements
    assert second_pass_rows > 0, "no row of the top_p-alone cases took the second launch"


def test_static_entry_point_rejects_sizes_beyond_its_limits():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from mako_b200 import BatchSampler, SamplingParams, lib
    from mako_b200._lib import SampleOutC
    big = BatchSampler(1000, 9, 0)
    logits = torch.zeros((9, 1000), dtype=torch.float32, device="cuda")
    u = torch.zeros(9, dtype=torch.float32, device="cuda")
    tok = torch.zeros(9, dtype=torch.int32, device="cuda")
    o = SampleOutC()
    o.token = tok.data_ptr()
    rows_c = big._rows(logits, SamplingParams())
    rc = lib.mk_sample_rows_static(0, C.byref(rows_c), u.data_ptr(), C.byref(o), None)
    assert rc == 1 and b"static limit" in lib.mk_last_error()
