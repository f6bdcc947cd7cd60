"""The decode loop around the sampler kept on the device (src/gen/session.cpp:416-444): sample, commit the token to
the row's history and to the next step's input, repeat — no host round trip between steps. The token streams must
equal the reference sampler's, fed the same logits, uniforms and forced tokens step by step."""
import numpy as np
import pytest

from mako_b200 import synth
from mako_b200.sampler import SamplingParams

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("params", [
    SamplingParams(temperature=0.8, top_p=0.9, min_p=0.05, repetition_penalty=1.1, presence_penalty=0.5,
                   frequency_penalty=0.3),
    SamplingParams(temperature=0.7, top_k=40, top_p=0.95, repetition_penalty=1.3),
    SamplingParams(temperature=0.0),
], ids=["penalised", "topk", "greedy"])
def test_device_resident_decode_loop(gpu_sampler_factory, ref, params):
    import torch
    v, b, steps, cap = 20011, 5, 24, 32
    s = gpu_sampler_factory(v, b, 0)
    logits = [synth.logits(901, b, v, step=k, n_spikes=3)[0] for k in range(steps)]
    u = [synth.uniforms(901, b, step=k) for k in range(steps)]
    forced = np.full((steps, b), -1, dtype=np.int32)
    forced[3, 1] = 17          # a forced token bypasses the sampler but is accepted like any other
    forced[4, 1] = 17
    forced[10, :] = 4242
    d_hist = torch.zeros((b, cap), dtype=torch.int32, device="cuda")
    d_len = torch.zeros(b, dtype=torch.int32, device="cuda")
    d_next = torch.full((b,), -1, dtype=torch.int32, device="cuda")
    d_logits = [torch.from_numpy(x).cuda() for x in logits]
    d_u = [torch.from_numpy(x).cuda() for x in u]
    d_forced = torch.from_numpy(forced).cuda()
    got = []
    for k in range(steps):    # nothing in this loop reads a result back
        res = s.sample(d_logits[k], params, d_u[k], history=d_hist, history_len=d_len)
        got.append(s.decode_commit(res.token, d_hist, d_len, forced=d_forced[k], next_input=d_next))
    torch.cuda.synchronize()
    got = torch.stack(got).cpu().numpy()
    hist = [[] for _ in range(b)]
    for k in range(steps):
        for i in range(b):
            if forced[k, i] >= 0:
                t = int(forced[k, i])
            else:
                h = np.array(hist[i], dtype=np.int32) if hist[i] else None
                t = ref.sample(params, logits[k][i], u[k][i], history=h)["token"]
            assert got[k, i] == t, f"step {k} row {i}: {got[k, i]} != {t}"
            hist[i].append(t)
    assert d_len.cpu().tolist() == [steps] * b
    assert d_hist.cpu().numpy()[:, :steps].tolist() == [h for h in hist]
    assert d_next.cpu().tolist() == [h[-1] for h in hist]


def test_decode_commit_full_history_and_failed_rows(gpu_sampler_factory):
    import torch
    s = gpu_sampler_factory(1024, 4, 0)
    hist = torch.zeros((4, 3), dtype=torch.int32, device="cuda")
    hlen = torch.tensor([0, 3, 2, 1], dtype=torch.int32, device="cuda")
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    sampled = torch.tensor([5, 6, -1, 8], dtype=torch.int32, device="cuda")
    out = s.decode_commit(sampled, hist, hlen, flags=flags)
    torch.cuda.synchronize()
    assert out.cpu().tolist() == [5, 6, -1, 8]
    assert hlen.cpu().tolist() == [1, 3, 2, 2]          # full row and failed row keep their length
    assert flags.cpu().tolist() == [0, 0x100, 0, 0]
    assert hist.cpu().numpy()[0, 0] == 5 and hist.cpu().numpy()[3, 1] == 8


def rank_force_cpu(logits, token, k=3):
    """ReasoningBudget::forced's logit test restated (src/server/openai.cpp:596-603): the loop counts logits strictly
    greater than the token's and gives up at k."""
    forced, above = [], []
    for row, t in zip(logits, token):
        if t < 0 or t >= row.shape[0]:
            forced.append(-1)
            above.append(-1)
            continue
        n = int((row > row[t]).sum())
        above.append(n)
        forced.append(int(t) if n < k else -1)
    return forced, above


def test_rank_force_known_answers_of_the_reference(gpu_sampler_factory):
    """tests/server_test.cpp:139-153: all logits 0 and the closing token at 1 closes; three logits above it do not
    close ("fourth is not closed early"); two above do ("third closes early")."""
    import torch
    nv, end = 4099, 4000
    s = gpu_sampler_factory(nv, 4, 0)
    rows = np.zeros((4, nv), dtype=np.float32)
    rows[:, end] = 1.0
    rows[1, :3] = 2.0
    rows[2, :2] = 2.0
    rows[3, 7] = np.nan                      # a NaN is never "greater"
    token = np.array([end, end, end, end], dtype=np.int32)
    forced, above = s.rank_force(torch.from_numpy(rows).cuda(), torch.from_numpy(token).cuda())
    torch.cuda.synchronize()
    assert forced.cpu().tolist() == [end, -1, end, end]
    assert above.cpu().tolist() == [0, 3, 2, 0]


def test_rank_force_random_rows(gpu_sampler_factory):
    import torch
    v, b = 129280, 12
    s = gpu_sampler_factory(v, b, 0)
    lg, spikes = synth.logits(77, b, v + 3, ld=v + 4)      # rows of v + 3 columns, 16-byte aligned
    token = np.array([int(spikes[i, i % 8]) if i % 3 else (i * 9973) % v for i in range(b)], dtype=np.int32)
    token[5], token[6] = -1, v + 3                          # no such token: nothing forced
    d = torch.from_numpy(lg).cuda()
    for view, nv in ((d[:, : v + 3], v + 3), (d[:, 1 : v + 2], v + 1)):   # aligned rows, then misaligned ones
        forced, above = s.rank_force(view, torch.from_numpy(token).cuda(), k=3)
        torch.cuda.synchronize()
        wf, wa = rank_force_cpu(view.cpu().numpy(), token)
        assert forced.cpu().tolist() == wf
        assert above.cpu().tolist() == wa
    # the forced tokens feed the commit step as they are
    hist = torch.zeros((b, 4), dtype=torch.int32, device="cuda")
    hlen = torch.zeros(b, dtype=torch.int32, device="cuda")
    sampled = torch.full((b,), 11, dtype=torch.int32, device="cuda")
    out = s.decode_commit(sampled, hist, hlen, forced=forced)
    assert out.cpu().tolist() == [f if f >= 0 else 11 for f in wf]
