"""Times the sampler on every benchmark configuration on one GPU and prints one line per configuration.

    python -m mako_b200.measure [--steps 200]

Configurations (synthetic, seeded; see mako_b200/csrc/synth.cpp):
  0  single-row sampling, V=151552, T 0.7 / top_k 40 / top_p 0.95, fresh logits every step (1000-row pool)
  1  256 x 129280, 4096-id histories, penalties, T 0.8 / top_p 0.9 / min_p 0.05
  2  128 x 151552, 2 % allowed-token mask + 64 bias pairs, T 1 / top_p 1 draw, and the greedy variant
  3  320 positions x 129280, target + drafter logits, p/q rejection sampling, T 0.6 / top_p 0.95
  4  1024 x 151552 as config 1 without min_p: one sample call (row-sharded, N=1) and the vocab-parallel path with
     8 column shards emulated on one GPU (8 local launches + merge; no all-gather on one GPU)
Time is CUDA-event time of the launches alone with inputs resident in HBM, at least four distinct input sets
(larger than L2 in total) cycled; bytes are the algorithmic bytes of the configuration.
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

from . import synth
from ._lib import lib
from .sampler import BatchSampler, SamplingParams, pack_bias

SEED = 777


def _time(fn, steps, warmup=5):
    for k in range(warmup):
        fn(k)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for k in range(steps):
        fn(k)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps * 1e3  # us per step


def _sets(n_sets, b, v, h=0, mask=False, nb=0):
    out = []
    for k in range(n_sets):
        lg, sp = synth.logits(SEED, b, v, step=k)
        d = dict(logits=torch.from_numpy(lg).cuda(), u=torch.from_numpy(synth.uniforms(SEED, b, step=k)).cuda(), kw={})
        if h:
            d["kw"]["history"] = torch.from_numpy(synth.history_zipf(SEED, b, v, h, step=k)).cuda()
        if mask:
            d["kw"]["mask"] = torch.from_numpy(synth.mask(SEED, b, v, spike_ids=sp, step=k).view(np.int32)).cuda()
        if nb:
            d["kw"]["bias"] = torch.from_numpy(pack_bias(*synth.bias(SEED, b, v, nb, step=k))).cuda()
        out.append(d)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    args = ap.parse_args()
    res = []

    def report(name, us, rows, nbytes):
        res.append(dict(config=name, us_per_step=round(us, 2), rows_per_s=round(rows / us * 1e6),
                        effective_gbs=round(nbytes / us / 1e3, 1)))
        print(json.dumps(res[-1]), flush=True)

    # 0: one row per step out of a pool of fresh rows
    v, pool = 151552, 1000
    lg, _ = synth.logits(SEED, pool, v)
    d_pool = torch.from_numpy(lg).cuda()
    d_u = torch.from_numpy(synth.uniforms(SEED, pool)).cuda()
    s = BatchSampler(v, 1)
    p = SamplingParams(temperature=0.7, top_k=40, top_p=0.95)
    us = _time(lambda k: s.sample(d_pool[k % pool:k % pool + 1], p, d_u[k % pool:k % pool + 1]), args.steps)
    report("0 single row, top_k 40 / top_p 0.95", us, 1, 4 * v + 12)
    del d_pool, s

    # 1
    v, b, h = 129280, 256, 4096
    sets = _sets(4, b, v, h)
    s = BatchSampler(v, b)
    p = SamplingParams(temperature=0.8, top_p=0.9, min_p=0.05, repetition_penalty=1.1, presence_penalty=0.5,
                       frequency_penalty=0.3)
    us = _time(lambda k: s.sample(sets[k % 4]["logits"], p, sets[k % 4]["u"], **sets[k % 4]["kw"]), args.steps)
    report("1 256 x 129280 penalised", us, b, b * lib.mk_row_bytes(v, h, 0, 0, 1))
    del sets, s

    # 2
    v, b, nb = 151552, 128, 64
    sets = _sets(8, b, v, 0, True, nb)
    s = BatchSampler(v, b)
    for name, p in (("2 128 x 151552 masked + biased draw", SamplingParams(temperature=1.0)),
                    ("2 same, greedy", SamplingParams(temperature=0.0))):
        us = _time(lambda k: s.sample(sets[k % 8]["logits"], p, sets[k % 8]["u"], **sets[k % 8]["kw"]), args.steps)
        report(name, us, b, b * lib.mk_row_bytes(v, 0, 1, nb, 1))
    del sets, s

    # 3
    v, b = 129280, 320
    sets = _sets(2, b, v)
    for k, d in enumerate(sets):
        d["drafter"] = torch.from_numpy(synth.add_noise(SEED, d["logits"].cpu().numpy(), v, step=k)).cuda()
        d["u2"] = torch.from_numpy(synth.uniforms(SEED, b, purpose=1, step=k)).cuda()
        d["u3"] = torch.from_numpy(synth.uniforms(SEED, b, purpose=2, step=k)).cuda()
    s = BatchSampler(v, b)
    p = SamplingParams(temperature=0.6, top_p=0.95)
    us = _time(lambda k: s.verify_pq(sets[k % 2]["logits"], sets[k % 2]["drafter"], p, sets[k % 2]["u"],
                                     sets[k % 2]["u2"], sets[k % 2]["u3"]), args.steps)
    report("3 320 positions p/q verification", us, b, b * (2 * 4 * v + 12 + 12))
    flagged = int(((s.flags[:b].cpu().numpy() & 0x50) != 0).sum())
    print(json.dumps(dict(config="3 rows overflowed", rows=flagged)), flush=True)
    del sets, s

    # reasoning-budget logit test over the same 256 x 129280 rows (one streaming pass, 4 bytes per column)
    v, b = 129280, 256
    sets = _sets(4, b, v)
    s = BatchSampler(v, b)
    tok = torch.full((b,), 1234, dtype=torch.int32, device="cuda")
    us = _time(lambda k: s.rank_force(sets[k % 4]["logits"], tok), args.steps)
    report("rank test (is the token among the 3 largest), 256 x 129280", us, b, b * (4 * v + 12))
    del sets, s

    # drafter pick: logits + head . embed[prev] -> argmax, confidence; head 129280 x 256 fp32 read once per step
    v, rank, dim = 129280, 256, 4096
    g = torch.Generator(device="cuda").manual_seed(SEED)
    head = torch.randn((v, rank), generator=g, device="cuda") * 0.05
    embed = torch.randn((v, rank), generator=g, device="cuda")
    w = torch.randn(dim + rank, generator=g, device="cuda") * 0.05
    s = BatchSampler(v, 8)
    for n_seq in (1, 8):
        lg = torch.randn((n_seq, v), generator=g, device="cuda") * 2
        x = torch.randn((n_seq, dim), generator=g, device="cuda")
        prev = torch.arange(n_seq, dtype=torch.int32, device="cuda") * 1000 + 5
        us = _time(lambda k: s.draft_pick(lg, head, embed, x, w, prev), args.steps)
        print(json.dumps(dict(config=f"drafter pick, {n_seq} sequence(s), head 129280 x 256", us_per_step=round(us, 2),
                              effective_gbs=round((4 * v * rank + n_seq * 4 * v) / us / 1e3, 1))), flush=True)
    del head, embed, s

    # 4
    v, b, h, n_sh, k_sh = 151552, 1024, 4096, 8, 64
    sets = _sets(2, b, v, h)
    s = BatchSampler(v, b)
    p = SamplingParams(temperature=0.8, top_p=0.9, repetition_penalty=1.1, presence_penalty=0.5, frequency_penalty=0.3)
    us = _time(lambda k: s.sample(sets[k % 2]["logits"], p, sets[k % 2]["u"], **sets[k % 2]["kw"]), max(args.steps // 4, 20))
    report("4 1024 x 151552 row-sharded, N=1 (first launch + second pass)", us, b, b * lib.mk_row_bytes(v, h, 0, 0, 1))
    fl = s.flags[:b].cpu().numpy()
    nc = s.n_cand[:b].cpu().numpy()
    print(json.dumps(dict(config="4 row flags", overflow=int(((fl & 0x10) != 0).sum()),
                          guard_band=int(((fl & 0x2) != 0).sum()), near_boundary=int((fl & 1).sum()),
                          nucleus_median=int(np.median(nc)), nucleus_max=int(nc.max()))), flush=True)
    vs = v // n_sh
    rb = lib.mk_vp_record_bytes(k_sh)
    gathered = torch.zeros((n_sh, b, rb), dtype=torch.uint8, device="cuda")
    shards = [[d["logits"][:, g * vs:(g + 1) * vs].contiguous() for g in range(n_sh)] for d in sets]

    def vp(k):
        d = sets[k % 2]
        for g in range(n_sh):
            s.vp_local(shards[k % 2][g], p, k_sh, gathered[g], id_offset=g * vs, history=d["kw"]["history"])
        s.vp_merge(gathered, n_sh, b, k_sh, v, p, d["u"])
    us = _time(vp, max(args.steps // 4, 20))
    report("4 vocab-parallel, 8 shards on one GPU (8 local + merge)", us, b, b * (4 * v + 8 * 4 * h + 12))


if __name__ == "__main__":
    main()
