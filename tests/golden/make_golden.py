"""Generates tests/golden/sampler_golden.npz from the reference's own sampler (oracle/_ref, i.e. the unmodified
src/gen/sampler.cpp of the reference compiled by oracle/Makefile). Run where the reference checkout is present:

    make -C oracle && python tests/golden/make_golden.py

Inputs are small seeded rows (V = 2048) covering the parameter families of the benchmark configurations; outputs
are the reference's tokens, candidate lists (ids and unnormalised weights q, bit patterns), verify() results and the
p/q rejection results of the checker's driver. The fixture travels with the repository; the reference does not."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from mako_b200 import synth  # noqa: E402
from mako_b200.sampler import SamplingParams  # noqa: E402
from oracle.oracle import Oracle  # noqa: E402

V, B, H, NB, CAP = 2048, 6, 96, 8, 2048
CASES = [
    dict(temperature=0.7, top_k=40, top_p=0.95),
    dict(temperature=0.8, top_p=0.9, min_p=0.05, repetition_penalty=1.1, presence_penalty=0.5, frequency_penalty=0.3),
    dict(temperature=1.0),
    dict(temperature=0.6, top_p=0.95),
    dict(temperature=0.0),
    dict(temperature=1.3, top_k=5, repetition_penalty=1.5, presence_penalty=-0.2),
    dict(temperature=1.0, top_k=50),                 # top_k alone, truncating: the list in canonical (sorted) order
    dict(temperature=2.5, top_k=200, min_p=0.018),   # fewer candidates than top_k: nothing reordered, ascending id
]


def main():
    ref = Oracle("reference")
    out = {"V": V, "B": B, "H": H, "NB": NB, "n_cases": len(CASES)}
    logits, spikes = synth.logits(4242, B, V, sigma=2.0, n_spikes=4)
    hist = synth.history_zipf(4242, B, V, H)
    mask = synth.mask(4242, B, V, fraction=0.3, spike_ids=spikes)
    bias_ids, bias_vals = synth.bias(4242, B, V, NB)
    drafter = synth.add_noise(4242, logits, V, sigma=1.0)
    u = [synth.uniforms(4242, B, purpose=k) for k in range(3)]
    out.update(logits=logits, history=hist, mask=mask, bias_ids=bias_ids, bias_vals=bias_vals, drafter=drafter,
               u0=u[0], u1=u[1], u2=u[2])
    for ci, kw in enumerate(CASES):
        p = SamplingParams(**kw)
        out[f"params{ci}"] = np.array([p.temperature, p.top_k, p.top_p, p.min_p, p.presence_penalty,
                                       p.frequency_penalty, p.repetition_penalty], dtype=np.float64)
        tok = np.zeros(B, np.int32); ncand = np.zeros(B, np.int32); prob = np.zeros(B, np.float32)
        ids = np.full((B, CAP), -1, np.int32); qs = np.zeros((B, CAP), np.float32)
        vtok = np.zeros(B, np.int32); vacc = np.zeros(B, np.int32); draft = np.zeros(B, np.int32)
        pq = np.zeros((B, 3), np.int32)
        for b in range(B):
            kwr = dict(history=hist[b])
            if b % 2 == 0:
                kwr.update(mask=mask[b], bias_ids=bias_ids[b], bias_vals=bias_vals[b])
            r = ref.sample(p, logits[b], u[0][b], cap=CAP, **kwr)
            tok[b], ncand[b], prob[b] = r["token"], r["n_cand"], r["prob"]
            ids[b, : r["n_cand"]] = r["cand_ids"]
            qs[b, : r["n_cand"]] = r["cand_q"]
            draft[b] = r["cand_ids"][min(1, r["n_cand"] - 1)]
            vtok[b], vacc[b] = ref.verify(p, logits[b], int(draft[b]), u[1][b], u[2][b], **kwr)
            pq[b] = ref.verify_pq(p, logits[b], drafter[b], u[0][b], u[1][b], u[2][b], **kwr)
        out.update({f"token{ci}": tok, f"ncand{ci}": ncand, f"prob{ci}": prob, f"ids{ci}": ids, f"q{ci}": qs,
                    f"draft{ci}": draft, f"vtoken{ci}": vtok, f"vacc{ci}": vacc, f"pq{ci}": pq})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "sampler_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
