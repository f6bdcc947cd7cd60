"""Benchmark of the token-sampling hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 1]

One step = one pass of the row pipeline over one batch of synthetic rows. The default workload is the batched
penalised configuration: 256 rows x V=129280 fp32 logits (N(0,2^2) + 8 spikes U(8,15)), a 4096-id Zipf(1.1) token
history per row, repetition 1.1 / presence 0.5 / frequency 0.3, temperature 0.8, top_p 0.9, min_p 0.05, one uniform
per row. Prints one JSON line (rank 0):

  value        rows/s over all GPUs with the inputs resident in HBM: a CUDA graph of 256 steps is replayed at least
               50 times (and for at least a quarter of a second), one CUDA-event pair per replay; ms_per_step is the
               median replay / 256, max over ranks, and value = rows / that; p10 / p90 / mean are given beside it
  e2e          the same through the host-buffer entry point: pinned host inputs copied in, results copied out,
               every step, inside the timed region
  roofline     algorithmic bytes of one launch / its median duration, against the measured HBM copy bandwidth
  cpu_baseline the reference's own CPU sampler (oracle/_ref when built, else the CPU restatement) timed on the host
               cores on a bounded sample of the same rows, rank 0 at N=1 only
  config4      the scale-out configuration (1024 rows x V=151552) on the N ranks of this run, in both modes:
               row-sharded (1024/N rows per rank, no collective: strong scaling) and vocab-parallel (V/N columns per
               rank, local step -> NCCL all-gather of the per-row records -> merge), each with its time split and
               its token mismatches against the CPU reference

With N > 1 (launched by torch.distributed.run) every rank samples its own 256 rows of a 256*N-row batch for the
headline: rows are independent, so there is no data-path collective (weak scaling). `--impl reference` times the CPU
reference alone. `--config 0|2|3|4` and `--aux` time the other configurations and the auxiliary kernels on one GPU.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

CONFIGS = {
    0: dict(batch=1, n_vocab=151552, n_history=0, mask=False, n_bias=0, pool=1000,
            params=dict(temperature=0.7, top_k=40, top_p=0.95), name="single-row top_k 40 / top_p 0.95"),
    1: dict(batch=256, n_vocab=129280, n_history=4096, mask=False, n_bias=0,
            params=dict(temperature=0.8, top_p=0.9, min_p=0.05, repetition_penalty=1.1, presence_penalty=0.5,
                        frequency_penalty=0.3), name="batched penalised sampling"),
    2: dict(batch=128, n_vocab=151552, n_history=0, mask=True, n_bias=64,
            params=dict(temperature=1.0, top_p=1.0), name="grammar-masked softmax draw"),
    3: dict(batch=320, n_vocab=129280, n_history=0, mask=False, n_bias=0,
            params=dict(temperature=0.6, top_p=0.95), name="speculative p/q verification, 64 seq x 5 pos"),
    4: dict(batch=1024, n_vocab=151552, n_history=4096, mask=False, n_bias=0,
            params=dict(temperature=0.8, top_p=0.9, repetition_penalty=1.1, presence_penalty=0.5,
                        frequency_penalty=0.3), name="scale-out 1024 x 151552"),
}
N_SETS = 4          # distinct input sets cycled between steps: 4 x 137 MB > the 126 MB L2
PER_GRAPH = 16      # steps captured in one CUDA graph (the other configurations, the scale-out block)
HEADLINE_PER_GRAPH = 256  # the headline: the streams drain where a graph ends, which a running server's do not;
                          # at 16 steps a graph that drain was 5 % of the time, at 256 it is 0.3 %
MIN_REPLAYS = 50
MIN_SECONDS = 0.25
SEED = 20240
VP_K = 64


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def launches_per_step(params, n_vocab: int) -> int:
    """Row-kernel launches one sample call makes: top_p alone (no min_p, no top_k) is followed by the second pass
    that streams again the rows whose nucleus the first launch could not settle (other CTAs return at once)."""
    top_p_alone = (params.temperature > 0 and params.top_p < 1.0 and not min(params.min_p, 1.0) > 0
                   and not 0 < params.top_k < n_vocab)
    return 2 if top_p_alone and n_vocab > 256 else 1


def committed_traffic(workload_key: str):
    """DRAM bytes per launch of the row kernel from the committed ncu capture, if one exists for this workload."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        with open(path) as f:
            return json.load(f).get(workload_key)
    except Exception:
        return None


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.tmp.flush()
        self.tmp.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.tmp.read().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.tmp.name)
        except OSError:
            pass
        if sm:
            out["sm_mhz"] = float(np.median(sm))
            out["sm_max_mhz"] = float(max(mx))
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
        return out


def make_inputs(cfg, rank: int, n_sets: int):
    from mako_b200 import synth
    b, v = cfg.get("pool", cfg["batch"]), cfg["n_vocab"]
    sets = []
    for k in range(n_sets):
        row0 = rank * b
        logits, spikes = synth.logits(SEED, b, v, step=k, row0=row0)
        d = dict(logits=logits, u=synth.uniforms(SEED, b, step=k, row0=row0))
        if cfg["n_history"]:
            d["history"] = synth.history_zipf(SEED, b, v, cfg["n_history"], step=k, row0=row0)
        if cfg["mask"]:
            d["mask"] = synth.mask(SEED, b, v, spike_ids=spikes, step=k, row0=row0)
        if cfg["n_bias"]:
            d["bias_ids"], d["bias_vals"] = synth.bias(SEED, b, v, cfg["n_bias"], step=k, row0=row0)
        sets.append(d)
    return sets


def row_bytes(cfg) -> int:
    v = cfg["n_vocab"]
    return (4 * v + 4 * cfg["n_history"] + (4 * ((v + 31) // 32) if cfg["mask"] else 0) + 8 * cfg["n_bias"] + 4 + 8)


def workload_name(cfg) -> str:
    return (f"{cfg['name']}: batch {cfg['batch']} x V={cfg['n_vocab']} fp32, history {cfg['n_history']}"
            + (", 2% mask" if cfg["mask"] else "") + (f", {cfg['n_bias']} bias" if cfg["n_bias"] else ""))


def workload_config(cfg, world: int) -> dict:
    """The keys both arms print under "config" (same names, same values for the same workload)."""
    return {"workload": workload_name(cfg), "batch_per_gpu": cfg["batch"], "n_vocab": cfg["n_vocab"],
            "n_history": cfg["n_history"], "parallelism": f"row-sharded x{world}, no collective", "seed": SEED}


# ---- the CPU reference alone ---------------------------------------------------------------------------------------
def run_reference(args, cfg, rank, world):
    """The reference's CPU sampler on the host cores; each step is one batch of the workload. Loads the input
    generator and the CPU checker only — none of the product's code."""
    if rank != 0:
        return
    from mako_b200.params import SamplingParams
    from oracle.oracle import Oracle
    params = SamplingParams(**cfg["params"])
    orc = Oracle("best")
    cores = os.cpu_count() or 1
    sets = make_inputs(cfg, 0, min(2, N_SETS))
    b = sets[0]["logits"].shape[0]

    def step(k):
        d = sets[k % len(sets)]
        sec, _ = orc.time_sample_batch(params, d["logits"], d["u"], history=d.get("history"), mask=d.get("mask"),
                                       bias_ids=d.get("bias_ids"), bias_vals=d.get("bias_vals"), n_threads=cores)
        return sec
    for k in range(args.warmup):
        step(k)
    times = [step(k) for k in range(args.steps)]
    total = sum(times)
    value = b * args.steps / total
    line = {
        "impl": "reference", "metric": "sampled rows/s", "value": value, "unit": "rows/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, world),
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": orc.kind,
                         "sample": f"{args.steps} steps of the full {b}-row batch, {cores} host threads, "
                                   "sample() only (sampler construction, history replay and one untimed pass that "
                                   "sizes the samplers' vectors are outside the timed region)"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "effective_gbs": value * row_bytes(cfg) / 1e9,
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- timing helpers ------------------------------------------------------------------------------------------------
class Timer:
    """Replays a callable (a CUDA graph replay, or a host-launched block of steps) with one event pair per replay."""

    def __init__(self, dev, world):
        self.dev, self.world = dev, world

    def barrier(self):
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize(self.dev)
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize(self.dev)

    def run(self, replay, steps_per_replay: int, want_steps: int, min_replays=MIN_REPLAYS, min_seconds=MIN_SECONDS):
        """Returns dict(steps, replays, total_ms, ms_per_step (median), p10, p90, mean) for this rank."""
        import torch
        replay()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        replay()
        e1.record()
        torch.cuda.synchronize(self.dev)
        est_ms = max(e0.elapsed_time(e1), 1e-3)
        n = max(min_replays, math.ceil(want_steps / steps_per_replay), math.ceil(min_seconds * 1e3 / est_ms))
        n = min(n, 20000)
        if self.world > 1:  # every rank replays the same number of times
            import torch.distributed as dist
            t = torch.tensor([n], dtype=torch.int64, device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            n = int(t.item())
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
        self.barrier()
        ev[0].record()
        for i in range(n):
            replay()
            ev[i + 1].record()
        self.barrier()
        per = np.array([ev[i].elapsed_time(ev[i + 1]) for i in range(n)]) / steps_per_replay
        return dict(steps=n * steps_per_replay, replays=n, total_ms=ev[0].elapsed_time(ev[n]),
                    ms_per_step=float(np.median(per)), p10=float(np.percentile(per, 10)),
                    p90=float(np.percentile(per, 90)), mean=float(ev[0].elapsed_time(ev[n]) / (n * steps_per_replay)))

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        import torch
        import torch.distributed as dist
        t = torch.tensor([x], dtype=torch.float64, device=self.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())


def capture(dev, body, n_streams: int = 1, n_steps: int = PER_GRAPH):
    """A CUDA graph of `body(k)` for k in range(n_steps), step k on side stream k % n_streams."""
    import torch
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            if n_streams == 1:
                for k in range(n_steps):
                    body(k)
            else:
                subs = [torch.cuda.Stream(device=dev) for _ in range(n_streams)]
                for sub in subs:
                    sub.wait_stream(side)
                for k in range(n_steps):
                    with torch.cuda.stream(subs[k % n_streams]):
                        body(k)
                for sub in subs:
                    side.wait_stream(sub)
    torch.cuda.current_stream(dev).wait_stream(side)
    return graph


def to_device(host_sets, dev):
    import torch
    from mako_b200 import pack_bias
    out = []
    for d in host_sets:
        g = dict(logits=torch.from_numpy(d["logits"]).to(dev), u=torch.from_numpy(d["u"]).to(dev), kw={})
        if "history" in d:
            g["kw"]["history"] = torch.from_numpy(d["history"]).to(dev)
        if "mask" in d:
            g["kw"]["mask"] = torch.from_numpy(d["mask"].view(np.int32)).to(dev)
        if "bias_ids" in d:
            g["kw"]["bias"] = torch.from_numpy(pack_bias(d["bias_ids"], d["bias_vals"])).to(dev)
        out.append(g)
    return out


def cpu_tokens(orc, params, d, rows=slice(None), threads=None):
    """(seconds, tokens) of the CPU reference over rows `rows` of host set d, on all host threads."""
    kw = {k: (d[k][rows] if d.get(k) is not None else None) for k in ("history", "mask", "bias_ids", "bias_vals")}
    return orc.time_sample_batch(params, d["logits"][rows], d["u"][rows], history=kw["history"], mask=kw["mask"],
                                 bias_ids=kw["bias_ids"], bias_vals=kw["bias_vals"],
                                 n_threads=threads or os.cpu_count() or 1)


# ---- the scale-out configuration: 1024 x 151552 over the ranks of this run, both modes -----------------------------
def config4_block(timer: Timer, dev, rank: int, world: int, local_rank: int, peak: float, with_cpu: bool):
    """Row-sharded (strong scaling, no collective) and vocab-parallel (local -> NCCL all-gather -> merge) sampling of
    one 1024-row batch. Every rank holds the whole synthetic batch in HBM (620 MB) and takes, at step j, the row block
    or column block (rank + j) mod N of it as its own shard of a fresh batch, so consecutive steps never re-read what
    L2 (126 MB) still holds; step 0 is the unrotated batch, which is the one compared with the CPU reference."""
    import torch
    import torch.distributed as dist
    from mako_b200 import BatchSampler, SamplingParams, lib, synth
    from mako_b200.parallel import row_shard, truncated_rows, vocab_parallel_sample, vocab_shard
    cfg = CONFIGS[4]
    b, v, h = cfg["batch"], cfg["n_vocab"], cfg["n_history"]
    params = SamplingParams(**cfg["params"])
    if b % world or (v // 32) % world:
        return {"skipped": f"1024 rows / {v} columns do not split evenly over {world} ranks"}
    host = dict(logits=synth.logits(SEED + 4, b, v)[0], u=synth.uniforms(SEED + 4, b),
                history=synth.history_zipf(SEED + 4, b, v, h))
    base = torch.from_numpy(host["logits"]).to(dev)
    hist = torch.from_numpy(host["history"]).to(dev)
    u = torch.from_numpy(host["u"]).to(dev)
    rb = row_bytes(cfg)
    n_launch = launches_per_step(params, v)
    out = {"workload": workload_name(cfg), "n_gpus": world,
           "l2": "every step reads another block of a 620 MB resident batch (> the 126 MB L2)"}
    want_cpu = None
    cpu_flat = None
    if with_cpu and rank == 0:
        from oracle.oracle import Oracle
        orc = Oracle("best")
        sec, want_cpu = cpu_tokens(orc, params, host)
        cpu_flat = {"rows_per_s": b / sec, "cores": os.cpu_count() or 1, "kind": orc.kind,
                    "sample": "one timed pass over the 1024 rows"}
        out["cpu_baseline"] = cpu_flat

    # -- row-sharded: rank r samples rows [r*1024/N, (r+1)*1024/N) ------------------------------------------------
    per = b // world
    rs = BatchSampler(v, per, local_rank)

    def rs_step(j):
        lo = ((rank + j) % world) * per
        return rs.sample(base[lo:lo + per], params, u[lo:lo + per], history=hist[lo:lo + per])
    rs_step(0)
    torch.cuda.synchronize(dev)
    rs_tok, rs_flags = rs.token[:per].cpu().numpy().copy(), rs.flags[:per].cpu().numpy().copy()
    g = capture(dev, rs_step)
    t = timer.run(g.replay, PER_GRAPH, 0, min_replays=20, min_seconds=0.15)
    ms = timer.max_over_ranks(t["ms_per_step"])
    blk = {"rows_per_gpu": per, "us_per_step": 1e3 * ms, "us_p10": 1e3 * t["p10"], "us_p90": 1e3 * t["p90"],
           "rows_per_s": b / (ms / 1e3), "effective_gbs": b * rb / (ms / 1e3) / 1e9,
           "roofline_frac_per_gpu": per * rb / (ms / 1e3) / 1e9 / peak, "gpu_launches_per_step": n_launch,
           "steps": t["steps"], "collective": "none", "scaling": "strong"}
    if want_cpu is not None:
        lo = rank * per
        sure = (rs_flags & 0x52) == 0
        blk.update(rows_compared=int(sure.sum()), rows_guard_band=int(((rs_flags & 0x2) != 0).sum()),
                   rows_overflow_or_timeout=int(((rs_flags & 0x50) != 0).sum()),
                   token_mismatches_vs_cpu=int((rs_tok[sure] != want_cpu[lo:lo + per][sure]).sum()))
    out["row_sharded"] = blk
    del rs, g

    # -- vocab-parallel: rank r holds columns [r*V/N, (r+1)*V/N) of every row -------------------------------------
    lo_c, hi_c = vocab_shard(v, rank, world)
    w = hi_c - lo_c
    vp = BatchSampler(v, b, local_rank)
    rec_b = lib.mk_vp_record_bytes(VP_K)
    records = torch.empty((b, rec_b), dtype=torch.uint8, device=dev)
    gathered = torch.empty((world, b, rec_b), dtype=torch.uint8, device=dev)

    def shard_of(j):
        c0 = ((rank + j) % world) * w
        return base[:, c0:c0 + w]          # a strided view: the kernel takes the row stride, nothing is copied

    def local(j):
        vp.vp_local(shard_of(j), params, VP_K, records, id_offset=lo_c, history=hist)

    def gather(j):
        local(j)
        if world > 1:
            dist.all_gather_into_tensor(gathered, records)
        else:
            gathered.copy_(records.unsqueeze(0))

    def full(j):
        gather(j)
        vp.vp_merge(gathered, world, b, VP_K, v, params, u)
    full(0)
    torch.cuda.synchronize(dev)
    vp_tok, vp_flags = vp.token[:b].cpu().numpy().copy(), vp.flags[:b].cpu().numpy().copy()
    split = {}
    for name, body in (("local", local), ("gather", gather), ("full", full)):
        try:
            g = capture(dev, body)
            launch, how = g.replay, "CUDA graph of 16 steps"
        except Exception as e:  # a collective that cannot be captured: launch from the host instead
            torch.cuda.synchronize(dev)
            how = f"host loop ({type(e).__name__})"

            def launch(body=body):
                for k in range(PER_GRAPH):
                    body(k)
        t = timer.run(launch, PER_GRAPH, 0, min_replays=20, min_seconds=0.15)
        split[name] = (timer.max_over_ranks(t["ms_per_step"]), t, how)
    ms_local, ms_gather, ms_full = split["local"][0], split["gather"][0], split["full"][0]
    n_trunc = int(((vp_flags & 0x20) != 0).sum())
    blk = {"columns_per_gpu": w, "k": VP_K, "record_bytes": rec_b, "all_gather_bytes_per_rank": world * b * rec_b,
           "us_local": 1e3 * ms_local, "us_all_gather": 1e3 * (ms_gather - ms_local),
           "us_merge": 1e3 * (ms_full - ms_gather), "us_per_step": 1e3 * ms_full,
           "us_p10": 1e3 * split["full"][1]["p10"], "us_p90": 1e3 * split["full"][1]["p90"],
           "rows_per_s": b / (ms_full / 1e3), "effective_gbs": b * rb / (ms_full / 1e3) / 1e9,
           "local_roofline_frac_per_gpu": b * (4 * w + 4 * h + 12) / (ms_local / 1e3) / 1e9 / peak,
           "steps": split["full"][1]["steps"], "launch": split["full"][2],
           "collective": "NCCL all_gather_into_tensor" if world > 1 else "none (one shard)", "scaling": "strong",
           "rows_vp_truncated": n_trunc, "rows_guard_band": int(((vp_flags & 0x2) != 0).sum())}
    if want_cpu is not None:
        sure = (vp_flags & 0x72) == 0
        blk.update(rows_compared=int(sure.sum()),
                   token_mismatches_vs_cpu=int((vp_tok[sure] != want_cpu[sure]).sum()))
    # the second round for rows whose nucleus reaches past a shard's list: whole rows gathered, single-device kernel
    res = vocab_parallel_sample(vp, shard_of(0), params, u, v, VP_K, history=hist, exact=True)  # untimed warm-up
    torch.cuda.synchronize(dev)
    timer.barrier()
    t0 = time.perf_counter()
    reps = 5
    for _ in range(reps):
        res = vocab_parallel_sample(vp, shard_of(0), params, u, v, VP_K, history=hist, exact=True)
        torch.cuda.synchronize(dev)
    ex_ms = timer.max_over_ranks((time.perf_counter() - t0) / reps * 1e3)
    ex_tok, ex_flags = res.token.cpu().numpy().copy(), res.flags.cpu().numpy().copy()
    ex = {"us_per_step": 1e3 * ex_ms, "rows_per_s": b / (ex_ms / 1e3), "rows_second_round": n_trunc,
          "timing": "host clock over whole calls (the second round reads the flags on the host)",
          "rows_still_truncated": int(((ex_flags & 0x20) != 0).sum())}
    if want_cpu is not None:
        sure = (ex_flags & 0x52) == 0
        ex.update(rows_compared=int(sure.sum()), token_mismatches_vs_cpu=int((ex_tok[sure] != want_cpu[sure]).sum()))
    blk["exact"] = ex
    out["vocab_parallel"] = blk
    return out


# ---- other configurations and the auxiliary kernels, one GPU -------------------------------------------------------
def run_other(args, cfg_id: int, dev, timer: Timer, peak: float, peak_kind: str):
    """--config 0|2|3|4: device-resident timing of one configuration, one JSON line."""
    import torch
    from mako_b200 import BatchSampler, SamplingParams, synth
    cfg = CONFIGS[cfg_id]
    params = SamplingParams(**cfg["params"])
    b, v = cfg["batch"], cfg["n_vocab"]
    lines = []

    def report(name, t, rows, nbytes, launches, extra=None):
        ms = t["ms_per_step"]
        line = {"metric": "sampled rows/s", "value": rows / (ms / 1e3), "unit": "rows/s", "n_gpus": 1,
                "steps": t["steps"], "warmup": args.warmup, "ms_per_step": ms, "ms_per_step_p10": t["p10"],
                "ms_per_step_p90": t["p90"], "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                "config": {"workload": name, "seed": SEED},
                "roofline": {"bound": "hbm", "achieved": nbytes / (ms / 1e3) / 1e9, "peak": peak, "unit": "GB/s",
                             "frac": nbytes / (ms / 1e3) / 1e9 / peak, "peak_kind": f"of {peak_kind}",
                             "traffic": committed_traffic(f"config{cfg_id}")},
                "gpu_launches": t["steps"] * launches}
        if extra:
            line.update(extra)
        lines.append(line)
        print(json.dumps(line), flush=True)

    if cfg_id == 0:
        # one row per step out of a pool of 1000 fresh rows (606 MB)
        pool = cfg["pool"]
        d = to_device(make_inputs(cfg, 0, 1), dev)[0]
        s = BatchSampler(v, 1, dev.index)
        s.set_overlap(args.overlap)
        for split, tag, launches in ((True, ", one row per step split over 37 CTAs", 3),
                                     (False, ", one row per step as one CTA", 1)):
            s.set_split(split)
            g = capture(dev, lambda k: s.sample(d["logits"][k % pool:k % pool + 1], params,
                                                d["u"][k % pool:k % pool + 1]))
            report(workload_name(cfg) + tag, timer.run(g.replay, PER_GRAPH, args.steps), 1, 4 * v + 12, launches)
    elif cfg_id in (2, 4):
        n_sets = 8 if cfg_id == 2 else 2
        sets = to_device(make_inputs(cfg, 0, n_sets), dev)
        s = BatchSampler(v, b, dev.index)
        variants = [("", params)] + ([(", greedy", SamplingParams(temperature=0.0))] if cfg_id == 2 else [])
        for tag, p in variants:
            def body(k, p=p):
                x = sets[k % n_sets]
                s.sample(x["logits"], p, x["u"], **x["kw"])
            g = capture(dev, body)
            t = timer.run(g.replay, PER_GRAPH, args.steps, min_replays=20)
            fl = s.flags[:b].cpu().numpy()
            nc = s.n_cand[:b].cpu().numpy()
            report(workload_name(cfg) + tag, t, b, b * row_bytes(cfg), launches_per_step(p, v),
                   {"rows_guard_band": int(((fl & 2) != 0).sum()), "rows_overflow_or_timeout": int(((fl & 0x50) != 0).sum()),
                    "candidates_median": int(np.median(nc)), "candidates_max": int(nc.max())})
    elif cfg_id == 3:
        host = make_inputs(cfg, 0, 2)
        sets = to_device(host, dev)
        for k, (d, hd) in enumerate(zip(sets, host)):
            d["drafter"] = torch.from_numpy(synth.add_noise(SEED, hd["logits"], v, step=k)).to(dev)
            d["u2"] = torch.from_numpy(synth.uniforms(SEED, b, purpose=1, step=k)).to(dev)
            d["u3"] = torch.from_numpy(synth.uniforms(SEED, b, purpose=2, step=k)).to(dev)
        s = BatchSampler(v, b, dev.index)

        def body(k):
            x = sets[k % 2]
            s.verify_pq(x["logits"], x["drafter"], params, x["u"], x["u2"], x["u3"])
        g = capture(dev, body)
        t = timer.run(g.replay, PER_GRAPH, args.steps, min_replays=20)
        fl = s.flags[:b].cpu().numpy()
        report(workload_name(cfg), t, b, b * (2 * 4 * v + 12 + 12), 5,
               {"rows_overflow_or_timeout": int(((fl & 0x50) != 0).sum()),
                "accepted": int(s.accepted[:b].sum().item())})
    return lines


def run_aux(args, dev, timer: Timer, peak: float, peak_kind: str):
    """--aux: the reasoning-budget logit test and the two drafter picks, one JSON line each."""
    import torch
    from mako_b200 import BatchSampler
    v, b = 129280, 256
    sets = to_device(make_inputs(CONFIGS[1], 0, N_SETS), dev)
    s = BatchSampler(v, b, dev.index)
    tok = torch.full((b,), 1234, dtype=torch.int32, device=dev)

    def line(name, t, nbytes, kernel):
        ms = t["ms_per_step"]
        print(json.dumps({"metric": "us per launch", "value": 1e3 * ms, "unit": "us", "higher_is_better": False,
                          "steps": t["steps"], "config": {"workload": name},
                          "roofline": {"bound": "hbm", "achieved": nbytes / (ms / 1e3) / 1e9, "peak": peak,
                                       "unit": "GB/s", "frac": nbytes / (ms / 1e3) / 1e9 / peak,
                                       "peak_kind": f"of {peak_kind}", "kernel": kernel}}), flush=True)
    g = capture(dev, lambda k: s.rank_force(sets[k % N_SETS]["logits"], tok))
    line("rank test (is the token among the 3 largest), 256 x 129280", timer.run(g.replay, PER_GRAPH, args.steps),
         b * (4 * v + 12), "rank_force_kernel")
    rank, dim = 256, 4096
    gen = torch.Generator(device=dev).manual_seed(SEED)
    head = torch.randn((v, rank), generator=gen, device=dev) * 0.05
    embed = torch.randn((v, rank), generator=gen, device=dev)
    w = torch.randn(dim + rank, generator=gen, device=dev) * 0.05
    s8 = BatchSampler(v, 8, dev.index)
    for n_seq in (1, 8):
        lg = torch.randn((n_seq, v), generator=gen, device=dev) * 2
        x = torch.randn((n_seq, dim), generator=gen, device=dev)
        prev = torch.arange(n_seq, dtype=torch.int32, device=dev) * 1000 + 5
        g = capture(dev, lambda k: s8.draft_pick(lg, head, embed, x, w, prev))
        line(f"drafter pick, {n_seq} sequence(s), head 129280 x 256", timer.run(g.replay, PER_GRAPH, args.steps),
             4 * v * rank + n_seq * 4 * v, "draft_score_kernel")
    h = torch.randn((8, dim), generator=gen, device=dev)
    cw = torch.randn(dim, generator=gen, device=dev) * 0.05
    lg = torch.randn((8, v), generator=gen, device=dev) * 2
    g = capture(dev, lambda k: s8.draft_pick_plain(lg, h, cw, 0.1))
    line("plain drafter pick, 8 sequences", timer.run(g.replay, PER_GRAPH, args.steps), 8 * 4 * v,
         "draft_pick_plain_kernel")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8192)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=1, choices=[0, 1, 2, 3, 4])
    ap.add_argument("--aux", action="store_true", help="time the auxiliary kernels instead (one GPU)")
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the host-buffer leg (default: 20)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-config4", action="store_true", help="skip the scale-out block of the JSON line")
    ap.add_argument("--streams", type=int, default=2, help="batches in flight (sampler handles and streams)")
    ap.add_argument("--no-graph", action="store_true", help="launch each step from the host instead of a CUDA graph")
    ap.add_argument("--overlap", type=int, default=2, choices=[0, 1, 2],
                    help="how a launch follows the previous kernel of its stream: 0 plain stream order, 1 programmatic "
                         "dependent launch, 2 the same with the history tables built before the wait")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = CONFIGS[args.config]

    if args.impl == "reference":
        run_reference(args, cfg, rank, world)
        return

    import torch
    import torch.distributed as dist
    from mako_b200 import BatchSampler, SamplingParams

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    timer = Timer(dev, world)
    peak, peak_kind = measured_hbm_peak()

    if args.aux or args.config != 1:
        assert world == 1, "--aux and --config 0|2|3|4 run on one GPU"
        if args.aux:
            run_aux(args, dev, timer, peak, peak_kind)
        else:
            run_other(args, args.config, dev, timer, peak, peak_kind)
        return

    params = SamplingParams(**cfg["params"])
    b, v = cfg["batch"], cfg["n_vocab"]
    host_sets = make_inputs(cfg, rank, N_SETS)
    dev_sets = to_device(host_sets, dev)
    # args.streams sampler handles (scratch and outputs of their own), step k on handle and stream k % streams: two
    # batches in flight, as a server that double-buffers its decode steps has them, so that one launch's set-up and
    # finish overlap the other's streaming instead of leaving the memory system idle.
    samplers = [BatchSampler(v, b, local_rank) for _ in range(max(1, args.streams))]
    for smp in samplers:
        smp.set_overlap(args.overlap)
    sampler = samplers[0]

    def step(k, handle=None):
        g = dev_sets[k % N_SETS]
        return (handle or samplers[k % len(samplers)]).sample(g["logits"], params, g["u"], **g["kw"])

    for k in range(args.warmup):
        step(k)
    timer.barrier()
    clocks = ClockSampler(local_rank) if rank == 0 else None
    # The timed loop replays a CUDA graph of 256 steps (64 cycles over the input sets), so that the host's launch
    # path (Python, ctypes) is not what is measured; --no-graph launches the same steps from the host instead.
    per_graph = HEADLINE_PER_GRAPH
    if args.no_graph:
        def replay():
            for k in range(per_graph):
                step(k)
        serial = None
    else:
        replay = capture(dev, step, len(samplers), per_graph).replay
        serial = capture(dev, lambda k: step(k, sampler), 1, per_graph).replay if len(samplers) > 1 else None
    t = timer.run(replay, per_graph, args.steps)
    ms_step = timer.max_over_ranks(t["ms_per_step"])
    ms_mean = timer.max_over_ranks(t["mean"])
    t1 = None
    if serial is not None:  # the same with one batch in flight: plain back-to-back launches on one stream
        t1 = timer.run(serial, per_graph, args.steps)
        replay()            # leave the outputs of the headline mode in place for the parity check below
        timer.barrier()
    last_k = per_graph - 1
    last = samplers[last_k % len(samplers)]
    flags = last.flags[:b].cpu().numpy()
    tokens_dev = last.token[:b].cpu().numpy().copy()

    # ---- end to end through the host-buffer entry point --------------------------------------------------------
    from mako_b200 import pack_bias
    e2e_steps = args.e2e_steps or 20
    pinned = []
    for d in host_sets[:2]:
        p = {k2: torch.from_numpy(a).pin_memory().numpy() for k2, a in d.items() if k2 in ("logits", "u", "history",
                                                                                         "mask")}
        if "bias_ids" in d:
            p["bias"] = torch.from_numpy(pack_bias(d["bias_ids"], d["bias_vals"])).pin_memory().numpy()
        pinned.append(p)

    def e2e_step(k):
        p = pinned[k % len(pinned)]
        return sampler.sample_host(p["logits"], params, p["u"], history=p.get("history"), mask=p.get("mask"),
                                   bias=p.get("bias"))
    for k in range(3):
        e2e_step(k + 1)
    timer.barrier()
    t0 = time.perf_counter()
    for k in range(e2e_steps):
        tok_e2e, _, flags_e2e = e2e_step(k)
    torch.cuda.synchronize()
    e2e_sec = timer.max_over_ranks(time.perf_counter() - t0)
    e2e_set = (e2e_steps - 1) % len(pinned)
    clk = clocks.stop() if clocks else None

    line = None
    if rank == 0:
        rb = row_bytes(cfg)
        achieved = rb * b / (t["ms_per_step"] / 1e3) / 1e9   # this rank's kernel, median launch
        h2d = b * (4 * v + 4 * cfg["n_history"] + (4 * ((v + 31) // 32) if cfg["mask"] else 0)
                   + 8 * cfg["n_bias"] + 4)
        conf = workload_config(cfg, world)
        conf.update(l2=f"{N_SETS} distinct input sets cycled ({N_SETS * rb * b / 1e6:.0f} MB > L2)",
                    launch="host loop" if args.no_graph else
                    f"CUDA graph of {per_graph} steps replayed {t['replays']} times, one event pair per replay, "
                    f"{len(samplers)} batches in flight",
                    overlap=["plain stream order", "programmatic dependent launch",
                             "programmatic dependent launch, history tables built before the wait (histories and "
                             "parameters are not written by the previous kernel)"][args.overlap])
        line = {
            "metric": "sampled rows/s", "value": world * b / (ms_step / 1e3), "unit": "rows/s", "n_gpus": world,
            "steps": t["steps"], "warmup": args.warmup, "ms_per_step": ms_step, "ms_per_step_p10": t["p10"],
            "ms_per_step_p90": t["p90"], "ms_per_step_mean": ms_mean, "timed_region_s": t["total_ms"] / 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": conf,
            "effective_gbs": world * b * rb / (ms_step / 1e3) / 1e9,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": committed_traffic(f"config{args.config}"),
                         "peak_kind": f"of {peak_kind}", "bytes_per_row": rb, "rows_per_launch": b,
                         "kernel": "row_pipeline_kernel",
                         "mode": f"{len(samplers)} independent batches in flight on {len(samplers)} streams"},
            "e2e": {"value": world * b * e2e_steps / e2e_sec, "unit": "rows/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 12 * b, "steps": e2e_steps,
                    "bound": "host-to-device copy of the logits (PCIe): the kernel is about 1 % of a step"},
            "gpu_launches": t["steps"] * launches_per_step(params, v),
            "one_batch_in_flight": None if t1 is None else {
                "ms_per_step": t1["ms_per_step"], "ms_per_step_p10": t1["p10"], "ms_per_step_p90": t1["p90"],
                "steps": t1["steps"], "value": b / (t1["ms_per_step"] / 1e3),
                "roofline_frac": rb * b / (t1["ms_per_step"] / 1e3) / 1e9 / peak},
            "clocks": clk,
            "parity": {"rows_flagged_near_cdf_boundary": int((flags & 1).sum()),
                       "rows_flagged_guard_band": int(((flags & 2) != 0).sum()),
                       "rows_overflow_or_timeout": int(((flags & 0x50) != 0).sum())},
        }
        if world == 1 and not args.no_cpu_baseline:
            from oracle.oracle import Oracle
            orc = Oracle("best")
            cores = os.cpu_count() or 1
            d = host_sets[last_k % N_SETS]
            reps, total, toks = 0, 0.0, None
            t_begin = time.perf_counter()
            while reps < 3 or (time.perf_counter() - t_begin < 8.0 and reps < 64):
                sec, toks = cpu_tokens(orc, params, d, threads=cores)
                total += sec
                reps += 1
            line["cpu_baseline"] = {"value": b * reps / total, "unit": "rows/s", "cores": cores, "kind": orc.kind,
                                    "sample": f"{reps} timed passes over the last step's {b} rows, {cores} host "
                                              "threads (each after an untimed pass that sizes the samplers' vectors)"}
            line["parity"]["token_mismatches_vs_cpu"] = int((toks != tokens_dev).sum())
            _, toks_e2e = cpu_tokens(orc, params, host_sets[e2e_set], threads=cores)
            line["parity"]["e2e_token_mismatches_vs_cpu"] = int((toks_e2e != tok_e2e).sum())
            line["parity"]["e2e_rows_overflow_or_timeout"] = int(((flags_e2e & 0x50) != 0).sum())
    del samplers, sampler, dev_sets
    if not args.no_config4:
        blk = config4_block(timer, dev, rank, world, local_rank, peak, with_cpu=not args.no_cpu_baseline)
        if line is not None:
            line["config4"] = blk
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
