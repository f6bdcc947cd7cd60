"""Benchmark of the token-sampling hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 1]

One step = one pass of the row pipeline over one batch of synthetic rows. The default workload is the batched
penalised configuration: 256 rows x V=129280 fp32 logits (N(0,2^2) + 8 spikes U(8,15)), a 4096-id Zipf(1.1) token
history per row, repetition 1.1 / presence 0.5 / frequency 0.3, temperature 0.8, top_p 0.9, min_p 0.05, one uniform
per row. Prints one JSON line (rank 0):

  value        rows/s over all GPUs with the inputs resident in HBM (CUDA events around K launches, max over ranks)
  e2e          the same through the host-buffer entry point: pinned host inputs copied in, results copied out,
               every step, inside the timed region
  roofline     algorithmic bytes of one launch / its mean duration, against the measured HBM copy bandwidth
  cpu_baseline the reference's own CPU sampler (oracle/_ref when built, else the CPU restatement) timed on the host
               cores on a bounded sample of the same rows, rank 0 at N=1 only

With N > 1 (launched by torch.distributed.run) every rank samples its own 256 rows of a 256*N-row batch: rows are
independent, so there is no data-path collective (weak scaling).  `--impl reference` times the CPU reference alone.
"""
from __future__ import annotations

import argparse
import json
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
    # name: (batch, V, history, mask, n_bias, params)
    0: dict(batch=1, n_vocab=151552, n_history=0, mask=False, n_bias=0,
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
                        frequency_penalty=0.3), name="row-sharded 1024 x 151552"),
}
N_SETS = 4  # distinct input sets cycled between steps: 4 x 137 MB > the 126 MB L2
SEED = 20240


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
    b, v = cfg["batch"], cfg["n_vocab"]
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


def run_reference(args, cfg, params, rank, world):
    """The reference's CPU sampler on the host cores; each step is one batch of the workload."""
    if rank != 0:
        return
    from oracle.oracle import Oracle
    orc = Oracle("best")
    cores = os.cpu_count() or 1
    sets = make_inputs(cfg, 0, min(2, N_SETS))
    b = cfg["batch"]

    def step(k):
        d = sets[k % len(sets)]
        sec, _ = orc.time_sample_batch(params, d["logits"], d["u"], history=d.get("history"), mask=d.get("mask"),
                                       bias_ids=d.get("bias_ids"), bias_vals=d.get("bias_vals"), n_threads=cores)
        return sec
    for k in range(args.warmup):
        step(k)
    total = sum(step(k) for k in range(args.steps))
    value = b * args.steps / total
    line = {
        "impl": "reference", "metric": "sampled rows/s", "value": value, "unit": "rows/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(cfg), "batch": b, "n_vocab": cfg["n_vocab"],
                   "n_history": cfg["n_history"]},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": orc.kind,
                         "sample": f"{args.steps} steps of the full {b}-row batch, {cores} host threads, "
                                   "sample() only (history replay outside the timed region)"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "effective_gbs": value * row_bytes(cfg) / 1e9,
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(cfg) -> str:
    return (f"{cfg['name']}: batch {cfg['batch']} x V={cfg['n_vocab']} fp32, history {cfg['n_history']}"
            + (", 2% mask" if cfg["mask"] else "") + (f", {cfg['n_bias']} bias" if cfg["n_bias"] else ""))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8192)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=1, choices=[0, 1, 2, 4])
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the host-buffer leg (default: min(steps, 20))")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--streams", type=int, default=2, help="batches in flight (sampler handles and streams)")
    ap.add_argument("--no-graph", action="store_true", help="launch each step from the host instead of a CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = CONFIGS[args.config]

    from mako_b200.sampler import SamplingParams
    params = SamplingParams(**cfg["params"])

    if args.impl == "reference":
        run_reference(args, cfg, params, rank, world)
        return

    import torch
    import torch.distributed as dist
    from mako_b200 import BatchSampler, pack_bias

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    b, v = cfg["batch"], cfg["n_vocab"]
    host_sets = make_inputs(cfg, rank, N_SETS)
    dev_sets = []
    for d in host_sets:
        g = dict(logits=torch.from_numpy(d["logits"]).to(dev), u=torch.from_numpy(d["u"]).to(dev), kw={})
        if "history" in d:
            g["kw"]["history"] = torch.from_numpy(d["history"]).to(dev)
        if "mask" in d:
            g["kw"]["mask"] = torch.from_numpy(d["mask"].view(np.int32)).to(dev)
        if "bias_ids" in d:
            g["kw"]["bias"] = torch.from_numpy(pack_bias(d["bias_ids"], d["bias_vals"])).to(dev)
        dev_sets.append(g)
    # args.streams sampler handles (scratch and outputs of their own), step k on handle and stream k % streams: two
    # batches in flight, as a server that double-buffers its decode steps has them, so that one launch's set-up and
    # finish overlap the other's streaming instead of leaving the memory system idle.
    samplers = [BatchSampler(v, b, local_rank) for _ in range(max(1, args.streams))]
    sampler = samplers[0]

    def step(k):
        g = dev_sets[k % N_SETS]
        return samplers[k % len(samplers)].sample(g["logits"], params, g["u"], **g["kw"])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for k in range(args.warmup):
        step(k)
    barrier()
    # The timed loop replays a CUDA graph of one cycle over the input sets, so that the host's launch path (Python,
    # ctypes) is not what is measured; --no-graph launches step by step instead.
    graph = None
    per_graph = N_SETS * 4   # steps captured in one graph
    cycles = max(1, args.steps // per_graph)
    if not args.no_graph:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                subs = [torch.cuda.Stream(device=dev) for _ in samplers]
                for sub in subs:
                    sub.wait_stream(side)
                for k in range(per_graph):
                    with torch.cuda.stream(subs[k % len(subs)]):
                        step(k)
                for sub in subs:
                    side.wait_stream(sub)
        torch.cuda.current_stream(dev).wait_stream(side)
        args.steps = cycles * per_graph
        graph.replay()
    barrier()
    clocks = ClockSampler(local_rank) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if graph is not None:
        for _ in range(cycles):
            graph.replay()
    else:
        for k in range(args.steps):
            step(k)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    # the same K steps with one batch in flight (plain back-to-back launches on one stream), for the record
    ms_serial = None
    if graph is not None and len(samplers) > 1:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            g1 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g1, stream=side):
                for k in range(per_graph):
                    samplers[0].sample(dev_sets[k % N_SETS]["logits"], params, dev_sets[k % N_SETS]["u"],
                                       **dev_sets[k % N_SETS]["kw"])
        torch.cuda.current_stream(dev).wait_stream(side)
        g1.replay()
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(cycles):
            g1.replay()
        s1.record()
        barrier()
        ms_serial = s0.elapsed_time(s1)
        graph.replay()          # leave the outputs of the headline mode in place for the parity check below
        barrier()
    last = samplers[(args.steps - 1) % len(samplers)]
    flags = last.flags[:b].cpu().numpy()
    tokens_dev = last.token[:b].cpu().numpy().copy()
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())

    # ---- end to end through the host-buffer entry point --------------------------------------------------------
    e2e_steps = args.e2e_steps or min(args.steps, 20)
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
        tok_host, _, _ = e2e_step(k + 1)
    barrier()
    t0 = time.perf_counter()
    for k in range(e2e_steps):
        tok_e2e, _, _ = e2e_step(k)
    torch.cuda.synchronize()
    e2e_sec = time.perf_counter() - t0
    te = torch.tensor([e2e_sec], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_sec = float(te.item())
    clk = clocks.stop() if clocks else None

    if rank == 0:
        rb = row_bytes(cfg)
        ms_per_step = ms_max / args.steps
        value = world * b * args.steps / (ms_max / 1e3)
        peak, peak_kind = measured_hbm_peak()
        achieved = rb * b / (ms / args.steps / 1e3) / 1e9   # this rank's kernel
        h2d = b * (4 * v + 4 * cfg["n_history"] + (4 * ((v + 31) // 32) if cfg["mask"] else 0)
                   + 8 * cfg["n_bias"] + 4)
        line = {
            "metric": "sampled rows/s", "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(cfg), "batch_per_gpu": b, "n_vocab": v,
                       "n_history": cfg["n_history"], "parallelism": f"row-sharded x{world}, no collective",
                       "l2": f"{N_SETS} distinct input sets cycled ({N_SETS * rb * b / 1e6:.0f} MB > L2)",
                       "seed": SEED, "launch": "host loop" if graph is None else f"CUDA graph of {per_graph} steps replayed, {len(samplers)} batches in flight"},
            "effective_gbs": value * rb / 1e9,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": committed_traffic(f"config{args.config}"),
                         "peak_kind": f"of {peak_kind}", "bytes_per_row": rb, "rows_per_launch": b,
                         "kernel": "row_pipeline_kernel"},
            "e2e": {"value": world * b * e2e_steps / e2e_sec, "unit": "rows/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 12 * b, "steps": e2e_steps},
            "gpu_launches": args.steps * launches_per_step(params, v),
            "one_batch_in_flight": None if ms_serial is None else {
                "ms_per_step": ms_serial / args.steps, "value": b * args.steps / (ms_serial / 1e3),
                "roofline_frac": rb * b / (ms_serial / args.steps / 1e3) / 1e9 / peak},
            "clocks": clk,
            "parity": {"rows_flagged_near_cdf_boundary": int((flags & 1).sum()),
                       "rows_flagged_guard_band": int(((flags & 2) != 0).sum()),
                       "rows_overflow_or_timeout": int(((flags & 0x50) != 0).sum())},
        }
        if world == 1 and not args.no_cpu_baseline:
            from oracle.oracle import Oracle
            orc = Oracle("best")
            cores = os.cpu_count() or 1
            d = host_sets[(args.steps - 1) % N_SETS]
            reps, total, toks = 0, 0.0, None
            t_begin = time.perf_counter()
            while reps < 3 or (time.perf_counter() - t_begin < 4.0 and reps < 64):
                sec, toks = orc.time_sample_batch(params, d["logits"], d["u"], history=d.get("history"),
                                                  mask=d.get("mask"), bias_ids=d.get("bias_ids"),
                                                  bias_vals=d.get("bias_vals"), n_threads=cores)
                total += sec
                reps += 1
            line["cpu_baseline"] = {"value": b * reps / total, "unit": "rows/s", "cores": cores, "kind": orc.kind,
                                    "sample": f"{reps} passes over the last step's {b} rows, {cores} host threads"}
            line["parity"]["token_mismatches_vs_cpu"] = int((toks != tokens_dev).sum())
            line["parity"]["e2e_token_mismatches_vs_cpu"] = None
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
