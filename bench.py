#!/usr/bin/env python
"""Decode benchmark: Qwen3-8B-geometry bf16 greedy decode through the megakernel.

  python bench.py --gpus 1 --steps K --warmup W [--batch B] [--layers L]
  python bench.py --impl reference ...   (the reference PyTorch path on the host cores)

A step is one decode iteration (one token per request).  The whole generation
(64-token prompt fed token by token, then W untimed + K timed decode steps) is
ONE persistent launch; step times are globaltimer stamps the kernel records at
each iteration boundary, so `value` is the mean time per output token over the
K timed steps with everything resident in HBM.  `e2e` repeats the generation
through the public API from pinned host prompts to host tokens and divides the
wall time by the tokens generated (prompt iterations included).  Synthetic
data: seeded random weights N(0, 0.02) in bf16 and uniform-random prompts with
the shapes of the reference's benchmark (no checkpoint or tokenizer here).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "Qwen3-8B bf16 decode TPOT"
PROMPT_LEN = 64
MAX_SEQ = 1200
PAGE = 64
DRAM_TRAFFIC_RATIO = 1.040


def geometry(layers):
    import fleet_chiplet_megakernel_b200 as mk
    return mk.Qwen3Geometry(layers=layers)


def weight_shapes(g):
    yield "embed", (g.vocab, g.hidden)
    for i in range(g.layers):
        yield f"l{i}.q", (g.n_q * g.head_dim, g.hidden)
        yield f"l{i}.k", (g.n_kv * g.head_dim, g.hidden)
        yield f"l{i}.v", (g.n_kv * g.head_dim, g.hidden)
        yield f"l{i}.o", (g.hidden, g.n_q * g.head_dim)
        yield f"l{i}.gate", (g.mlp, g.hidden)
        yield f"l{i}.up", (g.mlp, g.hidden)
        yield f"l{i}.down", (g.hidden, g.mlp)
    yield "lm_head", (g.vocab, g.hidden)


def make_weights(g, device, seed=0):
    """Seeded random-init weights in the fixed order embed, per layer q,k,v,o,gate,up,down, lm_head."""
    gen = torch.Generator(device=device).manual_seed(seed)
    w = {}
    for name, shape in weight_shapes(g):
        w[name] = (torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * 0.02).to(torch.bfloat16)
    for i in range(g.layers):
        w[f"l{i}.ln1"] = torch.ones(g.hidden, dtype=torch.bfloat16, device=device)
        w[f"l{i}.ln2"] = torch.ones(g.hidden, dtype=torch.bfloat16, device=device)
        w[f"l{i}.qn"] = torch.ones(g.head_dim, dtype=torch.bfloat16, device=device)
        w[f"l{i}.kn"] = torch.ones(g.head_dim, dtype=torch.bfloat16, device=device)
    w["norm"] = torch.ones(g.hidden, dtype=torch.bfloat16, device=device)
    return w


def make_prompts(g, batch):
    out = []
    for r in range(batch):
        gen = torch.Generator().manual_seed(1000 + r)
        out.append(torch.randint(0, g.vocab, (PROMPT_LEN,), generator=gen, dtype=torch.int64))
    return out


def algorithmic_bytes(g, batch, ctx_lens):
    """Weights read once + KV read/written + activations, per decode step."""
    per_layer = 2 * ((g.n_q + 2 * g.n_kv) * g.head_dim * g.hidden + g.hidden * g.n_q * g.head_dim +
                     2 * g.mlp * g.hidden + g.hidden * g.mlp) + 2 * (2 * g.hidden + 2 * g.head_dim)
    weights = g.layers * per_layer + 2 * g.vocab * g.hidden + 2 * g.hidden
    kv_unit = 2 * g.layers * g.n_kv * g.head_dim * 2
    kv = sum(kv_unit * (L + 1) for L in ctx_lens)
    act = batch * (2 * g.vocab + 40 * g.hidden * 2)
    return weights + kv + act, weights


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], None, set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
                power.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        busy = [c for c, p in zip(sm, power) if p > 0.5 * max(power)] if power else sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power) if power else None}


def cpu_baseline(g, w, threads=None, sample_layers=4, steps=4):
    """The oracle's restatement of the reference PyTorch model on the host cores:
    `sample_layers` layers + final norm + LM head, a 64-token prefill then `steps`
    decode steps at batch 1; the per-layer time is scaled to the full depth."""
    from oracle import qwen3_oracle as O
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    geom = O.Geometry(hidden=g.hidden, n_q=g.n_q, n_kv=g.n_kv, mlp=g.mlp, layers=g.layers, vocab=g.vocab)
    n = min(sample_layers, g.layers)
    keys = ["embed", "lm_head", "norm"] + [f"l{i}.{s}" for i in range(n)
                                           for s in ("q", "k", "v", "o", "gate", "up", "down", "ln1", "ln2", "qn", "kn")]
    wc = {k: w[k].cpu() for k in keys}
    m = O.TorchRefModel(geom, wc, PROMPT_LEN + steps + 2, layers=n)
    prompt = make_prompts(g, 1)[0]
    with torch.inference_mode():
        h = torch.nn.functional.embedding(prompt, wc["embed"])
        m.forward_hidden(h, 0)
        t_layers, t_head = [], []
        for s in range(steps):
            tok = torch.tensor([int(prompt[s])])
            t0 = time.perf_counter()
            h = torch.nn.functional.embedding(tok, wc["embed"])
            h = m.forward_hidden(h, PROMPT_LEN + s)
            t1 = time.perf_counter()
            lg = torch.nn.functional.linear(O.ref_rmsnorm(h, wc["norm"]), wc["lm_head"])
            int(lg.argmax(-1))
            t2 = time.perf_counter()
            t_layers.append(t1 - t0)
            t_head.append(t2 - t1)
    per_layer = statistics.median(t_layers) / n
    ms = (per_layer * g.layers + statistics.median(t_head)) * 1e3
    return {"value": ms, "unit": "ms/token", "cores": threads, "kind": "port",
            "sample": f"{n} of {g.layers} layers + LM head, 64-token prefill then {steps} decode steps at batch 1; "
                      f"median per-layer time x {g.layers} + head"}


def run_ours(args):
    import fleet_chiplet_megakernel_b200 as mk
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    g = geometry(args.layers)
    B = args.batch
    K, W = args.steps, args.warmup
    iters = PROMPT_LEN + W + K - 1
    assert PROMPT_LEN + W + K + 1 <= MAX_SEQ, "steps + warmup exceed the 1200-token sequence limit"
    w = make_weights(g, dev)
    if world > 1:
        # tensor parallel: every rank draws the same seeded weights and keeps its shard
        w_full = w
        w = mk.shard_qwen3_weights(w_full, world, rank)
        del w_full
        torch.cuda.empty_cache()
    prompts = make_prompts(g, B)
    dec = mk.Qwen3Decoder(g, w, max_seq_length=MAX_SEQ, max_requests=B, page_size=PAGE, device=dev,
                          max_iterations=iters, numerics=args.numerics, world_size=world, rank=rank)
    torch.cuda.synchronize()

    def generation(host_prompts):
        dec.set_prompts(host_prompts)
        dec.run()

    # untimed full pass first (page faults, clocks), then the measured one
    generation(prompts)
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dec.set_prompts(prompts)
    e0.record()
    dec.run()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    launch_ms = e0.elapsed_time(e1)
    stamps = dec.mpk.get_event_timing()
    assert stamps.shape[0] == iters + 1, (stamps.shape, iters)
    t = stamps[:, 0].astype("float64")
    first = PROMPT_LEN - 1 + W
    step_ns = t[first + 1: first + K + 1] - t[first: first + K]
    tpot_ms = float(step_ns.sum() / K / 1e6)
    import numpy as _np
    tpot_median_ms = float(_np.median(step_ns) / 1e6)
    tpot_first_ms, tpot_last_ms = float(step_ns[: max(1, K // 10)].mean() / 1e6), float(step_ns[-max(1, K // 10):].mean() / 1e6)
    # end to end through the public API: pinned host prompts in, host tokens out
    host_prompts = [p.pin_memory() for p in prompts]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    generation(host_prompts)
    out_tokens = dec.tokens[:, : PROMPT_LEN + W + K].to("cpu", non_blocking=False)
    t1 = time.perf_counter()
    clocks = sampler.stop()
    e2e_ms = (t1 - t0) * 1e3 / (W + K)
    if world > 1:
        v = torch.tensor([tpot_ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        tpot_ms, e2e_ms = float(v[0]), float(v[1])
    ctx = [PROMPT_LEN + W + j for j in range(K)]
    mean_bytes = statistics.mean(algorithmic_bytes(g, B, [L] * B)[0] for L in ctx)
    if world > 1:
        # per GPU under tensor parallelism: layer weights and KV are sharded, the LM head is replicated
        # (as in the reference, demo/qwen3/models/modeling_qwen3.py:514)
        head = 2 * g.vocab * g.hidden + 2 * g.hidden
        mean_bytes = (mean_bytes - head) / world + head
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = mean_bytes / (tpot_ms * 1e-3) / 1e9
    # DRAM read+write bytes per step: one ncu capture of the 4-layer case measured 1.040 x its
    # algorithmic bytes (profiles/megakernel_bs1_4layers_ncu.md); traffic grows in proportion to the
    # bytes a step streams, so the same ratio is applied to this workload
    traffic = DRAM_TRAFFIC_RATIO * mean_bytes if B <= 8 else None
    line = {
        "metric": METRIC, "value": tpot_ms, "unit": "ms/token", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": tpot_ms, "higher_is_better": False, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded random weights N(0,0.02), uniform-random 64-token prompts)",
        "config": {"workload": f"Qwen3-8B geometry, {g.layers} layers, vocab {g.vocab}, batch {B}, 64-token prompt, "
                               f"{K} greedy decode steps, paged KV (page 64), max seq 1200",
                   "batch": B, "l2": "inputs larger than L2 (15.1 GB of weights per step)",
                   "timing": "globaltimer stamp per iteration inside the single persistent launch",
                   "numerics": args.numerics, "grid": dec.mpk.grid_size(),
                   "parallelism": f"tp{world}" if world > 1 else "single GPU",
                   "launch_ms_total": launch_ms, "iterations": iters},
        "tokens_per_s": B * 1e3 / tpot_ms,
        "tpot_median_ms": tpot_median_ms,
        "tpot_first_tenth_ms": tpot_first_ms, "tpot_last_tenth_ms": tpot_last_ms,  # context grows during the run
        "clocks": clocks,
        "e2e": {"value": e2e_ms, "unit": "ms/token", "h2d_bytes_per_step": B * PROMPT_LEN * 8 / (W + K),
                "d2h_bytes_per_step": B * (PROMPT_LEN + W + K) * 8 / (W + K),
                "note": "wall time of set_prompts (H2D) + launch (64 prompt iterations + decode) + token readback, "
                        "per generated token"},
        "gpu_launches": 2,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "algorithmic_bytes_per_step": mean_bytes, "per": "GPU",
                     "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback",
                     "frac_of_nominal_8TBps": achieved / 8000.0},
    }
    if rank == 0:
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(g, w)
        print(json.dumps(line), flush=True)
    dec.finalize()
    if world > 1:
        dist.destroy_process_group()
    return out_tokens


def run_reference(args):
    """The reference's own CPU implementation of the path (its PyTorch model, restated in
    oracle/), timed on the host cores with all threads, on a bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    g = geometry(args.layers)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    n = min(4, g.layers)
    # only the sampled layers' weights are needed
    import dataclasses
    gs = dataclasses.replace(g, layers=n)
    w = make_weights(gs, dev)
    for i in range(n, g.layers):
        pass
    base = cpu_baseline(dataclasses.replace(g), w, sample_layers=n, steps=max(2, min(args.steps, 6)))
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": "ms/token",
            "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": base["value"], "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded random weights, uniform-random prompts)",
            "config": {"workload": f"Qwen3-8B geometry, {g.layers} layers, batch 1, host cores", "batch": 1},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "ms/token", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--numerics", default="torch", choices=["torch", "mpk"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
