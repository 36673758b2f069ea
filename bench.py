#!/usr/bin/env python
"""Decode benchmark: Qwen3-8B-geometry bf16 greedy decode through the megakernel.

  python bench.py --gpus 1 --steps K --warmup W [--batch B] [--layers L]
  python bench.py --impl reference ...   (the reference PyTorch path on the host cores)

A step is one decode iteration (one token per request).  The whole generation
(64-token prompt prefilled in one chunk, then W untimed + K timed decode steps)
is one generation call (two persistent launches: the prefill program, then the
decode program); step times are globaltimer stamps the kernel records at each iteration
boundary, so `value` is the mean time per output token over the K timed steps
with everything resident in HBM.  `e2e` repeats the generation through the
public API from pinned host prompts to host tokens and divides the wall time by
the tokens generated (prompt iterations included).  Synthetic data: seeded
random weights N(0, 0.02) in bf16 and uniform-random prompts with the shapes of
the reference's benchmark (no checkpoint or tokenizer here).

Under torchrun (N > 1) the model is split tensor-parallel over the ranks; before
the timed region every rank runs a small tensor-parallel parity case against a
fixture produced by the unmodified reference model and rank 0 reports it in the
`parity` key.
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
# DRAM read+write bytes per step over the algorithmic bytes, from an ncu capture of a 4-layer case of
# the same kernel at batch 1 (dram__bytes_read.sum + dram__bytes_write.sum of one launch, divided by
# the launch's iterations); traffic grows in proportion to the bytes a step streams.
DRAM_TRAFFIC_RATIO = 1.004


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


def make_weights(g, device, seed=0, norm_jitter=0.0, std=0.02):
    """Seeded random-init weights in the fixed order embed, per layer q,k,v,o,gate,up,down, lm_head,
    then the norm weights (1.0, or 1 + U(-j, j) drawn in the order ln1, ln2, qn, kn per layer, final norm)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    w = {}
    for name, shape in weight_shapes(g):
        w[name] = (torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * std).to(torch.bfloat16)

    def norm(n):
        if norm_jitter == 0.0:
            return torch.ones(n, dtype=torch.bfloat16, device=device)
        u = torch.rand(n, generator=gen, dtype=torch.float32, device=device)
        return (1.0 + norm_jitter * (2 * u - 1)).to(torch.bfloat16)

    for i in range(g.layers):
        w[f"l{i}.ln1"] = norm(g.hidden)
        w[f"l{i}.ln2"] = norm(g.hidden)
        w[f"l{i}.qn"] = norm(g.head_dim)
        w[f"l{i}.kn"] = norm(g.head_dim)
    w["norm"] = norm(g.hidden)
    return w


def make_prompts(g, batch):
    out = []
    for r in range(batch):
        gen = torch.Generator().manual_seed(1000 + r)
        out.append(torch.randint(0, g.vocab, (PROMPT_LEN,), generator=gen, dtype=torch.int64))
    return out


def algorithmic_bytes(g, batch, ctx_lens, world=1, lm_head_sharded=False):
    """Weights read once + KV read/written + activations, per decode step and per GPU.  Under tensor
    parallelism the layer weights and the KV cache are split over the ranks; the LM head is either
    replicated (as in the reference, demo/qwen3/models/modeling_qwen3.py:514) or split by vocabulary rows."""
    per_layer = 2 * ((g.n_q + 2 * g.n_kv) * g.head_dim * g.hidden + g.hidden * g.n_q * g.head_dim +
                     2 * g.mlp * g.hidden + g.hidden * g.mlp) + 2 * (2 * g.hidden + 2 * g.head_dim)
    head = 2 * g.vocab * g.hidden + 2 * g.hidden
    kv_unit = 2 * g.layers * g.n_kv * g.head_dim * 2
    kv = sum(kv_unit * (L + 1) for L in ctx_lens)
    act = batch * (2 * g.vocab + 40 * g.hidden * 2)
    total = g.layers * per_layer / world + (head / world if lm_head_sharded else head) + kv / world + act
    return total, g.layers * per_layer + head


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


def cpu_baseline(g, w, threads=None, steps=8, warm=2):
    """The oracle's restatement of the reference PyTorch model on the host cores, at full depth:
    all layers + final norm + LM head, a 64-token multi-token prefill (as the reference's driver
    does, demo/qwen3/demo.py:1196-1212), then `warm` untimed and `steps` timed decode steps at batch 1."""
    from oracle import qwen3_oracle as O
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    geom = O.Geometry(hidden=g.hidden, n_q=g.n_q, n_kv=g.n_kv, mlp=g.mlp, layers=g.layers, vocab=g.vocab)
    wc = {k: v.cpu() for k, v in w.items()}
    m = O.TorchRefModel(geom, wc, PROMPT_LEN + warm + steps + 2)
    prompt = make_prompts(g, 1)[0]
    times = []
    with torch.inference_mode():
        lg = m.forward(prompt, 0)
        tok = int(lg[-1].argmax(-1))
        for s in range(warm + steps):
            t0 = time.perf_counter()
            lg = m.forward(torch.tensor([tok]), PROMPT_LEN + s)
            tok = int(lg[-1].argmax(-1))
            times.append(time.perf_counter() - t0)
    ms = statistics.mean(times[warm:]) * 1e3
    return {"value": ms, "unit": "ms/token", "cores": threads, "kind": "port",
            "sample": f"all {g.layers} layers + LM head, 64-token prefill, {warm} untimed then {steps} timed greedy "
                      f"decode steps at batch 1 (mean)"}


def fixture_parity(rank, world, dev, n_new=20):
    """A small tensor-parallel run held against the fixture the unmodified reference model produced
    (tests/golden/kv8_generate.pt: 16 q / 8 kv heads, so it splits over 2, 4 and 8 ranks): the
    fixture's prompt, its tokens forced after every step, logits compared in units of the step's
    largest |logit|, tokens wherever the reference's top-2 margin exceeds the tolerance."""
    import fleet_chiplet_megakernel_b200 as mk
    fx = torch.load(os.path.join(ROOT, "tests", "golden", "kv8_generate.pt"))
    gd = fx["geometry"]
    g = mk.Qwen3Geometry(hidden=gd["hidden"], n_q=gd["n_q"], n_kv=gd["n_kv"], mlp=gd["mlp"], layers=gd["layers"],
                         vocab=gd["vocab"])
    w = make_weights(g, "cpu", seed=fx["seed"], norm_jitter=fx["norm_jitter"], std=gd["init_std"])
    mine = mk.shard_qwen3_weights({k: v.to(dev) for k, v in w.items()}, world, rank)
    P = len(fx["prompt"])
    dec = mk.Qwen3Decoder(g, mine, max_seq_length=P + n_new + 1, max_requests=1, page_size=16, keep_logits=True,
                          max_iterations=1, world_size=world, rank=rank, device=dev)
    dec.set_prompts([fx["prompt"]])
    ref_tok, ref_lg = fx["tokens"], fx["logits"]
    worst, firm, firm_equal = 0.0, 0, 0
    for it in range(P + n_new - 1):
        dec.run()
        if it >= P - 1:
            j = it - (P - 1)
            ours = dec.logits[0].float().cpu()  # this rank's slice of the vocabulary (the LM head is sharded by rows)
            ref = ref_lg[j].float()
            scale = float(ref.abs().max())
            off = rank * ours.shape[0]
            worst = max(worst, float((ours - ref[off:off + ours.shape[0]]).abs().max()) / scale)
            top2 = ref.topk(2).values
            if float(top2[0] - top2[1]) > 2e-2 * scale:
                firm += 1
                firm_equal += int(int(dec.tokens[0, P + j]) == int(ref_tok[P + j]))
            dec.tokens[0, P + j] = int(ref_tok[P + j])
    dec.finalize()
    import torch.distributed as dist
    v = torch.tensor([worst, float(firm_equal == firm)], device=dev, dtype=torch.float64)
    dist.all_reduce(v[:1], op=dist.ReduceOp.MAX)   # every rank checked its own slice of the logits
    dist.all_reduce(v[1:], op=dist.ReduceOp.MIN)
    return {"world": world, "max_rel_err": float(v[0]), "tolerance": 2e-2, "steps": n_new, "firm_steps": firm,
            "firm_tokens_equal": bool(v[1] > 0.5), "fixture": "tests/golden/kv8_generate.pt (reference model output)"}


def prefill_iterations(batch, budget):
    """Iterations until every request decodes, replaying the scheduler's chunking on the host: per
    iteration the requests, in slot order, get their whole remaining prompt or what is left of the token
    budget (decoding ones one token), and new requests are admitted while budget remains."""
    step = [0] * batch
    admitted = 0
    it = 0
    while True:
        if admitted == batch and all(s >= PROMPT_LEN for s in step):
            return it
        it += 1
        ntok = 0
        for r in range(admitted):
            left = PROMPT_LEN - step[r]
            n = min(left, budget - ntok) if left > 0 else min(1, budget - ntok)
            step[r] += n
            ntok += n
        while admitted < batch and ntok < budget:
            n = min(PROMPT_LEN, budget - ntok)
            step[admitted] = n
            ntok += n
            admitted += 1


def timed_generation(mk, g, w, dev, B, K, W, numerics, world, rank, sampler=None, e2e=True):
    """One decoder at batch B: an untimed full pass, the measured pass (in-kernel stamps) and, if asked,
    the end-to-end pass from pinned host prompts to host tokens.  Prompts are prefilled in chunks (a token
    budget of 64 per iteration, 128 above batch 32); the timed steps are the last K iterations, in which
    every request decodes one token.  Returns a dict of timings."""
    budget = 64 if B <= 32 else 128
    n_pf = prefill_iterations(B, budget)
    iters = n_pf + W + K - 1
    prompts = make_prompts(g, B)
    dec = mk.Qwen3Decoder(g, w, max_seq_length=MAX_SEQ, max_requests=B, page_size=PAGE, device=dev,
                          max_iterations=iters, numerics=numerics, world_size=world, rank=rank,
                          max_num_batched_tokens=budget)
    torch.cuda.synchronize()
    dec.set_prompts(prompts)
    dec.run()
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()
        time.sleep(0.3)
    if world > 1:
        import torch.distributed as dist
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
    first = iters - K
    assert all(int(n) == B for n in stamps[first: iters, 1]), "a timed iteration is not a pure decode step"
    step_ns = t[first + 1: first + K + 1] - t[first: first + K]
    out = {"tpot_ms": float(step_ns.sum() / K / 1e6), "launch_ms": launch_ms, "iters": iters, "prefill_iters": n_pf,
           "budget": budget, "prefill_ms": float((t[n_pf] - t[0]) / 1e6),
           "median_ms": float(statistics.median(step_ns.tolist()) / 1e6),
           "first_tenth_ms": float(step_ns[: max(1, K // 10)].mean() / 1e6),
           "last_tenth_ms": float(step_ns[-max(1, K // 10):].mean() / 1e6), "grid": dec.mpk.grid_size()}
    if e2e:
        host_prompts = [p.pin_memory() for p in prompts]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        dec.set_prompts(host_prompts)
        dec.run()
        out["tokens"] = dec.tokens[:, : PROMPT_LEN + W + K].to("cpu", non_blocking=False)
        out["e2e_ms"] = (time.perf_counter() - t0) * 1e3 / (W + K)
    dec.finalize()
    return out


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
    assert PROMPT_LEN + W + K + 1 <= MAX_SEQ, "steps + warmup exceed the 1200-token sequence limit"
    parity = None
    if world > 1 and not args.no_parity:
        parity = fixture_parity(rank, world, dev)
    w_full = make_weights(g, dev)
    w = w_full
    if world > 1:
        # tensor parallel: every rank draws the same seeded weights and keeps its shard
        w = mk.shard_qwen3_weights(w_full, world, rank)
        del w_full
        torch.cuda.empty_cache()
    sampler = ClockSampler(local)
    main = timed_generation(mk, g, w, dev, B, K, W, args.numerics, world, rank, sampler=sampler)
    clocks = sampler.stop()
    tpot_ms, e2e_ms = main["tpot_ms"], main["e2e_ms"]
    tokens_same = True
    if world > 1:
        v = torch.tensor([tpot_ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        tpot_ms, e2e_ms = float(v[0]), float(v[1])
        # every rank must have generated the same tokens
        mine = main["tokens"].to(dev)
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        tokens_same = bool(torch.equal(lo, hi))
    # context of the last request admitted (the earlier ones are up to prefill_iters tokens further: negligible)
    ctx = [PROMPT_LEN + W + j for j in range(K)]
    mean_bytes = statistics.mean(algorithmic_bytes(g, B, [L] * B, world, lm_head_sharded=True)[0] for L in ctx)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = mean_bytes / (tpot_ms * 1e-3) / 1e9
    traffic = DRAM_TRAFFIC_RATIO * mean_bytes if B <= 8 else None

    def frac_of(ms, batch, steps, warm):
        c = [PROMPT_LEN + warm + j for j in range(steps)]
        mb = statistics.mean(algorithmic_bytes(g, batch, [L] * batch, world, lm_head_sharded=True)[0] for L in c)
        return mb / (ms * 1e-3) / 1e9 / peak

    extra = {}
    if world == 1 and not args.no_sweep and B == 1:
        # config 3: the batch sweep, a short run per batch size (its own decoder: the path follows the batch)
        sweep = {"1": {"tpot_ms": tpot_ms, "frac": achieved / peak, "steps": K}}
        for b in (2, 4, 8, 16, 32, 64):
            r = timed_generation(mk, g, w, dev, b, args.sweep_steps, 3, args.numerics, 1, 0, e2e=False)
            sweep[str(b)] = {"tpot_ms": r["tpot_ms"], "frac": frac_of(r["tpot_ms"], b, args.sweep_steps, 3),
                             "steps": args.sweep_steps}
        extra["sweep"] = sweep
    if world > 1 and args.also_batch > 1 and B == 1:
        # config 4 names batch 1 and batch 32 under tensor parallelism
        b = args.also_batch
        ks = min(K, 32)
        r = timed_generation(mk, g, w, dev, b, ks, 3, args.numerics, world, rank, e2e=False)
        v = torch.tensor([r["tpot_ms"]], device=dev, dtype=torch.float64)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        extra[f"batch{b}"] = {"tpot_ms": float(v[0]), "frac": frac_of(float(v[0]), b, ks, 3), "steps": ks,
                              "tokens_per_s": b * 1e3 / float(v[0])}
    line = {
        "metric": METRIC, "value": tpot_ms, "unit": "ms/token", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": tpot_ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded random weights N(0,0.02), uniform-random 64-token prompts)",
        "config": {"workload": f"Qwen3-8B geometry, {g.layers} layers, vocab {g.vocab}, batch {B}, 64-token prompt, "
                               f"{K} greedy decode steps, paged KV (page 64), max seq 1200",
                   "batch": B, "l2": "inputs larger than L2 (15.1 GB of weights per step)",
                   "timing": "globaltimer stamp per iteration inside the single persistent launch",
                   "numerics": args.numerics, "grid": main["grid"],
                   "parallelism": f"tp{world} (heads, MLP columns and LM-head vocabulary rows split)" if world > 1 else "single GPU",
                   "launch_ms_total": main["launch_ms"], "iterations": main["iters"],
                   "prefill": f"chunked, {main['budget']} tokens per iteration: {main['prefill_iters']} iteration(s), "
                              f"{main['prefill_ms']:.2f} ms"},
        "tokens_per_s": B * 1e3 / tpot_ms,
        "tpot_median_ms": main["median_ms"],
        "tpot_first_tenth_ms": main["first_tenth_ms"], "tpot_last_tenth_ms": main["last_tenth_ms"],  # context grows during the run
        "clocks": clocks,
        "e2e": {"value": e2e_ms, "unit": "ms/token", "h2d_bytes_per_step": B * PROMPT_LEN * 8 / (W + K),
                "d2h_bytes_per_step": B * (PROMPT_LEN + W + K) * 8 / (W + K),
                "note": "wall time of set_prompts (H2D) + launch (chunked prefill + decode) + token readback, "
                        "per generated token"},
        "gpu_launches": 2,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "algorithmic_bytes_per_step": mean_bytes, "per": "GPU",
                     "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback",
                     "frac_of_nominal_8TBps": achieved / 8000.0},
    }
    line.update(extra)
    if world > 1:
        line["parity"] = parity
        line["ranks_generated_identical_tokens"] = tokens_same
    if rank == 0:
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(g, w)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    assert tokens_same, "the tensor-parallel ranks generated different tokens"
    return main.get("tokens")


def run_moe(args):
    """Config 5 of the benchmark list, single GPU, batch 1: Qwen3-30B-A3B geometry (48 layers, hidden 2048, 32 q /
    4 kv heads, 128 experts, top-8, expert MLP 768), seeded random weights, 64-token prompt, greedy decode.  The
    expert layers are built for one or two batched tokens and one GPU; prompts advance one token per iteration."""
    import fleet_chiplet_megakernel_b200 as mk
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    g = mk.Qwen3MoeGeometry(layers=args.layers if args.layers != 36 else 48)
    K, W = args.steps, args.warmup
    gen = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, std=0.02):
        return (torch.randn(shape, generator=gen, dtype=torch.float32, device=dev) * std).to(torch.bfloat16)

    w = {"embed": rnd(g.vocab, g.hidden), "lm_head": rnd(g.vocab, g.hidden), "norm": torch.ones(g.hidden, dtype=torch.bfloat16, device=dev)}
    for i in range(g.layers):
        w[f"l{i}.q"], w[f"l{i}.k"], w[f"l{i}.v"] = rnd(g.n_q * 128, g.hidden), rnd(g.n_kv * 128, g.hidden), rnd(g.n_kv * 128, g.hidden)
        w[f"l{i}.o"] = rnd(g.hidden, g.n_q * 128)
        w[f"l{i}.router"] = rnd(g.experts, g.hidden, std=2.0 / g.hidden ** 0.5)
        w[f"l{i}.w13"], w[f"l{i}.w2"] = rnd(g.experts, 2 * g.moe_mlp, g.hidden), rnd(g.experts, g.hidden, g.moe_mlp)
        for n, d in (("ln1", g.hidden), ("ln2", g.hidden), ("qn", 128), ("kn", 128)):
            w[f"l{i}.{n}"] = torch.ones(d, dtype=torch.bfloat16, device=dev)
    iters = PROMPT_LEN + W + K - 1
    dec = mk.Qwen3MoeDecoder(g, w, max_seq_length=MAX_SEQ, max_requests=1, page_size=PAGE, device=dev, max_iterations=iters,
                             numerics="mpk")
    prompt = make_prompts(g, 1)
    for _ in range(2):
        dec.set_prompts(prompt)
        dec.run()
    torch.cuda.synchronize()
    stamps = dec.mpk.get_event_timing()
    t = stamps[:, 0].astype("float64")
    first = iters - K
    step_ns = t[first + 1: first + K + 1] - t[first: first + K]
    tpot_ms = float(step_ns.sum() / K / 1e6)
    t0 = time.perf_counter()
    dec.set_prompts([p.pin_memory() for p in prompt])
    dec.run()
    toks = dec.tokens[:, : PROMPT_LEN + W + K].cpu()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / (W + K)
    per_layer = 2 * ((g.n_q + 2 * g.n_kv) * 128 * g.hidden + g.hidden * g.n_q * 128 + g.experts * g.hidden +
                     g.top_k * 3 * g.moe_mlp * g.hidden) + 2 * (2 * g.hidden + 256)
    ctx = PROMPT_LEN + W + K // 2
    nbytes = g.layers * per_layer + 2 * g.vocab * g.hidden + 2 * g.layers * g.n_kv * 128 * 2 * (ctx + 1)
    peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("hbm_gbs", 6650.0)) if \
        os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else 6650.0
    ach = nbytes / (tpot_ms * 1e-3) / 1e9
    print(json.dumps({"metric": "Qwen3-30B-A3B bf16 MoE decode TPOT", "value": tpot_ms, "unit": "ms/token", "n_gpus": 1, "steps": K,
                      "warmup": W, "ms_per_step": tpot_ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
                      "dtype": "bf16", "data": "synthetic (seeded random weights, uniform-random 64-token prompt)",
                      "config": {"workload": f"Qwen3-30B-A3B geometry, {g.layers} layers, {g.experts} experts top-{g.top_k}, batch 1, "
                                             f"64-token prompt, {K} greedy decode steps, single GPU", "batch": 1,
                                 "l2": "inputs larger than L2 (6 GB of weights per step)", "grid": dec.mpk.grid_size()},
                      "e2e": {"value": e2e_ms, "unit": "ms/token", "h2d_bytes_per_step": PROMPT_LEN * 8 / (W + K),
                              "d2h_bytes_per_step": toks.numel() * 8 / (W + K)},
                      "gpu_launches": 2,
                      "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                                   "traffic": None, "algorithmic_bytes_per_step": nbytes}}), flush=True)
    dec.finalize()


def run_reference(args):
    """The reference's own CPU implementation of the path (its PyTorch model, restated in
    oracle/), timed on the host cores with all threads: the full-depth model, a 64-token prefill
    and a bounded number of greedy decode steps."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    g = geometry(args.layers)
    dev = "cuda" if torch.cuda.is_available() else "cpu"  # only to draw the seeded weights quickly
    w = make_weights(g, dev)
    steps = max(8, min(args.steps, 16))
    base = cpu_baseline(g, w, steps=steps, warm=min(max(args.warmup, 1), 3))
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": "ms/token",
            "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": base["value"], "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded random weights N(0,0.02), uniform-random 64-token prompts)",
            "config": {"workload": f"Qwen3-8B geometry, {g.layers} layers, vocab {g.vocab}, batch 1, 64-token prompt, "
                                   f"{steps} greedy decode steps on the host cores", "batch": 1},
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
    ap.add_argument("--model", default="dense", choices=["dense", "moe"], help="dense: Qwen3-8B geometry (the headline); moe: Qwen3-30B-A3B geometry, batch 1")
    ap.add_argument("--numerics", default="torch", choices=["torch", "mpk"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sweep", action="store_true", help="skip the batch sweep (single GPU)")
    ap.add_argument("--sweep-steps", type=int, default=20)
    ap.add_argument("--no-parity", action="store_true", help="skip the tensor-parallel parity case (N > 1)")
    ap.add_argument("--also-batch", type=int, default=32, help="second batch size timed under tensor parallelism (0: none)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    elif args.model == "moe":
        run_moe(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
