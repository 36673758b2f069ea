"""Per-op time breakdown of one decode iteration, from the kernel's own trace.

  python -m fleet_chiplet_megakernel_b200.op_trace [--layers 36] [--batch 1] [--context 100]

Runs a seeded random-weight Qwen3-8B-geometry decode with a profiler tensor attached
(the reference's ``profiler_tensor`` argument, persistent_kernel.py:361-362), then prints,
per kind of device op, how long the CTAs waited at the op's barrier and how long the op
body took (mean and slowest CTA), all from ``%globaltimer`` stamps taken inside the
single persistent launch.  Tracing costs a few percent; the step time printed first is
measured with tracing on.
"""
import argparse
import collections

import torch

from . import Qwen3Decoder, Qwen3Geometry, Qwen3MoeDecoder, Qwen3MoeGeometry


def random_weights(g: Qwen3Geometry, device, seed=0):
    gen = torch.Generator(device=device).manual_seed(seed)

    def w(*shape):
        return (torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * 0.02).to(torch.bfloat16)

    d = g.head_dim
    out = {"embed": w(g.vocab, g.hidden), "lm_head": w(g.vocab, g.hidden),
           "norm": torch.ones(g.hidden, dtype=torch.bfloat16, device=device)}
    for i in range(g.layers):
        out[f"l{i}.q"], out[f"l{i}.k"], out[f"l{i}.v"] = w(g.n_q * d, g.hidden), w(g.n_kv * d, g.hidden), w(g.n_kv * d, g.hidden)
        out[f"l{i}.o"], out[f"l{i}.gate"], out[f"l{i}.up"] = w(g.hidden, g.n_q * d), w(g.mlp, g.hidden), w(g.mlp, g.hidden)
        out[f"l{i}.down"] = w(g.hidden, g.mlp)
        for n, k in (("ln1", g.hidden), ("ln2", g.hidden), ("qn", d), ("kn", d)):
            out[f"l{i}.{n}"] = torch.ones(k, dtype=torch.bfloat16, device=device)
    return out


def random_moe_weights(g: Qwen3MoeGeometry, device, seed=0):
    gen = torch.Generator(device=device).manual_seed(seed)

    def w(*shape, std=0.02):
        return (torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * std).to(torch.bfloat16)

    d = g.head_dim
    out = {"embed": w(g.vocab, g.hidden), "lm_head": w(g.vocab, g.hidden),
           "norm": torch.ones(g.hidden, dtype=torch.bfloat16, device=device)}
    for i in range(g.layers):
        out[f"l{i}.q"], out[f"l{i}.k"], out[f"l{i}.v"] = w(g.n_q * d, g.hidden), w(g.n_kv * d, g.hidden), w(g.n_kv * d, g.hidden)
        out[f"l{i}.o"] = w(g.hidden, g.n_q * d)
        out[f"l{i}.router"] = w(g.experts, g.hidden, std=2.0 / g.hidden ** 0.5)
        out[f"l{i}.w13"], out[f"l{i}.w2"] = w(g.experts, 2 * g.moe_mlp, g.hidden), w(g.experts, g.hidden, g.moe_mlp)
        for n, k in (("ln1", g.hidden), ("ln2", g.hidden), ("qn", d), ("kn", d)):
            out[f"l{i}.{n}"] = torch.ones(k, dtype=torch.bfloat16, device=device)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="dense", choices=["dense", "moe"],
                    help="dense: Qwen3-8B geometry; moe: Qwen3-30B-A3B geometry (batch 1; give --layers, 48 layers hold 60 GB)")
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=100, help="tokens in the KV cache at the traced iteration")
    ap.add_argument("--cluster", type=int, default=0, help="CTAs per cluster for the hierarchical grid barrier (0/1: flat)")
    ap.add_argument("--debug-flags", type=int, default=0,
                    help="measurement switches of the library (16: no tagged activations, every op keeps its grid barrier)")
    args = ap.parse_args()
    dev = torch.device("cuda")
    prompt_len = 16
    iters = args.context
    if args.model == "moe":
        g = Qwen3MoeGeometry(layers=args.layers)
        dec = Qwen3MoeDecoder(g, random_moe_weights(g, dev), max_seq_length=max(1200, iters + 8), max_requests=1, page_size=64,
                              device=dev, max_iterations=iters, trace=True)
        args.batch = 1
    else:
        g = Qwen3Geometry(layers=args.layers)
        w = random_weights(g, dev)
        dec = Qwen3Decoder(g, w, max_seq_length=max(1200, iters + 8), max_requests=args.batch, page_size=64,
                           max_iterations=iters, trace=True, cluster_size=args.cluster, debug_flags=args.debug_flags)
    gen = torch.Generator().manual_seed(1000)
    prompts = [torch.randint(0, g.vocab, (prompt_len,), generator=gen) for _ in range(args.batch)]
    for _ in range(2):
        dec.set_prompts(prompts)
        dec.run()
    st = dec.mpk.get_event_timing()[:, 0].astype("float64")
    n_tail = min(20, len(st) - 1)
    print(f"step time with tracing on: {(st[-1] - st[-1 - n_tail]) / n_tail / 1e6:.3f} ms "
          f"(batch {args.batch}, context ~{iters}, {args.layers} layers, grid {dec.mpk.grid_size()}, cluster {max(1, args.cluster)})")
    tr = dec.mpk.op_trace().double()  # [ops + 1, grid, 4]
    n = tr.shape[0] - 1
    # label every device op by its kind and shape, e.g. "linear 6144x4096" (QKV), "attention"
    names = []
    for line in dec.mpk.describe().strip().splitlines():
        f = line.split()
        kv = dict(x.split("=", 1) for x in f[2:] if "=" in x)
        names.append(f"{f[1]} {kv['n']}x{kv['k']}" if "linear" in f[1] else f[1])
    assert len(names) == n, (len(names), n)
    agg = collections.OrderedDict()
    for i in range(n):
        reach, passed, done = tr[i, :, 0], tr[i, :, 1], tr[i, :, 2]
        a = agg.setdefault(names[i], [0, 0.0, 0.0, 0.0, 0.0])
        a[0] += 1
        a[1] += float(passed.max() - reach.min())   # first CTA at the barrier -> barrier open
        a[2] += float(passed.max() - reach.max())   # last CTA at the barrier -> barrier open
        a[3] += float((done - passed).mean())
        a[4] += float((done - passed).max())
    print(f"{'op':22s} {'count':>5s} {'first arrival -> open':>22s} {'last arrival -> open':>21s} {'body mean':>10s} {'body max':>9s}   (us per op)")
    total = 0.0
    for k, a in agg.items():
        c = a[0]
        print(f"{k:22s} {c:5d} {a[1] / c / 1e3:22.2f} {a[2] / c / 1e3:21.2f} {a[3] / c / 1e3:10.2f} {a[4] / c / 1e3:9.2f}")
        total += a[2] + a[4]
    print(f"sum of (last arrival -> open) + (slowest body): {total / 1e6:.3f} ms per iteration")
    dec.finalize()


if __name__ == "__main__":
    main()
