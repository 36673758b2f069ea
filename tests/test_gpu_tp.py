"""Tensor-parallel decode on 2, 4 and 8 GPUs of one box: one process per GPU, weights sharded by
heads / MLP columns, the two allreduces per layer folded into the row-parallel linears' epilogues
(fp32 partial sums pushed over NVLink peer memory) and the next layers' input staging.
Teacher-forced logits and tokens against the fixtures the unmodified reference model produced,
at the single-GPU tolerance.  Each case is skipped where the box has fewer GPUs."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from oracle import qwen3_oracle as O

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL = 2e-2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def tp_teacher_forced(rank, ws, fixture, n_new, batch=1, fuse=True, device=None):
    """Runs on every rank (process group already initialised): the fixture's prompt in `batch`
    identical requests, the reference's tokens forced after every iteration.  Returns this rank's
    per-step logits [n_new, batch, its slice of the vocabulary] (the LM head is sharded by vocabulary
    rows), the greedy tokens [n_new][batch] all ranks agreed on, the device-op list and the slice's start."""
    import fleet_chiplet_megakernel_b200 as mk
    fx = torch.load(os.path.join(GOLD, fixture))
    geom = O.Geometry(**fx["geometry"])
    w = O.make_weights(geom, fx["seed"], norm_jitter=fx["norm_jitter"])
    g = mk.Qwen3Geometry(hidden=geom.hidden, n_q=geom.n_q, n_kv=geom.n_kv, mlp=geom.mlp, layers=geom.layers,
                         vocab=geom.vocab)
    dev = device or f"cuda:{rank}"
    mine = mk.shard_qwen3_weights({k: v.to(dev) for k, v in w.items()}, ws, rank)
    P = len(fx["prompt"])
    dec = mk.Qwen3Decoder(g, mine, max_seq_length=P + n_new + 1, max_requests=batch, page_size=16, keep_logits=True,
                          max_iterations=1, world_size=ws, rank=rank, device=dev, timeout_ms=3000, fuse=fuse,
                          max_tokens_per_request=1)
    dec.set_prompts([fx["prompt"]] * batch)
    logits, toks = [], []
    ref = fx["tokens"]
    for it in range(P + n_new - 1):
        dec.run()
        if it >= P - 1:
            j = it - (P - 1)
            logits.append(dec.logits.clone().cpu())
            toks.append([int(dec.tokens[r, P + j]) for r in range(batch)])
            dec.tokens[:, P + j] = int(ref[P + j])
    plan = dec.mpk.describe()
    dec.finalize()
    return torch.stack(logits), toks, plan, rank * mine["lm_head"].shape[0]


def check_tp_result(fixture, n_new, shards, toks):
    """shards: per rank (logits [n_new, batch, slice], first vocabulary index of the slice); toks [n_new][batch].
    Against the fixture: max error in units of the step's largest |logit| (over the whole vocabulary), tokens
    identical wherever the reference's top-2 margin is firm."""
    fx = torch.load(os.path.join(GOLD, fixture))
    ref = fx["logits"][:n_new]
    P = len(fx["prompt"])
    scale = ref.float().abs().amax(-1)
    margin = O.top2_margin(ref)
    worst, firm = 0.0, 0
    covered = sum(lg.shape[-1] for lg, _ in shards)
    assert covered == ref.shape[-1] or all(off == 0 for _, off in shards), "the ranks' slices must cover the vocabulary"
    for lg, off in shards:
        for b in range(lg.shape[1]):
            d = (lg[:, b].float() - ref[:, off:off + lg.shape[-1]].float()).abs().amax(-1) / scale
            worst = max(worst, float(d.max()))
    for b in range(len(toks[0])):
        for j in range(n_new):
            if margin[j] > TOL * scale[j]:
                firm += 1
                assert toks[j][b] == int(fx["tokens"][P + j]), f"step {j} request {b}"
    return worst, firm


def _worker(rank, ws, port, fixture, n_new, batch, fuse, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    ret[rank] = tp_teacher_forced(rank, ws, fixture, n_new, batch=batch, fuse=fuse)
    dist.barrier()
    dist.destroy_process_group()


def _run(ws, fixture, n_new, batch=1, fuse=True, tol=TOL):
    if torch.cuda.device_count() < ws:
        pytest.skip(f"needs {ws} GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(ws, _free_port(), fixture, n_new, batch, fuse, ret), nprocs=ws, join=True)
    l0, t0, plan, _ = ret[0]
    for r in range(1, ws):
        assert ret[r][1] == t0, f"rank {r} disagrees with rank 0 on the tokens"
    err, firm = check_tp_result(fixture, n_new, [(ret[r][0], ret[r][3]) for r in range(ws)], t0)
    assert err <= tol, f"TP={ws} {fixture}: logits off by {err:.4g}"
    print(f"TP={ws} batch {batch} {fixture}: max logit error {err:.4g}, {firm} firm token checks")
    return plan


@pytest.mark.parametrize("fixture", ["tiny_generate.pt", "small_generate.pt"])
def test_tp2_matches_reference_fixture(fixture):
    plan = _run(2, fixture, 24)
    kinds = [ln.split()[1] for ln in plan.strip().splitlines()]
    assert "allreduce folded" in plan and "allreduce" not in kinds  # no stand-alone exchange op is left
    assert "exchanged between the ranks" in plan  # the LM head is sharded by vocabulary rows


@pytest.mark.parametrize("ws", [2, 4, 8])
def test_tp_kv8_matches_reference_fixture(ws):
    _run(ws, "kv8_generate.pt", 32)


@pytest.mark.parametrize("batch", [4, 20])
def test_tp2_wider_batches(batch):
    """The stream-K (mma.sync) and tcgen05 paths under tensor parallelism: the rmsnorm task gathers."""
    _run(2, "kv8_generate.pt", 12, batch=batch)


def test_tp2_stand_alone_allreduce_op():
    """fuse=False keeps every layer as recorded: the allreduce runs as its own device op on the bf16
    outputs of the row-parallel linears, as the reference's allreduce task does
    (tasks/ampere/reduction.cuh:139-166).  That is one more bf16 rounding per exchange than the
    single-GPU model has, hence the wider bound here (the folded path above meets 2e-2)."""
    plan = _run(2, "tiny_generate.pt", 12, fuse=False, tol=2.5e-2)
    assert "allreduce" in [ln.split()[1] for ln in plan.strip().splitlines()]
