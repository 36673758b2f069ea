"""Tensor-parallel decode on 2 GPUs of one box: one process per GPU, weights sharded by
heads / MLP columns, the two allreduces per layer done inside the megakernel over NVLink
peer memory.  Teacher-forced logits and tokens against the reference fixture.  Skipped
with fewer than 2 GPUs."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from oracle import qwen3_oracle as O

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, ws, port, fixture, n_new, ret):
    import torch.distributed as dist
    import fleet_chiplet_megakernel_b200 as mk
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    fx = torch.load(os.path.join(GOLD, fixture))
    geom = O.Geometry(**fx["geometry"])
    w = O.make_weights(geom, fx["seed"], norm_jitter=fx["norm_jitter"])
    g = mk.Qwen3Geometry(hidden=geom.hidden, n_q=geom.n_q, n_kv=geom.n_kv, mlp=geom.mlp, layers=geom.layers,
                         vocab=geom.vocab)
    mine = mk.shard_qwen3_weights({k: v.cuda() for k, v in w.items()}, ws, rank)
    P = len(fx["prompt"])
    dec = mk.Qwen3Decoder(g, mine, max_seq_length=P + n_new + 1, max_requests=1, page_size=16, keep_logits=True,
                          max_iterations=1, world_size=ws, rank=rank, device=f"cuda:{rank}", timeout_ms=3000)
    dec.set_prompts([fx["prompt"]])
    logits, toks = [], []
    ref = fx["tokens"]
    for it in range(P + n_new - 1):
        dec.run()
        if it >= P - 1:
            j = it - (P - 1)
            logits.append(dec.logits[0].clone().cpu())
            toks.append(int(dec.tokens[0, P + j]))
            dec.tokens[0, P + j] = int(ref[P + j])
    dec.finalize()
    ret[rank] = (torch.stack(logits), toks)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("fixture", ["tiny_generate.pt", "small_generate.pt"])
def test_tp2_matches_reference_fixture(fixture):
    ws, n_new = 2, 24
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(ws, _free_port(), fixture, n_new, ret), nprocs=ws, join=True)
    fx = torch.load(os.path.join(GOLD, fixture))
    l0, t0 = ret[0]
    l1, t1 = ret[1]
    assert torch.equal(l0, l1) and t0 == t1, "ranks disagree on logits or tokens"
    # Against the single-GPU PyTorch fixture the tensor-parallel run carries one more bf16
    # rounding per row-parallel linear (the partial sums cross NVLink as bf16, as the
    # reference's allreduce on bf16 task outputs does), on top of a comparison whose noise
    # floor is already 0.0196: the fixture's own model re-run with fp64 linears.  Hence
    # 2.5e-2 here instead of the single-GPU tests' 2e-2; the tokens are still held to the
    # fixture wherever its top-2 margin exceeds 2e-2.
    err = O.max_rel_err(l0, fx["logits"][:n_new])
    assert err <= 2.5e-2, err
    P = len(fx["prompt"])
    scale = fx["logits"][:n_new].float().abs().amax(-1)
    margin = O.top2_margin(fx["logits"][:n_new])
    for j in range(n_new):
        if margin[j] > 2e-2 * scale[j]:
            assert t0[j] == int(fx["tokens"][P + j]), f"step {j}"
    print(f"TP=2 {fixture}: max logit error {err:.4g}")
