"""A device-side wait that runs out, by design, and what the host sees afterwards.

Two processes share GPU 0 as the two ranks of a tensor-parallel decoder.  Both compile
(exchange regions allocated, CUDA IPC handles swapped); then rank 1 never launches: it
stays on the host until rank 0 is finished.  Rank 0's megakernel reaches its first
allreduce, pushes its partial rows into the peer's region and waits for a sequence
number that nothing writes.  The wait is bounded (timeout_ms): the kernel records
{code, cta, op, iteration}, raises its abort flag, every CTA leaves, the launch returns
MK_E_DEVICE.  Nothing faults, traps or hangs: the context must still run kernels
afterwards.  Only one kernel is ever resident, so no two launches wait on each other."""
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


def _worker(rank, ws, port, ret):
    import time
    import torch.distributed as dist
    import fleet_chiplet_megakernel_b200 as mk
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(0)
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    fx = torch.load(os.path.join(GOLD, "tiny_generate.pt"))
    geom = O.Geometry(**fx["geometry"])
    w = O.make_weights(geom, fx["seed"], norm_jitter=fx["norm_jitter"])
    g = mk.Qwen3Geometry(hidden=geom.hidden, n_q=geom.n_q, n_kv=geom.n_kv, mlp=geom.mlp, layers=geom.layers,
                         vocab=geom.vocab)
    mine = mk.shard_qwen3_weights({k: v.cuda() for k, v in w.items()}, ws, rank)
    P = len(fx["prompt"])
    dec = mk.Qwen3Decoder(g, mine, max_seq_length=P + 4, max_requests=1, page_size=16, max_iterations=1,
                          world_size=ws, rank=rank, device="cuda:0", timeout_ms=400)
    dec.set_prompts([fx["prompt"]])
    if rank == 0:
        t0 = time.perf_counter()
        try:
            dec.run()
            ret["error"] = None
        except RuntimeError as e:
            ret["error"] = str(e)
        ret["seconds"] = time.perf_counter() - t0
        # the context is intact: an ordinary kernel still runs and gives the right answer
        ret["after"] = float((torch.arange(1000, device="cuda:0", dtype=torch.float32) * 2).sum())
    dist.barrier()  # rank 1 has been waiting here, on the host, all along
    dec.finalize()
    dist.destroy_process_group()


def test_peer_that_never_launches_ends_the_wait_cleanly():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret["error"] is not None, "the launch should have reported the missing rank"
    msg = ret["error"]
    assert "abort" in msg and "rank" in msg, msg
    assert "op" in msg and "cta" in msg, msg  # the decoded record says where it gave up
    assert 0.3 < ret["seconds"] < 5.0, ret["seconds"]
    assert ret["after"] == 999000.0
