"""Tensor-parallel host logic on CPU: two gloo ranks shard the weights the way the
megakernel's driver does, compute their partial layer outputs with the oracle's task
arithmetic (residual contributed by rank 0 only, as the reference's row-parallel linears
do, src/kernel/task_register.cc:553-555) and all-reduce them; the sum must equal the
unsharded layer.  No GPU."""
import ctypes as C
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fleet_chiplet_megakernel_b200.qwen3_graph import shard_qwen3_weights
from oracle import qwen3_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _partial_layer(geom, w, x, pos, ws, rank, kc, vc):
    """One decoder layer on rank `rank` of `ws`; returns the two pre-allreduce partial tensors
    given the already reduced inputs (x for attention, x_mid for the MLP is reduced by the caller)."""
    d = geom.head_dim
    n_q, n_kv = geom.n_q // ws, geom.n_kv // ws
    xn = O.mpk_rmsnorm(x, w["l0.ln1"], geom.eps)
    q = O.mpk_linear(xn, w["l0.q"]).view(n_q, d)
    k = O.mpk_linear(xn, w["l0.k"]).view(n_kv, d)
    v = O.mpk_linear(xn, w["l0.v"]).view(n_kv, d)
    q = O.mpk_qk_norm_rope(q, w["l0.qn"], kc["cos"][pos], kc["sin"][pos], geom.eps)
    k = O.mpk_qk_norm_rope(k, w["l0.kn"], kc["cos"][pos], kc["sin"][pos], geom.eps)
    a = O.mpk_attention_decode(q, k[None], v[None]).reshape(-1)  # context of one token
    return O.mpk_linear(a, w["l0.o"], residual=x if rank == 0 else None)


def _worker(rank, ws, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    geom = O.Geometry(hidden=512, n_q=4, n_kv=2, mlp=1024, layers=1, vocab=64)
    full = O.make_weights(geom, 0, norm_jitter=0.25)
    mine = shard_qwen3_weights(full, ws, rank)
    assert mine["l0.q"].shape[0] == geom.n_q * 128 // ws and mine["l0.o"].shape[1] == geom.n_q * 128 // ws
    assert mine["l0.gate"].shape[0] == geom.mlp // ws and mine["l0.down"].shape[1] == geom.mlp // ws
    assert mine["embed"] is full["embed"]
    g = torch.Generator().manual_seed(3)
    x = torch.randn(geom.hidden, generator=g).to(O.BF16)
    cos, sin = O.rope_tables(geom, 8)
    part = _partial_layer(geom, mine, x, 0, ws, rank, {"cos": cos, "sin": sin}, None).float()
    dist.all_reduce(part)  # fp32 sum over ranks
    x1 = part.to(O.BF16)
    # MLP half
    xn = O.mpk_rmsnorm(x1, mine["l0.ln2"], geom.eps)
    h = O.mpk_silu_mul(O.mpk_linear(xn, mine["l0.gate"]), O.mpk_linear(xn, mine["l0.up"]))
    part2 = O.mpk_linear(h, mine["l0.down"], residual=x1 if rank == 0 else None).float()
    dist.all_reduce(part2)
    if rank == 0:
        ref = O.MpkRefModel(geom, full, 8)
        want = ref.layer(0, x, 0)
        ret["err"] = O.max_rel_err(part2.to(O.BF16)[None], want[None])
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_and_rank0_residual_sum_to_the_full_layer():
    ws = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(ws, _free_port(), ret), nprocs=ws, join=True)
    assert ret["err"] < 2e-2, ret["err"]


def test_exchange_sequence_survives_long_launches_and_the_32_bit_wrap(native_lib):
    """Exchange numbers keep growing across launches by the number of exchanges each launch really ran
    (72 per iteration for a 36-layer model): consecutive exchanges alternate between the halves of the
    region, and nothing a slot can still hold from its earlier uses is mistaken for the awaited number,
    through a 20 000-iteration launch and across the 32-bit wrap."""
    lib = native_lib
    seq, word, stale = C.c_uint32(), C.c_int64(), C.c_int()
    world, tokens, cols = 8, 4, 4096
    half_words = world * tokens * cols
    for total in (0, 5, 2**20 - 3, 2**32 - 72 * 10_000 - 7):   # the last one wraps in the middle of the launch
        prev_half = None
        launch = 72 * 20_000
        # every exchange near the start, the end and the wrap; every 997th in between
        ks = set(range(1, 400)) | set(range(launch - 400, launch + 1)) | set(range(1, launch, 997))
        wrap_k = (2**32 - total) % 2**32
        ks |= {k for k in range(max(1, wrap_k - 200), wrap_k + 200) if 1 <= k <= launch}
        last = None
        for k in sorted(ks):
            assert lib.mk_debug_exchange_sequence(total, k, world, tokens, cols, C.byref(seq), C.byref(word), C.byref(stale)) == 0
            assert seq.value == (total + k) % 2**32
            assert word.value == (seq.value & 1) * half_words
            assert stale.value == 0
            if last is not None and k == last + 1:
                assert (seq.value & 1) != prev_half, "consecutive exchanges must use different halves"
            prev_half, last = seq.value & 1, k
        # the next launch continues where this one stopped
        assert lib.mk_debug_exchange_sequence((total + launch) % 2**32, 1, world, tokens, cols, C.byref(seq), None, None) == 0
        assert seq.value == (total + launch + 1) % 2**32


def test_barrier_counter_comparison_is_wrap_safe(native_lib):
    lib = native_lib
    grid = 148
    for epoch in (1, 1000, 2**32 // grid - 1, 2**32 // grid, 2**32 // grid + 1, 2**31 // grid, 181 * 200_000):
        target = (epoch * grid) % 2**32
        assert lib.mk_barrier_target_reached(target, epoch, grid) == 1
        assert lib.mk_barrier_target_reached((target - 1) % 2**32, epoch, grid) == 0
        assert lib.mk_barrier_target_reached((target - grid) % 2**32, epoch, grid) == 0
        assert lib.mk_barrier_target_reached((target + 5) % 2**32, epoch, grid) == 1
