"""Per-task parity on a B200: every device op of the megakernel, called through
the PersistentKernel mirror and the C ABI in single-pass mode, against the
oracle's restatement of the reference task arithmetic on the same seeded inputs."""
import math

import pytest
import torch

import fleet_chiplet_megakernel_b200 as mk
from oracle import qwen3_oracle as O
from tests.helpers import onepass_kernel, bf16_close

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(BF)


@pytest.mark.parametrize("T,N,K", [(1, 256, 512), (1, 6144, 4096), (2, 4096, 4096), (3, 384, 1024), (4, 4096, 12288),
                                   (1, 200, 264), (4, 136, 72), (7, 512, 512), (1, 64, 128)])
def test_linear_matches_oracle(T, N, K):
    x, w = _rand((T, K), 1), _rand((N, K), 2, 0.05)
    k, meta, _ = onepass_kernel(T)
    xd, wd = x.cuda(), w.cuda()
    od = torch.zeros(T, N, dtype=BF, device="cuda")
    k.linear_layer(input=k.attach_input(xd, "x"), weight=k.attach_input(wd, "w"), output=k.attach_input(od, "o"),
                   grid_dim=(max(1, N // 64), 1, 1), block_dim=(128, 1, 1))
    k.compile()
    k()
    bf16_close(od, O.mpk_linear(x, w), 1e-2, f"linear {T}x{N}x{K}")
    k()  # a compiled kernel is re-launchable
    bf16_close(od, O.mpk_linear(x, w), 1e-2, "linear, second launch")
    k.finalize()


@pytest.mark.parametrize("numerics", ["mpk", "torch"])
@pytest.mark.parametrize("T,N,K", [(1, 4096, 4096), (4, 512, 12288), (2, 328, 1024)])
def test_linear_with_residual(T, N, K, numerics):
    x, w, r = _rand((T, K), 3), _rand((N, K), 4, 0.05), _rand((T, N), 5)
    k, meta, _ = onepass_kernel(T, numerics=numerics)
    od = torch.zeros(T, N, dtype=BF, device="cuda")
    k.linear_with_residual_layer(input=k.attach_input(x.cuda(), "x"), weight=k.attach_input(w.cuda(), "w"),
                                 residual=k.attach_input(r.cuda(), "r"), output=k.attach_input(od, "o"),
                                 grid_dim=(max(1, N // 64), 1, 1), block_dim=(256, 1, 1))
    k.compile()
    k()
    ref = O.mpk_linear(x, w, residual=r) if numerics == "mpk" else (O.mpk_linear(x, w) + r)
    bf16_close(od, ref, 1e-2, "linear_with_residual")
    k.finalize()


@pytest.mark.parametrize("numerics", ["mpk", "torch"])
@pytest.mark.parametrize("fuse", [True, False])
@pytest.mark.parametrize("T", [2, 3])
def test_rmsnorm_then_linear(fuse, numerics, T):
    # the planner folds the norm into the linear for one or two batched tokens only
    N, K = 768, 1024
    x, wn, w = _rand((T, K), 6), (1 + 0.3 * _rand((K,), 7).float()).to(BF), _rand((N, K), 8, 0.05)
    k, meta, _ = onepass_kernel(T, fuse=fuse, numerics=numerics)
    od = torch.zeros(T, N, dtype=BF, device="cuda")
    mid = k.new_tensor(dims=(T, K), name="rmsnorm_out")
    k.rmsnorm_layer(input=k.attach_input(x.cuda(), "x"), weight=k.attach_input(wn.cuda(), "wn"), output=mid,
                    grid_dim=(T, 1, 1), block_dim=(128, 1, 1))
    k.linear_layer(input=mid, weight=k.attach_input(w.cuda(), "w"), output=k.attach_input(od, "o"),
                   grid_dim=(N // 64, 1, 1), block_dim=(128, 1, 1))
    assert len(k.plan().strip().splitlines()) == (1 if fuse and T <= 2 else 2)
    k.compile()
    k()
    xn = O.mpk_rmsnorm(x, wn) if numerics == "mpk" else O.ref_rmsnorm(x, wn)
    bf16_close(od, O.mpk_linear(xn, w), 1e-2, "rmsnorm+linear")
    k.finalize()


@pytest.mark.parametrize("numerics", ["mpk", "torch"])
@pytest.mark.parametrize("T,N,K", [(1, 768, 4096), (2, 640, 4096), (5, 768, 4096), (8, 256, 1024), (7, 384, 12288)])
def test_rmsnorm_linear_layer(T, N, K, numerics):
    # the reference's fused layer called directly (persistent_kernel.py:566): every CTA stages
    # and normalises the token rows itself; more rows than fit beside the weight ring take
    # several passes over the weights
    x, wn, w = _rand((T, K), 16), (1 + 0.3 * _rand((K,), 17).float()).to(BF), _rand((N, K), 18, 0.05)
    k, meta, _ = onepass_kernel(T, numerics=numerics)
    od = torch.zeros(T, N, dtype=BF, device="cuda")
    k.rmsnorm_linear_layer(input=k.attach_input(x.cuda(), "x"), weight_norm=k.attach_input(wn.cuda(), "wn"),
                           weight_linear=k.attach_input(w.cuda(), "w"), output=k.attach_input(od, "o"),
                           grid_dim=(N // 64, 1, 1), block_dim=(128, 1, 1))
    assert len(k.plan().strip().splitlines()) == 1
    k.compile()
    k()
    xn = O.mpk_rmsnorm(x, wn) if numerics == "mpk" else O.ref_rmsnorm(x, wn)
    bf16_close(od, O.mpk_linear(xn, w), 1e-2, "rmsnorm_linear")
    k.finalize()


@pytest.mark.parametrize("numerics", ["mpk", "torch"])
def test_rmsnorm_alone(numerics):
    T, K = 5, 4096
    x, wn = _rand((T, K), 9, 3.0), (1 + 0.3 * _rand((K,), 10).float()).to(BF)
    k, meta, _ = onepass_kernel(T, numerics=numerics)
    od = torch.zeros(T, K, dtype=BF, device="cuda")
    k.rmsnorm_layer(input=k.attach_input(x.cuda(), "x"), weight=k.attach_input(wn.cuda(), "wn"),
                    output=k.attach_input(od, "o"), grid_dim=(T, 1, 1), block_dim=(128, 1, 1))
    k.compile()
    k()
    ref = O.mpk_rmsnorm(x, wn) if numerics == "mpk" else O.ref_rmsnorm(x, wn)
    bf16_close(od, ref, 8e-3, "rmsnorm")
    k.finalize()


@pytest.mark.parametrize("fuse", [True, False])
def test_gate_up_silu_mul(fuse):
    T, K, I = 2, 512, 1024
    x, wg, wu = _rand((T, K), 11), _rand((I, K), 12, 0.05), _rand((I, K), 13, 0.05)
    k, meta, _ = onepass_kernel(T, fuse=fuse)
    od = torch.zeros(T, I, dtype=BF, device="cuda")
    groups = I // 128
    g, u = k.attach_input(wg.cuda(), "wg"), k.attach_input(wu.cuda(), "wu")
    wgu = k.shuffle_tensors([g, u], 0, groups, "wgu")
    mid = k.new_tensor(dims=(T, 2 * I), name="mlp_mid")
    k.linear_layer(input=k.attach_input(x.cuda(), "x"), weight=wgu, output=mid, grid_dim=(2 * I // 64, 1, 1),
                   block_dim=(128, 1, 1))
    k.silu_mul_layer(input=mid, output=k.attach_input(od, "o"), grid_dim=(groups, 1, 1), block_dim=(128, 1, 1))
    assert len(k.plan().strip().splitlines()) == (1 if fuse and T <= 2 else 2)
    k.compile()
    k()
    ref = O.mpk_silu_mul(O.mpk_linear(x, wg), O.mpk_linear(x, wu))
    bf16_close(od, ref, 1e-2, "gate/up + silu_mul")
    k.finalize()


@pytest.mark.parametrize("T,N,K", [(9, 512, 512), (16, 4096, 4096), (24, 384, 1024), (33, 1024, 12288), (64, 6144, 4096),
                                   (64, 200, 264), (12, 136, 72)])
def test_linear_wide_batches(T, N, K):
    """Above 8 tokens the activations ride along with the weight stages (16/32/64-row boxes)."""
    x, w, r = _rand((T, K), 31), _rand((N, K), 32, 0.05), _rand((T, N), 33)
    k, meta, _ = onepass_kernel(T)
    od = torch.zeros(T, N, dtype=BF, device="cuda")
    k.linear_with_residual_layer(input=k.attach_input(x.cuda(), "x"), weight=k.attach_input(w.cuda(), "w"),
                                 residual=k.attach_input(r.cuda(), "r"), output=k.attach_input(od, "o"),
                                 grid_dim=(max(1, N // 64), 1, 1), block_dim=(256, 1, 1))
    k.compile()
    k()
    bf16_close(od, O.mpk_linear(x, w, residual=r), 1e-2, f"wide linear {T}x{N}x{K}")
    k.finalize()


def test_wide_rmsnorm_gate_up_silu_mul():
    T, K, I = 20, 512, 1024
    x, wn = _rand((T, K), 34), (1 + 0.3 * _rand((K,), 35).float()).to(BF)
    wg, wu = _rand((I, K), 36, 0.05), _rand((I, K), 37, 0.05)
    k, meta, _ = onepass_kernel(T)
    od = torch.zeros(T, I, dtype=BF, device="cuda")
    groups = I // 128
    mid0 = k.new_tensor(dims=(T, K), name="rmsnorm_out")
    k.rmsnorm_layer(input=k.attach_input(x.cuda(), "x"), weight=k.attach_input(wn.cuda(), "wn"), output=mid0,
                    grid_dim=(T, 1, 1), block_dim=(128, 1, 1))
    wgu = k.shuffle_tensors([k.attach_input(wg.cuda(), "wg"), k.attach_input(wu.cuda(), "wu")], 0, groups, "wgu")
    mid = k.new_tensor(dims=(T, 2 * I), name="mlp_mid")
    k.linear_layer(input=mid0, weight=wgu, output=mid, grid_dim=(2 * I // 64, 1, 1), block_dim=(128, 1, 1))
    k.silu_mul_layer(input=mid, output=k.attach_input(od, "o"), grid_dim=(groups, 1, 1), block_dim=(128, 1, 1))
    assert [ln.split()[1] for ln in k.plan().strip().splitlines()] == ["rmsnorm", "linear"]
    k.compile()
    k()
    xn = O.mpk_rmsnorm(x, wn)
    bf16_close(od, O.mpk_silu_mul(O.mpk_linear(xn, wg), O.mpk_linear(xn, wu)), 1e-2, "wide norm + gate/up + silu")
    k.finalize()


def test_embedding_is_exact():
    T, V, H = 6, 1000, 512
    tab = _rand((V, H), 14)
    ids = torch.tensor([[3], [999], [0], [512], [3], [77]], dtype=torch.int64)
    k, meta, _ = onepass_kernel(T)
    meta["input_tokens"].copy_(ids)
    od = torch.zeros(T, H, dtype=BF, device="cuda")
    k.embed_layer(input=k.attach_input(meta["input_tokens"], "ids"), weight=k.attach_input(tab.cuda(), "tab"),
                  output=k.attach_input(od, "o"), grid_dim=(1, 1, 1), block_dim=(128, 1, 1), input_source=1)
    k.compile()
    k()
    assert torch.equal(od.cpu(), tab[ids[:, 0]])
    k.finalize()


def test_embedding_refuses_bad_token_id():
    T, V, H = 2, 100, 256
    k, meta, _ = onepass_kernel(T)
    meta["input_tokens"].copy_(torch.tensor([[5], [100]]))
    od = torch.zeros(T, H, dtype=BF, device="cuda")
    k.embed_layer(input=k.attach_input(meta["input_tokens"], "ids"), weight=k.attach_input(_rand((V, H), 15).cuda(), "tab"),
                  output=k.attach_input(od, "o"), grid_dim=(1, 1, 1), block_dim=(128, 1, 1), input_source=1)
    k.compile()
    with pytest.raises(RuntimeError, match="token id out of range"):
        k()
    k.finalize()


@pytest.mark.parametrize("V", [2048, 151936, 1000])
def test_argmax_lowest_index_wins_ties(V):
    T = 3
    lg = _rand((T, V), 16)
    lg[0, 17] = 50.0          # unique max
    lg[1, 900] = 60.0         # tie: the lower index must win
    lg[1, 333] = 60.0
    lg[2] = -5.0              # all equal: index 0
    k, meta, _ = onepass_kernel(T)
    out = meta["output_tokens"]
    k.argmax_layer(input=k.attach_input(lg.cuda(), "lg"), output=k.attach_input(out, "tok"), grid_dim=(1, 1, 1),
                   block_dim=(128, 1, 1))
    k.compile()
    k()
    assert out[:, 0].tolist() == [17, 333, 0]
    k.finalize()


def test_lm_head_with_fused_argmax():
    T, V, K = 2, 5000, 512
    x, w = _rand((T, K), 17), _rand((V, K), 18, 0.05)
    k, meta, _ = onepass_kernel(T)
    lg = torch.zeros(T, V, dtype=BF, device="cuda")
    lgt = k.attach_input(lg, "argmax_in")
    pv = k.new_tensor(dims=(T, 8), name="pv")
    pi = k.new_tensor(dims=(T, 8), dtype=mk.int64, name="pi")
    k.linear_layer(input=k.attach_input(x.cuda(), "x"), weight=k.attach_input(w.cuda(), "w"), output=lgt,
                   grid_dim=(8, 1, 1), block_dim=(128, 1, 1))
    k.argmax_partial_layer(input=lgt, output=(pv, pi), grid_dim=(8, 1, 1), block_dim=(128, 1, 1))
    k.argmax_reduce_layer(input=(pv, pi), output=k.attach_input(meta["output_tokens"], "tok"), grid_dim=(1, 1, 1),
                          block_dim=(128, 1, 1))
    assert "argmax partials fused" in k.plan()
    k.compile()
    k()
    ref = O.mpk_linear(x, w)
    bf16_close(lg, ref, 1e-2, "lm head")
    assert meta["output_tokens"][:, 0].tolist() == lg.float().argmax(-1).tolist()
    k.finalize()


def _attention_case(seq_lens, n_q, n_kv, page_size, numerics, seed):
    T = len(seq_lens)
    D = 128
    max_seq = max(seq_lens) + 3
    qkv = _rand((T, (n_q + 2 * n_kv) * D), seed)
    qn, kn = (1 + 0.2 * _rand((D,), seed + 1).float()).to(BF), (1 + 0.2 * _rand((D,), seed + 2).float()).to(BF)
    geom = O.Geometry(n_q=n_q, n_kv=n_kv)
    cos, sin = O.rope_tables(geom, max_seq)
    k, meta, (indptr, indices) = onepass_kernel(T, max_seq=max_seq, page_size=page_size, seq_lens=seq_lens,
                                               numerics=numerics)
    kc = _rand((k.max_num_pages, page_size, n_kv, D), seed + 3)
    vc = _rand((k.max_num_pages, page_size, n_kv, D), seed + 4)
    kcd, vcd = kc.cuda(), vc.cuda()
    od = torch.zeros(T, n_q * D, dtype=BF, device="cuda")
    k.paged_attention_layer(input=k.attach_input(qkv.cuda(), "qkv"), k_cache=k.attach_input(kcd, "kc"),
                            v_cache=k.attach_input(vcd, "vc"), q_norm=k.attach_input(qn.cuda(), "qn"),
                            k_norm=k.attach_input(kn.cuda(), "kn"), cos_pos_embed=k.attach_input(cos.cuda(), "cos"),
                            sin_pos_embed=k.attach_input(sin.cuda(), "sin"), output=k.attach_input(od, "o"),
                            grid_dim=(T, n_kv, 1), block_dim=(128, 1, 1))
    k.compile()
    k()
    qpk = n_q // n_kv
    for t, L in enumerate(seq_lens):
        pos = L - 1
        row = qkv[t].view(n_kv, qpk + 2, D)
        q, knew, vnew = row[:, :qpk].reshape(n_q, D), row[:, qpk], row[:, qpk + 1]
        pages = indices[indptr[t]:indptr[t + 1]]
        kk = torch.cat([kc[p] for p in pages])[:L].clone()
        vv = torch.cat([vc[p] for p in pages])[:L].clone()
        if numerics == "mpk":
            qr = O.mpk_qk_norm_rope(q, qn, cos[pos], sin[pos])
            kr = O.mpk_qk_norm_rope(knew, kn, cos[pos], sin[pos])
        else:
            qr, kr = O.ref_rope(O.ref_rmsnorm(q, qn), O.ref_rmsnorm(knew, kn), cos[pos][None], sin[pos][None], 0)
            qr, kr = qr.reshape(n_q, D), kr.reshape(n_kv, D)
        kk[pos], vv[pos] = kr, vnew
        ref = O.mpk_attention_decode(qr, kk, vv).reshape(-1)
        bf16_close(od[t], ref, 1e-2, f"attention token {t} L={L}")
        # the new K/V landed in the right page slot, other slots untouched
        pg, slot = pages[pos // page_size], pos % page_size
        assert torch.equal(kcd[pg, slot].cpu(), kr), "appended K"
        assert torch.equal(vcd[pg, slot].cpu(), vnew), "appended V"
        if slot > 0:
            assert torch.equal(kcd[pg, slot - 1].cpu(), kc[pg, slot - 1])
    k.finalize()


@pytest.mark.parametrize("numerics", ["mpk", "torch"])
@pytest.mark.parametrize("seq_lens,n_q,n_kv,page", [([1], 4, 2, 16), ([65], 32, 8, 64), ([1025], 32, 8, 64),
                                                    ([64, 1, 17, 200], 8, 2, 16), ([1200], 32, 8, 64),
                                                    ([300, 299, 301], 4, 1, 32), ([128], 16, 2, 64),
                                                    # more (request, kv head) pairs than SMs: several rounds of tasks
                                                    ([3 + (i * 7) % 60 for i in range(40)], 32, 8, 16),
                                                    ([1 + (i * 13) % 90 for i in range(24)], 16, 8, 32),
                                                    ([5 + i for i in range(64)], 8, 8, 64)])
def test_paged_attention(seq_lens, n_q, n_kv, page, numerics):
    _attention_case(seq_lens, n_q, n_kv, page, numerics, seed=100 + len(seq_lens) + n_q)


def test_batch_rows_are_independent():
    """The reference driver's cross-batch check (demo.py:1281-1301): identical rows give identical outputs."""
    T, N, K = 4, 1024, 1024
    x1, w = _rand((1, K), 20), _rand((N, K), 21, 0.05)
    x = x1.repeat(T, 1)
    k, meta, _ = onepass_kernel(T)
    od = torch.zeros(T, N, dtype=BF, device="cuda")
    k.linear_layer(input=k.attach_input(x.cuda(), "x"), weight=k.attach_input(w.cuda(), "w"), output=k.attach_input(od, "o"),
                   grid_dim=(N // 64, 1, 1), block_dim=(128, 1, 1))
    k.compile()
    k()
    for t in range(1, T):
        assert torch.equal(od[t], od[0])
    k.finalize()


# ---- the reference's other spellings of the linear layers ----------------------------------
@pytest.mark.parametrize("T", [1, 5, 24])
def test_split_k_linear_accumulates_into_its_output(T):
    """splitk_linear_layer on sm_100: output += input * W^T, the output holding the residual stream
    (python/mirage/mpk/models/qwen3/builder.py:556-563)."""
    N, K = 1024, 2048
    x, w, r = _rand((T, K), 41), _rand((N, K), 42, 0.05), _rand((T, N), 43)
    k, meta, _ = onepass_kernel(T)
    od = r.clone().cuda()
    k.splitk_linear_layer(input=k.attach_input(x.cuda(), "x"), weight=k.attach_input(w.cuda(), "w"),
                          output=k.attach_input(od, "o"), grid_dim=(N // 128, 128 * 128 // N, 1), block_dim=(256, 1, 1))
    k.compile()
    k()
    bf16_close(od, O.mpk_linear(x, w, residual=r), 1e-2, "split-k linear into the residual stream")
    k.finalize()


def test_split_k_workspace_and_reduce():
    T, N, K, S = 3, 512, 1024, 4
    x, w, r = _rand((T, K), 44), _rand((N, K), 45, 0.05), _rand((T, N), 46)
    k, meta, _ = onepass_kernel(T)
    od = torch.zeros(T, N, dtype=BF, device="cuda")
    ws = k.new_tensor(dims=(S * T, N), name="splitk_ws")
    k.splitk_linear_layer(input=k.attach_input(x.cuda(), "x"), weight=k.attach_input(w.cuda(), "w"), output=ws,
                          grid_dim=(N // 128, S, 1), block_dim=(256, 1, 1))
    k.splitk_reduce_layer(workspace=ws, residual=k.attach_input(r.cuda(), "r"), output=k.attach_input(od, "o"),
                          k_splits=S, grid_dim=(N // 128, 1, 1), block_dim=(256, 1, 1))
    k.compile()
    k()
    bf16_close(od, O.mpk_linear(x, w, residual=r), 1e-2, "split-k workspace + reduce")
    k.finalize()


@pytest.mark.parametrize("T,groups", [(2, 1), (2, 8), (6, 1)])
def test_silu_mul_linear_with_residual(T, groups):
    """The fused SiLU*up + down projection layer (persistent_kernel.py:2174): its input row is
    [gate | up] halves, so the gate/up weight is shuffled in ONE group for it; with more groups the
    layer still reads halves of whatever the linear before it wrote."""
    K, I, N = 512, 1024, 384
    x, wg, wu = _rand((T, K), 47), _rand((I, K), 48, 0.05), _rand((I, K), 49, 0.05)
    wd, r = _rand((N, I), 50, 0.05), _rand((T, N), 51)
    k, meta, _ = onepass_kernel(T)
    od = torch.zeros(T, N, dtype=BF, device="cuda")
    wgu = k.shuffle_tensors([k.attach_input(wg.cuda(), "wg"), k.attach_input(wu.cuda(), "wu")], 0, groups, "wgu")
    mid = k.new_tensor(dims=(T, 2 * I), name="mlp_mid")
    k.linear_layer(input=k.attach_input(x.cuda(), "x"), weight=wgu, output=mid, grid_dim=(2 * I // 64, 1, 1),
                   block_dim=(128, 1, 1))
    k.silu_mul_linear_with_residual_layer(input=mid, weight=k.attach_input(wd.cuda(), "wd"),
                                          residual=k.attach_input(r.cuda(), "r"), output=k.attach_input(od, "o"),
                                          grid_dim=(N // 64, 1, 1), block_dim=(256, 1, 1))
    kinds = [ln.split()[1] for ln in k.plan().strip().splitlines()]
    assert kinds == (["linear", "linear"] if groups == 1 else ["linear", "silu_mul", "linear"])
    k.compile()
    k()
    # the mid tensor as the reference lays it out: `groups` blocks of [gate rows | up rows]
    per = I // groups
    wcat = torch.cat([torch.cat((wg[g * per:(g + 1) * per], wu[g * per:(g + 1) * per])) for g in range(groups)])
    midref = O.mpk_linear(x, wcat)
    h = O.mpk_silu_mul(midref[:, :I], midref[:, I:])
    bf16_close(od, O.mpk_linear(h, wd, residual=r), 1e-2, "silu_mul_linear_with_residual")
    k.finalize()


@pytest.mark.parametrize("T", [1, 12])
def test_gang_spellings_run_the_same_arithmetic(T):
    """gang_rmsnorm -> gang_linear_silu -> gang_splitk_linear_with_residual: Fleet's MLP half
    (demo/qwen3/demo.py:925-1075 with USE_GANG and USE_FUSED_SILU), tiling arguments as hints."""
    K, I = 512, 1024
    x, wn = _rand((T, K), 52), (1 + 0.3 * _rand((K,), 53).float()).to(BF)
    wg, wu, wd = _rand((I, K), 54, 0.05), _rand((I, K), 55, 0.05), _rand((K, I), 56, 0.05)
    k, meta, _ = onepass_kernel(T)
    od = torch.zeros(T, K, dtype=BF, device="cuda")
    xt = k.attach_input(x.cuda(), "x")
    rms = k.new_tensor(dims=(T, K), name="rmsnorm_out")
    act = k.new_tensor(dims=(T, I), name="silu_mul_out")
    ws = k.new_tensor(dims=(4 * T, K), dtype=mk.float32, name="splitk_ws")
    wgu = k.shuffle_tensors([k.attach_input(wg.cuda(), "wg"), k.attach_input(wu.cuda(), "wu")], 0, I // 64, "wgu")
    k.gang_rmsnorm_layer(input=xt, weight=k.attach_input(wn.cuda(), "wn"), output=rms)
    k.gang_linear_silu_layer(input=rms, weight=wgu, output=act, tile_n=64, output_stride=I, m_tiles=1, wgm=4)
    k.gang_splitk_linear_with_residual_layer(input=act, weight=k.attach_input(wd.cuda(), "wd"), residual=xt, workspace=ws,
                                             output=k.attach_input(od, "o"), tile_n=64, output_stride=K, k_splits=4)
    k.compile()
    k()
    xn = O.mpk_rmsnorm(x, wn)
    h = O.mpk_silu_mul(O.mpk_linear(xn, wg), O.mpk_linear(xn, wu))
    bf16_close(od, O.mpk_linear(h, wd, residual=x), 1e-2, "gang MLP half")
    k.finalize()


@pytest.mark.parametrize("T", [2, 9])
def test_mlp_half_written_in_the_fleet_dsl(T):
    """The MLP half of a layer through the task DSL (decorated op functions on a fleet.Graph)."""
    import fleet_chiplet_megakernel_b200.fleet as fleet
    K, I = 512, 1024
    x, wn = _rand((T, K), 61), (1 + 0.3 * _rand((K,), 62).float()).to(BF)
    wg, wu, wd = _rand((I, K), 63, 0.05), _rand((I, K), 64, 0.05), _rand((K, I), 65, 0.05)
    k, meta, _ = onepass_kernel(T)
    od = torch.zeros(T, K, dtype=BF, device="cuda")

    @fleet.task(level="cu")
    def norm(a, w, o):
        return fleet.ops.rmsnorm(a, w, o)

    @fleet.task(level="xcd", tiling="split_k")
    def down(a, w, o, r):
        return fleet.ops.linear(a, w, o, residual=r, strategy=fleet.strategy_from_meta(fleet.get_meta(down)))

    g = fleet.Graph(k)
    xt = g.input(x.cuda(), "x")
    rms = g.intermediate((T, K), name="rmsnorm_out")
    act = g.intermediate((T, I), name="silu_mul_out")
    wgu = g.shuffle_inputs([g.input(wg.cuda(), "wg"), g.input(wu.cuda(), "wu")], I // 64, "wgu")
    norm(xt, g.input(wn.cuda(), "wn"), rms)
    fleet.ops.linear_silu(rms, wgu, act)
    down(act, g.input(wd.cuda(), "wd"), g.input(od, "o"), xt)
    k.compile()
    k()
    xn = O.mpk_rmsnorm(x, wn)
    h = O.mpk_silu_mul(O.mpk_linear(xn, wg), O.mpk_linear(xn, wu))
    bf16_close(od, O.mpk_linear(h, wd, residual=x), 1e-2, "MLP half through the DSL")
    k.finalize()
