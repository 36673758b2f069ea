"""The Fleet task DSL on the PersistentKernel mirror: decorators carry metadata, the cost model names the
B200 strategies, and a decoder layer written with the DSL (the pattern of the reference's
demo/qwen3/demo_dsl.py:182-383) lowers to the same device program as the plain layer calls.  No GPU."""
import pytest
import torch

import fleet_chiplet_megakernel_b200 as mk
import fleet_chiplet_megakernel_b200.fleet as fleet
from tests.test_cabi_host import _kernel, _weights, _variant_graph, _shape_of


def test_decorators_attach_metadata_and_map_to_strategies():
    @fleet.affinity(placement="inherit_xcd")
    @fleet.task(level="warp")
    def act(i, o):
        return fleet.ops.silu_mul(i, o)

    @fleet.distribute(dim=0, num_xcds=8)
    @fleet.task(level="xcd", tiling="split_k", l2_budget="4MB")
    def down(x, w, o, r):
        return None

    m = fleet.get_meta(act)
    assert m["level"] == "warp" and m["scope"] == "warp" and m["placement"] == "inherit_xcd"
    assert fleet.strategy_from_meta(m) == "standard"
    d = fleet.get_meta(down)
    assert d["scope"] == "gpu" and d["l2_budget"] == 4 << 20 and d["partition"] == {"dim": 0, "num_xcds": 8}
    assert fleet.strategy_from_meta(d) == "gang_splitk"
    assert fleet.strategy_from_meta(fleet.get_meta(fleet.task(level="cluster")(lambda: None))) == "gang"
    assert fleet.strategy_from_meta({}) == "auto"
    with pytest.raises(ValueError):
        fleet.task(level="planet")
    assert repr(fleet.Tile[4, 8]) == "Tile[4, 8]" and repr(fleet.Partition[512, 64]) == "Partition[512, 64]"


def test_cost_model_names_the_b200_paths():
    assert [fleet.select_strategy(4096, 4096, b) for b in (1, 2, 3, 16, 17, 64)] == \
        ["row_owner", "row_owner", "stream_k", "stream_k", "tcgen05", "tcgen05"]
    assert fleet.select_strategy(4096, 4096, 1, target_cc=94) == "standard"
    assert fleet.select_k_splits(4096, 32) == 5      # 32 row blocks on 148 SMs: a block is shared by about 5 CTAs
    assert fleet.select_k_splits(4096, 1187) == 1    # the LM head: more row blocks than SMs, no block is split
    assert fleet.select_k_splits(256, 1) == 2        # never more pieces than k tiles


def _dsl_graph(k, layers=2):
    geom = mk.Qwen3Geometry(hidden=512, n_q=4, n_kv=2, mlp=1024, layers=layers, vocab=2048)
    w = _weights(geom, layers)
    T, H, D = k.max_num_batched_tokens, geom.hidden, 128
    kc = torch.zeros(layers, k.max_num_pages, k.page_size, geom.n_kv, D, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    cos = torch.zeros(k.max_seq_length, D, dtype=torch.bfloat16)
    sin = cos.clone()
    keep = [w, kc, vc, cos, sin]

    @fleet.task(level="cu")
    def norm(x, wt, out):
        return fleet.ops.rmsnorm(x, wt, out)

    @fleet.distribute(dim=0, num_xcds=8)
    @fleet.task(level="xcd")
    def proj(x, wt, out, res=None):
        return fleet.ops.linear(x, wt, out, residual=res, strategy=fleet.strategy_from_meta(fleet.get_meta(proj)))

    @fleet.task(level="auto")
    def auto_proj(x, wt, out, res=None):
        return fleet.ops.linear(x, wt, out, residual=res)

    g = fleet.Graph(k)
    x = g.input(k.meta_tensors["input_tokens"], "input_token")
    cos_t, sin_t = g.input(cos, "cos"), g.input(sin, "sin")
    y = g.intermediate((T, H), name="embed_out")
    rms = g.intermediate((T, H), name="rmsnorm_out")
    attn_in = g.intermediate((T, (geom.n_q + 2 * geom.n_kv) * D), name="attn_in")
    attn_out = g.intermediate((T, geom.n_q * D), name="attn_out")
    attn_proj = g.intermediate((T, H), name="attn_proj_out")
    silu_out = g.intermediate((T, geom.mlp), name="silu_mul_out")
    mlp_out = g.intermediate((T, H), name="mlp_out")
    fleet.ops.embed(x, g.input(w["embed"], "embed"), y)
    x = y
    for i in range(layers):
        wqkv = g.shuffle_inputs([g.input(w[f"l{i}.{n}"], f"l{i}{n}") for n in "qkv"], geom.n_kv, f"l{i}qkv")
        norm(x, g.input(w[f"l{i}.ln1"], f"l{i}ln1"), rms)
        proj(rms, wqkv, attn_in)
        fleet.ops.paged_attention(attn_in, g.input(kc[i], f"l{i}kc"), g.input(vc[i], f"l{i}vc"),
                                  g.input(w[f"l{i}.qn"], f"l{i}qn"), g.input(w[f"l{i}.kn"], f"l{i}kn"), cos_t, sin_t,
                                  attn_out, geom.n_kv)
        proj(attn_out, g.input(w[f"l{i}.o"], f"l{i}o"), attn_proj, res=x)
        x = attn_proj
        wgu = g.shuffle_inputs([g.input(w[f"l{i}.gate"], f"l{i}g"), g.input(w[f"l{i}.up"], f"l{i}u")], geom.mlp // 64,
                               f"l{i}gu")
        norm(x, g.input(w[f"l{i}.ln2"], f"l{i}ln2"), rms)
        fleet.ops.linear_silu(rms, wgu, silu_out)
        auto_proj(silu_out, g.input(w[f"l{i}.down"], f"l{i}d"), mlp_out, res=x)
        x = mlp_out
    return keep


@pytest.mark.parametrize("R", [1, 4])
def test_a_layer_written_in_the_dsl_lowers_to_the_plain_program(native_lib, R):
    k = _kernel(R=R, pages=4 * R, fuse=True)
    keep = _variant_graph(k, "plain")
    base = _shape_of(k.plan())
    k.finalize()
    k = _kernel(R=R, pages=4 * R, fuse=True)
    keep2 = _dsl_graph(k)
    assert _shape_of(k.plan()) == base
    k.finalize()
    del keep, keep2
