"""The oracle against the fixtures the unmodified reference model produced
(tests/golden/make_golden.py).  CPU only."""
import os

import torch

from oracle import qwen3_oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _checksum(t):
    return int(t.view(torch.int16).to(torch.int64).sum())


def _load(name):
    return torch.load(os.path.join(GOLD, name))


def _generate_case(name):
    fx = _load(name)
    geom = O.Geometry(**fx["geometry"])
    w = O.make_weights(geom, fx["seed"], norm_jitter=fx["norm_jitter"])
    for k, v in fx["weights_checksum"].items():
        assert _checksum(w[k]) == v, f"seeded weight {k} differs from the fixture's"
    n_new = fx["logits"].shape[0]
    m = O.TorchRefModel(geom, w, fx["max_seq"])
    toks, logits = m.generate(fx["prompt"], n_new)
    assert toks == fx["tokens"].tolist()
    assert torch.equal(logits, fx["logits"]), "restatement is not bit-exact against the reference's logits"
    return fx, geom, w


def test_torch_restatement_matches_reference_tiny():
    _generate_case("tiny_generate.pt")


def test_torch_restatement_matches_reference_small():
    _generate_case("small_generate.pt")


def test_torch_restatement_matches_reference_kv8():
    _generate_case("kv8_generate.pt")


def test_task_arithmetic_within_tolerance_of_reference():
    """The megakernel-task arithmetic (fp32 norms) stays inside the 2e-2 logit
    tolerance of the reference PyTorch model under teacher forcing."""
    fx = _load("tiny_generate.pt")
    geom = O.Geometry(**fx["geometry"])
    w = O.make_weights(geom, fx["seed"], norm_jitter=fx["norm_jitter"])
    m = O.MpkRefModel(geom, w, fx["max_seq"])
    P = len(fx["prompt"])
    ref = fx["tokens"].tolist()
    worst = 0.0
    for p in range(P + 15):
        lg = m.step(ref[p], p)
        if p >= P - 1:
            worst = max(worst, O.max_rel_err(lg[None], fx["logits"][p - P + 1][None]))
    assert worst < 2.5e-2, worst


def test_single_layer_config_matches_reference():
    """Config 1: one Qwen3-8B-geometry layer, one decode step over 1024 cached positions."""
    from tests.golden.make_golden import config1_inputs
    fx = _load("config1_layer.pt")
    w, hidden, kc, vc, L = config1_inputs()
    assert _checksum(hidden) == fx["in_checksum"] and _checksum(kc) == fx["k_checksum"]
    for k, v in fx["w_checksum"].items():
        assert _checksum(w[k]) == v
    g1 = O.Geometry(layers=1, vocab=8)
    m = O.TorchRefModel(g1, w, L + 8)
    m.k_cache[0, :L] = kc
    m.v_cache[0, :L] = vc
    with torch.inference_mode():
        out = m.layer(0, hidden[None, :], L)[0]
    assert torch.equal(out, fx["out_hidden"])
    assert torch.equal(m.k_cache[0, L], fx["new_k"])
    # the task arithmetic on the same inputs
    m2 = O.MpkRefModel(g1, w, L + 8)
    m2.k_cache[0, :L] = kc
    m2.v_cache[0, :L] = vc
    out2 = m2.layer(0, hidden, L)
    assert O.max_rel_err(out2[None], fx["out_hidden"][None]) < 2e-2


def test_argmax_tie_rule():
    lg = torch.tensor([1.0, 3.0, 3.0, 2.0], dtype=torch.bfloat16)
    assert int(O.mpk_argmax(lg)) == 1


def test_moe_restatement_matches_transformers_fixture():
    """Qwen3-MoE: the oracle against the fixture transformers' Qwen3MoeForCausalLM produced (make_golden_moe.py)."""
    fx = _load("moe_tiny_generate.pt")
    g = O.MoeGeometry(**fx["geometry"])
    w = O.make_moe_weights(g, fx["seed"], norm_jitter=fx["norm_jitter"])
    n_new = fx["logits"].shape[0]
    m = O.TorchMoeRefModel(g, w, fx["max_seq"])
    toks, logits = m.generate(fx["prompt"], n_new)
    assert toks == fx["tokens"].tolist()
    assert torch.equal(logits, fx["logits"]), "restatement is not bit-exact against transformers' logits"


def test_moe_routing_semantics():
    """softmax -> top-k -> renormalise (the reference's tests/runtime_python/blackwell/sm100_moe/test_gate_topk.py:34-78)."""
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(5, 128, generator=g).to(torch.bfloat16)
    val, idx = O.moe_route(logits, 8)
    p = torch.softmax(logits.float(), -1)
    top = p.topk(8, -1)
    assert torch.equal(idx, top.indices)
    assert torch.allclose(val.sum(-1), torch.ones(5), atol=1e-6)
    assert torch.allclose(val, top.values / top.values.sum(-1, keepdim=True))
