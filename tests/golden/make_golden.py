"""Generate the golden fixtures in this folder from the UNMODIFIED reference model.

Run once in a container that has the reference checkout (it does not travel to
the GPU box):  ``python tests/golden/make_golden.py [reference_root]``.

It imports the reference's demo/qwen3/models/modeling_qwen3.py with five
external shims (nothing in the reference tree is touched):
  1. a stub ``mirage`` module (the file imports it, the forward never uses it);
  2. the 'default' RoPE initialiser, which newer transformers dropped
     (inv_freq = theta^(-2i/d), scaling 1.0);
  3. ``device="cuda"`` allocations redirected to the CPU;
  4. ``config.pad_token_id = None``;
  5. the Triton RoPE replaced by the file's own pure-torch apply_rotary_pos_emb.
It then loads the oracle's seeded weights into the reference model, runs the
reference, checks the oracle's restatement against it, and stores the
REFERENCE's outputs:
  tiny_generate.pt   TINY geometry: prompt, greedy tokens, per-step logits
  small_generate.pt  SMALL geometry: same
  kv8_generate.pt    KV8 geometry (16 q / 8 kv heads: splits over 2, 4 and 8 tensor-parallel ranks): same
  config1_layer.pt   one Qwen3-8B-geometry decoder layer, one decode step at
                     position 1024 over a seeded N(0,1) KV cache: output hidden
                     state, plus checksums of the seeded inputs
"""
import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import qwen3_oracle as O  # noqa: E402


def import_reference(ref_root):
    sys.modules.setdefault("mirage", types.ModuleType("mirage"))
    from transformers import modeling_rope_utils as mru

    if "default" not in mru.ROPE_INIT_FUNCTIONS:
        def _default(config, device=None, **kw):
            d = config.head_dim
            inv = 1.0 / (config.rope_theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
            return inv, 1.0
        mru.ROPE_INIT_FUNCTIONS["default"] = _default
    # Triton import in rope.py must not need a GPU: stub the module it defines.
    demo = os.path.join(ref_root, "demo", "qwen3")
    sys.path.insert(0, demo)
    rope_stub = types.ModuleType("models.rope")
    rope_stub.apply_rotary_pos_emb_triton = None
    import importlib
    pkg = importlib.import_module("models")  # demo/qwen3/models/__init__.py
    return pkg


def build_reference(ref_root, geom, weights, max_seq, layers=None):
    _orig_empty, _orig_tensor = torch.empty, torch.tensor

    def _cpu(fn):
        def wrapped(*a, **k):
            if k.get("device") == "cuda":
                k["device"] = "cpu"
            return fn(*a, **k)
        return wrapped

    torch.empty, torch.tensor = _cpu(_orig_empty), _cpu(_orig_tensor)
    try:
        sys.modules.setdefault("mirage", types.ModuleType("mirage"))
        from transformers import modeling_rope_utils as mru
        if "default" not in mru.ROPE_INIT_FUNCTIONS:
            def _default(config, device=None, **kw):
                d = config.head_dim
                inv = 1.0 / (config.rope_theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
                return inv, 1.0
            mru.ROPE_INIT_FUNCTIONS["default"] = _default
        demo = os.path.join(ref_root, "demo", "qwen3")
        if demo not in sys.path:
            sys.path.insert(0, demo)
        # rope.py needs triton at import; it imports fine on CPU, only launch needs a GPU
        from models import modeling_qwen3 as M
        from models.configuration_qwen3 import Qwen3Config
        M.apply_rotary_pos_emb_triton = M.apply_rotary_pos_emb  # shim 5
        n_layers = geom.layers if layers is None else layers
        cfg = Qwen3Config(vocab_size=geom.vocab, hidden_size=geom.hidden, intermediate_size=geom.mlp,
                          num_hidden_layers=n_layers, num_attention_heads=geom.n_q,
                          num_key_value_heads=geom.n_kv, head_dim=geom.head_dim,
                          rope_theta=geom.rope_theta, max_position_embeddings=32768,
                          attention_bias=False, tie_word_embeddings=False)
        cfg.pad_token_id = None
        if not hasattr(cfg, "rope_scaling"):
            cfg.rope_scaling = None
        torch.set_default_dtype(torch.bfloat16)
        model = M.Qwen3ForCausalLM(cfg, 1, 1, max_seq)
        torch.set_default_dtype(torch.float32)
    finally:
        torch.empty, torch.tensor = _orig_empty, _orig_tensor
    sd = {"model.embed_tokens.weight": weights["embed"], "model.norm.weight": weights["norm"],
          "lm_head.weight": weights["lm_head"]}
    for i in range(n_layers):
        p = f"model.layers.{i}."
        sd[p + "self_attn.q_proj.weight"] = weights[f"l{i}.q"]
        sd[p + "self_attn.k_proj.weight"] = weights[f"l{i}.k"]
        sd[p + "self_attn.v_proj.weight"] = weights[f"l{i}.v"]
        sd[p + "self_attn.o_proj.weight"] = weights[f"l{i}.o"]
        sd[p + "self_attn.q_norm.weight"] = weights[f"l{i}.qn"]
        sd[p + "self_attn.k_norm.weight"] = weights[f"l{i}.kn"]
        sd[p + "mlp.gate_proj.weight"] = weights[f"l{i}.gate"]
        sd[p + "mlp.up_proj.weight"] = weights[f"l{i}.up"]
        sd[p + "mlp.down_proj.weight"] = weights[f"l{i}.down"]
        sd[p + "input_layernorm.weight"] = weights[f"l{i}.ln1"]
        sd[p + "post_attention_layernorm.weight"] = weights[f"l{i}.ln2"]
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not [m for m in missing if "inv_freq" not in m], missing
    assert not unexpected, unexpected
    model.eval()
    return model


def reference_generate(model, geom, prompt, n_new, max_seq):
    """demo/qwen3/demo.py:1196-1212 on CPU."""
    pos = torch.arange(max_seq).unsqueeze(0)
    cos, sin = model.model.rotary_emb(pos)
    toks = torch.zeros(1, max_seq, dtype=torch.long)
    P = len(prompt)
    toks[0, :P] = prompt
    step = torch.zeros(1, dtype=torch.int32)
    prev = 0
    logits_out = []
    for cur in range(P, P + n_new):
        step.fill_(cur - 1)
        out = model.forward(input_ids=toks[:, prev:cur],
                            position_embeddings=(cos[:, prev:cur], sin[:, prev:cur]), step=step)
        logits = out[0] if isinstance(out, tuple) else getattr(out, "logits", out)
        last = logits[0, -1]
        logits_out.append(last.clone())
        toks[0, cur] = int(last.argmax(-1))
        prev = cur
    return toks[0, :P + n_new].tolist(), torch.stack(logits_out)


def checksum(t):
    return int(t.view(torch.int16).to(torch.int64).sum())


def gen_generate_fixture(ref_root, geom, name, prompt_len, n_new, max_seq, norm_jitter):
    w = O.make_weights(geom, seed=0, norm_jitter=norm_jitter)
    prompt = O.make_prompt(geom, prompt_len, 0)
    ref = build_reference(ref_root, geom, w, max_seq)
    toks, logits = reference_generate(ref, geom, prompt, n_new, max_seq)
    mine = O.TorchRefModel(geom, w, max_seq)
    toks2, logits2 = mine.generate(prompt, n_new)
    exact = toks == toks2 and torch.equal(logits, logits2)
    print(f"[{name}] restatement bit-exact vs reference: {exact}; "
          f"max|dlogit|={float((logits.float() - logits2.float()).abs().max()):.3e}")
    assert toks == toks2
    torch.save({"geometry": geom.asdict(), "seed": 0, "norm_jitter": norm_jitter, "prompt": prompt,
                "tokens": torch.tensor(toks), "logits": logits, "max_seq": max_seq,
                "weights_checksum": {k: checksum(v) for k, v in list(w.items())[:4]},
                "restatement_bit_exact": exact}, os.path.join(HERE, name))


def gen_config1(ref_root):
    geom = O.QWEN3_8B
    L = 1024
    w = O.make_weights(O.Geometry(layers=1, vocab=8), seed=0)  # one layer; embed/lm_head unused here
    g = torch.Generator().manual_seed(0)
    hidden = torch.randn(geom.hidden, generator=g, dtype=torch.float32).to(O.BF16)
    kc = torch.randn(L, geom.n_kv, geom.head_dim, generator=g, dtype=torch.float32).to(O.BF16)
    vc = torch.randn(L, geom.n_kv, geom.head_dim, generator=g, dtype=torch.float32).to(O.BF16)
    g1 = O.Geometry(layers=1, vocab=8)
    ref = build_reference(ref_root, g1, w, L + 8)
    ref.model.kv_cache[0][0, 0, :L] = kc
    ref.model.kv_cache[1][0, 0, :L] = vc
    pos = torch.arange(L + 8).unsqueeze(0)
    cos, sin = ref.model.rotary_emb(pos)
    step = torch.full((1,), L, dtype=torch.int32)
    with torch.inference_mode():
        out = ref.model.layers[0](hidden[None, None, :], position_embeddings=(cos[:, L:L + 1], sin[:, L:L + 1]),
                                  step=step)[0][0, 0]
    mine = O.TorchRefModel(g1, w, L + 8)
    mine.k_cache[0, :L] = kc
    mine.v_cache[0, :L] = vc
    with torch.inference_mode():
        out2 = mine.layer(0, hidden[None, :], L)[0]
    exact = torch.equal(out, out2)
    print(f"[config1] restatement bit-exact vs reference: {exact}")
    torch.save({"position": L, "out_hidden": out.clone(), "in_checksum": checksum(hidden),
                "k_checksum": checksum(kc), "v_checksum": checksum(vc),
                "w_checksum": {k: checksum(v) for k, v in w.items() if k.startswith("l0.")},
                "new_k": ref.model.kv_cache[0][0, 0, L].clone(), "new_v": ref.model.kv_cache[1][0, 0, L].clone(),
                "restatement_bit_exact": exact}, os.path.join(HERE, "config1_layer.pt"))


def config1_inputs():
    """The seeded inputs of config 1, shared by the generator and the tests."""
    geom = O.QWEN3_8B
    L = 1024
    w = O.make_weights(O.Geometry(layers=1, vocab=8), seed=0)
    g = torch.Generator().manual_seed(0)
    hidden = torch.randn(geom.hidden, generator=g, dtype=torch.float32).to(O.BF16)
    kc = torch.randn(L, geom.n_kv, geom.head_dim, generator=g, dtype=torch.float32).to(O.BF16)
    vc = torch.randn(L, geom.n_kv, geom.head_dim, generator=g, dtype=torch.float32).to(O.BF16)
    return w, hidden, kc, vc, L


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py <root of the reference checkout>")
    ref_root = sys.argv[1]
    torch.manual_seed(0)
    gen_generate_fixture(ref_root, O.TINY, "tiny_generate.pt", prompt_len=8, n_new=40, max_seq=64, norm_jitter=0.25)
    gen_generate_fixture(ref_root, O.SMALL, "small_generate.pt", prompt_len=16, n_new=40, max_seq=96, norm_jitter=0.0)
    gen_generate_fixture(ref_root, O.KV8, "kv8_generate.pt", prompt_len=12, n_new=40, max_seq=96, norm_jitter=0.1)
    gen_config1(ref_root)
