"""Generate the Qwen3-MoE fixture from transformers' Qwen3MoeForCausalLM.

The reference's MoE demo (demo/qwen3/demo_30B_A3B.py:1, 381-392) takes its PyTorch model from the
transformers package (pinned 4.57.1 in the reference's requirements.txt; this image holds 5.5.0), so that
model, run here on the oracle's seeded weights with its default attention (torch's scaled_dot_product_attention)
and its per-expert loop, is the reference output:

  python tests/golden/make_golden_moe.py      ->  tests/golden/moe_tiny_generate.pt

It also checks the oracle's restatement (oracle/qwen3_oracle.py: TorchMoeRefModel) against it."""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import qwen3_oracle as O  # noqa: E402


def build_hf(g, w):
    from transformers.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeForCausalLM
    cfg = Qwen3MoeConfig(vocab_size=g.vocab, hidden_size=g.hidden, intermediate_size=4 * g.hidden,
                         moe_intermediate_size=g.moe_mlp, num_hidden_layers=g.layers, num_attention_heads=g.n_q,
                         num_key_value_heads=g.n_kv, head_dim=g.head_dim, num_experts=g.experts,
                         num_experts_per_tok=g.top_k, norm_topk_prob=True, rope_theta=g.rope_theta,
                         max_position_embeddings=4096, tie_word_embeddings=False, decoder_sparse_step=1,
                         mlp_only_layers=[], attention_bias=False, rms_norm_eps=g.eps)
    cfg._attn_implementation = "sdpa"       # the library's default, what the reference's demo runs
    cfg._experts_implementation = "eager"   # the published per-expert loop (5.x would otherwise pick a grouped GEMM)
    m = Qwen3MoeForCausalLM(cfg).to(torch.bfloat16).eval()
    # .to(bfloat16) also rounds the rotary embedding's inv_freq buffer; a checkpoint loaded with
    # from_pretrained(torch_dtype=bfloat16), as the reference's demo does, keeps it in fp32
    d = g.head_dim
    m.model.rotary_emb.inv_freq = 1.0 / (g.rope_theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
    sd = {"model.embed_tokens.weight": w["embed"], "model.norm.weight": w["norm"], "lm_head.weight": w["lm_head"]}
    for i in range(g.layers):
        p = f"model.layers.{i}."
        sd.update({p + "self_attn.q_proj.weight": w[f"l{i}.q"], p + "self_attn.k_proj.weight": w[f"l{i}.k"],
                   p + "self_attn.v_proj.weight": w[f"l{i}.v"], p + "self_attn.o_proj.weight": w[f"l{i}.o"],
                   p + "self_attn.q_norm.weight": w[f"l{i}.qn"], p + "self_attn.k_norm.weight": w[f"l{i}.kn"],
                   p + "mlp.gate.weight": w[f"l{i}.router"], p + "mlp.experts.gate_up_proj": w[f"l{i}.w13"],
                   p + "mlp.experts.down_proj": w[f"l{i}.w2"], p + "input_layernorm.weight": w[f"l{i}.ln1"],
                   p + "post_attention_layernorm.weight": w[f"l{i}.ln2"]})
    missing, unexpected = m.load_state_dict(sd, strict=False)
    assert not [k for k in missing if "inv_freq" not in k], missing
    assert not unexpected, unexpected
    return m


@torch.inference_mode()
def hf_generate(m, prompt, n_new):
    from transformers import DynamicCache
    cache = DynamicCache(config=m.config)
    toks = prompt.tolist()
    out = m(input_ids=prompt[None], past_key_values=cache, use_cache=True)
    logits = []
    for j in range(n_new):
        last = out.logits[0, -1]
        logits.append(last.clone())
        toks.append(int(last.argmax(-1)))
        if j + 1 < n_new:
            out = m(input_ids=torch.tensor([[toks[-1]]]), past_key_values=cache, use_cache=True)
    return toks, torch.stack(logits)


def main():
    g, name, P, n_new = O.MOE_TINY, "moe_tiny_generate.pt", 10, 32
    w = O.make_moe_weights(g, seed=0, norm_jitter=0.1)
    prompt = O.make_prompt(O.Geometry(vocab=g.vocab), P, 0)
    toks, logits = hf_generate(build_hf(g, w), prompt, n_new)
    mine = O.TorchMoeRefModel(g, w, P + n_new + 2)
    toks2, logits2 = mine.generate(prompt, n_new)
    exact = toks == toks2 and torch.equal(logits, logits2)
    err = O.max_rel_err(logits2, logits)
    print(f"[{name}] restatement vs transformers {__import__('transformers').__version__}: bit-exact {exact}, "
          f"max error {err:.3e} of the step's largest |logit|, tokens equal {toks == toks2}")
    torch.save({"geometry": g.asdict(), "seed": 0, "norm_jitter": 0.1, "prompt": prompt, "tokens": torch.tensor(toks),
                "logits": logits, "max_seq": P + n_new + 2, "restatement_bit_exact": exact,
                "route_margin": torch.tensor(mine.margins),  # per generated step: smallest top-k routing gap over the layers
                "transformers_version": __import__("transformers").__version__}, os.path.join(HERE, name))


if __name__ == "__main__":
    torch.manual_seed(0)
    main()
