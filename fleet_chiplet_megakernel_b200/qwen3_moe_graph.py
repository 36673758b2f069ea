"""Qwen3-MoE decode graph on the ``PersistentKernel`` API.

The layer sequence follows the reference's MoE driver demo/qwen3/demo_30B_A3B.py:430-790: the attention
half of a layer as in the dense model, then rmsnorm -> linear(router) -> moe_topk_softmax_routing ->
moe_w13_linear -> moe_silu_mul -> moe_w2_linear -> moe_mul_sum_add (weighted sum + residual).  Expert
weights are [experts, 2 * inter, hidden] ([gate | up] halves) and [experts, hidden, inter], the layout of
transformers' Qwen3MoeExperts.  Built for one or two batched tokens (every (token, expert) pair a GEMV)."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .persistent_kernel import PersistentKernel, bfloat16, float32, int32, int64
from .qwen3_graph import rope_tables


@dataclass(frozen=True)
class Qwen3MoeGeometry:
    hidden: int = 2048
    n_q: int = 32
    n_kv: int = 4
    head_dim: int = 128
    experts: int = 128
    top_k: int = 8
    moe_mlp: int = 768
    layers: int = 48
    vocab: int = 151936
    rope_theta: float = 1e6


def build_qwen3_moe_graph(mpk: PersistentKernel, geom: Qwen3MoeGeometry, weights: dict, k_cache, v_cache, cos, sin,
                          input_tokens, output_tokens, logits=None, num_layers=None):
    """``weights``: embed, l{i}.{q,k,v,o,router,w13,w2,ln1,ln2,qn,kn}, norm, lm_head (device bf16 tensors)."""
    T, R = mpk.max_num_batched_tokens, mpk.max_num_batched_requests
    H, D, E, K, I = geom.hidden, geom.head_dim, geom.experts, geom.top_k, geom.moe_mlp
    n_q, n_kv = geom.n_q, geom.n_kv
    qkv_out = (n_q + 2 * n_kv) * D
    L = geom.layers if num_layers is None else num_layers

    x = mpk.attach_input(torch_tensor=input_tokens, name="input_token")
    cos_t = mpk.attach_input(torch_tensor=cos, name="cos_position_embedding")
    sin_t = mpk.attach_input(torch_tensor=sin, name="sin_position_embedding")
    y = mpk.new_tensor(dims=(T, H), dtype=bfloat16, name="embed_out")
    rmsnorm_out = mpk.new_tensor(dims=(T, H), dtype=bfloat16, name="rmsnorm_out")
    attn_in = mpk.new_tensor(dims=(T, qkv_out), dtype=bfloat16, name="attn_in")
    attn_out = mpk.new_tensor(dims=(T, n_q * D), dtype=bfloat16, name="attn_out")
    attn_proj_out = mpk.new_tensor(dims=(T, H), dtype=bfloat16, name="attn_proj_out")
    moe_gate_out = mpk.new_tensor(dims=(T, E), dtype=bfloat16, name="moe_gate_out")
    moe_topk_weight = mpk.new_tensor(dims=(T, K), dtype=float32, name="moe_topk_weight")
    moe_routing_indices = mpk.new_tensor(dims=(E, T), dtype=int32, name="moe_routing_indices")
    moe_mask = mpk.new_tensor(dims=(E + 1,), dtype=int32, name="moe_mask")
    mlp_mid = mpk.new_tensor(dims=(T, K, 2 * I), dtype=bfloat16, name="mlp_mid")
    silu_mul_out = mpk.new_tensor(dims=(T, K, I), dtype=bfloat16, name="silu_mul_out")
    mlp_out = mpk.new_tensor(dims=(T, K, H), dtype=bfloat16, name="mlp_out")
    mlp_sum = mpk.new_tensor(dims=(T, H), dtype=bfloat16, name="mlp_weighted_sum_out")

    w = mpk.attach_input(torch_tensor=weights["embed"], name="embed_tokens")
    mpk.embed_layer(input=x, weight=w, output=y, grid_dim=(1, 1, 1), block_dim=(128, 1, 1), input_source=1)
    x = y
    for i in range(L):
        w_norm = mpk.attach_input(torch_tensor=weights[f"l{i}.ln1"], name=f"layer_{i}_input_layernorm")
        w_q = mpk.attach_input(torch_tensor=weights[f"l{i}.q"], name=f"layer_{i}_q_proj")
        w_k = mpk.attach_input(torch_tensor=weights[f"l{i}.k"], name=f"layer_{i}_k_proj")
        w_v = mpk.attach_input(torch_tensor=weights[f"l{i}.v"], name=f"layer_{i}_v_proj")
        w_qkv = mpk.shuffle_tensors(inputs=[w_q, w_k, w_v], shuffled_dim=0, num_groups=n_kv, name=f"layer_{i}_qkv_proj")
        mpk.rmsnorm_layer(input=x, weight=w_norm, output=rmsnorm_out, grid_dim=(T, 1, 1), block_dim=(128, 1, 1))
        mpk.linear_layer(input=rmsnorm_out, weight=w_qkv, output=attn_in, grid_dim=(qkv_out // 64, 1, 1), block_dim=(128, 1, 1))
        w_qn = mpk.attach_input(torch_tensor=weights[f"l{i}.qn"], name=f"layer_{i}_q_norm")
        w_kn = mpk.attach_input(torch_tensor=weights[f"l{i}.kn"], name=f"layer_{i}_k_norm")
        kc = mpk.attach_input(torch_tensor=k_cache[i], name=f"layer_{i}_k_cache")
        vc = mpk.attach_input(torch_tensor=v_cache[i], name=f"layer_{i}_v_cache")
        mpk.paged_attention_layer(input=attn_in, k_cache=kc, v_cache=vc, q_norm=w_qn, k_norm=w_kn, cos_pos_embed=cos_t,
                                  sin_pos_embed=sin_t, output=attn_out, grid_dim=(R, n_kv, 1), block_dim=(128, 1, 1))
        w_o = mpk.attach_input(torch_tensor=weights[f"l{i}.o"], name=f"layer_{i}_o_proj")
        mpk.linear_with_residual_layer(input=attn_out, weight=w_o, residual=x, output=attn_proj_out,
                                       grid_dim=(H // 64, 1, 1), block_dim=(128, 1, 1))
        x = attn_proj_out
        w_norm = mpk.attach_input(torch_tensor=weights[f"l{i}.ln2"], name=f"layer_{i}_post_attn_layernorm")
        w_gate = mpk.attach_input(torch_tensor=weights[f"l{i}.router"], name=f"layer_{i}_moe_gate")
        w13 = mpk.attach_input(torch_tensor=weights[f"l{i}.w13"], name=f"layer_{i}_gateup_proj")
        w2 = mpk.attach_input(torch_tensor=weights[f"l{i}.w2"], name=f"layer_{i}_down_proj")
        mpk.rmsnorm_layer(input=x, weight=w_norm, output=rmsnorm_out, grid_dim=(T, 1, 1), block_dim=(256, 1, 1))
        mpk.linear_layer(input=rmsnorm_out, weight=w_gate, output=moe_gate_out, grid_dim=(1, 1, 1), block_dim=(256, 1, 1))
        mpk.moe_topk_softmax_routing_layer(input=moe_gate_out, output=(moe_topk_weight, moe_routing_indices, moe_mask),
                                           grid_dim=(1, 1, 1), block_dim=(256, 1, 1))
        mpk.moe_w13_linear_layer(input=rmsnorm_out, weight=w13, moe_routing_indices=moe_routing_indices, moe_mask=moe_mask,
                                 output=mlp_mid, grid_dim=(10, 2 * I // 64, 1), block_dim=(256, 1, 1))
        mpk.moe_silu_mul_layer(input=mlp_mid, output=silu_mul_out, grid_dim=(T, K, 1), block_dim=(256, 1, 1))
        mpk.moe_w2_linear_layer(input=silu_mul_out, weight=w2, moe_routing_indices=moe_routing_indices, moe_mask=moe_mask,
                                output=mlp_out, grid_dim=(8, H // 64, 1), block_dim=(256, 1, 1))
        mpk.moe_mul_sum_add_layer(input=mlp_out, weight=moe_topk_weight, residual=x, output=mlp_sum,
                                  grid_dim=(T, max(1, H // 256), 1), block_dim=(256, 1, 1))
        x = mlp_sum
    w_norm = mpk.attach_input(torch_tensor=weights["norm"], name="model_norm_weight")
    w_proj = mpk.attach_input(torch_tensor=weights["lm_head"], name="lm_head")
    vocab = weights["lm_head"].shape[0]
    argmax_in = mpk.attach_input(torch_tensor=logits, name="argmax_in") if logits is not None else \
        mpk.new_tensor(dims=(T, vocab), dtype=bfloat16, name="argmax_in")
    tasks = 128
    part_v = mpk.new_tensor(dims=(T, tasks), dtype=bfloat16, name="argmax_part_value")
    part_i = mpk.new_tensor(dims=(T, tasks), dtype=int64, name="argmax_part_index")
    argmax_out = mpk.attach_input(torch_tensor=output_tokens, name="output_token")
    mpk.rmsnorm_layer(input=x, weight=w_norm, output=rmsnorm_out, grid_dim=(T, 1, 1), block_dim=(256, 1, 1))
    mpk.linear_layer(input=rmsnorm_out, weight=w_proj, output=argmax_in, grid_dim=(tasks, 1, 1), block_dim=(256, 1, 1))
    mpk.argmax_partial_layer(input=argmax_in, output=(part_v, part_i), grid_dim=(tasks, 1, 1), block_dim=(128, 1, 1))
    mpk.argmax_reduce_layer(input=(part_v, part_i), output=argmax_out, grid_dim=(1, 1, 1), block_dim=(128, 1, 1))
    return argmax_in


class Qwen3MoeDecoder:
    """Offline-mode greedy generation for the MoE model (the driver's ``--use-mirage`` path)."""

    def __init__(self, geom: Qwen3MoeGeometry, weights: dict, max_seq_length: int, max_requests: int = 1,
                 total_requests: int | None = None, page_size: int = 64, device="cuda", numerics=None, keep_logits=False,
                 eos_token_id: int = 0x7FFFFFFF, max_iterations: int = 0, num_layers=None, timeout_ms: int = 0,
                 trace: bool = False):
        self.geom, self.device = geom, torch.device(device)
        R = max_requests
        total = total_requests if total_requests is not None else R
        self.max_num_pages = R * math.ceil(max_seq_length / page_size)
        L = geom.layers if num_layers is None else num_layers
        dev = self.device
        self.tokens = torch.zeros(total, max_seq_length, dtype=torch.int64, device=dev)
        self.prompt_lengths = torch.zeros(total, dtype=torch.int32, device=dev)
        self.step = torch.zeros(total, dtype=torch.int32, device=dev)
        self.input_tokens = torch.zeros(R, 1, dtype=torch.int64, device=dev)
        self.output_tokens = torch.zeros(R, 1, dtype=torch.int64, device=dev)
        self.num_new_tokens = torch.ones(total, dtype=torch.int32, device=dev)
        self.qo_indptr = torch.zeros(R + 1, dtype=torch.int32, device=dev)
        self.kv_indptr = torch.zeros(R + 1, dtype=torch.int32, device=dev)
        self.kv_indices = torch.zeros(self.max_num_pages, dtype=torch.int32, device=dev)
        self.kv_last_page_len = torch.zeros(R, dtype=torch.int32, device=dev)
        self.k_cache = torch.zeros(L, self.max_num_pages, page_size, geom.n_kv, geom.head_dim, dtype=torch.bfloat16, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.cos, self.sin = rope_tables(geom, max(max_seq_length, 8), dev)
        self.logits = torch.zeros(R, weights["lm_head"].shape[0], dtype=torch.bfloat16, device=dev) if keep_logits else None
        self.profiler = torch.zeros(1 << 21, dtype=torch.int64, device=dev) if trace else None
        self.mpk = PersistentKernel(
            mode="offline", world_size=1, mpi_rank=0, num_workers=0, num_local_schedulers=0, num_remote_schedulers=0,
            max_seq_length=max_seq_length, max_num_batched_requests=R, max_num_batched_tokens=R,
            max_num_pages=self.max_num_pages, page_size=page_size,
            meta_tensors={"step": self.step, "tokens": self.tokens, "input_tokens": self.input_tokens,
                          "output_tokens": self.output_tokens, "num_new_tokens": self.num_new_tokens,
                          "prompt_lengths": self.prompt_lengths, "qo_indptr_buffer": self.qo_indptr,
                          "paged_kv_indptr_buffer": self.kv_indptr, "paged_kv_indices_buffer": self.kv_indices,
                          "paged_kv_last_page_len_buffer": self.kv_last_page_len},
            profiler_tensor=self.profiler, trace_name="", spec_decode_config=None, use_cutlass_kernel=True,
            eos_token_id=eos_token_id, numerics=numerics, max_iterations=max_iterations, timeout_ms=timeout_ms,
            max_tokens_per_request=1)
        build_qwen3_moe_graph(self.mpk, geom, weights, self.k_cache, self.v_cache, self.cos, self.sin, self.input_tokens,
                              self.output_tokens, logits=self.logits, num_layers=num_layers)
        self.mpk.compile()

    def set_prompts(self, prompts):
        self.tokens.zero_()
        for r, p in enumerate(prompts):
            self.tokens[r, : len(p)] = p.to(self.device)
            self.prompt_lengths[r] = len(p)
        self.mpk.init_requests()

    def run(self):
        self.mpk()

    def generated(self, r):
        return self.tokens[r, : int(self.step[r]) + 1]

    def finalize(self):
        self.mpk.finalize()
