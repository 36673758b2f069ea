"""Qwen3 decode graph on the ``PersistentKernel`` API.

The layer sequence and tensor names follow the reference's benchmark driver
demo/qwen3/demo.py:314-1185 (and python/mirage/mpk/models/qwen3/builder.py):
embedding, then per layer rmsnorm -> linear(QKV, group-interleaved by
shuffle_tensors) -> paged attention (split-KV + merge) -> linear_with_residual(O)
-> rmsnorm -> linear(gate/up, block-interleaved) -> silu_mul ->
linear_with_residual(down), then rmsnorm -> linear(LM head) -> argmax partial /
reduce.  ``Qwen3Decoder`` owns the meta tensors and KV cache the way the driver
does (demo.py:246-352) and runs offline-mode generation.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .persistent_kernel import PersistentKernel, bfloat16, float32, int64


@dataclass(frozen=True)
class Qwen3Geometry:
    hidden: int = 4096
    n_q: int = 32
    n_kv: int = 8
    head_dim: int = 128
    mlp: int = 12288
    layers: int = 36
    vocab: int = 151936
    rope_theta: float = 1e6


def rope_tables(geom: Qwen3Geometry, max_pos: int, device):
    """bf16 cos/sin of cat(freqs, freqs), as the reference's rotary embedding
    builds them (demo/qwen3/models/modeling_qwen3.py:95-117)."""
    d = geom.head_dim
    inv_freq = 1.0 / (geom.rope_theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
    freqs = torch.arange(max_pos, dtype=torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(torch.bfloat16).to(device).contiguous(), emb.sin().to(torch.bfloat16).to(device).contiguous()


def shard_qwen3_weights(weights: dict, world_size: int, rank: int, shard_lm_head: bool = True) -> dict:
    """Tensor-parallel shard of a full weight dict, as the reference's converter cuts a checkpoint
    (demo/qwen3/models/convert.py:13-28): q/k/v/gate/up by output rows (column parallel), o/down by
    input columns (row parallel), everything else replicated.  Beyond the reference, the LM head is cut by
    vocabulary rows as well (``shard_lm_head``): the reference replicates it (modeling_qwen3.py:514), which
    leaves every rank streaming the full 1.2 GB head however many ranks there are."""
    if world_size == 1:
        return weights
    out = {}
    for name, t in weights.items():
        leaf = name.split(".")[-1]
        if leaf in ("q", "k", "v", "gate", "up") or (name == "lm_head" and shard_lm_head and t.shape[0] % world_size == 0):
            out[name] = t.chunk(world_size, dim=0)[rank].contiguous()
        elif leaf in ("o", "down"):
            out[name] = t.chunk(world_size, dim=1)[rank].contiguous()
        else:
            out[name] = t
    return out


def build_qwen3_graph(mpk: PersistentKernel, geom: Qwen3Geometry, weights: dict, k_cache, v_cache, cos, sin,
                      input_tokens, output_tokens, logits=None, num_layers=None, lm_head=True):
    """Record the decode graph.  ``weights`` uses the keys embed, l{i}.{q,k,v,o,gate,up,down,ln1,ln2,qn,kn},
    norm, lm_head (device bf16 tensors); ``k_cache``/``v_cache`` are [layers, pages, page, kv_heads, 128]."""
    T = mpk.max_num_batched_tokens
    R = mpk.max_num_batched_requests
    H, D = geom.hidden, geom.head_dim
    ws = mpk.world_size
    n_q, n_kv = geom.n_q // ws, geom.n_kv // ws
    qkv_out = (n_q + 2 * n_kv) * D
    inter = geom.mlp // ws
    L = geom.layers if num_layers is None else num_layers
    chunks = max(1, (mpk.max_seq_length + 127) // 128)
    cat = "nvshmem_tensor" if ws > 1 else "cuda_tensor"

    x = mpk.attach_input(torch_tensor=input_tokens, name="input_token")
    cos_t = mpk.attach_input(torch_tensor=cos, name="cos_position_embedding")
    sin_t = mpk.attach_input(torch_tensor=sin, name="sin_position_embedding")
    y = mpk.new_tensor(dims=(T, H), dtype=bfloat16, name="embed_out")
    rmsnorm_out = mpk.new_tensor(dims=(T, H), dtype=bfloat16, name="rmsnorm_out")
    attn_in = mpk.new_tensor(dims=(T, qkv_out), dtype=bfloat16, name="attn_in")
    lse = mpk.new_tensor(dims=(T, chunks * n_q // n_kv, n_kv), strides=(chunks * n_q, 1, chunks * n_q // n_kv),
                         dtype=float32, name="lse")
    attn_out_tmp = mpk.new_tensor(dims=(T, chunks * n_q // n_kv * D, n_kv),
                                  strides=(chunks * n_q * D, 1, chunks * n_q // n_kv * D), dtype=bfloat16,
                                  name="attn_out_tmp")
    attn_out = mpk.new_tensor(dims=(T, n_q * D), dtype=bfloat16, name="attn_out")
    attn_proj_out = mpk.new_tensor(dims=(T, H), dtype=bfloat16, name="attn_proj_out", io_category=cat)
    mlp_mid = mpk.new_tensor(dims=(T, 2 * inter), dtype=bfloat16, name="mlp_mid")
    silu_mul_out = mpk.new_tensor(dims=(T, inter), dtype=bfloat16, name="silu_mul_out")
    mlp_out = mpk.new_tensor(dims=(T, H), dtype=bfloat16, name="mlp_out", io_category=cat)
    if ws > 1:
        allreduce_buf = mpk.new_tensor(dims=(ws, T, H), dtype=bfloat16, name="all_reduce_buf", io_category=cat)
        attn_allreduce_out = mpk.new_tensor(dims=(T, H), dtype=bfloat16, name="attn_allreduce_out", io_category=cat)
        mlp_final = mpk.new_tensor(dims=(T, H), dtype=bfloat16, name="mlp_final", io_category=cat)

    w = mpk.attach_input(torch_tensor=weights["embed"], name="embed_tokens")
    mpk.embed_layer(input=x, weight=w, output=y, grid_dim=(1, 1, 1), block_dim=(128, 1, 1), input_source=1)
    x = y
    gateup_tasks = max(2, 2 * inter // 128)  # [gate|up] blocks of 64 columns each
    for i in range(L):
        w_norm = mpk.attach_input(torch_tensor=weights[f"l{i}.ln1"], name=f"layer_{i}_input_layernorm")
        w_q = mpk.attach_input(torch_tensor=weights[f"l{i}.q"], name=f"layer_{i}_q_proj")
        w_k = mpk.attach_input(torch_tensor=weights[f"l{i}.k"], name=f"layer_{i}_k_proj")
        w_v = mpk.attach_input(torch_tensor=weights[f"l{i}.v"], name=f"layer_{i}_v_proj")
        w_qkv = mpk.shuffle_tensors(inputs=[w_q, w_k, w_v], shuffled_dim=0, num_groups=n_kv,
                                    name=f"layer_{i}_qkv_proj")
        mpk.rmsnorm_layer(input=x, weight=w_norm, output=rmsnorm_out, grid_dim=(T, 1, 1), block_dim=(128, 1, 1))
        mpk.linear_layer(input=rmsnorm_out, weight=w_qkv, output=attn_in, grid_dim=(qkv_out // 64, 1, 1),
                         block_dim=(128, 1, 1))
        w_qn = mpk.attach_input(torch_tensor=weights[f"l{i}.qn"], name=f"layer_{i}_q_norm")
        w_kn = mpk.attach_input(torch_tensor=weights[f"l{i}.kn"], name=f"layer_{i}_k_norm")
        kc = mpk.attach_input(torch_tensor=k_cache[i], name=f"layer_{i}_k_cache")
        vc = mpk.attach_input(torch_tensor=v_cache[i], name=f"layer_{i}_v_cache")
        mpk.paged_attention_split_kv_layer(input=attn_in, k_cache=kc, v_cache=vc, q_norm=w_qn, k_norm=w_kn,
                                           cos_pos_embed=cos_t, sin_pos_embed=sin_t, lse=lse, output=attn_out_tmp,
                                           attention_params=(n_q, chunks), grid_dim=(R, n_kv, chunks),
                                           block_dim=(128, 1, 1))
        mpk.paged_attention_split_kv_merge_layer(lse=lse, output_tmp=attn_out_tmp, output=attn_out,
                                                 attention_params=(n_q, D), grid_dim=(R, n_kv, 1),
                                                 block_dim=(128, 1, 1))
        w_o = mpk.attach_input(torch_tensor=weights[f"l{i}.o"], name=f"layer_{i}_o_proj")
        mpk.linear_with_residual_layer(input=attn_out, weight=w_o, residual=x, output=attn_proj_out,
                                       grid_dim=(H // 64, 1, 1), block_dim=(256, 1, 1))
        x = attn_proj_out
        if ws > 1:
            mpk.allreduce_layer(input=attn_proj_out, buffer=allreduce_buf, output=attn_allreduce_out,
                                grid_dim=(H // 64, 1, 1), block_dim=(128, 1, 1))
            x = attn_allreduce_out
        w_norm = mpk.attach_input(torch_tensor=weights[f"l{i}.ln2"], name=f"layer_{i}_post_attn_layernorm")
        w_g = mpk.attach_input(torch_tensor=weights[f"l{i}.gate"], name=f"layer_{i}_gate_proj")
        w_u = mpk.attach_input(torch_tensor=weights[f"l{i}.up"], name=f"layer_{i}_up_proj")
        w_gu = mpk.shuffle_tensors(inputs=[w_g, w_u], shuffled_dim=0, num_groups=gateup_tasks // 2,
                                   name=f"layer_{i}_gatedup_proj")
        mpk.rmsnorm_layer(input=x, weight=w_norm, output=rmsnorm_out, grid_dim=(T, 1, 1), block_dim=(128, 1, 1))
        mpk.linear_layer(input=rmsnorm_out, weight=w_gu, output=mlp_mid, grid_dim=(2 * inter // 64, 1, 1),
                         block_dim=(128, 1, 1))
        mpk.silu_mul_layer(input=mlp_mid, output=silu_mul_out, grid_dim=(gateup_tasks // 2, 1, 1),
                           block_dim=(128, 1, 1))
        w_d = mpk.attach_input(torch_tensor=weights[f"l{i}.down"], name=f"layer_{i}_down_proj")
        mpk.linear_with_residual_layer(input=silu_mul_out, weight=w_d, residual=x, output=mlp_out,
                                       grid_dim=(H // 64, 1, 1), block_dim=(256, 1, 1))
        x = mlp_out
        if ws > 1:
            mpk.allreduce_layer(input=mlp_out, buffer=allreduce_buf, output=mlp_final, grid_dim=(H // 64, 1, 1),
                                block_dim=(128, 1, 1))
            x = mlp_final
    if not lm_head:
        return x
    w_norm = mpk.attach_input(torch_tensor=weights["norm"], name="model_norm_weight")
    w_proj = mpk.attach_input(torch_tensor=weights["lm_head"], name="lm_head")
    vocab = weights["lm_head"].shape[0]  # this rank's rows: the whole vocabulary, or its slice of a sharded head
    head_sharded = ws > 1 and vocab * ws == geom.vocab
    if logits is not None:
        argmax_in = mpk.attach_input(torch_tensor=logits, name="argmax_in")
    else:
        argmax_in = mpk.new_tensor(dims=(T, vocab), dtype=bfloat16, name="argmax_in")
    tasks = 128
    argmax_part_value = mpk.new_tensor(dims=(T, tasks), dtype=bfloat16, name="argmax_part_value")
    argmax_part_index = mpk.new_tensor(dims=(T, tasks), dtype=int64, name="argmax_part_index")
    argmax_out = mpk.attach_input(torch_tensor=output_tokens, name="output_token")
    mpk.rmsnorm_layer(input=x, weight=w_norm, output=rmsnorm_out, grid_dim=(T, 1, 1), block_dim=(128, 1, 1))
    mpk.linear_layer(input=rmsnorm_out, weight=w_proj, output=argmax_in, grid_dim=(tasks, 1, 1),
                     block_dim=(128, 1, 1))
    mpk.argmax_partial_layer(input=argmax_in, output=(argmax_part_value, argmax_part_index), grid_dim=(tasks, 1, 1),
                             block_dim=(128, 1, 1))
    mpk.argmax_reduce_layer(input=(argmax_part_value, argmax_part_index), output=argmax_out, grid_dim=(1, 1, 1),
                            block_dim=(128, 1, 1), vocab_offset=mpk.mpi_rank * vocab if head_sharded else 0,
                            across_ranks=head_sharded)
    return argmax_in


class Qwen3Decoder:
    """Offline-mode greedy generation for a batch of requests (the reference
    driver's ``--use-mirage`` path, demo.py:1247-1276)."""

    def __init__(self, geom: Qwen3Geometry, weights: dict, max_seq_length: int, max_requests: int,
                 total_requests: int | None = None, page_size: int = 64, max_num_pages: int | None = None,
                 device="cuda", numerics=None, fuse=None, keep_logits=False, eos_token_id: int = 0x7FFFFFFF,
                 max_iterations: int = 0, num_layers=None, timeout_ms: int = 0, trace: bool = False,
                 trace_op: int = -1, debug_flags: int = 0, world_size: int = 1, rank: int = 0, cluster_size: int = 0,
                 test_barrier_epoch: int = 0, max_num_batched_tokens: int | None = None,
                 max_tokens_per_request: int = 0, prefetch_kb: int = 0, max_stages: int = 0):
        """``weights`` are this rank's shard (see ``shard_qwen3_weights``) when world_size > 1.
        ``max_num_batched_tokens`` (default: max_requests, one token per request and iteration) is the
        token budget of an iteration: above max_requests, a request that is still inside its prompt is fed
        a chunk of it per iteration (the reference's chunked prefill, persistent_kernel.cuh:380-536).
        ``max_tokens_per_request`` caps a request's chunk (1: every request advances one token per iteration)."""
        self.geom, self.device = geom, torch.device(device)
        R = max_requests
        T = max(R, max_num_batched_tokens or R)
        total = total_requests if total_requests is not None else R
        pages_per_req = math.ceil(max_seq_length / page_size)
        self.max_num_pages = max_num_pages if max_num_pages is not None else R * pages_per_req
        L = geom.layers if num_layers is None else num_layers
        dev = self.device
        self.tokens = torch.zeros(total, max_seq_length, dtype=torch.int64, device=dev)
        self.prompt_lengths = torch.zeros(total, dtype=torch.int32, device=dev)
        self.step = torch.zeros(total, dtype=torch.int32, device=dev)
        self.input_tokens = torch.zeros(T, 1, dtype=torch.int64, device=dev)
        self.output_tokens = torch.zeros(T, 1, dtype=torch.int64, device=dev)
        self.num_new_tokens = torch.ones(total, dtype=torch.int32, device=dev)
        self.qo_indptr = torch.zeros(R + 1, dtype=torch.int32, device=dev)
        self.kv_indptr = torch.zeros(R + 1, dtype=torch.int32, device=dev)
        self.kv_indices = torch.zeros(self.max_num_pages, dtype=torch.int32, device=dev)
        self.kv_last_page_len = torch.zeros(R, dtype=torch.int32, device=dev)
        self.k_cache = torch.zeros(L, self.max_num_pages, page_size, geom.n_kv // world_size, geom.head_dim,
                                   dtype=torch.bfloat16, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.cos, self.sin = rope_tables(geom, max(max_seq_length, 8), dev)
        self.logits = torch.zeros(T, weights["lm_head"].shape[0], dtype=torch.bfloat16, device=dev) if keep_logits else None
        self.profiler = torch.zeros(1 << 20, dtype=torch.int64, device=dev) if trace else None
        self.mpk = PersistentKernel(
            mode="offline", world_size=world_size, mpi_rank=rank, num_workers=0, num_local_schedulers=0,
            num_remote_schedulers=0, max_seq_length=max_seq_length, max_num_batched_requests=R,
            max_num_batched_tokens=T, max_num_pages=self.max_num_pages, page_size=page_size,
            meta_tensors={"step": self.step, "tokens": self.tokens, "input_tokens": self.input_tokens,
                          "output_tokens": self.output_tokens, "num_new_tokens": self.num_new_tokens,
                          "prompt_lengths": self.prompt_lengths, "qo_indptr_buffer": self.qo_indptr,
                          "paged_kv_indptr_buffer": self.kv_indptr, "paged_kv_indices_buffer": self.kv_indices,
                          "paged_kv_last_page_len_buffer": self.kv_last_page_len},
            profiler_tensor=self.profiler, trace_name="", spec_decode_config=None, use_cutlass_kernel=True,
            eos_token_id=eos_token_id, numerics=numerics, fuse=fuse, max_iterations=max_iterations,
            timeout_ms=timeout_ms, trace_op=trace_op, debug_flags=debug_flags, cluster_size=cluster_size,
            test_barrier_epoch=test_barrier_epoch, max_tokens_per_request=max_tokens_per_request,
            prefetch_kb=prefetch_kb, max_stages=max_stages)
        build_qwen3_graph(self.mpk, geom, weights, self.k_cache, self.v_cache, self.cos, self.sin,
                          self.input_tokens, self.output_tokens, logits=self.logits, num_layers=num_layers)
        self.mpk.compile()

    def set_prompts(self, prompts):
        """prompts: list of 1-D int64 tensors, one per request.  Host prompts travel in one copy
        (a padded [requests, longest] block) plus one for the lengths."""
        n = len(prompts)
        lens = [len(p) for p in prompts]
        width = max(lens)
        self.tokens.zero_()
        if all(p.device.type == "cpu" for p in prompts):
            block = torch.zeros(n, width, dtype=torch.int64).pin_memory() if torch.cuda.is_available() else \
                torch.zeros(n, width, dtype=torch.int64)
            for r, p in enumerate(prompts):
                block[r, : lens[r]] = p
            self.tokens[:n, :width].copy_(block, non_blocking=True)
        else:
            for r, p in enumerate(prompts):
                self.tokens[r, : lens[r]] = p.to(self.device)
        self.prompt_lengths[:n].copy_(torch.tensor(lens, dtype=torch.int32), non_blocking=False)
        self.mpk.init_requests()

    def run(self):
        """One launch: the whole generation (or ``max_iterations`` iterations of it)."""
        self.mpk()

    def generated(self, r):
        return self.tokens[r, : int(self.step[r]) + 1]

    def finalize(self):
        self.mpk.finalize()
