"""``MPK`` and ``MPKMetadata``: the reference's serving-side wrapper around ``PersistentKernel``
(python/mirage/mpk/mpk.py:15-429), the entry a host framework uses: describe the deployment in a metadata
record, hand over weights, KV cache and position embeddings in a model config, ``build()`` the model graph,
``compile()``, then call it.

Differences that follow from this runtime: ranks come from ``torch.distributed`` when it is initialised (the
reference asks mpi4py); there is no tokenizer or checkpoint download offline, so ``load_new_request`` takes
token ids and ``weight_from_model`` is refused; the Qwen3 graph is recorded by ``build_qwen3_graph``."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from .persistent_kernel import PersistentKernel, get_configurations_from_gpu
from .qwen3_graph import Qwen3Geometry, build_qwen3_graph


@dataclass
class MirageModelConfig:
    """python/mirage/mpk/models/graph_builder.py:7-27: architecture, caches, position embeddings, weights.
    ``state_dict`` uses the checkpoint's names (model.layers.N.self_attn.q_proj.weight, ...), already cut for
    this rank under tensor parallelism; ``k_cache`` / ``v_cache`` are lists of per-layer tensors
    [max_num_pages, page_size, local_kv_heads, head_dim]."""
    hidden_size: int = None
    intermediate_size: int = None
    vocab_size: int = None
    local_num_q_heads: int = None
    local_num_kv_heads: int = None
    head_dim: int = None
    num_layers: int = None
    k_cache: list = None
    v_cache: list = None
    position_embeddings: tuple = None
    state_dict: dict | None = None
    with_lm_head: bool = True


@dataclass
class MPKMetadata:
    """python/mirage/mpk/mpk.py:15-63: everything outside the model itself.  Meta tensors left None are
    allocated by ``MPK`` with the shapes the kernel expects."""
    mode: str = "offline"
    total_num_requests: int = 1
    num_remote_schedulers: int = 0
    max_seq_length: int = 0
    max_num_batched_requests: int = 0
    max_num_batched_tokens: int = 0
    max_num_pages: int = 0
    page_size: int = 0
    max_sm_num: int = 148
    device: str = "cuda"
    weight_from_model: bool = False
    model_name: Optional[str] = "qwen3"
    model_path: Optional[str] = None
    world_size: int = 1
    rank: int = 0
    num_workers: int = -1
    num_schedulers: int = -1
    step: Optional[torch.Tensor] = None
    tokens: Optional[torch.Tensor] = None
    input_tokens: Optional[torch.Tensor] = None
    output_tokens: Optional[torch.Tensor] = None
    num_new_tokens: Optional[torch.Tensor] = None
    prompt_lengths: Optional[torch.Tensor] = None
    qo_indptr_buffer: Optional[torch.Tensor] = None
    paged_kv_indptr_buffer: Optional[torch.Tensor] = None
    paged_kv_indices_buffer: Optional[torch.Tensor] = None
    paged_kv_last_page_len_buffer: Optional[torch.Tensor] = None
    model_config: Optional[MirageModelConfig] = None
    profiling: bool = False
    profiler_tensor: Optional[torch.Tensor] = None
    trace_name: Optional[str] = None
    spec_decode: Optional[str] = None
    spec_decode_config: Optional[object] = None
    use_cutlass_kernel: bool = True
    eos_token_id: int = -1
    extra: dict = field(default_factory=dict)  # further PersistentKernel arguments (numerics, max_iterations, ...)

    def check_valid(self):
        if self.weight_from_model:
            raise NotImplementedError("weight_from_model needs a checkpoint download; pass model_config.state_dict")
        mc = self.model_config
        assert mc is not None and mc.state_dict is not None, "state_dict is required when weight_from_model is False"
        assert mc.k_cache is not None, "k_cache is required when weight_from_model is False"
        assert mc.v_cache is not None, "v_cache is required when weight_from_model is False"

    def info_as_string(self):
        keys = ("mode", "total_num_requests", "max_seq_length", "max_num_batched_requests", "max_num_batched_tokens",
                "max_num_pages", "page_size", "device", "model_name", "world_size", "rank")
        return "MPKMetadata info:\n" + "".join(f"{k}: {getattr(self, k)}\n" for k in keys)


_CHECKPOINT_NAMES = {"q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight", "v": "self_attn.v_proj.weight",
                     "o": "self_attn.o_proj.weight", "qn": "self_attn.q_norm.weight", "kn": "self_attn.k_norm.weight",
                     "gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight", "down": "mlp.down_proj.weight",
                     "ln1": "input_layernorm.weight", "ln2": "post_attention_layernorm.weight"}


def weights_from_state_dict(sd: dict, num_layers: int) -> dict:
    """Checkpoint names -> the short keys ``build_qwen3_graph`` uses."""
    w = {"embed": sd["model.embed_tokens.weight"], "norm": sd["model.norm.weight"]}
    if "lm_head.weight" in sd:
        w["lm_head"] = sd["lm_head.weight"]
    for i in range(num_layers):
        for short, long in _CHECKPOINT_NAMES.items():
            w[f"l{i}.{short}"] = sd[f"model.layers.{i}.{long}"]
    return w


class MPK:
    def __init__(self, meta: MPKMetadata):
        meta.check_valid()
        self.metadata = meta
        self.world_size, self.rank = meta.world_size, meta.rank
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            self.world_size, self.rank = torch.distributed.get_world_size(), torch.distributed.get_rank()
        self.device = torch.device(meta.device)
        self.max_seq_length = meta.max_seq_length
        self.max_num_batched_requests = meta.max_num_batched_requests
        self.max_num_batched_tokens = meta.max_num_batched_tokens or meta.max_num_batched_requests
        self.max_num_pages = meta.max_num_pages
        self.total_num_requests = meta.total_num_requests
        self.model_config = meta.model_config
        self.with_lm_head = self.model_config.with_lm_head
        for k in ("step", "tokens", "input_tokens", "output_tokens", "num_new_tokens", "prompt_lengths", "qo_indptr_buffer",
                  "paged_kv_indptr_buffer", "paged_kv_indices_buffer", "paged_kv_last_page_len_buffer"):
            setattr(self, k, getattr(meta, k))
        self.need_cpy_input = False
        if self.input_tokens is not None and self.input_tokens.dtype != torch.int64:
            # a host framework with int32 token ids: the kernel reads an int64 copy refreshed at every call
            self.need_cpy_input, self.src_input_tokens = True, self.input_tokens
            self.input_tokens = torch.empty_like(self.input_tokens, dtype=torch.int64)
        self.profiler_tensor = meta.profiler_tensor
        self.compensate_meta_tensors()
        workers = meta.num_workers
        if workers <= 0 and torch.cuda.is_available():
            workers, _ = get_configurations_from_gpu(self.device.index or 0)
        self.num_workers = min(max(workers, 0), meta.max_sm_num) if workers > 0 else 0
        self.persistent_kernel = PersistentKernel(
            mode=meta.mode, world_size=self.world_size, mpi_rank=self.rank, num_workers=self.num_workers,
            num_local_schedulers=0, num_remote_schedulers=0, max_seq_length=self.max_seq_length,
            max_num_batched_requests=self.max_num_batched_requests, max_num_batched_tokens=self.max_num_batched_tokens,
            max_num_pages=self.max_num_pages, page_size=meta.page_size,
            meta_tensors={"step": self.step, "tokens": self.tokens, "input_tokens": self.input_tokens,
                          "output_tokens": self.output_tokens, "num_new_tokens": self.num_new_tokens,
                          "prompt_lengths": self.prompt_lengths, "qo_indptr_buffer": self.qo_indptr_buffer,
                          "paged_kv_indptr_buffer": self.paged_kv_indptr_buffer,
                          "paged_kv_indices_buffer": self.paged_kv_indices_buffer,
                          "paged_kv_last_page_len_buffer": self.paged_kv_last_page_len_buffer},
            profiler_tensor=self.profiler_tensor, trace_name=meta.trace_name or "", spec_decode_config=meta.spec_decode_config,
            use_cutlass_kernel=meta.use_cutlass_kernel, eos_token_id=meta.eos_token_id, **meta.extra)
        self.is_built = self.is_compiled = False
        self.returned_hidden_state = None

    def compensate_meta_tensors(self):
        """mpk.py:237-268: allocate the meta tensors the caller left out."""
        dev, R, T = self.device, self.max_num_batched_requests, self.max_num_batched_tokens
        make = {
            "step": lambda: torch.zeros(self.total_num_requests, dtype=torch.int32, device=dev),
            "tokens": lambda: torch.zeros(self.total_num_requests, self.max_seq_length, dtype=torch.int64, device=dev),
            "input_tokens": lambda: torch.zeros(T, 1, dtype=torch.int64, device=dev),
            "output_tokens": lambda: torch.zeros(T, 1, dtype=torch.int64, device=dev),
            "num_new_tokens": lambda: torch.ones(self.total_num_requests, dtype=torch.int32, device=dev),
            "prompt_lengths": lambda: torch.zeros(self.total_num_requests, dtype=torch.int32, device=dev),
            "qo_indptr_buffer": lambda: torch.zeros(R + 1, dtype=torch.int32, device=dev),
            "paged_kv_indptr_buffer": lambda: torch.zeros(R + 1, dtype=torch.int32, device=dev),
            "paged_kv_indices_buffer": lambda: torch.zeros(self.max_num_pages, dtype=torch.int32, device=dev),
            "paged_kv_last_page_len_buffer": lambda: torch.zeros(R, dtype=torch.int32, device=dev),
        }
        for k, fn in make.items():
            if getattr(self, k) is None:
                setattr(self, k, fn())

    def build(self):
        """Record the model graph (mpk.py:370-380 -> Qwen3Builder.build_from_config)."""
        mc = self.model_config
        geom = Qwen3Geometry(hidden=mc.hidden_size, n_q=mc.local_num_q_heads * self.world_size,
                             n_kv=mc.local_num_kv_heads * self.world_size, head_dim=mc.head_dim,
                             mlp=mc.intermediate_size, layers=mc.num_layers, vocab=mc.vocab_size)
        w = weights_from_state_dict(mc.state_dict, mc.num_layers)
        cos, sin = mc.position_embeddings
        out = build_qwen3_graph(self.persistent_kernel, geom, w, mc.k_cache, mc.v_cache, cos, sin, self.input_tokens,
                                self.output_tokens, lm_head=self.with_lm_head)
        if not self.with_lm_head:
            self.returned_hidden_state = out  # online_notoken without a head: the last hidden state (a DTensor)
        self.is_built = True

    def compile(self, output_dir: str = None):
        if not self.is_built:
            raise ValueError("Model is not built yet")
        self.persistent_kernel.compile(output_dir=output_dir)
        self.is_compiled = True

    def init_request_func(self):
        self.persistent_kernel.init_requests()

    init_per_request = init_request_func

    def load_new_request(self, prompt, use_template: bool = True):
        """The same prompt for every request slot (mpk.py:302-325); ``prompt`` is a 1-D tensor or list of token ids."""
        if isinstance(prompt, str):
            raise NotImplementedError("no tokenizer offline: pass token ids")
        ids = torch.as_tensor(prompt, dtype=torch.int64)
        self.tokens.zero_()
        self.tokens[:, : len(ids)] = ids.to(self.device)[None, :]
        self.prompt_lengths.fill_(len(ids))

    def clear_buffers(self):
        for t in (self.step, self.tokens, self.input_tokens, self.output_tokens, self.num_new_tokens, self.prompt_lengths,
                  self.qo_indptr_buffer, self.paged_kv_indptr_buffer, self.paged_kv_indices_buffer,
                  self.paged_kv_last_page_len_buffer):
            t.fill_(0)

    def run(self, prompt):
        """One generation for the prompt in every slot; returns the token ids of each request (mpk.py:354-368)."""
        self.load_new_request(prompt)
        self.init_request_func()
        self()
        torch.cuda.synchronize()
        return [self.tokens[r, : int(self.step[r]) + 1].clone() for r in range(self.total_num_requests)]

    def __call__(self, **kwargs):
        if not self.is_compiled:
            self.compile()
        if self.need_cpy_input:
            self.input_tokens.copy_(self.src_input_tokens.to(torch.int64))
        self.persistent_kernel(**kwargs)
        if not self.with_lm_head and self.persistent_kernel.mode == "online_notoken":
            return self.persistent_kernel.read_tensor(self.returned_hidden_state)

    def finalize(self):
        if not getattr(self.persistent_kernel, "__finalized__", True):
            self.persistent_kernel.finalize()

    def __del__(self):
        try:
            self.finalize()
        except Exception:
            pass
