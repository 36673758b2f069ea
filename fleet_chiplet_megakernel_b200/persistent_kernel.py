"""``PersistentKernel``: the reference's operator/plugin API for the decode path.

Mirror of python/mirage/mpk/persistent_kernel.py:367-2786 (constructor :368-387,
attach_input :469, new_tensor :482, fuse_tensors :505, shuffle_tensors :513,
embed_layer :521, rmsnorm_layer :544, rmsnorm_linear_layer :566,
paged_attention_layer :724, paged_attention_split_kv_layer :804, its merge :894,
linear_layer :2045, linear_with_residual_layer :2077, allreduce_layer :2115,
silu_mul_layer :2137, argmax_layer :2195, argmax_partial_layer :2207,
argmax_reduce_layer :2232, compile :2404, __call__ :2622, finalize :2782).

Same names, argument meaning and error behaviour; ``grid_dim``/``block_dim``
are accepted as hints of the reference's tiling (only silu_mul's grid carries
meaning: it fixes the [gate|up] block width).  Instead of generating and
JIT-compiling CUDA, the layers are recorded into the ahead-of-time native
runtime through the C ABI in include/b200mk.h.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np
import torch

from . import _cabi

valid_persistent_kernel_modes = {"offline", "online", "online_notoken", "onepass", "online_multi_turn"}


class dtype:
    def __init__(self, name, code, torch_dtype):
        self.name, self.code, self.torch_dtype = name, code, torch_dtype

    def __repr__(self):
        return f"mk.{self.name}"


bfloat16 = dtype("bfloat16", _cabi.MK_BF16, torch.bfloat16)
float16 = dtype("float16", _cabi.MK_F16, torch.float16)
float32 = dtype("float32", _cabi.MK_F32, torch.float32)
int32 = dtype("int32", _cabi.MK_I32, torch.int32)
int64 = dtype("int64", _cabi.MK_I64, torch.int64)
uint64 = dtype("uint64", _cabi.MK_U64, torch.uint64)
_ALL = [bfloat16, float16, float32, int32, int64, uint64]


def convert_torch_type_to_dtype(t):
    for d in _ALL:
        if d.torch_dtype == t:
            return d
    raise RuntimeError(f"Unsupported torch dtype: {t}")


class DTensor:
    """Handle of a tensor known to the runtime (the reference's DTensor)."""

    def __init__(self, tid, dims, dt, name):
        self.id, self.dims, self.dtype, self.name = tid, tuple(int(d) for d in dims), dt, name

    @property
    def num_dims(self):
        return len(self.dims)

    def dim(self, i):
        return self.dims[i]

    def __repr__(self):
        return f"DTensor({self.name}, {self.dims}, {self.dtype})"


def get_configurations_from_gpu(rank=0):
    """(num_workers, num_schedulers) for the device (python/mirage/utils.py:38-101).
    On B200 every SM is a worker; the static schedule needs no scheduler SMs."""
    if not torch.cuda.is_available():
        raise RuntimeError("get_configurations_from_gpu needs a CUDA device")
    return torch.cuda.get_device_properties(rank).multi_processor_count, 0


_META_ORDER = ["step", "tokens", "input_tokens", "output_tokens", "num_new_tokens", "prompt_lengths",
               "qo_indptr_buffer", "paged_kv_indptr_buffer", "paged_kv_indices_buffer",
               "paged_kv_last_page_len_buffer"]


class PersistentKernel:
    def __init__(
        self,
        mode: str,
        world_size: int,
        mpi_rank: int,
        num_workers: int,
        num_local_schedulers: int,
        num_remote_schedulers: int,
        max_seq_length: int,
        max_num_batched_requests: int,
        max_num_batched_tokens: int,
        max_num_pages: int,
        page_size: int,
        meta_tensors: dict,
        profiler_tensor: torch.Tensor = None,
        trace_name: str = "",
        spec_decode_config=None,
        use_cutlass_kernel: bool = True,
        eos_token_id: int = -1,
        numerics: str | None = None,
        fuse: bool | None = None,
        max_iterations: int = 0,
        timeout_ms: int = 0,
        trace_op: int = -1,
        debug_flags: int = 0,
        cluster_size: int = 0,
        max_stages: int = 0,
        prefetch_kb: int = 0,
        test_barrier_epoch: int = 0,
        max_tokens_per_request: int = 0,
    ):
        self.__finalized__ = False
        self._is_compiled = False
        self._h = None
        if mode not in valid_persistent_kernel_modes:
            raise ValueError(f"Invalid persistent kernel mode: {mode}")
        if mode == "online":
            # the reference's single-request loop that advances `step` by new_token_nums[0] and never touches the
            # paging metadata (persistent_kernel.cuh:538-567): superseded there by offline / online_notoken
            raise NotImplementedError("mode 'online' is not built; use 'offline' or 'online_notoken'")
        # 'online_multi_turn' is one pass per call over the caller's metadata, like 'online_notoken': the reference's
        # runtime reads its MODE_MULTI_TURN switch only beside MODE_ONLINE_NOTOKEN (runtime_header.h:43) and gives it
        # no batching code of its own
        if spec_decode_config is not None:
            raise NotImplementedError("speculative decoding is outside the greedy decode path")
        self.mode = mode
        self.world_size = world_size
        self.mpi_rank = mpi_rank
        self.num_workers = num_workers
        self.num_local_schedulers = num_local_schedulers
        self.num_remote_schedulers = num_remote_schedulers
        self.max_seq_length = max_seq_length
        self.max_num_batched_requests = max_num_batched_requests
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_num_pages = max_num_pages
        self.page_size = page_size
        self.eos_token_id = eos_token_id
        self.meta_tensors = meta_tensors
        self.profiler_tensor = profiler_tensor
        self.trace_name = trace_name
        self.use_nvshmem = world_size > 1
        self.use_cutlass_kernel = use_cutlass_kernel
        self.target_cc = 100
        for k in _META_ORDER:
            if k not in meta_tensors:
                raise KeyError(f"meta_tensors['{k}'] is required")
        self.total_num_requests = meta_tensors["tokens"].shape[0]
        assert self.max_seq_length == meta_tensors["tokens"].shape[1]
        qo = meta_tensors["qo_indptr_buffer"]
        assert qo.shape[0] <= max_num_batched_requests + 1, f"qo_indptr_buffer.shape: {qo.shape}"
        kvp = meta_tensors["paged_kv_indptr_buffer"]
        assert kvp.shape[0] <= max_num_batched_requests + 1, f"paged_kv_indptr_buffer.shape: {kvp.shape}"
        assert meta_tensors["paged_kv_indices_buffer"].shape[0] <= max_num_pages
        assert meta_tensors["paged_kv_last_page_len_buffer"].shape[0] <= max_num_batched_requests
        # the runtime writes max_num_batched_requests+1 index pointers
        assert qo.shape[0] == max_num_batched_requests + 1 and kvp.shape[0] == max_num_batched_requests + 1, \
            "qo_indptr_buffer / paged_kv_indptr_buffer must hold max_num_batched_requests + 1 entries"
        assert meta_tensors["paged_kv_indices_buffer"].shape[0] == max_num_pages
        for k, dt in (("tokens", torch.int64), ("input_tokens", torch.int64), ("output_tokens", torch.int64),
                      ("num_new_tokens", torch.int32), ("prompt_lengths", torch.int32), ("step", torch.int32),
                      ("qo_indptr_buffer", torch.int32), ("paged_kv_indptr_buffer", torch.int32),
                      ("paged_kv_indices_buffer", torch.int32), ("paged_kv_last_page_len_buffer", torch.int32)):
            assert meta_tensors[k].dtype == dt, f"{k}.dtype: {meta_tensors[k].dtype}"

        if numerics is None:
            numerics = os.environ.get("B200MK_NUMERICS", "torch")
        if numerics not in ("torch", "mpk"):
            raise ValueError("numerics must be 'torch' or 'mpk'")
        if fuse is None:
            fuse = os.environ.get("B200MK_FUSE", "1") != "0"
        self.numerics = numerics
        self._lib = _cabi.load()
        cfg = _cabi.MkConfig()
        cfg.mode = _cabi.MK_MODE_OFFLINE if mode == "offline" else _cabi.MK_MODE_ONEPASS
        cfg.world_size, cfg.rank = world_size, mpi_rank
        cfg.num_workers = int(num_workers or 0)
        cfg.max_seq_length = max_seq_length
        cfg.max_num_batched_requests = max_num_batched_requests
        cfg.max_num_batched_tokens = max_num_batched_tokens
        cfg.max_num_pages, cfg.page_size = max_num_pages, page_size
        cfg.numerics = _cabi.MK_NUMERICS_TORCH if numerics == "torch" else _cabi.MK_NUMERICS_MPK
        cfg.eos_token_id = int(eos_token_id)
        cfg.fuse = 1 if fuse else 0
        cfg.max_iterations = int(max_iterations)
        cfg.timeout_ms = int(timeout_ms)
        cfg.device = -1
        cfg.max_tokens_per_request = int(max_tokens_per_request)
        cfg.trace_op = int(trace_op) + 1
        # measurement / test aids: explicit arguments only (never read from the environment)
        cfg.debug_flags = int(debug_flags)
        cfg.max_stages = int(max_stages)
        cfg.prefetch_kb = int(prefetch_kb)
        cfg.cluster_size = int(cluster_size)
        cfg.test_barrier_epoch = int(test_barrier_epoch) & 0xFFFFFFFF
        self._h = self._lib.mk_create(C.byref(cfg))
        if not self._h:
            raise RuntimeError("mk_create failed")
        self._keepalive = []
        self._names = set()

    # -- helpers -------------------------------------------------------------------------
    def _err(self):
        buf = C.create_string_buffer(1024)
        self._lib.mk_last_error(self._h, buf, 1024)
        return buf.value.decode()

    def _check(self, rc, what):
        if rc >= 0:
            return rc
        msg = f"{what}: {self._err()}"
        if rc == _cabi.MK_E_UNSUPPORTED:
            raise NotImplementedError(msg)
        if rc == _cabi.MK_E_INVALID:
            raise ValueError(msg)
        raise RuntimeError(msg)

    def _op(self, name, tensors, params=(), grid_dim=(1, 1, 1), block_dim=(1, 1, 1)):
        ids = _cabi.int_array([t.id for t in tensors])
        prm = _cabi.i64_array(list(params)) if len(params) else None
        g = _cabi.int_array(list(grid_dim) + [1] * (3 - len(grid_dim)))
        b = _cabi.int_array(list(block_dim) + [1] * (3 - len(block_dim)))
        self._check(self._lib.mk_op(self._h, name.encode(), ids, len(tensors), prm, len(params), g, b), name)

    # -- tensors -------------------------------------------------------------------------
    def attach_input(self, torch_tensor: torch.Tensor, name: str = None) -> DTensor:
        dims = tuple(int(d) for d in torch_tensor.shape)
        strides = tuple(int(s) for s in torch_tensor.stride())
        for d in range(len(dims) - 1):
            assert strides[d] == strides[d + 1] * dims[d + 1]
        dt = convert_torch_type_to_dtype(torch_tensor.dtype)
        assert name is not None
        tid = self._check(self._lib.mk_tensor_attach(self._h, name.encode(), C.c_void_p(torch_tensor.data_ptr()),
                                                     dt.code, len(dims), _cabi.i64_array(dims),
                                                     _cabi.i64_array(strides)), f"attach_input({name})")
        self._keepalive.append(torch_tensor)  # borrowed by raw pointer until finalize
        return DTensor(tid, dims, dt, name)

    def new_tensor(self, dims: tuple, strides: tuple = None, dtype: dtype = bfloat16, name: str = None,
                   io_category: str = "cuda_tensor") -> DTensor:
        assert name is not None
        if io_category == "cuda_tensor":
            cat = _cabi.MK_CAT_CUDA
        elif io_category == "nvshmem_tensor":
            cat = _cabi.MK_CAT_SYMMETRIC
        else:
            raise RuntimeError(f"Invalid io_category: {io_category}")
        st = _cabi.i64_array(strides) if strides is not None else None
        tid = self._check(self._lib.mk_tensor_new(self._h, name.encode(), dtype.code, len(dims),
                                                  _cabi.i64_array(dims), st, cat), f"new_tensor({name})")
        return DTensor(tid, dims, dtype, name)

    def fuse_tensors(self, inputs: list, fused_dim: int, num_groups: int, name: str = None) -> DTensor:
        assert fused_dim == 0
        ids = _cabi.int_array([t.id for t in inputs])
        tid = self._check(self._lib.mk_tensor_fuse(self._h, (name or "fused").encode(), ids, len(inputs), fused_dim,
                                                   num_groups), "fuse_tensors")
        return DTensor(tid, (sum(t.dim(0) for t in inputs),) + inputs[0].dims[1:], inputs[0].dtype, name)

    def shuffle_tensors(self, inputs: list, shuffled_dim: int, num_groups: int, name: str = None) -> DTensor:
        assert shuffled_dim == 0
        ids = _cabi.int_array([t.id for t in inputs])
        tid = self._check(self._lib.mk_tensor_shuffle(self._h, (name or "shuffled").encode(), ids, len(inputs),
                                                      shuffled_dim, num_groups), "shuffle_tensors")
        return DTensor(tid, (sum(t.dim(0) for t in inputs),) + inputs[0].dims[1:], inputs[0].dtype, name)

    # -- layers --------------------------------------------------------------------------
    def embed_layer(self, input: DTensor, weight: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple,
                    input_source: int = 0):
        self._op("embedding", [input, weight, output], [input_source], grid_dim, block_dim)

    def rmsnorm_layer(self, input: DTensor, weight: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2
        assert output.num_dims == 2
        self._op("rmsnorm", [input, weight, output], (), grid_dim, block_dim)

    def rmsnorm_linear_layer(self, input: DTensor, weight_norm: DTensor, weight_linear: DTensor, output: DTensor,
                             grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2
        assert weight_linear.num_dims == 2
        assert output.num_dims == 2
        self._op("rmsnorm_linear", [input, weight_norm, weight_linear, output], (), grid_dim, block_dim)

    def _attention_params(self, k_cache, q_norm, k_norm, cos_pos_embed, sin_pos_embed, num_q_heads):
        head_dim = k_cache.dim(3)
        num_kv_heads = k_cache.dim(2)
        rotary_embed = 0
        if cos_pos_embed is not None or sin_pos_embed is not None:
            assert cos_pos_embed.num_dims == 2
            assert sin_pos_embed.num_dims == 2
            assert cos_pos_embed.dim(1) == head_dim
            assert sin_pos_embed.dim(1) == head_dim
            rotary_embed = 1
        qk_norm = 0
        if q_norm is not None or k_norm is not None:
            assert q_norm.num_dims == 1
            assert k_norm.num_dims == 1
            qk_norm = 1
            assert q_norm.dim(0) == head_dim
            assert k_norm.dim(0) == head_dim
        if not (rotary_embed and qk_norm):
            raise NotImplementedError("the attention task is built with QK-norm and RoPE (Qwen3)")
        return [num_q_heads, num_kv_heads, qk_norm, rotary_embed, self.max_seq_length, self.page_size]

    def paged_attention_layer(self, input: DTensor, k_cache: DTensor, v_cache: DTensor, q_norm: DTensor,
                              k_norm: DTensor, cos_pos_embed: DTensor, sin_pos_embed: DTensor, output: DTensor,
                              grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2
        assert output.num_dims == 2
        assert k_cache.num_dims == 4
        assert v_cache.num_dims == 4
        assert k_cache.dim(0) == self.max_num_pages
        assert v_cache.dim(0) == self.max_num_pages
        assert k_cache.dim(1) == self.page_size
        assert v_cache.dim(1) == self.page_size
        num_q_heads = output.dim(1) // k_cache.dim(3)
        params = self._attention_params(k_cache, q_norm, k_norm, cos_pos_embed, sin_pos_embed, num_q_heads)
        assert grid_dim[0] == self.max_num_batched_requests
        assert grid_dim[1] == k_cache.dim(2)
        self._op("paged_attention", [input, k_cache, v_cache, q_norm, k_norm, cos_pos_embed, sin_pos_embed, output],
                 params, grid_dim, block_dim)

    def paged_attention_split_kv_layer(self, input: DTensor, k_cache: DTensor, v_cache: DTensor, q_norm: DTensor,
                                       k_norm: DTensor, cos_pos_embed: DTensor, sin_pos_embed: DTensor,
                                       lse: DTensor, output: DTensor, attention_params: tuple, grid_dim: tuple,
                                       block_dim: tuple):
        assert input.num_dims == 2
        assert k_cache.num_dims == 4
        assert v_cache.num_dims == 4
        assert k_cache.dim(0) == self.max_num_pages
        assert v_cache.dim(0) == self.max_num_pages
        assert k_cache.dim(1) == self.page_size
        assert v_cache.dim(1) == self.page_size
        assert output.num_dims == 3
        assert lse.num_dims == 3
        num_q_heads, num_kv_chunks = attention_params[0], attention_params[1]
        params = self._attention_params(k_cache, q_norm, k_norm, cos_pos_embed, sin_pos_embed, num_q_heads)
        params.append(num_kv_chunks)
        assert grid_dim[0] == self.max_num_batched_requests
        assert grid_dim[1] == k_cache.dim(2)
        self._op("paged_attention_split_kv",
                 [input, k_cache, v_cache, q_norm, k_norm, cos_pos_embed, sin_pos_embed, lse, output],
                 params, grid_dim, block_dim)

    def paged_attention_split_kv_merge_layer(self, lse: DTensor, output_tmp: DTensor, output: DTensor,
                                             attention_params: tuple, grid_dim: tuple, block_dim: tuple):
        assert lse.num_dims == 3
        assert output_tmp.num_dims == 3
        assert output.num_dims == 2
        num_q_heads, head_dim = attention_params[0], attention_params[1]
        params = [num_q_heads // grid_dim[1], head_dim, self.max_seq_length, self.page_size, grid_dim[1]]
        self._op("paged_attention_split_kv_merge", [lse, output_tmp, output], params, grid_dim, block_dim)

    def linear_layer(self, input: DTensor, weight: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2
        assert weight.num_dims == 2
        assert output.num_dims == 2
        self._op("linear", [input, weight, output], (), grid_dim, block_dim)

    def linear_with_residual_layer(self, input: DTensor, weight: DTensor, residual: DTensor, output: DTensor,
                                   grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2
        assert weight.num_dims == 2
        assert residual.num_dims == 2
        assert output.num_dims == 2
        self._op("linear_with_residual", [input, weight, residual, output], (), grid_dim, block_dim)

    def allreduce_layer(self, input: DTensor, buffer: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2
        assert buffer.num_dims == 3
        assert output.num_dims == 2
        self._op("allreduce", [input, buffer, output], [self.world_size, self.mpi_rank], grid_dim, block_dim)

    def silu_mul_layer(self, input: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2
        assert output.num_dims == 2
        self._op("silu_mul", [input, output], (), grid_dim, block_dim)

    # -- aliases of the layers above ----------------------------------------------------
    # The reference has one method per tiling strategy of the same operator: the split-K
    # linears its model builder picks on Hopper/Blackwell (persistent_kernel.py:1437, 1901,
    # 1920), the fused SiLU/linear forms (:1716, :2174) and Fleet's gang_* family for MI300
    # (:1064-1899), whose extra arguments (tile_n, m_tiles, wgm/wgn, k_splits, workspaces,
    # done counters) describe how ITS kernels tile the work.  Here the runtime chooses the
    # split of every linear itself (row-owner, stream-K or tcgen05 tiles by batch size), so
    # these methods accept the same arguments, keep the tensors' meaning, and record the
    # reference's task name; the native planner folds each onto the plain device op.  The
    # reference asserts target_cc == 94 in the gang_* methods; that check is dropped because
    # the layers are architecture-neutral here.
    def attention_layer(self, input: DTensor, k_cache: DTensor, v_cache: DTensor, q_norm: DTensor, k_norm: DTensor,
                        cos_pos_embed: DTensor, sin_pos_embed: DTensor, output: DTensor, grid_dim: tuple,
                        block_dim: tuple):
        """persistent_kernel.py:587-651: decode attention over a per-request contiguous cache
        [requests, seq_len, kv_heads, head_dim].  Served by the paged task with one page per
        request, so the cache must be laid out as [max_num_pages, page_size, kv_heads, head_dim]
        with page_size >= max_seq_length."""
        assert input.num_dims == 2
        assert output.num_dims == 2
        assert k_cache.num_dims == 4
        assert v_cache.num_dims == 4
        num_q_heads = output.dim(1) // k_cache.dim(3)
        params = self._attention_params(k_cache, q_norm, k_norm, cos_pos_embed, sin_pos_embed, num_q_heads)[:4]
        if k_cache.dim(0) != self.max_num_pages or k_cache.dim(1) != self.page_size or \
                self.page_size < self.max_seq_length:
            raise NotImplementedError("attention_layer: the contiguous cache must be [max_num_pages, page_size >= "
                                      "max_seq_length, kv_heads, head_dim] (one page per request)")
        self._op("attention", [input, k_cache, v_cache, q_norm, k_norm, cos_pos_embed, sin_pos_embed, output],
                 params, grid_dim, block_dim)

    def gang_paged_attention_split_kv_layer(self, input: DTensor, k_cache: DTensor, v_cache: DTensor, q_norm: DTensor,
                                            k_norm: DTensor, cos_pos_embed: DTensor, sin_pos_embed: DTensor,
                                            lse: DTensor, output: DTensor, q_workspace: DTensor,
                                            attention_params: tuple, block_dim: tuple):
        """persistent_kernel.py:1064-1139."""
        assert input.num_dims == 2
        assert k_cache.num_dims == 4
        assert v_cache.num_dims == 4
        num_q_heads, num_kv_chunks = attention_params[0], attention_params[1]
        params = self._attention_params(k_cache, q_norm, k_norm, cos_pos_embed, sin_pos_embed, num_q_heads)
        params.append(num_kv_chunks)
        self._op("gang_attn_split_kv_mi300",
                 [input, k_cache, v_cache, q_norm, k_norm, cos_pos_embed, sin_pos_embed, lse, output, q_workspace],
                 params, (8, 1, 1), block_dim)

    def gang_paged_attention_split_kv_merge_layer(self, lse: DTensor, output_tmp: DTensor, output: DTensor,
                                                  attention_params: tuple, block_dim: tuple):
        """persistent_kernel.py:1141-1181."""
        assert lse.num_dims == 2
        assert output_tmp.num_dims == 2
        assert output.num_dims == 2
        num_q_heads, head_dim, num_kv_heads, num_kv_chunks = attention_params[:4]
        params = [num_q_heads // num_kv_heads, head_dim, self.max_seq_length, self.page_size, num_kv_heads,
                  num_kv_chunks]
        self._op("gang_attn_merge_mi300", [lse, output_tmp, output], params, (8, 1, 1), block_dim)

    def splitk_linear_layer(self, input: DTensor, weight: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        """persistent_kernel.py:1437-1466.  On sm_100 the reference's k-splits add into ``output``
        (which holds the residual stream); followed by ``splitk_reduce_layer`` the output is a
        workspace instead.  Either way: one linear-with-residual device op."""
        assert input.num_dims == 2
        assert weight.num_dims == 2
        assert output.num_dims == 2
        self._op("splitk_linear_sm100", [input, weight, output], (), grid_dim, block_dim)

    def splitk_reduce_layer(self, workspace: DTensor, residual: DTensor, output: DTensor, k_splits: int,
                            grid_dim: tuple, block_dim: tuple):
        """persistent_kernel.py:1901-1918; must directly follow the splitk_linear_layer that writes ``workspace``."""
        assert workspace.num_dims == 2
        assert residual.num_dims == 2
        assert output.num_dims == 2
        self._op("splitk_reduce_mi300", [workspace, residual, output], [k_splits], grid_dim, block_dim)

    def splitk_linear_res_atomic_layer(self, input: DTensor, weight: DTensor, residual: DTensor, workspace: DTensor,
                                       done_counter: DTensor, output: DTensor, k_splits: int, grid_dim: tuple,
                                       block_dim: tuple):
        """persistent_kernel.py:1920-1951."""
        assert input.num_dims == 2
        assert weight.num_dims == 2
        self._op("splitk_linear_res_atomic_mi300", [input, weight, residual, workspace, done_counter, output],
                 [k_splits], grid_dim, block_dim)

    def silu_mul_linear_with_residual_layer(self, input: DTensor, weight: DTensor, residual: DTensor, output: DTensor,
                                            grid_dim: tuple, block_dim: tuple):
        """persistent_kernel.py:2174-2193: SiLU(gate) * up of an input row [gate | up], then the
        linear layer with residual."""
        assert input.num_dims == 2
        assert weight.num_dims == 2
        assert residual.num_dims == 2
        self._op("silu_mul_linear_with_residual", [input, weight, residual, output], (), grid_dim, block_dim)

    def linear_silu_layer(self, input: DTensor, weight: DTensor, output: DTensor, output_stride: int, tile_n: int = 64,
                          m_tiles: int = 1, wgm: int = 0, block_dim: tuple = (256, 1, 1)):
        """persistent_kernel.py:1716-1735: gate/up linear with SiLU(gate) * up in the epilogue;
        ``weight`` is shuffle_tensors([gate, up])."""
        assert input.num_dims == 2
        assert weight.num_dims == 2
        assert output.num_dims == 2
        self._op("linear_silu_mi300", [input, weight, output], [output_stride, tile_n, m_tiles, wgm], (1, 1, 1), block_dim)

    def gang_rmsnorm_layer(self, input: DTensor, weight: DTensor, output: DTensor, block_dim: tuple = (128, 1, 1)):
        """persistent_kernel.py:1553-1569."""
        self._op("gang_rmsnorm_mi300", [input, weight, output], [input.dim(0)], (8, 1, 1), block_dim)

    def _gang_linear(self, task, input, weight, residual, output, hints, block_dim, workspace=None):
        assert input.num_dims == 2
        assert weight.num_dims == 2
        assert output.num_dims == 2
        tensors = [input, weight] + ([residual] if residual is not None else []) + \
                  ([workspace] if workspace is not None else []) + [output]
        self._op(task, tensors, [int(h) for h in hints], (8, 1, 1), block_dim)

    def gang_linear_layer(self, input: DTensor, weight: DTensor, output: DTensor, tile_n: int, output_stride: int,
                          m_tiles: int = 1, wgm: int = 0, block_dim: tuple = (256, 1, 1)):
        """persistent_kernel.py:1571-1616."""
        self._gang_linear("gang_linear_mi300", input, weight, None, output, (output_stride, tile_n, m_tiles, wgm), block_dim)

    def gang_linear_n_tiling_layer(self, input: DTensor, weight: DTensor, output: DTensor, tile_n: int,
                                   output_stride: int, m_tiles: int = 1, wgn: int = 0, block_dim: tuple = (256, 1, 1)):
        """persistent_kernel.py:1618-1668."""
        self._gang_linear("gang_linear_n_tiling_mi300", input, weight, None, output, (output_stride, tile_n, m_tiles, wgn), block_dim)

    def gang_linear_msplit_layer(self, input: DTensor, weight: DTensor, output: DTensor, tile_n: int,
                                 output_stride: int, m_tiles: int = 2, block_dim: tuple = (256, 1, 1)):
        """persistent_kernel.py:1782-1815."""
        self._gang_linear("gang_linear_msplit_mi300", input, weight, None, output, (output_stride, tile_n, m_tiles), block_dim)

    def gang_linear_silu_layer(self, input: DTensor, weight: DTensor, output: DTensor, tile_n: int, output_stride: int,
                               m_tiles: int = 1, wgm: int = 0, block_dim: tuple = (256, 1, 1)):
        """persistent_kernel.py:1852-1899: gate/up linear with SiLU(gate) * up in the epilogue."""
        self._gang_linear("gang_linear_silu_mi300", input, weight, None, output, (output_stride, tile_n, m_tiles, wgm), block_dim)

    def gang_linear_with_residual_layer(self, input: DTensor, weight: DTensor, residual: DTensor, output: DTensor,
                                        tile_n: int, output_stride: int, m_tiles: int = 1, wgm: int = 0,
                                        block_dim: tuple = (256, 1, 1)):
        """persistent_kernel.py:1670-1714."""
        self._gang_linear("gang_linear_res_mi300", input, weight, residual, output, (output_stride, tile_n, m_tiles, wgm), block_dim)

    def gang_linear_with_residual_n_tiling_layer(self, input: DTensor, weight: DTensor, residual: DTensor,
                                                 output: DTensor, tile_n: int, output_stride: int, m_tiles: int = 1,
                                                 wgn: int = 0, block_dim: tuple = (256, 1, 1)):
        """persistent_kernel.py:1737-1780."""
        self._gang_linear("gang_linear_res_n_tiling_mi300", input, weight, residual, output, (output_stride, tile_n, m_tiles, wgn), block_dim)

    def gang_linear_with_residual_msplit_layer(self, input: DTensor, weight: DTensor, residual: DTensor,
                                               output: DTensor, tile_n: int, output_stride: int, m_tiles: int = 2,
                                               block_dim: tuple = (256, 1, 1)):
        """persistent_kernel.py:1817-1850."""
        self._gang_linear("gang_linear_res_msplit_mi300", input, weight, residual, output, (output_stride, tile_n, m_tiles), block_dim)

    def gang_ksplit_linear_with_residual_layer(self, input: DTensor, weight: DTensor, residual: DTensor,
                                               workspace: DTensor, output: DTensor, tile_n: int, output_stride: int,
                                               k_splits: int = 8, block_dim: tuple = (256, 1, 1)):
        """persistent_kernel.py:1468-1513."""
        self._gang_linear("gang_ksplit_gemm_mi300", input, weight, residual, output, (output_stride, tile_n, k_splits), block_dim,
                          workspace=workspace)

    def gang_splitk_linear_with_residual_layer(self, input: DTensor, weight: DTensor, residual: DTensor,
                                               workspace: DTensor, output: DTensor, tile_n: int, output_stride: int,
                                               k_splits: int = 4, block_dim: tuple = (256, 1, 1)):
        """persistent_kernel.py:1515-1551."""
        self._gang_linear("gang_splitk_linear_res_mi300", input, weight, residual, output, (output_stride, tile_n, k_splits), block_dim,
                          workspace=workspace)

    # -- mixture of experts (persistent_kernel.py:1183-1435) ---------------------------------
    def tensor_init_layer(self, input: DTensor, dummy_input: DTensor, dummy_output: DTensor, grid_dim: tuple,
                          block_dim: tuple):
        """persistent_kernel.py:1183-1201: the reference zeroes a buffer its expert tasks accumulate into.
        Accepted and dropped: nothing accumulates in place in this runtime."""
        assert input.num_dims == 2
        self._op("tensor_init", [input, dummy_input, dummy_output], (), grid_dim, block_dim)

    def moe_topk_softmax_routing_layer(self, input: DTensor, output: tuple, grid_dim: tuple, block_dim: tuple):
        """persistent_kernel.py:1203-1227: router logits [tokens, experts] -> softmax, top-k, renormalised weights.
        ``output`` = (topk weights [tokens, k], routing indices [experts, tokens], mask [experts + 1]); the last two
        describe the reference's grouping of tokens per expert and are accepted, not written."""
        assert input.num_dims == 2
        assert len(output) == 3
        moe_topk_weight, moe_routing_indices, moe_masks = output
        assert moe_topk_weight.num_dims == 2
        assert moe_routing_indices.num_dims == 2
        assert moe_masks.num_dims == 1
        self._op("moe_topk_softmax_sm100", [input, moe_topk_weight, moe_routing_indices, moe_masks], (), grid_dim, block_dim)

    def moe_w13_linear_layer(self, input: DTensor, weight: DTensor, moe_routing_indices: DTensor, moe_mask: DTensor,
                             output: DTensor, grid_dim: tuple, block_dim: tuple):
        """persistent_kernel.py:1229-1260: per (token, slot): [gate | up] = W13[expert] x."""
        assert input.num_dims == 2
        assert weight.num_dims == 3
        assert moe_routing_indices.num_dims == 2
        assert moe_mask.num_dims == 1
        assert output.num_dims == 3
        self._op("moe_w13_linear_sm100", [input, weight, moe_routing_indices, moe_mask, output], (), grid_dim, block_dim)

    def moe_silu_mul_layer(self, input: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        """persistent_kernel.py:1262-1276."""
        assert input.num_dims == 3
        assert output.num_dims == 3
        self._op("moe_silu_mul", [input, output], (), grid_dim, block_dim)

    def moe_w2_linear_layer(self, input: DTensor, weight: DTensor, moe_routing_indices: DTensor, moe_mask: DTensor,
                            output: DTensor, grid_dim: tuple, block_dim: tuple):
        """persistent_kernel.py:1278-1309: per (token, slot): W2[expert] act."""
        assert input.num_dims == 3
        assert weight.num_dims == 3
        assert moe_routing_indices.num_dims == 2
        assert moe_mask.num_dims == 1
        assert output.num_dims == 3
        self._op("moe_w2_linear_sm100", [input, weight, moe_routing_indices, moe_mask, output], (), grid_dim, block_dim)

    def gang_moe_w13_linear_layer(self, input: DTensor, weight: DTensor, moe_routing_indices: DTensor, moe_mask: DTensor,
                                  output: DTensor, block_dim: tuple = (256, 1, 1)):
        """persistent_kernel.py:1311-1359 (Fleet's per-XCD expert ganging: the plain layer here)."""
        self.moe_w13_linear_layer(input, weight, moe_routing_indices, moe_mask, output, (8, 1, 1), block_dim)

    def gang_moe_w2_linear_layer(self, input: DTensor, weight: DTensor, moe_routing_indices: DTensor, moe_mask: DTensor,
                                 output: DTensor, block_dim: tuple = (256, 1, 1)):
        """persistent_kernel.py:1361-1409."""
        self.moe_w2_linear_layer(input, weight, moe_routing_indices, moe_mask, output, (8, 1, 1), block_dim)

    def moe_mul_sum_add_layer(self, input: DTensor, weight: DTensor, residual: DTensor, output: DTensor, grid_dim: tuple,
                              block_dim: tuple):
        """persistent_kernel.py:1411-1435: out[t] = sum over slots of weight[t, slot] * input[t, slot] + residual[t]."""
        assert input.num_dims == 3
        assert weight.num_dims == 2
        assert residual.num_dims == 2
        assert output.num_dims == 2
        self._op("moe_mul_sum_add_sm100", [input, weight, residual, output], (), grid_dim, block_dim)

    def argmax_layer(self, input: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2
        assert output.num_dims == 2
        self._op("argmax", [input, output], (), grid_dim, block_dim)

    def argmax_partial_layer(self, input: DTensor, output: tuple, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2
        assert len(output) == 2
        output_value, output_index = output
        assert output_value.num_dims == 2
        assert output_index.num_dims == 2
        num_tasks = grid_dim[0]
        self.argmax_partial_output_size = input.dim(1) // num_tasks
        self._op("argmax_partial", [input, output_value, output_index], [num_tasks], grid_dim, block_dim)

    def argmax_reduce_layer(self, input: tuple, output: DTensor, grid_dim: tuple, block_dim: tuple,
                            vocab_offset: int = 0, across_ranks: bool = False):
        """persistent_kernel.py:2232-2257.  Beyond the reference (which replicates the LM head on every
        rank): with ``across_ranks`` the input holds the partials of this rank's slice of the vocabulary,
        starting at ``vocab_offset``; the ranks exchange their best (value, index) pairs over NVLink inside
        the kernel and every rank writes the same global token."""
        assert len(input) == 2
        input_value, input_index = input
        assert input_value.num_dims == 2
        assert input_index.num_dims == 2
        assert output.num_dims == 2
        self._op("argmax_reduce", [input_value, input_index, output],
                 [getattr(self, "argmax_partial_output_size", 0), int(vocab_offset), 1 if across_ranks else 0],
                 grid_dim, block_dim)

    # -- compile / run -------------------------------------------------------------------
    def plan(self) -> str:
        """Host-only lowering; returns one line per device op (no GPU needed)."""
        self._check(self._lib.mk_plan(self._h), "plan")
        buf = C.create_string_buffer(1 << 20)
        self._check(self._lib.mk_describe(self._h, buf, 1 << 20), "describe")
        return buf.value.decode()

    def describe(self) -> str:
        """The device-op list of a planned or compiled graph, one line per op."""
        buf = C.create_string_buffer(1 << 20)
        self._check(self._lib.mk_describe(self._h, buf, 1 << 20), "describe")
        return buf.value.decode()

    def compile(self, output_dir: str = None, **kwargs):
        assert not self._is_compiled
        if not torch.cuda.is_available():
            raise RuntimeError("compile() needs a CUDA device (sm_100); there is no CPU fallback")
        ptrs = (C.c_void_p * 10)(*[C.c_void_p(self.meta_tensors[k].data_ptr()) for k in _META_ORDER])
        prof = C.c_void_p(self.profiler_tensor.data_ptr()) if self.profiler_tensor is not None else None
        self._check(self._lib.mk_set_meta(self._h, ptrs, self.total_num_requests, prof), "set_meta")
        if self.profiler_tensor is not None:
            assert self.profiler_tensor.dtype in (torch.uint64, torch.int64)
            self._check(self._lib.mk_set_profiler(self._h, prof, self.profiler_tensor.numel()), "set_profiler")
        if self.world_size > 1:
            self._exchange_handles()
        self._check(self._lib.mk_compile(self._h), "compile")
        self._is_compiled = True
        if self.world_size > 1:
            import torch.distributed as dist
            dist.barrier()  # every rank's exchange region exists and is mapped before anyone launches

    def _exchange_handles(self):
        """Tensor parallel set-up: gather the CUDA IPC handles of all ranks' exchange regions over
        torch.distributed (the reference bootstraps NVSHMEM over MPI, persistent_kernel.cuh:2002-2015)."""
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError("world_size > 1 needs an initialised torch.distributed process group")
        if dist.get_world_size() != self.world_size or dist.get_rank() != self.mpi_rank:
            raise ValueError("world_size / mpi_rank differ from the torch.distributed group")
        mine = (C.c_ubyte * 64)()
        need = self._check(self._lib.mk_comm_prepare(self._h, mine), "comm_prepare")
        if need == 0:
            return
        gathered = [None] * self.world_size
        dist.all_gather_object(gathered, bytes(mine))
        blob = b"".join(gathered)
        arr = (C.c_ubyte * len(blob)).from_buffer_copy(blob)
        self._check(self._lib.mk_comm_connect(self._h, arr, self.world_size), "comm_connect")

    def init_requests(self, stream=None):
        s = stream if stream is not None else torch.cuda.current_stream()
        self._check(self._lib.mk_init_requests(self._h, C.c_void_p(s.cuda_stream)), "init_requests")

    def __call__(self, **kwargs):
        stream = kwargs.get("default_stream", None)
        if stream is None:
            stream = torch.cuda.current_stream()
        elif not isinstance(stream, torch.cuda.Stream):
            raise ValueError("default_stream must be a torch.cuda.Stream")
        assert self._is_compiled, "compile() must be called first"
        self._check(self._lib.mk_launch(self._h, C.c_void_p(stream.cuda_stream)), "launch")

    def launch_async(self, stream=None):
        s = stream if stream is not None else torch.cuda.current_stream()
        self._check(self._lib.mk_launch_async(self._h, C.c_void_p(s.cuda_stream)), "launch")

    def wait(self, stream=None):
        s = stream if stream is not None else torch.cuda.current_stream()
        self._check(self._lib.mk_wait(self._h, C.c_void_p(s.cuda_stream)), "megakernel")

    def get_event_timing(self, max_entries=16384):
        """Per-iteration (start time ns, active tokens) of the last launch; the last
        row is the time the generation ended."""
        buf = (C.c_uint64 * (2 * max_entries))()
        n = self._check(self._lib.mk_get_event_timing(self._h, buf, max_entries), "get_event_timing")
        return np.ctypeslib.as_array(buf)[: 2 * n].reshape(n, 2).copy()

    def num_device_ops(self):
        return self._check(self._lib.mk_num_device_ops(self._h), "num_device_ops")

    def op_trace(self):
        """The profiler tensor as [ops + 1, grid, 4] int64 ns (row `ops` = iteration prologue)."""
        assert self.profiler_tensor is not None and self._is_compiled
        n, g = self.num_device_ops() + 1, self.grid_size()
        return self.profiler_tensor.view(torch.int64)[: n * g * 4].reshape(n, g, 4).cpu()

    def grid_size(self):
        return self._check(self._lib.mk_grid_size(self._h), "grid_size")

    def weight_bytes_per_step(self):
        return int(self._lib.mk_weight_bytes_per_step(self._h))

    def tensor_ptr(self, t: DTensor):
        return self._lib.mk_tensor_ptr(self._h, t.id)

    def read_tensor(self, t: DTensor) -> torch.Tensor:
        """Host copy of a tensor the runtime knows (its own intermediates included)."""
        out = torch.empty(t.dims, dtype=t.dtype.torch_dtype)
        self._check(self._lib.mk_tensor_read(self._h, t.id, C.c_void_p(out.data_ptr()),
                                             out.numel() * out.element_size()), "read_tensor")
        return out

    def finalize(self):
        assert not self.__finalized__
        if self.world_size > 1 and self._is_compiled:
            import torch.distributed as dist
            if dist.is_initialized():
                dist.barrier()  # nobody unmaps a region a peer may still be writing
        if self._h:
            self._lib.mk_finalize(self._h)
            self._h = None
        self._keepalive = []
        self.__finalized__ = True

    def __del__(self):
        if not getattr(self, "__finalized__", True) and getattr(self, "_h", None):
            try:
                self.finalize()
            except Exception:
                pass
