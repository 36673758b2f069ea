"""Op functions of the DSL (python/mirage/mpk/dsl/ops.py of the reference): each records one or two
layers on the graph's PersistentKernel and returns its output tensor.

``linear`` takes a ``strategy``: "auto" asks the cost model (on B200: row_owner / stream_k / tcgen05, all
recorded as the plain layer, because the native runtime makes that split itself), the reference's names
("standard", "gang", "gang_splitk", "gang_coop") record the reference's corresponding layer method, whose
tiling arguments the runtime accepts as hints."""
import torch

from .cost_model import B200_STRATEGIES, select_k_splits, select_strategy


def _mpk(t):
    return t.graph.mpk


def rmsnorm(x, weight, output):
    mpk = _mpk(x)
    mpk.rmsnorm_layer(input=x.dt, weight=weight.dt, output=output.dt, grid_dim=(mpk.max_num_batched_tokens, 1, 1),
                      block_dim=(128, 1, 1))
    return output


def embed(x, weight, output, input_source=1):
    _mpk(x).embed_layer(input=x.dt, weight=weight.dt, output=output.dt, grid_dim=(1, 1, 1), block_dim=(128, 1, 1),
                        input_source=input_source)
    return output


def silu_mul(input, output, block=128):
    """input [tokens, 2 * inter] in [gate | up] blocks of ``block`` columns, output [tokens, inter]."""
    cols = output.dim(output.num_dims - 1)
    _mpk(input).silu_mul_layer(input=input.dt, output=output.dt, grid_dim=(max(1, cols // block), 1, 1),
                               block_dim=(128, 1, 1))
    return output


def silu_mul_linear(input, weight, output, residual=None):
    """SiLU(gate) * up of an input row [gate | up], then the down projection (+ residual)."""
    mpk = _mpk(input)
    if residual is None:
        raise NotImplementedError("silu_mul_linear without a residual is not built; pass residual=")
    mpk.silu_mul_linear_with_residual_layer(input=input.dt, weight=weight.dt, residual=residual.dt, output=output.dt,
                                            grid_dim=(max(1, weight.dim(0) // 64), 1, 1), block_dim=(256, 1, 1))
    return output


def linear_silu(input, weight, output, output_stride=None, m_tiles=None, tile_n=64):
    """Gate/up linear with SiLU(gate) * up in its epilogue; ``weight`` is shuffle_inputs([gate, up], ...)."""
    mpk = _mpk(input)
    inter = output.dim(output.num_dims - 1)
    mpk.gang_linear_silu_layer(input=input.dt, weight=weight.dt, output=output.dt, tile_n=tile_n,
                               output_stride=output_stride if output_stride is not None else inter,
                               m_tiles=m_tiles or max(1, mpk.max_num_batched_tokens // 16), block_dim=(256, 1, 1))
    return output


def argmax(input, part_val, part_idx, output, num_tasks=None):
    mpk = _mpk(input)
    nt = num_tasks or max(1, input.dim(1) // 1024)
    mpk.argmax_partial_layer(input=input.dt, output=(part_val.dt, part_idx.dt), grid_dim=(nt, 1, 1), block_dim=(128, 1, 1))
    mpk.argmax_reduce_layer(input=(part_val.dt, part_idx.dt), output=output.dt, grid_dim=(1, 1, 1), block_dim=(128, 1, 1))
    return output


def linear(input, weight, output, residual=None, strategy="auto", k_splits=None, output_stride=None, m_tiles=None,
           tile_n=64, num_tasks=None):
    """input [tokens, K] x weight [N, K] -> output [tokens, N] (+ residual)."""
    g = input.graph
    mpk = g.mpk
    N, K = weight.dim(0), weight.dim(1)
    tokens = mpk.max_num_batched_tokens
    stride = output_stride if output_stride is not None else N
    if strategy == "auto":
        strategy = select_strategy(N, K, tokens, mpk.target_cc)
    if strategy in B200_STRATEGIES or strategy == "standard":
        grid = (num_tasks or max(1, N // 64), 1, 1)
        if residual is not None:
            mpk.linear_with_residual_layer(input=input.dt, weight=weight.dt, residual=residual.dt, output=output.dt,
                                           grid_dim=grid, block_dim=(128, 1, 1))
        else:
            mpk.linear_layer(input=input.dt, weight=weight.dt, output=output.dt, grid_dim=grid, block_dim=(128, 1, 1))
    elif strategy == "gang":
        if residual is not None:
            mpk.gang_linear_with_residual_layer(input=input.dt, weight=weight.dt, residual=residual.dt, output=output.dt,
                                                tile_n=tile_n, output_stride=stride, m_tiles=m_tiles or 1)
        else:
            mpk.gang_linear_layer(input=input.dt, weight=weight.dt, output=output.dt, tile_n=tile_n, output_stride=stride,
                                  m_tiles=m_tiles or 1)
    elif strategy in ("gang_splitk", "gang_coop"):
        if residual is None:
            raise NotImplementedError(f"strategy {strategy!r} is only built with a residual (the reference uses it for the "
                                      "O and down projections)")
        ks = k_splits or select_k_splits(K, max(1, N // 128), mpk.num_workers or 148)
        ws = g.get_workspace(tokens, N, torch.float32, f"splitk_{N}")
        mpk.gang_splitk_linear_with_residual_layer(input=input.dt, weight=weight.dt, residual=residual.dt, workspace=ws,
                                                   output=output.dt, tile_n=tile_n, output_stride=stride, k_splits=ks)
    else:
        raise ValueError(f"unknown linear strategy {strategy!r}")
    return output


def paged_attention_split_kv(input, k_cache, v_cache, q_norm, k_norm, cos_pe, sin_pe, lse, attn_tmp, attn_out, num_q_heads,
                             num_kv_chunks, num_kv_heads, head_dim, gang=None):
    """QK-norm + RoPE + KV append + paged split-KV GQA attention + merge (two layers of the reference, one device op)."""
    mpk = _mpk(input)
    opt = lambda t: t.dt if t is not None else None
    R = mpk.max_num_batched_requests
    mpk.paged_attention_split_kv_layer(input=input.dt, k_cache=k_cache.dt, v_cache=v_cache.dt, q_norm=opt(q_norm),
                                       k_norm=opt(k_norm), cos_pos_embed=opt(cos_pe), sin_pos_embed=opt(sin_pe),
                                       lse=lse.dt, output=attn_tmp.dt, attention_params=(num_q_heads, num_kv_chunks),
                                       grid_dim=(R, num_kv_heads, num_kv_chunks), block_dim=(128, 1, 1))
    mpk.paged_attention_split_kv_merge_layer(lse=lse.dt, output_tmp=attn_tmp.dt, output=attn_out.dt,
                                             attention_params=(num_q_heads, head_dim), grid_dim=(R, num_kv_heads, 1),
                                             block_dim=(128, 1, 1))
    return attn_out


def paged_attention(input, k_cache, v_cache, q_norm, k_norm, cos_pe, sin_pe, attn_out, num_kv_heads):
    mpk = _mpk(input)
    mpk.paged_attention_layer(input=input.dt, k_cache=k_cache.dt, v_cache=v_cache.dt, q_norm=q_norm.dt, k_norm=k_norm.dt,
                              cos_pos_embed=cos_pe.dt, sin_pos_embed=sin_pe.dt, output=attn_out.dt,
                              grid_dim=(mpk.max_num_batched_requests, num_kv_heads, 1), block_dim=(128, 1, 1))
    return attn_out
