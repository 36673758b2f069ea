"""Shared helpers of the tests: meta tensors for single-pass graphs, comparators."""
import math

import torch

import fleet_chiplet_megakernel_b200 as mk


def onepass_kernel(T, max_seq=256, page_size=64, max_pages=None, seq_lens=None, device="cuda", numerics="mpk",
                   fuse=True, timeout_ms=2000):
    """A PersistentKernel in single-pass mode with T active tokens (one per request).
    seq_lens[r] = tokens of request r INCLUDING the new one."""
    R = T
    pages_per = math.ceil(max_seq / page_size)
    max_pages = max_pages or R * pages_per
    dev = torch.device(device)
    meta = {
        "step": torch.zeros(R, dtype=torch.int32, device=dev),
        "tokens": torch.zeros(R, max_seq, dtype=torch.int64, device=dev),
        "input_tokens": torch.zeros(T, 1, dtype=torch.int64, device=dev),
        "output_tokens": torch.zeros(T, 1, dtype=torch.int64, device=dev),
        "num_new_tokens": torch.ones(R, dtype=torch.int32, device=dev),
        "prompt_lengths": torch.ones(R, dtype=torch.int32, device=dev),
        "qo_indptr_buffer": torch.arange(R + 1, dtype=torch.int32, device=dev),
        "paged_kv_indptr_buffer": torch.zeros(R + 1, dtype=torch.int32, device=dev),
        "paged_kv_indices_buffer": torch.zeros(max_pages, dtype=torch.int32, device=dev),
        "paged_kv_last_page_len_buffer": torch.ones(R, dtype=torch.int32, device=dev),
    }
    page_table = None
    if seq_lens is not None:
        # scatter the pages of the requests over the pool in a shuffled order
        g = torch.Generator().manual_seed(7)
        perm = torch.randperm(max_pages, generator=g).tolist()
        indptr, indices, last = [0], [], []
        for L in seq_lens:
            n = math.ceil(L / page_size)
            indices += [perm.pop() for _ in range(n)]
            indptr.append(len(indices))
            last.append(L - (n - 1) * page_size)
        meta["paged_kv_indptr_buffer"].copy_(torch.tensor(indptr, dtype=torch.int32))
        meta["paged_kv_indices_buffer"][: len(indices)] = torch.tensor(indices, dtype=torch.int32, device=dev)
        meta["paged_kv_last_page_len_buffer"].copy_(torch.tensor(last, dtype=torch.int32))
        page_table = (indptr, indices)
    k = mk.PersistentKernel(
        mode="online_notoken", world_size=1, mpi_rank=0, num_workers=0, num_local_schedulers=0,
        num_remote_schedulers=0, max_seq_length=max_seq, max_num_batched_requests=R, max_num_batched_tokens=T,
        max_num_pages=max_pages, page_size=page_size, meta_tensors=meta, profiler_tensor=None, trace_name="",
        spec_decode_config=None, use_cutlass_kernel=True, numerics=numerics, fuse=fuse, timeout_ms=timeout_ms)
    return k, meta, page_table


def bf16_close(a, b, rel=2e-2, what=""):
    """max |a-b| over the largest |b| of the row, the unit the logit tolerance uses."""
    a, b = a.float().cpu(), b.float().cpu()
    scale = b.abs().amax(-1, keepdim=True).clamp_min(1e-20)
    err = float(((a - b).abs() / scale).max())
    assert err <= rel, f"{what}: max normalised error {err:.4g} > {rel}"
    return err
