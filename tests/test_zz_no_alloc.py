"""mk_linear_static, the entry point that allocates nothing.

Some hosts of the library cannot call cudaMalloc where they need a linear layer (a
server whose arena already owns the whole GPU, a loop that must not hit cudaMalloc's
device-wide synchronisation), so this variant keeps the partial sums of its k-splits in
a fixed array inside the library.  It is checked here against the oracle's linear task and against the regular path (a
linear_with_residual layer run through the PersistentKernel mirror and the C ABI) on
calls in a row with different inputs: the second call must not see anything the first
one left in the shared scratch.  The file sorts last so that a run stopping at the first
failure has already run every other test."""
import ctypes as C

import pytest
import torch

from fleet_chiplet_megakernel_b200 import _cabi
from oracle import qwen3_oracle as O
from tests.helpers import onepass_kernel, bf16_close

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _regular_path(x, w, r):
    T, N = x.shape[0], w.shape[0]
    k, meta, _ = onepass_kernel(T)
    od = torch.zeros(T, N, dtype=BF, device="cuda")
    k.linear_with_residual_layer(input=k.attach_input(x, "x"), weight=k.attach_input(w, "w"),
                                 residual=k.attach_input(r, "r"), output=k.attach_input(od, "o"),
                                 grid_dim=(max(1, N // 64), 1, 1), block_dim=(256, 1, 1))
    k.compile()
    k()
    k.finalize()
    return od


def test_static_scratch_linear_matches_regular_path_twice():
    lib = _cabi.load()
    stream = torch.cuda.current_stream()
    g = torch.Generator().manual_seed(5)
    for call, (T, N, K) in enumerate([(3, 4096, 4096), (3, 4096, 4096), (1, 1000, 12288)]):
        xh = torch.randn(T, K, generator=g).to(BF)
        wh = (torch.randn(N, K, generator=g) * 0.05).to(BF)
        rh = torch.randn(T, N, generator=g).to(BF)
        x, w, r = xh.cuda(), wh.cuda(), rh.cuda()
        out = torch.full((T, N), 7.0, dtype=BF, device="cuda")
        rc = lib.mk_linear_static(C.c_void_p(x.data_ptr()), C.c_void_p(w.data_ptr()), C.c_void_p(r.data_ptr()),
                                  C.c_void_p(out.data_ptr()), T, N, K, C.c_void_p(stream.cuda_stream))
        assert rc == 0
        torch.cuda.synchronize()
        bf16_close(out, O.mpk_linear(xh, wh, residual=rh), 1e-2, f"static-scratch linear vs the oracle, call {call}")
        ref = _regular_path(x, w, r)
        bf16_close(out, ref, 1e-2, f"static-scratch linear vs the regular path, call {call}")


def test_static_scratch_linear_rejects_oversize():
    lib = _cabi.load()
    x = torch.zeros(1, 64, dtype=BF, device="cuda")
    p = C.c_void_p(x.data_ptr())
    assert lib.mk_linear_static(p, p, None, p, 9, 64, 64, None) == _cabi.MK_E_TOO_LARGE
    assert lib.mk_linear_static(p, p, None, p, 1, 16385, 64, None) == _cabi.MK_E_TOO_LARGE
    assert lib.mk_linear_static(p, p, None, p, 1, 64, 60, None) == _cabi.MK_E_INVALID
