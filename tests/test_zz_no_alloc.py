"""rd_gmm_static_scratch: the entry point for hosts that can neither pass a workspace nor
allocate one (a fixed inputs/outputs operator slot inside a framework that owns the device's
memory).  Its scratch is an array inside the library, so the test checks that it gives the same
answer as rd_gmm with a caller-owned workspace -- twice in a row, because the array is shared
between calls and still holds the first call's metadata when the second one starts.

Collected last on purpose (file name), and written to pass both alone and after the rest.
"""

import ctypes

import pytest
import torch

from gpu_ragged_dot_b200 import _lib, ops
from oracle import ragged_dot_oracle as oracle

pytestmark = pytest.mark.gpu

RTOL = ATOL = 2e-2
BF16 = _lib.RD_DTYPE_BF16


def _inputs(seed, m, k, n, g, dev):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(m, k, generator=gen).to(torch.bfloat16).to(dev)
    A = (torch.randn(g, k, n, generator=gen) / k ** 0.5).to(torch.bfloat16).to(dev)
    return x, A


def _both(lib, x, A, gs, trans_rhs):
    m, k = x.shape
    g = A.shape[0]
    n = A.shape[1] if trans_rhs else A.shape[2]
    dev = x.device
    stream = torch.cuda.current_stream(dev).cuda_stream
    want = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    ws = ops._workspace(m, g, dev)
    rc = lib.rd_gmm(x.data_ptr(), A.data_ptr(), gs.data_ptr(), want.data_ptr(), ws.data_ptr(), ws.numel(),
                    m, k, n, g, int(trans_rhs), BF16, None, stream)
    assert rc == 0, _lib.status_string(rc)
    got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
    rc = lib.rd_gmm_static_scratch(x.data_ptr(), A.data_ptr(), gs.data_ptr(), got.data_ptr(),
                                   m, k, n, g, int(trans_rhs), BF16, None, stream)
    assert rc == 0, _lib.status_string(rc)
    torch.cuda.synchronize(dev)
    return got, want


def _check(got, want, what):
    assert bool(torch.isfinite(got.float()).all()), f"{what}: output not fully written"
    diff = (got.float() - want.float()).abs()
    assert bool((diff <= ATOL + RTOL * want.float().abs()).all()), f"{what}: max diff {float(diff.max())}"


def test_static_scratch_matches_workspace_variant_twice():
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    # first call: many groups and row tiles, so the shared array is left full of metadata
    x, A = _inputs(1, 1300, 256, 384, 12, dev)
    gs = torch.tensor([100, 0, 257, 1, 128, 64, 0, 300, 90, 10, 200, 100], dtype=torch.int32, device=dev)
    got, want = _both(lib, x, A, gs, trans_rhs=False)
    _check(got, want, "first call")
    _check(got, oracle.ragged_dot(x, A, gs).to(dev), "first call vs the CPU oracle")
    assert float(got[int(gs.sum()):].float().abs().max()) == 0.0
    # second call, straight after: fewer groups, fewer rows, transposed weights
    x2, A2 = _inputs(2, 300, 128, 264, 3, dev)
    gs2 = torch.tensor([37, 0, 200], dtype=torch.int32, device=dev)
    got2, want2 = _both(lib, x2, A2.transpose(1, 2).contiguous(), gs2, trans_rhs=True)
    _check(got2, want2, "second call")
    _check(got2, oracle.ragged_dot(x2, A2, gs2).to(dev), "second call vs the CPU oracle")
    assert float(got2[237:].float().abs().max()) == 0.0


def test_static_scratch_rejects_oversized_problems():
    lib = _lib.load()
    a16 = 0x1000  # never dereferenced: the size check comes first
    rc = lib.rd_gmm_static_scratch(a16, a16, a16, a16, 1 << 20, 64, 64, 4096, 0, BF16, None, None)
    assert rc == 10
    assert "too large" in _lib.status_string(rc)
    rc = lib.rd_gmm_static_scratch(a16, a16, a16, a16, 128, 64, 64, 5000, 0, BF16, None, None)
    assert rc == 10
