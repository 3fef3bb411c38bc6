"""GPU parity of the pipelined host-buffer path (HostRaggedDot): pinned host operands, expert
chunks copied in / multiplied / copied out on three streams, through rd_gmm and rd_tgmm.  Checked
against the CPU oracle and against the one-call device path on the same inputs."""

import numpy as np
import pytest
import torch

import gpu_ragged_dot_b200 as rd
from gpu_ragged_dot_b200.host_pipeline import HostRaggedDot
from oracle import ragged_dot_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None
RTOL = ATOL = 2e-2  # bf16 tolerance of the elementwise check


def _close(got, want, what):
    ok, worst = oracle.allclose_report(got, want, RTOL, ATOL)
    assert ok, f"{what}: worst violation {worst:.2f}x of |a-b| <= {ATOL} + {RTOL}|b|"


def _inputs(seed, m, k, n, g, fill, trans_rhs):
    rng = np.random.default_rng(seed)
    bf = lambda a: torch.from_numpy(a.astype(np.float32)).to(torch.bfloat16).pin_memory()  # noqa: E731
    x = bf(rng.standard_normal((m, k)))
    a_shape = (g, n, k) if trans_rhs else (g, k, n)
    A = bf(rng.standard_normal(a_shape) / np.sqrt(k))
    dout = bf(rng.standard_normal((m, n)))
    target = int(round(m * fill))
    p = rng.dirichlet(np.full(g, 0.5))
    gs = rng.multinomial(target, p).astype(np.int32)
    if g > 2:
        gs[-1] += gs[1]
        gs[1] = 0  # an empty group inside a chunk
    return x, A, dout, torch.from_numpy(gs)


CASES = [
    # m, k, n, g, fill, experts per chunk
    (512, 256, 384, 8, 1.0, 1),
    (700, 136, 264, 8, 0.7, 3),
    (300, 64, 72, 5, 0.5, 2),
    (256, 128, 128, 4, 1.0, 16),
]


@pytest.mark.parametrize("m,k,n,g,fill,per_chunk", CASES)
@pytest.mark.parametrize("trans_rhs", [False, True])
def test_host_pipeline_matches_oracle_and_device_path(m, k, n, g, fill, per_chunk, trans_rhs):
    x, A, dout, gs = _inputs(11, m, k, n, g, fill, trans_rhs)
    pipe = HostRaggedDot(m, k, n, g, device=DEV, trans_rhs=trans_rhs, chunk_bytes=per_chunk * k * n * 2)
    assert pipe.experts_per_chunk == per_chunk
    for step in range(2):  # the second call reuses the device buffers of the first
        if step == 1:
            x = (x.float() * 0.5).to(torch.bfloat16).pin_memory()
        y, dlhs, drhs = pipe(x, A, gs, dout)
        torch.cuda.synchronize()
        y_ref = oracle.ragged_dot(x, A, gs, trans_rhs=trans_rhs)
        dlhs_ref, drhs_ref = oracle.ragged_dot_vjp(x, A, gs, dout, trans_rhs=trans_rhs)
        _close(y, y_ref, "y")
        _close(dlhs, dlhs_ref, "dlhs")
        _close(drhs, drhs_ref, "drhs")
        total = int(gs.sum())
        assert not y[total:].any() and not dlhs[total:].any()
        assert not drhs[gs == 0].any()
        # one-call device path on the same inputs
        xd = x.to(DEV).requires_grad_(True)
        Ad = A.to(DEV).requires_grad_(True)
        yd = rd.ragged_dot(xd, Ad, gs.to(DEV), trans_rhs=trans_rhs)
        yd.backward(dout.to(DEV))
        _close(y, yd.detach().cpu(), "y vs device path")
        _close(dlhs, xd.grad.cpu(), "dlhs vs device path")
        _close(drhs, Ad.grad.cpu(), "drhs vs device path")


def test_host_pipeline_forward_only_and_all_empty():
    m, k, n, g = 256, 64, 64, 4
    x, A, _, _ = _inputs(3, m, k, n, g, 1.0, False)
    gs = torch.zeros(g, dtype=torch.int32)
    pipe = HostRaggedDot(m, k, n, g, device=DEV, backward=False)
    y = pipe(x, A, gs)
    torch.cuda.synchronize()
    assert not y.any()
    gs = torch.tensor([100, 0, 56, 7], dtype=torch.int32)
    y = pipe(x, A, gs, y=y)
    torch.cuda.synchronize()
    _close(y, oracle.ragged_dot(x, A, gs), "y")


def test_host_pipeline_refuses_bad_operands():
    m, k, n, g = 128, 64, 64, 2
    pipe = HostRaggedDot(m, k, n, g, device=DEV, backward=False)
    x, A, _, gs = _inputs(5, m, k, n, g, 1.0, False)
    with pytest.raises(ValueError, match="pinned"):
        pipe(x.clone(), A, gs)
    with pytest.raises(ValueError, match="host tensor"):
        pipe(x.to(DEV), A, gs)
    with pytest.raises(ValueError, match="sum to at most m"):
        pipe(x, A, torch.tensor([100, 100], dtype=torch.int32))
    with pytest.raises(ValueError, match="16-byte rows"):
        HostRaggedDot(m, 60, n, g, device=DEV)
