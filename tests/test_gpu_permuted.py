"""GPU parity of the permutation-fused entry points (rd_gmm_permuted / rd_tgmm_permuted) through
the C ABI: against the CPU oracle, and bit-for-bit against the un-fused path (gather rows, then
rd_gmm / rd_tgmm on the sorted copy), which runs the same arithmetic in the same order."""

import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))

import gpu_ragged_dot_b200 as rd  # noqa: E402
from gpu_ragged_dot_b200 import _lib, ops  # noqa: E402
from oracle import ragged_dot_oracle as oracle  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None
RTOL = ATOL = 2e-2  # bf16 tolerance of the elementwise check


def _routing(seed, tokens, top_k, g, capacity_extra=0):
    """Top-k routing -> (group_sizes[g], in_rows[m], out_rows[m]) with m = tokens*top_k + extra.
    in_rows[r]: token feeding sorted row r; out_rows[r]: its slot token*top_k + j in the
    token-major expanded layout.  Entries past sum(group_sizes) are filled with junk."""
    rng = np.random.default_rng(seed)
    experts = np.stack([rng.permutation(g)[:top_k] for _ in range(tokens)])  # [tokens, top_k]
    flat = experts.reshape(-1)
    order = np.argsort(flat, kind="stable")
    gs = np.bincount(flat, minlength=g).astype(np.int32)
    in_rows = (order // top_k).astype(np.int32)
    out_rows = order.astype(np.int32)
    if capacity_extra:
        junk = rng.integers(-5, tokens + 5, size=capacity_extra).astype(np.int32)
        in_rows = np.concatenate([in_rows, junk])
        out_rows = np.concatenate([out_rows, junk])
    return torch.from_numpy(gs), torch.from_numpy(in_rows), torch.from_numpy(out_rows)


def _close(got, want, what):
    ok, worst = oracle.allclose_report(got, want, RTOL, ATOL)
    assert ok, f"{what}: worst violation {worst:.2f}x of |a-b| <= {ATOL} + {RTOL}|b|"


CASES = [
    # tokens, top_k, k, n, g, extra, tile_n
    (64, 2, 64, 64, 4, 0, None),
    (200, 2, 256, 384, 8, 0, None),
    (333, 4, 200, 328, 16, 37, None),
    (512, 1, 128, 256, 3, 0, 256),
    (300, 2, 192, 136, 8, 11, 128),
    (300, 2, 72, 72, 8, 0, 64),
]


@pytest.mark.parametrize("tokens,top_k,k,n,g,extra,tile_n", CASES)
@pytest.mark.parametrize("trans_rhs", [False, True])
def test_gmm_permuted(tokens, top_k, k, n, g, extra, tile_n, trans_rhs):
    gs, in_rows, out_rows = _routing(7, tokens, top_k, g, extra)
    m = in_rows.numel()
    total = int(gs.sum())
    x = oracle.reference_normal(11, (tokens, k), torch.bfloat16)
    A = oracle.reference_normal(12, (g, n, k) if trans_rhs else (g, k, n), torch.bfloat16)
    cfg = _lib.TileCfg(tile_n, 0, 0, 0, 0) if tile_n else None
    xd, Ad, gd, ird, ord_ = (t.to(DEV) for t in (x, A, gs, in_rows, out_rows))
    safe_in = in_rows.clamp(0, tokens - 1)

    # gather only: rows come back in sorted order, rows past sum(group_sizes) are zero
    ws = ops._workspace(m, g, DEV)
    y1 = ops.gmm_permuted_forward(xd, Ad, gd, in_rows=ird, trans_rhs=trans_rhs, cfg=cfg, workspace=ws)
    assert ops.device_status(ws) == 0
    want1 = oracle.ragged_dot(x[safe_in.long()], A, gs, trans_rhs=trans_rhs)
    _close(y1.cpu(), want1, "gather")
    if total < m:
        assert float(y1[total:].float().abs().max()) == 0.0
    unfused = ops.gmm_forward(ops.gather_rows(xd, ird.clamp(0, tokens - 1)), Ad, gd, trans_rhs=trans_rhs,
                              cfg=_lib.TileCfg(tile_n or 0, 0, 1, 128, 0))
    assert torch.equal(y1[:total], unfused[:total]), "fused gather differs from gather_rows + rd_gmm"

    # gather + scatter into the token-major expanded layout
    y_rows = tokens * top_k
    y2 = ops.gmm_permuted_forward(xd, Ad, gd, in_rows=ird, out_rows=ord_, y_rows=y_rows, trans_rhs=trans_rhs,
                                  cfg=cfg)
    want2 = oracle.ragged_dot_permuted(x, A, gs, in_rows=safe_in, out_rows=out_rows, y_rows=y_rows,
                                       trans_rhs=trans_rhs)
    _close(y2.cpu(), want2, "gather+scatter")
    inv = out_rows[:total].long().to(DEV)
    assert torch.equal(y2[inv], y1[:total]), "scattered rows differ from the sorted result"

    # scatter only, into a buffer that already holds data: untouched rows keep it
    xs = x[safe_in.long()].contiguous().to(DEV)
    base = torch.full((y_rows + 3, n), 7.0, dtype=torch.bfloat16, device=DEV)
    y3 = ops.gmm_permuted_forward(xs, Ad, gd, out_rows=ord_, out=base, m=m, trans_rhs=trans_rhs, cfg=cfg)
    assert y3.data_ptr() == base.data_ptr() or (n % 8)
    assert torch.equal(y3[inv], y1[:total])
    assert float((y3[y_rows:] - 7.0).float().abs().max()) == 0.0


@pytest.mark.parametrize("tokens,top_k,k,n,g,extra,tile_n", CASES)
def test_tgmm_permuted(tokens, top_k, k, n, g, extra, tile_n):
    gs, in_rows, out_rows = _routing(9, tokens, top_k, g, extra)
    m = in_rows.numel()
    x = oracle.reference_normal(21, (tokens, k), torch.bfloat16)
    dy = oracle.reference_normal(22, (tokens * top_k, n), torch.bfloat16)
    cfg = _lib.TileCfg(tile_n, 0, 0, 0, 0) if tile_n else None
    safe_in = in_rows.clamp(0, tokens - 1).long()
    safe_out = out_rows.clamp(0, tokens * top_k - 1).long()
    xs, dys = x[safe_in].contiguous(), dy[safe_out].contiguous()
    want = oracle.trans_ragged_dot(xs, dys, gs)
    xd, dyd, gd = x.to(DEV), dy.to(DEV), gs.to(DEV)
    ws = ops._workspace(m, g, DEV)
    got = ops.tgmm_permuted_forward(xd, dyd, gd, x_rows_index=in_rows.to(DEV), y_rows_index=out_rows.to(DEV),
                                    cfg=cfg, workspace=ws)
    assert ops.device_status(ws) == 0
    _close(got.cpu(), want, "tgmm both gathered")
    err = oracle.rel_l2_err(got.cpu(), want, axis=(-1, -2), mask=gs != 0)
    assert float(err.max()) < 2e-3
    for gi in (gs == 0).nonzero().flatten().tolist():
        assert float(got[gi].float().abs().max()) == 0.0
    unfused = ops.tgmm_forward(xs.to(DEV), dys.to(DEV), gd, cfg=_lib.TileCfg(tile_n or 0, 0, 1, 128, 0))
    assert torch.equal(got, unfused), "fused gathers differ from rd_tgmm on the sorted copies"
    # one side only
    got_x = ops.tgmm_permuted_forward(xd, dys.to(DEV), gd, x_rows_index=in_rows.to(DEV), m=m, cfg=cfg)
    assert torch.equal(got_x, unfused)
    got_y = ops.tgmm_permuted_forward(xs.to(DEV), dyd, gd, y_rows_index=out_rows.to(DEV), m=m, cfg=cfg)
    assert torch.equal(got_y, unfused)


@pytest.mark.parametrize("fused", [True, False, None])
def test_ragged_dot_permuted_vjp(fused):
    tokens, top_k, k, n, g = 150, 2, 96, 136, 6
    gs, in_rows, out_rows = _routing(3, tokens, top_k, g)
    x = oracle.reference_normal(31, (tokens, k), torch.bfloat16)
    A = oracle.reference_normal(32, (g, k, n), torch.bfloat16)
    dy = oracle.reference_normal(33, (tokens * top_k, n), torch.bfloat16)
    xd = x.to(DEV).requires_grad_(True)
    Ad = A.to(DEV).requires_grad_(True)
    y = rd.ops.ragged_dot_permuted(xd, Ad, gs.to(DEV), in_rows=in_rows.to(DEV), out_rows=out_rows.to(DEV),
                                   fused=fused)
    y.backward(dy.to(DEV))
    # oracle: the same composition, differentiated by hand with the reference's VJP wiring
    xs = x[in_rows.long()]
    dys = dy[out_rows.long()]
    dxs, dA = oracle.ragged_dot_vjp(xs, A, gs, dys)
    dx = torch.zeros((tokens, k), dtype=torch.float32).index_add_(0, in_rows.long(), dxs.float())
    _close(y.detach().cpu(), oracle.ragged_dot_permuted(x, A, gs, in_rows, out_rows, tokens * top_k), "fwd")
    _close(xd.grad.cpu(), dx.to(torch.bfloat16), "dx")
    _close(Ad.grad.cpu(), dA, "dA")


def test_permuted_argument_checks():
    lib = _lib.load()
    x = torch.zeros((16, 64), dtype=torch.bfloat16, device=DEV)
    A = torch.zeros((2, 64, 64), dtype=torch.bfloat16, device=DEV)
    gs = torch.tensor([8, 8], dtype=torch.int32, device=DEV)
    y = torch.zeros((16, 64), dtype=torch.bfloat16, device=DEV)
    ws = ops._workspace(16, 2, DEV)

    def call(**kw):
        a = dict(x_rows=16, in_rows=None, y_rows=16, out_rows=None, m=16, k=64, dtype=_lib.RD_DTYPE_BF16, cfg=None)
        a.update(kw)
        return lib.rd_gmm_permuted(x.data_ptr(), a["x_rows"], a["in_rows"], A.data_ptr(), 2, gs.data_ptr(), None,
                                   y.data_ptr(), a["y_rows"], a["out_rows"], ws.data_ptr(), ws.numel(), a["m"],
                                   a["k"], 64, 2, 0, a["dtype"], a["cfg"], None)

    assert call() == 0
    assert call(x_rows=8) == _lib.RD_ERR_BAD_SHAPE       # identity gather needs x_rows >= m
    assert call(y_rows=8) == _lib.RD_ERR_BAD_SHAPE       # identity scatter needs y_rows == m
    assert call(k=60) == _lib.RD_ERR_BAD_SHAPE
    assert call(dtype=_lib.RD_DTYPE_F32) == _lib.RD_ERR_BAD_DTYPE
    import ctypes
    pair = _lib.TileCfg(256, 0, 2, 0, 0)
    assert call(cfg=ctypes.byref(pair)) == _lib.RD_ERR_BAD_CONFIG
    torch.cuda.synchronize()
