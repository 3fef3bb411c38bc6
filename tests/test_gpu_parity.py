"""GPU parity tests: the CUDA path (through the C ABI, via the Python host layer) against the
CPU oracle on the same seeded inputs.

Tolerances: elementwise |a-b| <= 2e-2 + 2e-2*|b| for bf16 inputs with fp32 accumulation, and
the reference's own relative-L2 gates (tests.py:127,144,168,183): 5e-3 per row for gmm and its
gradients, 2e-3 per group for tgmm.  Group metadata must match bit for bit.
"""

import itertools
import random

import numpy as np
import pytest
import torch

import gpu_ragged_dot_b200 as rd
from gpu_ragged_dot_b200 import _lib, ops, workloads
from oracle import ragged_dot_oracle as oracle

pytestmark = pytest.mark.gpu

RTOL = ATOL = 2e-2
EPS_ROWS_BF16 = 5e-3
EPS_GROUPS_BF16 = 2e-3
DEV = "cuda:0"


def _assert_close(got, want, what):
    ok, worst = oracle.allclose_report(got, want, RTOL, ATOL)
    assert ok, f"{what}: elementwise rtol/atol 2e-2 violated, worst ratio {worst:.3f}"


def _inputs(seed, m, k, n, g, dtype=torch.bfloat16, random_inputs=True):
    if random_inputs:
        x = oracle.reference_normal(seed * 7 + 1, (m, k), dtype)
        A = oracle.reference_normal(seed * 7 + 2, (g, k, n), dtype)
        dout = oracle.reference_normal(seed * 7 + 3, (m, n), dtype)
    else:
        x, A, dout = (torch.ones(s, dtype=dtype) for s in ((m, k), (g, k, n), (m, n)))
    return x, A, dout


def _to_dev(*ts):
    return tuple(t.to(DEV) for t in ts)


# ------------------------------------------------------------------ metadata (bit exact)
META_CASES = [
    ([5, 0, 12, 3, 0, 0, 9, 1], 32, 8),
    ([0, 0, 0, 0], 16, 8),
    ([128], 128, 128),
    ([127, 1, 128, 129, 0, 255], 640, 128),
    ([512, 0, 0, 512], 1024, 512),
    ([3] * 300, 1024, 8),
]


@pytest.mark.parametrize("gs,m,chunk", META_CASES)
def test_metadata_bit_exact(gs, m, chunk):
    want = oracle.make_group_metadata(gs, m, chunk)
    got = rd.make_group_metadata(torch.tensor(gs, dtype=torch.int32, device=DEV), m, chunk)
    torch.cuda.synchronize()
    assert np.array_equal(got.group_offsets.cpu().numpy(), want.group_offsets)
    assert np.array_equal(got.row_it2group.cpu().numpy(), want.row_it2group)
    assert np.array_equal(got.row_it2it_in_group.cpu().numpy(), want.row_it2it_in_group)
    assert int(got.total_row_its.cpu()) == int(want.total_row_its)


@pytest.mark.parametrize("seed", [0, 1, 2])
@pytest.mark.parametrize("g,m,chunk", [(8, 8192, 128), (256, 32768, 128), (64, 256, 128), (2500, 40000, 64)])
def test_metadata_random_bit_exact(seed, g, m, chunk):
    rng = np.random.default_rng(seed)
    gs = rng.multinomial(int(m * 0.9), rng.dirichlet(0.3 * np.ones(g))).astype(np.int32)
    want = oracle.make_group_metadata(gs, m, chunk)
    got = rd.make_group_metadata(torch.from_numpy(gs).to(DEV), m, chunk)
    assert np.array_equal(got.group_offsets.cpu().numpy(), want.group_offsets)
    assert np.array_equal(got.row_it2group.cpu().numpy(), want.row_it2group)
    assert np.array_equal(got.row_it2it_in_group.cpu().numpy(), want.row_it2it_in_group)
    assert int(got.total_row_its.cpu()) == int(want.total_row_its)


# ------------------------------------------------------------------ forward
def _check_gmm(x, A, gs, trans_rhs=False, cfg=None, what="gmm"):
    gs_t = torch.as_tensor(gs, dtype=torch.int32)
    want = oracle.ragged_dot(x, A, gs_t, trans_rhs=trans_rhs)
    xd, Ad, gd = _to_dev(x, A, gs_t)
    m, g = x.shape[0], A.shape[0]
    ws = ops._workspace(m, g, xd.device)
    got = ops.gmm_forward(xd, Ad, gd, trans_rhs=trans_rhs, cfg=cfg, workspace=ws)
    assert ops.device_status(ws) == 0, "device reported an expired wait"
    got = got.cpu()
    total = int(min(int(np.sum(np.maximum(np.asarray(gs), 0))), m))
    _assert_close(got, want, what)
    err = oracle.rel_l2_err(got, want, axis=-1, mask=torch.arange(m) < total)
    assert float(err.max()) < EPS_ROWS_BF16, f"{what}: rel-L2 per row {float(err.max()):.2e}"
    if total < m:
        assert not bool(got[total:].float().abs().max() > 0), f"{what}: rows past sum(group_sizes) not zero"
    return got


def _check_tgmm(x, dout, gs, cfg=None, what="tgmm"):
    gs_t = torch.as_tensor(gs, dtype=torch.int32)
    want = oracle.trans_ragged_dot(x, dout, gs_t)
    xd, dd, gd = _to_dev(x, dout, gs_t)
    m, g = x.shape[0], gs_t.numel()
    ws = ops._workspace(m, g, xd.device)
    got = ops.tgmm_forward(xd, dd, gd, cfg=cfg, workspace=ws)
    assert ops.device_status(ws) == 0, "device reported an expired wait"
    got = got.cpu()
    _assert_close(got, want, what)
    err = oracle.rel_l2_err(got, want, axis=(-1, -2), mask=gs_t != 0)
    assert float(err.max()) < EPS_GROUPS_BF16, f"{what}: rel-L2 per group {float(err.max()):.2e}"
    empty = (gs_t == 0).nonzero().flatten().tolist()
    for gi in empty:
        assert not bool(got[gi].float().abs().max() > 0), f"{what}: empty group {gi} not zero"
    return got


def test_small_config_forward_backward():
    s = workloads.SMALL
    gs = workloads.group_sizes_small(0)
    assert gs.sum() == s.m and (gs == 0).any()
    rng_x = oracle.reference_normal(101, (s.m, s.k), torch.bfloat16)
    A = (oracle.reference_normal(102, (s.g, s.k, s.n), torch.float32) / s.k ** 0.5).to(torch.bfloat16)
    dout = oracle.reference_normal(103, (s.m, s.n), torch.bfloat16)
    _check_gmm(rng_x, A, gs, what="small fwd")
    _check_gmm(dout, A, gs, trans_rhs=True, what="small dlhs")
    _check_tgmm(rng_x, dout, gs, what="small drhs")


def _reference_grid(samples, seed=1234):
    grid = dict(
        m=[128, 256, 171], k=[256, 512, 58], n=[64, 128, 77], g=[8, 16],
        fill_in=[1.0, 0.7, 0.5], seed=[0, 1], random_inputs=[True, False],
    )
    keys = list(grid)
    prod = list(itertools.product(*grid.values()))
    random.Random(seed).shuffle(prod)
    return [dict(zip(keys, v)) for v in prod[:samples]]


GRID = _reference_grid(24)


@pytest.mark.parametrize("case", GRID, ids=lambda c: "-".join(f"{k}{v}" for k, v in c.items()))
def test_reference_grid_forward(case):
    m, k, n, g = case["m"], case["k"], case["n"], case["g"]
    x, A, _ = _inputs(case["seed"], m, k, n, g, random_inputs=case["random_inputs"])
    target_m = max(min(round(m * case["fill_in"]), m), 0)
    gs = oracle.reference_group_sizes(case["seed"] + 17, g, target_m)
    _check_gmm(x, A, gs, what="grid fwd")


@pytest.mark.parametrize("case", GRID[:12], ids=lambda c: "-".join(f"{k}{v}" for k, v in c.items()))
def test_reference_grid_trans_rhs(case):
    m, k, n, g = case["m"], case["k"], case["n"], case["g"]
    x, A, _ = _inputs(case["seed"], m, k, n, g, random_inputs=case["random_inputs"])
    target_m = max(min(round(m * case["fill_in"]), m), 0)
    gs = oracle.reference_group_sizes(case["seed"] + 17, g, target_m)
    _check_gmm(x, A.transpose(1, 2).contiguous(), gs, trans_rhs=True, what="grid fwd trans_rhs")


@pytest.mark.parametrize("case", GRID[:16], ids=lambda c: "-".join(f"{k}{v}" for k, v in c.items()))
def test_reference_grid_trans_ragged_dot(case):
    m, k, n, g = case["m"], case["k"], case["n"], case["g"]
    x, _, dout = _inputs(case["seed"], m, k, n, g, random_inputs=case["random_inputs"])
    target_m = max(min(round(m * case["fill_in"]), m), 0)
    gs = oracle.reference_group_sizes(case["seed"] + 17, g, target_m)
    _check_tgmm(x, dout, gs, what="grid tgmm")


@pytest.mark.parametrize("tile_n,cta_group,tile_m",
                         [(64, 1, 128), (128, 1, 128), (256, 1, 128), (256, 2, 128), (256, 1, 256)])
@pytest.mark.parametrize("trans_rhs", [False, True])
def test_every_tile_shape(tile_n, cta_group, tile_m, trans_rhs):
    """Every kernel instantiation, forced through rd_tile_cfg: tile widths 64/128/256 on one CTA,
    the 256x256 tile on a CTA pair, and the 256x256 two-half tile on one CTA."""
    m, k, n, g = 700, 320, 520, 5
    x, A, dout = _inputs(3, m, k, n, g)
    gs = [130, 0, 257, 1, 300]
    cfg = _lib.TileCfg(tile_n, 0, cta_group, tile_m)
    Aa = A.transpose(1, 2).contiguous() if trans_rhs else A
    _check_gmm(x, Aa, gs, trans_rhs=trans_rhs, cfg=cfg, what=f"tile_n={tile_n} ctas={cta_group}")
    if not trans_rhs:
        _check_tgmm(x, dout, gs, cfg=cfg, what=f"tgmm tile_n={tile_n} ctas={cta_group}")


@pytest.mark.parametrize("cta_group,tile_m", [(2, 128), (1, 256)])
@pytest.mark.parametrize("trans_rhs", [False, True])
def test_256_row_tiles_ragged_boundaries(cta_group, tile_m, trans_rhs):
    """256-row tiles (CTA pair, and two-half on one CTA) against groups that end inside the
    first or the second half, empty groups, and k / n that are not multiples of the tile."""
    sizes = [1, 127, 128, 129, 255, 256, 257, 0, 300, 64, 0, 513]
    m, k, n = sum(sizes) + 40, 200, 392
    x, A, dout = _inputs(6, m, k, n, len(sizes))
    cfg = _lib.TileCfg(256, 0, cta_group, tile_m)
    Aa = A.transpose(1, 2).contiguous() if trans_rhs else A
    _check_gmm(x, Aa, sizes, trans_rhs=trans_rhs, cfg=cfg, what="pair ragged gmm")
    if not trans_rhs:
        _check_tgmm(x, dout, sizes, cfg=cfg, what="pair ragged tgmm")


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("k,n", [(136, 392), (264, 392), (392, 392), (520, 392), (1032, 392),
                                 (64, 64), (128, 192), (320, 448), (576, 256), (1024, 512)])
def test_tgmm_256_row_tiles_all_load_paths(k, n, cta_group):
    """tgmm with 256-row tiles on one CTA and with 512 x 256 tiles on CTA pairs (tile_m 256,
    cta_group 1 / 2).  k values that end inside the first CTA's rows, the second CTA's rows, the
    second half and the second tile; k and n that are multiples of 64 (one column-blocked TMA box
    per operand and stage, also where the box is wider than the tensor) and that are not (one box
    per 64 columns); group sizes around the 64-row reduction step and the 16-row MMA depth (the
    fixer warp of either CTA clears the tail rows); empty groups; rows past the last group hold
    NaN and must not reach any output."""
    sizes = [1, 63, 64, 65, 0, 130, 15, 16, 17, 0, 300, 77]
    m = sum(sizes) + 40
    x, _, dout = _inputs(8, m, k, n, len(sizes))
    x[sum(sizes):] = float("nan")
    dout[sum(sizes):] = float("nan")
    got = _check_tgmm(x, dout, sizes, cfg=_lib.TileCfg(256, 0, cta_group, 256),
                      what=f"256-row tgmm k={k} n={n} ctas={cta_group}")
    assert torch.isfinite(got.float()).all()


def test_group_boundaries_every_residue():
    """Group sizes 1..40 and 120..136: every boundary residue around the 64-row reduction
    step and the 128-row tile."""
    sizes = list(range(1, 41)) + list(range(120, 137))
    m, k, n = sum(sizes) + 5, 128, 64
    x, A, dout = _inputs(5, m, k, n, len(sizes))
    _check_gmm(x, A, sizes, what="residues fwd")
    _check_tgmm(x, dout, sizes, what="residues tgmm")


def test_all_groups_empty():
    m, k, n, g = 200, 64, 72, 4
    x, A, dout = _inputs(7, m, k, n, g)
    got = _check_gmm(x, A, [0, 0, 0, 0], what="all-empty fwd")
    assert float(got.float().abs().max()) == 0.0
    got = _check_tgmm(x, dout, [0, 0, 0, 0], what="all-empty tgmm")
    assert float(got.float().abs().max()) == 0.0


def test_single_giant_group():
    m, k, n, g = 1500, 256, 264, 3
    x, A, dout = _inputs(9, m, k, n, g)
    _check_gmm(x, A, [0, 1500, 0], what="giant fwd")
    _check_tgmm(x, dout, [0, 1500, 0], what="giant tgmm")


def test_nan_rows_outside_groups_do_not_leak():
    """Rows past sum(group_sizes) may hold anything (here NaN): they must not reach any output."""
    m, k, n, g = 300, 128, 128, 3
    x, A, dout = _inputs(11, m, k, n, g)
    gs = [70, 50, 33]
    x[153:] = float("nan")
    dout[153:] = float("nan")
    got = _check_gmm(x, A, gs, what="nan-tail fwd")
    assert torch.isfinite(got.float()).all()
    got = _check_tgmm(x, dout, gs, what="nan-tail tgmm")
    assert torch.isfinite(got.float()).all()


def test_float16_inputs():
    m, k, n, g = 256, 128, 192, 4
    x, A, dout = _inputs(13, m, k, n, g, dtype=torch.float16)
    A = (A.float() / k ** 0.5).to(torch.float16)
    _check_gmm(x, A, [64, 100, 0, 92], what="fp16 fwd")
    _check_tgmm(x, (dout.float() / 8).to(torch.float16), [64, 100, 0, 92], what="fp16 tgmm")


# ------------------------------------------------------------------ custom VJP wiring
@pytest.mark.parametrize("trans_rhs", [False, True])
def test_vjp_matches_oracle(trans_rhs):
    m, k, n, g = 384, 256, 192, 6
    x, A, dout = _inputs(21, m, k, n, g)
    A = (A.float() / k ** 0.5).to(torch.bfloat16)
    gs = torch.tensor([100, 0, 37, 128, 60, 40], dtype=torch.int32)
    Aa = A.transpose(1, 2).contiguous() if trans_rhs else A
    dx_ref, dA_ref = oracle.ragged_dot_vjp(x, Aa, gs, dout, trans_rhs=trans_rhs)
    xd, Ad, dd, gd = _to_dev(x, Aa, dout, gs)
    xd.requires_grad_(True)
    Ad.requires_grad_(True)
    y = rd.ragged_dot(xd, Ad, gd, block_m=32, block_k=32, block_n=32, trans_rhs=trans_rhs)
    y.backward(dd)
    total = int(gs.sum())
    _assert_close(y.detach().cpu(), oracle.ragged_dot(x, Aa, gs, trans_rhs=trans_rhs), "vjp fwd")
    _assert_close(xd.grad.cpu(), dx_ref, "dlhs")
    _assert_close(Ad.grad.cpu(), dA_ref, "drhs")
    e = oracle.rel_l2_err(xd.grad.cpu(), dx_ref, axis=-1, mask=torch.arange(m) < total)
    assert float(e.max()) < EPS_ROWS_BF16
    e = oracle.rel_l2_err(Ad.grad.cpu(), dA_ref, axis=(-1, -2), mask=gs != 0)
    assert float(e.max()) < EPS_ROWS_BF16


def test_tgmm_vjp_matches_oracle():
    m, k, n, g = 256, 128, 64, 4
    x, _, y = _inputs(23, m, k, n, g)
    gs = torch.tensor([60, 0, 100, 96], dtype=torch.int32)
    dA = oracle.reference_normal(99, (g, k, n), torch.bfloat16)
    dx_ref = oracle.ragged_dot(y, dA, gs, trans_rhs=True)
    dy_ref = oracle.ragged_dot(x, dA, gs, trans_rhs=False)
    xd, yd, gd, dAd = _to_dev(x, y, gs, dA)
    xd.requires_grad_(True)
    yd.requires_grad_(True)
    out = rd.trans_ragged_dot(xd, yd, gd)
    out.backward(dAd)
    _assert_close(xd.grad.cpu(), dx_ref, "tgmm dx")
    _assert_close(yd.grad.cpu(), dy_ref, "tgmm dy")


def test_interpret_and_dtype_arguments_raise():
    x = torch.zeros(8, 8, dtype=torch.bfloat16, device=DEV)
    A = torch.zeros(1, 8, 8, dtype=torch.bfloat16, device=DEV)
    gs = torch.tensor([8], dtype=torch.int32, device=DEV)
    with pytest.raises(NotImplementedError):
        rd.gmm(x, A, gs, interpret=True)
    with pytest.raises(NotImplementedError):
        rd.gmm(x, A, gs, acc_dtype=torch.float16)
    with pytest.raises(RuntimeError):
        rd.gmm(x.cpu(), A, gs)


# ------------------------------------------------------------------ full-size parity
def _assert_close_blocks(got, want, what, rows_per_block=4096):
    """Elementwise tolerance over whole tensors, a block of rows at a time (bounded host memory)."""
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    for lo in range(0, got.shape[0], rows_per_block):
        _assert_close(got[lo:lo + rows_per_block].cpu(), want[lo:lo + rows_per_block], f"{what} rows {lo}..")


def test_mixtral_shape_full_parity():
    """The benchmark size, forward: EVERY element of y against the oracle (its 16-bit CPU matmul
    mode, which test_native_16bit_mode_agrees holds to the fp32 mode), plus exact linearity under
    scaling by a power of two and the zero tail."""
    s = workloads.MIXTRAL
    gs_np = workloads.group_sizes_mixtral_ragged(0)
    gs_np[-1] -= 200  # leave a tail of unowned rows
    x, A, _ = workloads.make_inputs(s, DEV, seed=0, with_dout=False)
    gs = torch.from_numpy(gs_np).to(DEV)
    ws = ops._workspace(s.m, s.g, DEV)
    y = ops.gmm_forward(x, A, gs, workspace=ws)
    assert ops.device_status(ws) == 0
    y2 = ops.gmm_forward(x * 2, A, gs)
    torch.cuda.synchronize()
    total = int(gs_np.sum())
    assert float(y[total:].float().abs().max()) == 0.0
    assert torch.equal((y.float() * 2).to(torch.bfloat16), y2)
    want = oracle.ragged_dot(x, A, gs_np, native_16bit=True)
    _assert_close_blocks(y, want, "mixtral y")
    err = oracle.rel_l2_err(y.cpu(), want, axis=-1, mask=torch.arange(s.m) < total)
    assert float(err.max()) < EPS_ROWS_BF16


def test_mixtral_shape_backward_full_parity():
    """dlhs and drhs at the benchmark size with ragged group sizes: every element of both against
    the oracle (so every k tile and column tile of every group, whatever order the kernel takes
    them in), and drhs additive over a split of the rows."""
    s = workloads.MIXTRAL
    gs_np = workloads.group_sizes_mixtral_ragged(0)
    x, A, dout = workloads.make_inputs(s, DEV, seed=0)
    gs = torch.from_numpy(gs_np).to(DEV)
    ws = ops._workspace(s.m, s.g, DEV)
    dx = ops.gmm_forward(dout, A, gs, trans_rhs=True, workspace=ws)
    assert ops.device_status(ws) == 0
    want_dx = oracle.ragged_dot(dout, A, gs_np, trans_rhs=True, native_16bit=True)
    _assert_close_blocks(dx, want_dx, "mixtral dlhs")
    assert float(oracle.rel_l2_err(dx.cpu(), want_dx, axis=-1).max()) < EPS_ROWS_BF16
    del dx, want_dx, A
    dA = ops.tgmm_forward(x, dout, gs, workspace=ws)
    assert ops.device_status(ws) == 0
    want_dA = oracle.trans_ragged_dot(x, dout, gs_np, native_16bit=True)
    for gi in range(s.g):
        _assert_close_blocks(dA[gi], want_dA[gi], f"mixtral drhs block {gi}")
        assert float(oracle.rel_l2_err(dA[gi].cpu(), want_dA[gi], axis=(-1, -2))) < EPS_GROUPS_BF16
    del want_dA
    # rows of group gi split in two halves as two groups: the two blocks add up to the one block
    # (fp32 sums rounded once vs twice: within two bf16 ulps of the larger magnitude)
    gs2 = np.zeros(2 * s.g, dtype=np.int32)
    gs2[0::2] = gs_np // 2
    gs2[1::2] = gs_np - gs_np // 2
    dA2 = ops.tgmm_forward(x, dout, torch.from_numpy(gs2).to(DEV))
    summed = dA2[0::2].float() + dA2[1::2].float()
    err = (summed - dA.float()).abs()
    tol = 2.0 ** -6 * torch.maximum(dA2[0::2].float().abs(), dA2[1::2].float().abs()) + 1e-3
    assert bool((err <= tol).all()), f"drhs not additive over a row split: worst {float((err / tol).max()):.2f}x"
    del dA2, summed, err, tol


def test_deepseek_shape_full_parity():
    """The largest configuration (m 32768, k 7168, n 2048, 256 experts, heavy-tailed sizes with
    empty experts; 7.5 GB of weights and as much of drhs): every element of y and of dlhs against
    the oracle; for drhs every element of the blocks of the three largest, the three smallest
    non-empty and ALL empty experts (zeros), the zero tail, and the device status word."""
    s = workloads.DEEPSEEK_V3
    gs_np = workloads.group_sizes_deepseek(0)
    gs_np[int(np.argmax(gs_np))] -= 100  # leave a tail of unowned rows
    x, A, dout = workloads.make_inputs(s, DEV, seed=0)
    gs = torch.from_numpy(gs_np).to(DEV)
    ws = ops._workspace(s.m, s.g, DEV)
    y = ops.gmm_forward(x, A, gs, workspace=ws)
    assert ops.device_status(ws) == 0
    total = int(gs_np.sum())
    assert float(y[total:].float().abs().max()) == 0.0
    _assert_close_blocks(y, oracle.ragged_dot(x, A, gs_np, native_16bit=True), "deepseek y")
    del y
    dx = ops.gmm_forward(dout, A, gs, trans_rhs=True, workspace=ws)
    assert ops.device_status(ws) == 0
    _assert_close_blocks(dx, oracle.ragged_dot(dout, A, gs_np, trans_rhs=True, native_16bit=True), "deepseek dlhs")
    del dx, A
    torch.cuda.empty_cache()
    dA = ops.tgmm_forward(x, dout, gs, workspace=ws)
    assert ops.device_status(ws) == 0
    offs = np.concatenate([[0], np.cumsum(gs_np)])
    empty = np.nonzero(gs_np == 0)[0]
    assert len(empty) > 0
    for gi in empty:
        assert float(dA[int(gi)].float().abs().max()) == 0.0
    order = np.argsort(gs_np, kind="stable")
    nonempty = [int(i) for i in order if gs_np[i] > 0]
    xc, dc = x.cpu(), dout.cpu()
    for gi in nonempty[:3] + nonempty[-3:]:
        lo, hi = int(offs[gi]), int(offs[gi + 1])
        want = (xc[lo:hi].T @ dc[lo:hi])
        _assert_close_blocks(dA[gi], want, f"deepseek drhs block {gi} ({hi - lo} rows)")


# ------------------------------------------------------------------ against the reference's own outputs
from tests import golden_io  # noqa: E402

GOLDEN = golden_io.gemm_cases()


@pytest.mark.parametrize("case", GOLDEN, ids=lambda c: c["name"])
def test_cuda_matches_reference_golden(case):
    """The CUDA path against outputs produced by the reference's own kernels
    (tests/golden/make_golden.py)."""
    gs = case["group_sizes"]
    x, A, dout, gd = _to_dev(case["x"], case["A"], case["dout"], gs)
    At = A.transpose(1, 2).contiguous()
    pairs = [
        ("y", ops.gmm_forward(x, A, gd), case["y"]),
        ("y_trans_rhs", ops.gmm_forward(x, At, gd, trans_rhs=True), case.get("y_trans_rhs")),
        ("tgmm", ops.tgmm_forward(x, dout, gd), case.get("tgmm")),
        ("dlhs", ops.gmm_forward(dout, A, gd, trans_rhs=True), case["dlhs"]),
        ("drhs", ops.tgmm_forward(x, dout, gd), case["drhs"]),
        ("dlhs_trans_rhs", ops.gmm_forward(dout, At, gd, trans_rhs=False), case.get("dlhs_trans_rhs")),
        ("drhs_trans_rhs", ops.tgmm_forward(dout, x, gd), case.get("drhs_trans_rhs")),
    ]
    for name, got, want in pairs:
        if want is None:
            continue
        assert bool(torch.isfinite(want.float()).all())
        _assert_close(got.cpu(), want, f"{case['name']}:{name}")


@pytest.mark.parametrize("case", golden_io.metadata_cases(),
                         ids=lambda c: f"gs{len(c['group_sizes'])}_m{c['m_chunk'][0]}_c{c['m_chunk'][1]}")
def test_cuda_metadata_matches_reference_golden(case):
    m, chunk = (int(v) for v in case["m_chunk"])
    got = rd.make_group_metadata(torch.from_numpy(case["group_sizes"]).to(DEV), m, chunk)
    assert np.array_equal(got.group_offsets.cpu().numpy(), case["group_offsets"])
    assert np.array_equal(got.row_it2group.cpu().numpy(), case["row_it2group"])
    assert np.array_equal(got.row_it2it_in_group.cpu().numpy(), case["row_it2it_in_group"])
    assert int(got.total_row_its.cpu()) == int(case["total_row_its"])


# ------------------------------------------------------------------ expert-parallel building blocks
def test_gather_rows_bit_exact():
    src = oracle.reference_normal(31, (300, 136), torch.bfloat16)
    idx = torch.tensor(np.random.default_rng(0).integers(0, 300, size=777), dtype=torch.int32)
    got = ops.gather_rows(src.to(DEV), idx.to(DEV)).cpu()
    assert torch.equal(got.view(torch.int16), src[idx.long()].view(torch.int16))
    idx[5] = -1
    idx[6] = 300
    got = ops.gather_rows(src.to(DEV), idx.to(DEV)).cpu()
    assert float(got[5].float().abs().max()) == 0.0 and float(got[6].float().abs().max()) == 0.0


def test_gmm_indexed_shares_weights_between_segments():
    m, k, n, experts = 640, 128, 136, 3
    x, A, _ = _inputs(41, m, k, n, experts)
    seg_sizes = [100, 0, 60, 130, 90, 1, 0, 200, 30]  # 3 sources x 3 experts, source-major
    seg2e = [0, 1, 2] * 3
    want = oracle.ragged_dot(x, A[torch.tensor(seg2e)], torch.tensor(seg_sizes))
    got = ops.gmm_forward(x.to(DEV), A.to(DEV), torch.tensor(seg_sizes, dtype=torch.int32, device=DEV),
                          group_to_weight=torch.tensor(seg2e, dtype=torch.int32, device=DEV)).cpu()
    _assert_close(got, want, "gmm_indexed")
    assert float(got[sum(seg_sizes):].float().abs().max()) == 0.0


def test_expert_parallel_single_rank_matches_oracle():
    from gpu_ragged_dot_b200 import ep

    E, k, n, T, top_k = 16, 128, 72, 300, 4
    layer = ep.ExpertParallelRaggedDot(E, k, n, torch.device(DEV), seed=5)
    x = workloads.normal_tensor((T, k), 1.0, 77, DEV)
    routing = torch.from_numpy(workloads.topk_routing(T, E, top_k, seed=9)).to(DEV)
    y, plan = layer.forward(x, routing)
    flat = routing.reshape(-1).cpu()
    order = torch.sort(flat, stable=True).indices
    rows = x.cpu()[(order // top_k)]
    gs = torch.bincount(flat, minlength=E).to(torch.int32)
    assert plan.segment_sizes.cpu().tolist() == gs.tolist()
    want = oracle.ragged_dot(rows, layer.weights.cpu(), gs)
    _assert_close(y.cpu(), want, "ep single rank")


# ------------------------------------------------------------------ peer-store dispatch (one GPU stands in for W ranks)
def _plan_oracle(counts_all, rank):
    world, experts = counts_all.shape
    local = experts // world
    dest_offset = np.zeros(experts, dtype=np.int64)
    for e in range(experts):
        owner = e // local
        first = owner * local
        dest_offset[e] = counts_all[:rank, first:first + local].sum() + counts_all[rank, first:e].sum()
    seg = counts_all[:, rank * local:(rank + 1) * local].reshape(-1)
    return dest_offset, seg, int(seg.sum())


@pytest.mark.parametrize("world", [1, 2, 4])
def test_ep_plan_and_dispatch_emulated_ranks(world):
    """W ranks emulated on one GPU: each rank's count / plan / dispatch kernels run one after the
    other (none waits for another), all writing into W receive buffers on this device.  The
    buffers must hold exactly the rows the routing says, grouped (source, expert), and the local
    rd_gmm_indexed over them must match the oracle."""
    E, k, n, T, top_k = 16, 128, 72, 200, 4
    local = E // world
    xs = [workloads.normal_tensor((T, k), 1.0, 1000 + r, DEV) for r in range(world)]
    routings = [torch.from_numpy(workloads.topk_routing(T, E, top_k, seed=3000 + r)).to(DEV) for r in range(world)]
    counts = [ops.ep_count(routings[r], E) for r in range(world)]
    counts_all = torch.stack(counts).contiguous()
    want_counts = np.stack([np.bincount(routings[r].cpu().numpy().reshape(-1), minlength=E) for r in range(world)])
    assert np.array_equal(counts_all.cpu().numpy(), want_counts)
    capacity = T * top_k * world
    bufs = [torch.full((capacity, k), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    peer_base = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=DEV)
    plans, poss = [], []
    for r in range(world):
        dest_offset, seg, fill, totals = ops.ep_plan(counts_all, r)
        off_ref, seg_ref, tot_ref = _plan_oracle(want_counts, r)
        assert np.array_equal(dest_offset.cpu().numpy(), off_ref)
        assert np.array_equal(seg.cpu().numpy(), seg_ref) and int(totals.cpu()) == tot_ref
        poss.append(ops.ep_dispatch(xs[r], routings[r], E, world, dest_offset, fill, peer_base, capacity))
        plans.append((seg, tot_ref))
    torch.cuda.synchronize()
    weights = workloads.normal_tensor((E, k, n), k ** -0.5, 7, DEV)
    for d in range(world):
        seg, total = plans[d]
        got = bufs[d][:total].cpu()
        assert bool(torch.isfinite(got.float()).all()), "a received row was never written"
        assert bool(torch.isnan(bufs[d][total:].float()).all()), "rows written past the received total"
        # every (source, token, slot) routed to an expert of rank d sits at its recorded position
        off = 0
        seg_np = seg.cpu().numpy()
        for s in range(world):
            flat = routings[s].cpu().reshape(-1)
            pos = poss[s].cpu().reshape(-1)
            for j in range(local):
                e = d * local + j
                idx = (flat == e).nonzero().flatten()
                cnt = int(seg_np[s * local + j])
                assert len(idx) == cnt
                p = pos[idx]
                assert int(p.min()) >= off and int(p.max()) < off + cnt and len(set(p.tolist())) == cnt
                assert torch.equal(got[p.long()].view(torch.int16), xs[s].cpu()[idx // top_k].view(torch.int16))
                off += cnt
        # local grouped GEMM over the received segments, rows past `total` left unwritten
        seg2e = torch.arange(local, dtype=torch.int32, device=DEV).repeat(world)
        y = torch.full((capacity, n), float("nan"), dtype=torch.bfloat16, device=DEV)
        cfg = _lib.TileCfg(0, 0, 0, 0, _lib.RD_CFG_NO_ZERO_TAIL)
        ops.gmm_forward(bufs[d], weights[d * local:(d + 1) * local], seg, group_to_weight=seg2e, cfg=cfg, out=y)
        want = oracle.ragged_dot(got, weights[d * local:(d + 1) * local].cpu()[seg2e.cpu().long()], seg.cpu())
        _assert_close(y[:total].cpu(), want, f"ep p2p rank {d}")
        assert bool(torch.isnan(y[total:].float()).all()), "NO_ZERO_TAIL: rows past the total must stay untouched"


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_ep_ring_phases_emulated_ranks(world):
    """The ring-phased exchange with W ranks emulated on one GPU, everything on one stream so that
    no kernel ever waits for a later one: all ranks' send lists are copied first, phase by phase
    (each raises its flag on the destination), then every rank's flag-gated GEMM finds its flags up.  Checks the ring
    layout (position q = (dest - source) mod W), the flags, and the GEMM against the oracle; two
    epochs in a row."""
    E, k, n, T, top_k = 16, 128, 72, 200, 4
    local = E // world
    capacity = T * top_k * world
    weights = workloads.normal_tensor((E, k, n), k ** -0.5, 7, DEV)
    bufs = [torch.full((capacity, k), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    flags = [torch.zeros(max(world, 4), dtype=torch.int32, device=DEV) for _ in range(world)]
    for epoch in (1, 2):
        xs = [workloads.normal_tensor((T, k), 1.0, 1000 * epoch + r, DEV) for r in range(world)]
        routings = [torch.from_numpy(workloads.topk_routing(T, E, top_k, seed=3000 * epoch + r)).to(DEV)
                    for r in range(world)]
        counts_all = torch.stack([ops.ep_count(routings[r], E) for r in range(world)]).contiguous()
        cnt = counts_all.cpu().numpy()
        plans, poss = [], []
        for r in range(world):
            plan = ops.ep_plan_ring(counts_all, r)
            # oracle of the ring plan
            seg_ref = np.array([cnt[(r - q) % world, r * local + j] for q in range(world) for j in range(local)])
            assert np.array_equal(plan["segment_sizes"].cpu().numpy(), seg_ref)
            off_ref = np.zeros(E, dtype=np.int64)
            for e in range(E):
                owner, first = e // local, (e // local) * local
                before = (owner - r) % world
                off_ref[e] = sum(int(cnt[(owner - q) % world, first:first + local].sum()) for q in range(before)) \
                    + int(cnt[r, first:e].sum())
            assert np.array_equal(plan["dest_offset"].cpu().numpy(), off_ref)
            assert int(plan["totals"].cpu()) == int(cnt[:, r * local:(r + 1) * local].sum())
            dest_pos = torch.full((T * top_k,), -7, dtype=torch.int32, device=DEV)
            send_index = torch.full((T * top_k,), -7, dtype=torch.int32, device=DEV)
            ops.ep_assign(routings[r].to(torch.int32).contiguous(), E, world, r, plan, capacity, dest_pos,
                          send_index)
            for p in range(world):
                d = (r + p) % world
                ops.ep_send_list(xs[r], top_k, send_index, plan, p, world, dest_pos, bufs[d].data_ptr(),
                                 capacity, flags[d].data_ptr() + 4 * p, epoch)
            plans.append(plan)
            poss.append(dest_pos)
        for d in range(world):
            assert flags[d][:world].cpu().tolist() == [epoch] * world
            seg = plans[d]["segment_sizes"]
            total = int(plans[d]["totals"].cpu())
            got = bufs[d][:total].cpu()
            off = 0
            seg_np = seg.cpu().numpy()
            for q in range(world):
                s_rank = (d - q) % world
                flat = routings[s_rank].cpu().reshape(-1)
                pos = poss[s_rank].cpu().reshape(-1)
                assert int(pos.min()) >= 0
                for j in range(local):
                    idx = (flat == d * local + j).nonzero().flatten()
                    c = int(seg_np[q * local + j])
                    assert len(idx) == c
                    if c:
                        pp = pos[idx]
                        assert int(pp.min()) >= off and int(pp.max()) < off + c and len(set(pp.tolist())) == c
                        assert torch.equal(got[pp.long()].view(torch.int16),
                                           xs[s_rank].cpu()[idx // top_k].view(torch.int16))
                    off += c
            seg2e = torch.arange(local, dtype=torch.int32, device=DEV).repeat(world)
            y = torch.full((capacity, n), float("nan"), dtype=torch.bfloat16, device=DEV)
            for tile_m in (128, 256) if n >= 256 else (128,):
                cfg = _lib.TileCfg(0, 0, 1, tile_m, _lib.RD_CFG_NO_ZERO_TAIL)
                ws = ops._workspace(capacity, E, DEV)
                ops.gmm_forward(bufs[d], weights[d * local:(d + 1) * local], seg, group_to_weight=seg2e, cfg=cfg,
                                out=y, workspace=ws, ready=(flags[d], local, epoch))
                assert ops.device_status(ws) == 0
                want = oracle.ragged_dot(got, weights[d * local:(d + 1) * local].cpu()[seg2e.cpu().long()], seg.cpu())
                _assert_close(y[:total].cpu(), want, f"ep ring rank {d}")


def test_ep_assign_send_lists_and_fused_single_rank():
    """Fused exchange on one rank: assign + own-row copy + rd_gmm_ep_fused (whose sender CTAs have
    nothing to send when world == 1), checked against the NCCL-free reference path."""
    from gpu_ragged_dot_b200 import ep

    E, k, n, T, top_k = 16, 128, 264, 300, 4
    x = workloads.normal_tensor((T, k), 1.0, 77, DEV)
    routing = torch.from_numpy(workloads.topk_routing(T, E, top_k, seed=9)).to(DEV)
    a = ep.ExpertParallelRaggedDot(E, k, n, torch.device(DEV), seed=5)
    b = ep.ExpertParallelRaggedDot(E, k, n, torch.device(DEV), seed=5, dispatch="fused")
    ya, plan = a.forward(x, routing)
    for step in range(2):
        yb, seg, dest_pos, totals = b.forward(x, routing)
    assert ops.device_status(b._ring["ws"]) == 0
    assert int(totals.cpu()) == T * top_k and seg.cpu().tolist() == plan.segment_sizes.cpu().tolist()
    order = torch.sort(routing.reshape(-1).cpu().long(), stable=True).indices
    pos = dest_pos.reshape(-1).cpu().long()
    assert sorted(pos.tolist()) == list(range(T * top_k))
    _assert_close(yb.cpu()[pos[order]], ya.cpu(), "fused vs nccl path")


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ep_assign_send_lists_emulated_ranks(world):
    """rd_ep_plan_ring + rd_ep_assign for W emulated ranks: every phase's send list holds exactly the
    entries routed to rank + p, and positions at the owners are a permutation of each segment."""
    E, T, top_k = 16, 200, 4
    local = E // world
    capacity = T * top_k * world
    routings = [torch.from_numpy(workloads.topk_routing(T, E, top_k, seed=40 + r)).to(DEV) for r in range(world)]
    counts_all = torch.stack([ops.ep_count(routings[r], E) for r in range(world)]).contiguous()
    for r in range(world):
        plan = ops.ep_plan_ring(counts_all, r)
        dest_pos = torch.full((T * top_k,), -9, dtype=torch.int32, device=DEV)
        send_index = torch.full((T * top_k,), -9, dtype=torch.int32, device=DEV)
        ops.ep_assign(routings[r].to(torch.int32).contiguous(), E, world, r, plan, capacity, dest_pos, send_index)
        flat = routings[r].cpu().reshape(-1).numpy()
        start = plan["send_start"].cpu().numpy()
        idx = send_index.cpu().numpy()
        pos = dest_pos.cpu().numpy()
        off = plan["dest_offset"].cpu().numpy()
        assert start[0] == 0 and start[world] == T * top_k
        for p in range(world):
            d = (r + p) % world
            want = np.nonzero((flat // local) == d)[0]
            got = np.sort(idx[start[p]:start[p + 1]])
            assert np.array_equal(got, want)
        for e in range(E):
            mine = np.nonzero(flat == e)[0]
            assert sorted(pos[mine].tolist()) == list(range(off[e], off[e] + len(mine)))


def test_flag_gated_gmm_256_row_tiles():
    """rd_gmm_indexed_when_ready through the 256-row kernel, flags already up."""
    m, k, n, g = 1500, 128, 512, 6
    x, A, _ = _inputs(5, m, k, n, 3)
    gs = torch.tensor([300, 0, 411, 256, 1, 500], dtype=torch.int32)
    g2w = torch.tensor([0, 1, 2, 0, 1, 2], dtype=torch.int32)
    flags = torch.tensor([3, 3, 3, 0], dtype=torch.int32, device=DEV)
    cfg = _lib.TileCfg(256, 0, 1, 256, 0)
    ws = ops._workspace(m, g, DEV)
    y = ops.gmm_forward(x.to(DEV), A.to(DEV), gs.to(DEV), group_to_weight=g2w.to(DEV), cfg=cfg, workspace=ws,
                        ready=(flags, 2, 3))
    assert ops.device_status(ws) == 0
    want = oracle.ragged_dot(x, A[g2w.long()], gs)
    _assert_close(y.cpu(), want, "flag-gated 256-row")


def test_expert_parallel_p2p_single_rank_matches_nccl_path():
    from gpu_ragged_dot_b200 import ep

    E, k, n, T, top_k = 16, 128, 72, 300, 4
    x = workloads.normal_tensor((T, k), 1.0, 77, DEV)
    routing = torch.from_numpy(workloads.topk_routing(T, E, top_k, seed=9)).to(DEV)
    a = ep.ExpertParallelRaggedDot(E, k, n, torch.device(DEV), seed=5)
    b = ep.ExpertParallelRaggedDot(E, k, n, torch.device(DEV), seed=5, dispatch="p2p")
    ya, plan = a.forward(x, routing)
    yb, seg, dest_pos, totals = b.forward(x, routing)
    assert int(totals.cpu()) == T * top_k and seg.cpu().tolist() == plan.segment_sizes.cpu().tolist()
    # same rows, possibly in another order inside a segment: compare per (token, slot)
    order = torch.sort(routing.reshape(-1).cpu().long(), stable=True).indices  # sorted row -> entry
    pos = dest_pos.reshape(-1).cpu().long()
    _assert_close(yb.cpu()[pos[order]], ya.cpu(), "p2p vs nccl path")


# ------------------------------------------------------------------ float32 inputs (TF32 on the tensor cores)
def _f32_err(got, x, A, gs, fn, axis, mask):
    """Relative-L2 error against the fp32 oracle fed TF32-reduced operands, for both ways the
    hardware might reduce them; returns the smaller (and which)."""
    errs = {}
    for mode in ("truncate", "nearest"):
        want = fn(oracle.to_tf32(x, mode), oracle.to_tf32(A, mode), gs)
        errs[mode] = float(oracle.rel_l2_err(got, want, axis=axis, mask=mask).max())
    best = min(errs, key=errs.get)
    return errs[best], best, errs


@pytest.mark.parametrize("case", GRID[:10], ids=lambda c: "-".join(f"{k}{v}" for k, v in c.items()))
def test_reference_grid_float32(case):
    """float32 cases of the reference grid (tests.py:93): rel-L2 5e-4 per row for gmm and its
    transposed form, 1e-4 per group for tgmm, against an oracle with TF32 operands; and within
    2e-3 of the exact fp32 product."""
    m, k, n, g = case["m"], case["k"], case["n"], case["g"]
    x, A, dout = _inputs(case["seed"], m, k, n, g, dtype=torch.float32, random_inputs=case["random_inputs"])
    target_m = max(min(round(m * case["fill_in"]), m), 0)
    gs = torch.from_numpy(oracle.reference_group_sizes(case["seed"] + 17, g, target_m))
    rows = torch.arange(m) < target_m
    xd, Ad, dd, gd = _to_dev(x, A, dout, gs)

    y = ops.gmm_forward(xd, Ad, gd).cpu()
    assert y.dtype == torch.float32
    e, mode, all_e = _f32_err(y, x, A, gs, lambda a, b, c: oracle.ragged_dot(a, b, c), -1, rows)
    assert e < 5e-4, f"gmm f32 rel-L2 {all_e}"
    exact = float(oracle.rel_l2_err(y, oracle.ragged_dot(x, A, gs), axis=-1, mask=rows).max())
    assert exact < 2e-3, f"gmm f32 vs exact fp32: {exact:.2e}"
    if target_m < m:
        assert float(y[target_m:].abs().max()) == 0.0

    At = A.transpose(1, 2).contiguous()
    yt = ops.gmm_forward(xd, At.to(DEV), gd, trans_rhs=True).cpu()
    e, _, all_e = _f32_err(yt, x, At, gs, lambda a, b, c: oracle.ragged_dot(a, b, c, trans_rhs=True), -1, rows)
    assert e < 5e-4, f"gmm trans f32 rel-L2 {all_e}"

    out = ops.tgmm_forward(xd, dd, gd).cpu()
    e, _, all_e = _f32_err(out, x, dout, gs, lambda a, b, c: oracle.trans_ragged_dot(a, b, c), (-1, -2), gs != 0)
    assert e < 1e-4, f"tgmm f32 rel-L2 {all_e}"
    for gi in (gs == 0).nonzero().flatten().tolist():
        assert float(out[gi].abs().max()) == 0.0


def test_float32_vjp_and_tile_widths():
    m, k, n, g = 600, 200, 328, 5
    x, A, dout = _inputs(51, m, k, n, g, dtype=torch.float32)
    gs = torch.tensor([130, 0, 257, 1, 200], dtype=torch.int32)
    rows = torch.arange(m) < int(gs.sum())
    for tile_n in (64, 128, 256):
        cfg = _lib.TileCfg(tile_n, 0, 0, 0, 0)
        y = ops.gmm_forward(x.to(DEV), A.to(DEV), gs.to(DEV), cfg=cfg).cpu()
        e, _, all_e = _f32_err(y, x, A, gs, lambda a, b, c: oracle.ragged_dot(a, b, c), -1, rows)
        assert e < 5e-4, f"tile_n={tile_n}: {all_e}"
    xd, Ad = x.to(DEV).requires_grad_(True), A.to(DEV).requires_grad_(True)
    y = rd.ragged_dot(xd, Ad, gs.to(DEV))
    y.backward(dout.to(DEV))
    dx_ref, dA_ref = oracle.ragged_dot_vjp(x, A, gs, dout)
    assert float(oracle.rel_l2_err(xd.grad.cpu(), dx_ref, axis=-1, mask=rows).max()) < 2e-3
    assert float(oracle.rel_l2_err(Ad.grad.cpu(), dA_ref, axis=(-1, -2), mask=gs != 0).max()) < 2e-3


def test_ragged_dot_general_matches_oracle():
    """ragged_dot_general with the dimension numbers of the reference's own oracle calls
    (tests.py:31-48): both modes, and the rhs-transposed form of the first."""
    m, k, n, g = 300, 136, 200, 5
    rng = np.random.default_rng(21)
    bf = lambda a: torch.from_numpy(a.astype(np.float32)).to(torch.bfloat16)  # noqa: E731
    x, A, y = bf(rng.standard_normal((m, k))), bf(rng.standard_normal((g, k, n)) / np.sqrt(k)), bf(rng.standard_normal((m, n)))
    gs = torch.tensor([100, 0, 57, 120, 3], dtype=torch.int32)
    DN = rd.RaggedDotDimensionNumbers
    got = rd.ragged_dot_general(x.to(DEV), A.to(DEV), gs.to(DEV), DN((([1], [1]), ([], [])), [0], [0]))
    want = oracle.ragged_dot(x, A, gs)
    ok, worst = oracle.allclose_report(got.cpu(), want, 2e-2, 2e-2)
    assert ok, worst
    At = A.transpose(1, 2).contiguous()
    got = rd.ragged_dot_general(x.to(DEV), At.to(DEV), gs.to(DEV), DN((([1], [2]), ([], [])), [0], [0]))
    ok, worst = oracle.allclose_report(got.cpu(), want, 2e-2, 2e-2)
    assert ok, worst
    got = rd.ragged_dot_general(x.to(DEV), y.to(DEV), gs.to(DEV), DN((([0], [0]), ([], [])), [0], []))
    ok, worst = oracle.allclose_report(got.cpu(), oracle.trans_ragged_dot(x, y, gs), 2e-2, 2e-2)
    assert ok, worst


# ------------------------------------------------------------------ strided tgmm, overshooting sizes, expiry
@pytest.mark.parametrize("n,tile_m", [(264, 128), (264, 256), (72, 0), (136, 0)])
def test_tgmm_strided_matches_oracle(n, tile_m):
    """rd_tgmm_strided: block i sums the groups i, i + g, i + 2g, ... (segments with ragged ends,
    empty segments, one block whose segments are all empty)."""
    m, k, g, seg = 1100, 256, 4, 3
    x, _, dout = _inputs(61, m, k, n, 1)
    sizes = [130, 0, 64, 77,   0, 0, 200, 1,   63, 0, 129, 300]  # segment-major: [q][i]
    assert sum(sizes) <= m and all(sizes[q * g + 1] == 0 for q in range(seg))
    offs = np.concatenate([[0], np.cumsum(sizes)])
    want = torch.zeros((g, k, n), dtype=torch.float32)
    for q in range(seg):
        for i in range(g):
            lo, hi = int(offs[q * g + i]), int(offs[q * g + i + 1])
            want[i] += x[lo:hi].float().T @ dout[lo:hi].float()
    cfg = _lib.TileCfg(256 if tile_m else 0, 0, 1, tile_m, 0) if tile_m else None
    ws = ops._workspace(m, len(sizes), DEV)
    got = ops.tgmm_forward(x.to(DEV), dout.to(DEV), torch.tensor(sizes, dtype=torch.int32, device=DEV),
                           cfg=cfg, workspace=ws, seg_count=seg)
    assert ops.device_status(ws) == 0
    _assert_close(got.cpu(), want.to(torch.bfloat16), "tgmm strided")
    assert float(got[1].float().abs().max()) == 0.0
    e = oracle.rel_l2_err(got.cpu(), want, axis=(-1, -2), mask=torch.tensor([True, False, True, True]))
    assert float(e.max()) < EPS_GROUPS_BF16
    # one segment per block is plain tgmm
    plain = ops.tgmm_forward(x.to(DEV), dout.to(DEV), torch.tensor(sizes[:g], dtype=torch.int32, device=DEV))
    one = ops.tgmm_forward(x.to(DEV), dout.to(DEV), torch.tensor(sizes[:g], dtype=torch.int32, device=DEV),
                           seg_count=1, cfg=cfg)
    assert torch.equal(plain.view(torch.int16), one.view(torch.int16))


@pytest.mark.parametrize("sizes,m,n", [([1000], 256, 1024), ([100, 300, 50], 256, 520), ([0, 5000, 7], 700, 264)])
@pytest.mark.parametrize("tile_m", [128, 256])
def test_group_sizes_overshooting_m(sizes, m, n, tile_m):
    """sum(group_sizes) > m: every row below m belongs to the group whose range covers it and
    must be written for all n columns (a group is clamped to the rows that exist)."""
    k, g = 128, len(sizes)
    x, A, dout = _inputs(71, m, k, n, g)
    gs = torch.tensor(sizes, dtype=torch.int32)
    cfg = _lib.TileCfg(256, 0, 1, tile_m, 0)
    y = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    ws = ops._workspace(m, g, DEV)
    ops.gmm_forward(x.to(DEV), A.to(DEV), gs.to(DEV), cfg=cfg, out=y, workspace=ws)
    assert ops.device_status(ws) == 0
    assert bool(torch.isfinite(y.float()).all()), "rows below m left unwritten"
    _assert_close(y.cpu(), oracle.ragged_dot(x, A, gs), "gmm, sizes overshooting m")
    dA = ops.tgmm_forward(x.to(DEV), dout.to(DEV), gs.to(DEV), cfg=cfg)
    _assert_close(dA.cpu(), oracle.trans_ragged_dot(x, dout, gs), "tgmm, sizes overshooting m")


@pytest.mark.parametrize("tile_m", [128, 256])
def test_bounded_wait_expiry_is_reported_and_recoverable(tile_m, monkeypatch):
    """A wait that can never be satisfied (ready flags that nothing raises) must end by itself: the
    kernel gives up after rd_tile_cfg.wait_limit_ms, returns, and the status word says so; the
    next ordinary call on the same workspace is correct.  Nothing traps, faults or hangs."""
    import time

    monkeypatch.delenv("RD_CHECK_STATUS", raising=False)  # the first call must return, not raise
    m, k, n, g = 700, 128, 512, 4
    x, A, _ = _inputs(81, m, k, n, 2)
    gs = torch.tensor([300, 0, 250, 150], dtype=torch.int32)
    g2w = torch.tensor([0, 1, 0, 1], dtype=torch.int32, device=DEV)
    flags = torch.zeros(4, dtype=torch.int32, device=DEV)
    cfg = _lib.TileCfg(256, 0, 1, tile_m, 0, 5)  # five milliseconds
    ws = ops._workspace(m, g, DEV)
    xd, Ad, gd = _to_dev(x, A, gs)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ops.gmm_forward(xd, Ad, gd, group_to_weight=g2w, cfg=cfg, workspace=ws, ready=(flags, 1, 1))
    status = ops.device_status(ws)  # synchronises
    waited = time.perf_counter() - t0
    assert status == _lib.RD_ERR_DEVICE_WAIT
    assert waited < 1.0, f"the kernel took {waited:.2f} s to give up on a 5 ms limit"
    # the same call raises when the caller asks for the check
    monkeypatch.setenv("RD_CHECK_STATUS", "1")
    with pytest.raises(_lib.RaggedDotError) as ei:
        ops.gmm_forward(xd, Ad, gd, group_to_weight=g2w, cfg=cfg, workspace=ws, ready=(flags, 1, 1))
    assert ei.value.code == _lib.RD_ERR_DEVICE_WAIT
    monkeypatch.delenv("RD_CHECK_STATUS")
    # once the flags are up the same kernel runs through, and so does a plain call
    flags.fill_(1)
    y = ops.gmm_forward(xd, Ad, gd, group_to_weight=g2w, cfg=cfg, workspace=ws, ready=(flags, 1, 1))
    assert ops.device_status(ws) == 0
    _assert_close(y.cpu(), oracle.ragged_dot(x, A[g2w.cpu().long()], gs), "flag-gated gmm after an expiry")
    y2 = ops.gmm_forward(xd, Ad[:1].expand(4, -1, -1).contiguous(), gd, workspace=ws)
    assert ops.device_status(ws) == 0
    _assert_close(y2.cpu(), oracle.ragged_dot(x, A[:1].expand(4, -1, -1), gs), "plain gmm after an expiry")


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_ep_combine_pull_emulated_ranks(world):
    """rd_ep_combine_pull with the W owners' gradient buffers all on this GPU: each token's row is
    the fp32 sum of its top_k rows at the recorded positions, rounded once."""
    E, k, T, top_k = 16, 264, 300, 4
    local = E // world
    capacity = T * top_k * world
    bufs = [oracle.reference_normal(90 + d, (capacity, k), torch.bfloat16).to(DEV) for d in range(world)]
    base = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=DEV)
    routing = torch.from_numpy(workloads.topk_routing(T, E, top_k, seed=5)).to(DEV).to(torch.int32)
    pos = torch.from_numpy(np.random.default_rng(3).integers(0, capacity, size=(T, top_k)).astype(np.int32)).to(DEV)
    pos[7, 2] = -1          # a dropped row adds nothing
    routing[9, 0] = E + 3   # an expert that does not exist adds nothing
    got = ops.ep_combine_pull(routing, pos, E, world, base, capacity, k, torch.bfloat16)
    want = torch.zeros((T, k), dtype=torch.float32)
    r_cpu, p_cpu = routing.cpu(), pos.cpu()
    for t in range(T):
        for s_ in range(top_k):
            e, q = int(r_cpu[t, s_]), int(p_cpu[t, s_])
            if 0 <= e < E and q >= 0:
                want[t] += bufs[e // local][q].float().cpu()
    assert torch.equal(got.cpu().view(torch.int16), want.to(torch.bfloat16).view(torch.int16))


@pytest.mark.parametrize("mode", ["nccl", "p2p", "fused"])
def test_expert_parallel_backward_single_rank(mode):
    """ExpertParallelRaggedDot.backward on one rank against the oracle's VJP of the same routed
    product: dx[t] = sum over the token's experts of dy_row @ W[e]^T, dW[e] = x_e^T dy_e."""
    from gpu_ragged_dot_b200 import ep

    E, k, n, T, top_k = 8, 256, 264, 200, 2
    layer = ep.ExpertParallelRaggedDot(E, k, n, torch.device(DEV), seed=5, dispatch=mode)
    x = workloads.normal_tensor((T, k), 1.0, 77, DEV)
    routing = torch.from_numpy(workloads.topk_routing(T, E, top_k, seed=9)).to(DEV)
    for step in range(2):
        out = layer.forward(x, routing)
        y = out[0]
        dy = workloads.normal_tensor(tuple(y.shape), 1.0, 500 + step, DEV)
        dx, dW = layer.backward(dy)
    torch.cuda.synchronize()
    assert layer.device_status() == 0
    flat = routing.reshape(-1).cpu().long()
    if mode == "nccl":
        order = torch.sort(flat, stable=True).indices
        pos = torch.empty_like(order)
        pos[order] = torch.arange(order.numel())
    else:
        pos = out[2].reshape(-1).cpu().long()
    W = layer.weights.float().cpu()
    dyc, xc = dy.float().cpu(), x.float().cpu()
    want_dx = torch.zeros((T, k))
    want_dW = torch.zeros((E, k, n))
    for i in range(T * top_k):
        e, t = int(flat[i]), i // top_k
        row = (dyc[pos[i]] @ W[e].T).to(torch.bfloat16).float()  # the owner rounds each gradient row
        want_dx[t] += row
        want_dW[e] += torch.outer(xc[t], dyc[pos[i]])
    _assert_close(dx.cpu(), want_dx.to(torch.bfloat16), f"ep backward dx ({mode})")
    _assert_close(dW.cpu(), want_dW.to(torch.bfloat16), f"ep backward dW ({mode})")


# ------------------------------------------------------------------ compute_dtype and float32 precision
def test_compute_dtype_casts_like_the_reference():
    """compute_dtype != input dtype: both operands are cast before the product, the result comes
    back in x's type (gpu_ragged_dot.py:116,145,149), in the forward and in both gradients."""
    m, k, n, g = 300, 136, 72, 4
    x, A, dout = _inputs(91, m, k, n, g)
    gs = torch.tensor([100, 0, 150, 40], dtype=torch.int32)
    xd, Ad, gd, dd = _to_dev(x, A, gs, dout)
    # bf16 inputs multiplied as float32 (TF32 holds every bf16 value exactly): same product
    xd.requires_grad_(True)
    Ad.requires_grad_(True)
    y = rd.gmm(xd, Ad, gd, compute_dtype=torch.float32)
    assert y.dtype == torch.bfloat16
    y.backward(dd)
    dx_ref, dA_ref = oracle.ragged_dot_vjp(x, A, gs, dout)
    _assert_close(y.detach().cpu(), oracle.ragged_dot(x, A, gs), "bf16 in, f32 compute: y")
    _assert_close(xd.grad.cpu(), dx_ref, "bf16 in, f32 compute: dx")
    _assert_close(Ad.grad.cpu(), dA_ref, "bf16 in, f32 compute: dA")
    assert xd.grad.dtype == torch.bfloat16 and Ad.grad.dtype == torch.bfloat16
    # float32 inputs multiplied as bf16: the oracle on the rounded operands, float32 out
    x32 = oracle.reference_normal(5, (m, k), torch.float32)
    A32 = oracle.reference_normal(6, (g, k, n), torch.float32)
    y = rd.gmm(x32.to(DEV), A32.to(DEV), gd, compute_dtype=torch.bfloat16)
    assert y.dtype == torch.float32
    want = oracle.ragged_dot(x32.to(torch.bfloat16), A32.to(torch.bfloat16), gs).float()
    _assert_close(y.cpu(), want, "f32 in, bf16 compute")
    # operands of different types: A is cast to x's type
    y = rd.gmm(xd.detach(), A32.to(DEV), gd)
    _assert_close(y.cpu(), oracle.ragged_dot(x, A32.to(torch.bfloat16), gs), "bf16 x, f32 A")
    out = rd.tgmm(x32.to(DEV), dd, gd, compute_dtype=torch.bfloat16)
    assert out.dtype == torch.float32
    _assert_close(out.cpu(), oracle.trans_ragged_dot(x32.to(torch.bfloat16), dout, gs).float(), "tgmm f32 in, bf16 compute")


def test_float32_highest_precision_three_tf32_passes():
    """precision="highest": float32 results within 2e-5 relative L2 of the exact product (float64
    on the CPU), twenty times tighter than the reference's float32 gate of 5e-4 (tests.py:127),
    where one TF32 pass sits at about 5e-4; forward, trans_rhs, tgmm and the VJP."""
    m, k, n, g = 500, 264, 136, 5
    gs = torch.tensor([120, 0, 200, 77, 90], dtype=torch.int32)
    x = oracle.reference_normal(1, (m, k), torch.float32)
    A = oracle.reference_normal(2, (g, k, n), torch.float32)
    dout = oracle.reference_normal(3, (m, n), torch.float32)
    total = int(gs.sum())

    def oracle64(a, b, trans=False):
        y = torch.zeros((m, b.shape[-2] if trans else b.shape[-1]), dtype=torch.float64)
        off = 0
        for gi, s_ in enumerate(gs.tolist()):
            w = b[gi].double()
            y[off:off + s_] = a[off:off + s_].double() @ (w.T if trans else w)
            off += s_
        return y

    xd, Ad, gd, dd = _to_dev(x, A, gs, dout)
    mask = torch.arange(m) < total
    y_hi = rd.gmm(xd, Ad, gd, precision="highest")
    y_lo = rd.gmm(xd, Ad, gd)
    want = oracle64(x, A)
    e_hi = float(oracle.rel_l2_err(y_hi.cpu().double().float(), want.float(), mask=mask).max())
    e_lo = float(oracle.rel_l2_err(y_lo.cpu(), want.float(), mask=mask).max())
    assert e_hi < 2e-5, e_hi
    assert e_lo > 5 * e_hi  # the single pass really is the coarser one
    assert float(y_hi[total:].abs().max()) == 0.0
    At = A.transpose(1, 2).contiguous()
    y_t = rd.gmm(xd, At.to(DEV), gd, trans_rhs=True, precision="highest")
    assert float(oracle.rel_l2_err(y_t.cpu(), want.float(), mask=mask).max()) < 2e-5
    out = rd.tgmm(xd, dd, gd, precision="highest")
    want_t = torch.zeros((g, k, n), dtype=torch.float64)
    off = 0
    for gi, s_ in enumerate(gs.tolist()):
        want_t[gi] = x[off:off + s_].double().T @ dout[off:off + s_].double()
        off += s_
    assert float(oracle.rel_l2_err(out.cpu(), want_t.float(), axis=(-1, -2), mask=gs != 0).max()) < 2e-5
    assert float(out[1].abs().max()) == 0.0
    xg, Ag = xd.clone().requires_grad_(True), Ad.clone().requires_grad_(True)
    rd.gmm(xg, Ag, gd, precision="highest").backward(dd)
    want_dx = oracle64(dout, A, trans=True)
    assert float(oracle.rel_l2_err(xg.grad.cpu(), want_dx.float(), mask=mask).max()) < 2e-5
    assert float(oracle.rel_l2_err(Ag.grad.cpu(), want_t.float(), axis=(-1, -2), mask=gs != 0).max()) < 2e-5


# ------------------------------------------------------------------ ragged_dot_general: batch dimension, ragged batch
def test_ragged_dot_general_batched_and_ragged_batch():
    """The three modes of jax.lax.ragged_dot_general with one batch dimension, in permuted layouts
    too, against the oracle's loops over the batch."""
    b, m, k, n, g = 3, 200, 72, 136, 4
    rng = np.random.default_rng(33)
    bf = lambda a: torch.from_numpy(a.astype(np.float32)).to(torch.bfloat16)  # noqa: E731
    lhs = bf(rng.standard_normal((b, m, k)))
    w = bf(rng.standard_normal((b, g, k, n)) / np.sqrt(k))
    y = bf(rng.standard_normal((b, m, n)))
    gs = torch.tensor([[50, 0, 100, 30], [200, 0, 0, 0], [1, 64, 65, 70]], dtype=torch.int32)
    DN = rd.RaggedDotDimensionNumbers
    close = lambda got, want, what: _assert_close(got.cpu(), want, what)  # noqa: E731
    # ragged m, rhs [b, g, k, n]
    got = rd.ragged_dot_general(lhs.to(DEV), w.to(DEV), gs.to(DEV), DN((([2], [2]), ([0], [0])), [1], [1]))
    want = oracle.ragged_dot_general_batched("ragged_m", lhs, w, gs)
    assert got.shape == (b, m, n)
    close(got, want, "general: ragged m, batched")
    # the same with rhs stored [g, b, n, k] (group first, contracting last)
    w2 = w.permute(1, 0, 3, 2).contiguous()
    got = rd.ragged_dot_general(lhs.to(DEV), w2.to(DEV), gs.to(DEV), DN((([2], [3]), ([0], [1])), [1], [0]))
    close(got, want, "general: ragged m, batched, rhs [g, b, n, k]")
    # ragged k -> [g, b, k, n]
    got = rd.ragged_dot_general(lhs.to(DEV), y.to(DEV), gs.to(DEV), DN((([1], [1]), ([0], [0])), [1], []))
    want = oracle.ragged_dot_general_batched("ragged_k", lhs, y, gs)
    assert got.shape == (g, b, k, n)
    close(got, want, "general: ragged k, batched")
    # ragged batch: group sizes partition b; elements past their sum are zero
    w3 = bf(rng.standard_normal((b, k, n)) / np.sqrt(k))
    for sizes in ([1, 1], [3], [0, 2, 1], [5]):
        gsb = torch.tensor(sizes, dtype=torch.int32)
        got = rd.ragged_dot_general(lhs.to(DEV), w3.to(DEV), gsb.to(DEV), DN((([2], [1]), ([0], [0])), [0], []))
        want = oracle.ragged_dot_general_batched("ragged_batch", lhs, w3, gsb)
        assert got.shape == (b, m, n)
        close(got, want, f"general: ragged batch {sizes}")
        live = min(sum(sizes), b)
        assert float(got[live:].float().abs().max() if live < b else 0.0) == 0.0


def test_group_by_weight_order_gives_identical_results():
    """RD_CFG_GROUP_BY_WEIGHT only changes the order in which tiles are taken: many small segments
    over few weight matrices (the decode-sized expert-parallel layout), with empty segments, a
    segment over one tile, and both tile kernels; bit-identical output, oracle-checked."""
    experts, world, k, n = 6, 5, 136, 520
    rng = np.random.default_rng(17)
    sizes = rng.integers(0, 9, size=experts * world).astype(np.int32)
    sizes[3] = 0
    sizes[7] = 300
    m = int(sizes.sum()) + 40
    x, A, _ = _inputs(19, m, k, n, experts)
    seg2e = torch.arange(experts, dtype=torch.int32).repeat(world)
    gs = torch.from_numpy(sizes)
    want = oracle.ragged_dot(x, A[seg2e.long()], gs)
    xd, Ad, gd, sd = _to_dev(x, A, gs, seg2e)
    for tile_m in (128, 256):
        outs = []
        for flags in (0, _lib.RD_CFG_GROUP_BY_WEIGHT):
            ws = ops._workspace(m, len(sizes), DEV)
            y = ops.gmm_forward(xd, Ad, gd, group_to_weight=sd, cfg=_lib.TileCfg(256, 0, 1, tile_m, flags), workspace=ws)
            assert ops.device_status(ws) == 0
            outs.append(y)
        assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
        _assert_close(outs[1].cpu(), want, f"group-by-weight order, tile_m {tile_m}")
        assert float(outs[1][int(sizes.sum()):].float().abs().max()) == 0.0
    # with ready flags too (the flag of a later segment is waited for early: it is already up)
    flags_t = torch.full((8,), 2, dtype=torch.int32, device=DEV)
    ws = ops._workspace(m, len(sizes), DEV)
    y = ops.gmm_forward(xd, Ad, gd, group_to_weight=sd, workspace=ws, ready=(flags_t, experts, 2),
                        cfg=_lib.TileCfg(256, 0, 1, 128, _lib.RD_CFG_GROUP_BY_WEIGHT))
    assert ops.device_status(ws) == 0
    _assert_close(y.cpu(), want, "group-by-weight order with ready flags")


# ------------------------------------------------------------------ 8-bit (e4m3) inputs
@pytest.mark.parametrize("m,k,n,tile_n", [(700, 256, 520, 0), (700, 144, 72, 0), (300, 128, 136, 128),
                                           (300, 1040, 264, 64), (1, 16, 8, 0)])
def test_gmm_fp8_matches_oracle(m, k, n, tile_n):
    """rd_gmm_fp8: e4m3 x [m,k] and A [g,n,k], fp32 accumulation, per-weight scale, bf16 out; every
    tile width, k not a multiple of the 128-byte stage, empty groups, tiles of at most 64 rows,
    the zero tail."""
    g = 5
    rng = np.random.default_rng(7)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(torch.float8_e4m3fn)
    A = torch.from_numpy(rng.standard_normal((g, n, k)).astype(np.float32)).to(torch.float8_e4m3fn)
    scale = torch.tensor([0.5, 2.0, 1.0, 0.03125, 3.0], dtype=torch.float32) / k ** 0.5
    sizes = [m // 3, 0, m // 2, 0, max(m - m // 3 - m // 2 - 7, 0)]
    gs = torch.tensor(sizes, dtype=torch.int32)
    cfg = _lib.TileCfg(tile_n, 0, 0, 0, 0) if tile_n else None
    ws = ops._workspace(m, g, DEV)
    y = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gmm_fp8_forward(x.to(DEV), A.to(DEV), gs.to(DEV), weight_scale=scale.to(DEV), cfg=cfg, out=y, workspace=ws)
    assert ops.device_status(ws) == 0
    want = oracle.ragged_dot_fp8(x, A, gs, scale)
    _assert_close(y.cpu(), want, "gmm fp8")
    total = int(gs.sum())
    assert float(y[total:].float().abs().max() if total < m else 0.0) == 0.0
    err = oracle.rel_l2_err(y.cpu(), want, axis=-1, mask=torch.arange(m) < total)
    assert float(err.max()) < EPS_ROWS_BF16
    # no scale, and segments sharing weights through an index
    g2w = torch.tensor([2, 0, 2, 1, 0], dtype=torch.int32)
    y2 = ops.gmm_fp8_forward(x.to(DEV), A[:3].contiguous().to(DEV), gs.to(DEV), group_to_weight=g2w.to(DEV))
    want2 = oracle.ragged_dot_fp8(x, A[:3], gs, None, g2w)
    ok, worst = oracle.allclose_report(y2.cpu(), want2, 2e-2, 2e-2 * max(float(want2.float().abs().max()), 1.0))
    assert ok, f"gmm fp8 indexed, unscaled: worst ratio {worst:.3f}"


def test_gmm_fp8_rejects_what_it_does_not_do():
    x = torch.zeros(8, 32, dtype=torch.float8_e4m3fn, device=DEV)
    A = torch.zeros(1, 8, 32, dtype=torch.float8_e4m3fn, device=DEV)
    gs = torch.tensor([8], dtype=torch.int32, device=DEV)
    with pytest.raises(NotImplementedError):
        ops.gmm_fp8_forward(x.to(torch.bfloat16), A, gs)
    with pytest.raises(NotImplementedError):
        ops.gmm_fp8_forward(x[:, :24].contiguous(), A[:, :, :24].contiguous(), gs)  # k not a multiple of 16
    with pytest.raises(_lib.RaggedDotError):
        ops.gmm_fp8_forward(x, A, gs, cfg=_lib.TileCfg(256, 0, 2, 0, 0))  # no CTA pairs for 8-bit inputs


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ep_count_share_emulated_ranks(world):
    """rd_ep_count_share + rd_ep_plan_ring_when_counted with W ranks emulated on one GPU (every
    rank's count kernel first, then every rank's plan: no kernel waits for a later one): every
    rank's table ends up holding all ranks' counts, the flags carry the epoch, the scratch is left
    zero, and the plan equals the one made from an all-gathered table; two epochs, two tables."""
    E, T, top_k = 64, 300, 4
    tables = [torch.zeros((2, world, E), dtype=torch.int32, device=DEV) for _ in range(world)]
    flags = [torch.zeros(max(world, 4), dtype=torch.int32, device=DEV) for _ in range(world)]
    scratch = [torch.zeros(E + 1, dtype=torch.int32, device=DEV) for _ in range(world)]
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    peer_flags = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=DEV)
    for epoch in (1, 2):
        par = epoch & 1
        peer_counts = torch.tensor([t[par].data_ptr() for t in tables], dtype=torch.int64, device=DEV)
        routings = [torch.from_numpy(workloads.topk_routing(T, E, top_k, seed=100 * epoch + r)).to(DEV).to(torch.int32)
                    for r in range(world)]
        routings[0][5, 1] = E + 7  # an expert id that does not exist is not counted
        for r in range(world):
            ops.ep_count_share(routings[r], E, scratch[r], world, r, peer_counts, peer_flags, epoch)
        want = torch.stack([ops.ep_count(routings[r], E) for r in range(world)])
        for r in range(world):
            assert torch.equal(tables[r][par], want), f"rank {r}: table of epoch {epoch}"
            assert flags[r][:world].tolist() == [epoch] * world
            assert int(scratch[r].abs().sum()) == 0
            got = ops.ep_plan_ring_when_counted(tables[r][par], flags[r], epoch, r, ops.ep_plan_ring(want, r), status)
            ref = ops.ep_plan_ring(want.contiguous(), r)
            for name in ("dest_offset", "segment_sizes", "totals", "send_start"):
                assert torch.equal(got[name], ref[name]), name
        assert ops.device_status(status) == 0
    # a count that never arrives: the plan kernel gives up after its limit and says so
    late = torch.zeros(max(world, 4), dtype=torch.int32, device=DEV)
    ops.ep_plan_ring_when_counted(tables[0][0], late, 1, 0, ops.ep_plan_ring(want, 0), status, wait_limit_ms=5)
    assert ops.device_status(status) == _lib.RD_ERR_DEVICE_WAIT
