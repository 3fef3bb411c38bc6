"""Pins the CPU oracle against fixtures produced by running the reference's own code
(tests/golden/make_golden.py).  Runs without a GPU."""

import numpy as np
import pytest
import torch

from oracle import ragged_dot_oracle as oracle
from tests import golden_io

GEMM = golden_io.gemm_cases()
META = golden_io.metadata_cases()

# The reference accumulates one block_k slab at a time in fp32 and rounds once to bf16; the
# oracle does one fp32 matmul per group.  The two can differ by an ulp of bf16 (2^-8 relative).
RTOL = ATOL = 1e-2


def _close(got, want, what):
    got, want = got.float(), want.float()
    written = torch.isfinite(want)
    viol = ((got - want).abs() / (ATOL + RTOL * want.abs()))[written]
    assert viol.numel() > 0
    assert float(viol.max()) <= 1.0, f"{what}: worst ratio {float(viol.max()):.3f}"
    return written


def test_fixtures_present():
    assert len(GEMM) >= 6 and len(META) >= 8
    names = {c["name"] for c in GEMM}
    assert {"empty_groups", "baseline_small"} <= names
    # the reference's own output pins the empty-group branches: at least two fixtures hold zeros
    assert sum(bool((c["group_sizes"] == 0).any()) for c in GEMM) >= 2


@pytest.mark.parametrize("case", META, ids=lambda c: f"gs{len(c['group_sizes'])}_m{c['m_chunk'][0]}_c{c['m_chunk'][1]}")
def test_metadata_bit_exact(case):
    m, chunk = (int(v) for v in case["m_chunk"])
    got = oracle.make_group_metadata(case["group_sizes"], m, chunk)
    assert np.array_equal(got.group_offsets, case["group_offsets"])
    assert np.array_equal(got.row_it2group, case["row_it2group"])
    assert np.array_equal(got.row_it2it_in_group, case["row_it2it_in_group"])
    assert int(got.total_row_its) == int(case["total_row_its"])


def test_metadata_worked_example():
    got = oracle.make_group_metadata([5, 0, 12, 3, 0, 0, 9, 1], 32, 8)
    assert got.group_offsets.tolist() == [0, 5, 5, 17, 20, 20, 20, 29]
    assert got.row_it2group.tolist() == [0, 2, 2, 3, 6, 6, 7, 0, 0, 0, 0, 0]
    assert got.row_it2it_in_group.tolist() == [0, 0, 1, 0, 0, 1, 0, 0, 0, 0, 0, 0]
    assert int(got.total_row_its) == 7


@pytest.mark.parametrize("case", GEMM, ids=lambda c: c["name"])
def test_forward_matches_reference(case):
    gs = case["group_sizes"]
    got = oracle.ragged_dot(case["x"], case["A"], gs)
    written = _close(got, case["y"], "y")
    # the reference writes every row here: the owned ones and the zero tail
    assert bool(written.all())
    tail = int(gs.sum())
    assert float(case["y"][tail:].float().abs().max() if tail < case["m"] else 0.0) == 0.0
    if "y_trans_rhs" in case:
        got_t = oracle.ragged_dot(case["x"], case["A"].transpose(1, 2).contiguous(), gs, trans_rhs=True)
        _close(got_t, case["y_trans_rhs"], "y (trans_rhs)")
    err = oracle.rel_l2_err(got, case["y"], axis=-1, mask=torch.arange(case["m"]) < case["target_m"])
    assert float(err.max()) < 5e-3


@pytest.mark.parametrize("case", GEMM, ids=lambda c: c["name"])
def test_trans_ragged_dot_matches_reference(case):
    gs = case["group_sizes"]
    want = case["tgmm"] if "tgmm" in case else case["drhs"]  # the same product (gpu_ragged_dot.py:401)
    got = oracle.trans_ragged_dot(case["x"], case["dout"], gs)
    _close(got, want, "tgmm")
    err = oracle.rel_l2_err(got, want, axis=(-1, -2), mask=gs != 0)
    assert float(err.max()) < 2e-3
    for gi in (gs == 0).nonzero().flatten().tolist():
        # an empty group's block is written by the reference itself, as zeros
        assert bool(torch.isfinite(want[gi].float()).all())
        assert float(want[gi].float().abs().max()) == 0.0


@pytest.mark.parametrize("case", GEMM, ids=lambda c: c["name"])
def test_vjp_wiring_matches_reference(case):
    gs = case["group_sizes"]
    dx, dA = oracle.ragged_dot_vjp(case["x"], case["A"], gs, case["dout"], trans_rhs=False)
    _close(dx, case["dlhs"], "dlhs")
    _close(dA, case["drhs"], "drhs")
    if "dlhs_trans_rhs" not in case:
        return
    At = case["A"].transpose(1, 2).contiguous()
    dx_t, dA_t = oracle.ragged_dot_vjp(case["x"], At, gs, case["dout"], trans_rhs=True)
    _close(dx_t, case["dlhs_trans_rhs"], "dlhs (trans_rhs)")
    _close(dA_t, case["drhs_trans_rhs"], "drhs (trans_rhs)")
    assert dA_t.shape == (case["g"], case["n"], case["k"])


def test_native_16bit_mode_agrees():
    case = GEMM[0]
    gs = case["group_sizes"]
    a = oracle.ragged_dot(case["x"], case["A"], gs)
    b = oracle.ragged_dot(case["x"], case["A"], gs, native_16bit=True)
    ok, worst = oracle.allclose_report(b, a, 1e-2, 1e-2)
    assert ok, worst
    a = oracle.trans_ragged_dot(case["x"], case["dout"], gs)
    b = oracle.trans_ragged_dot(case["x"], case["dout"], gs, native_16bit=True)
    ok, worst = oracle.allclose_report(b, a, 1e-2, 1e-2)
    assert ok, worst
