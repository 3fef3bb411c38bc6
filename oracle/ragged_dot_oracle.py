"""CPU oracle for the ragged-dot hot path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and the cpu_baseline / --impl reference legs of bench.py
may import this module; the product (gpu_ragged_dot_b200) never does and has no CPU path.

It restates, in NumPy / torch-CPU, what the reference computes:
  * make_group_metadata  -- _make_gmm_group_metadata, gpu_ragged_dot.py:70-90
  * ragged_dot           -- _gpu_gmm_kernel, gpu_ragged_dot.py:112-165 (row ranges, cast ->
                            dot in acc dtype -> cast, zero rows past sum(group_sizes)), i.e. the
                            semantics of jax.lax.ragged_dot the reference is tested against
                            (tests.py:31-33,39-42)
  * trans_ragged_dot     -- _gpu_tgmm_kernel, gpu_ragged_dot.py:250-281 (zero block for an
                            empty group), dimension numbers of tests.py:34-36
  * ragged_dot_vjp       -- _gpu_gmm_bwd, gpu_ragged_dot.py:399-402
  * ragged_dot_general_batched -- the op of tests.py:39-48 with a batch dimension / ragged batch
                            (jax.lax.ragged_dot_general's published semantics; the reference
                            itself has no batched form)
  * rel_l2_err           -- err_fn, tests.py:74-79
  * reference_group_sizes / reference_normal -- the generators of tests.py:51-62

The arithmetic the reference compares itself with lives in a dependency that is not under the
reference tree: jax (jax.lax.ragged_dot_general), not pinned by the reference (pyproject.toml
has no dependency table; README.md:5 links jax commit 713ea3caa17b506a6b485224c88f35e74ff6a297).
jax is not installed here, so this oracle is pinned instead against golden vectors produced by
executing the reference's own metadata builder and kernel bodies under a NumPy stand-in for
jax/pallas (tests/golden/make_golden.py; fixtures in tests/golden/*.npz).
"""

from __future__ import annotations

from typing import NamedTuple, Optional, Tuple

import numpy as np
import torch


class GroupMetadata(NamedTuple):
    group_sizes: np.ndarray
    group_offsets: np.ndarray
    row_it2group: np.ndarray
    row_it2it_in_group: np.ndarray
    total_row_its: np.ndarray


def make_group_metadata(group_sizes, m: int, chunk_m: int) -> GroupMetadata:
    """Loop restatement of gpu_ragged_dot.py:73-89 (int32, zero-filled past the live chunks)."""
    gs = np.asarray(group_sizes, dtype=np.int32)
    g = gs.size
    blocks = (gs + chunk_m - 1) // chunk_m
    upper = (m + chunk_m - 1) // chunk_m + g
    it2group = np.zeros(upper, dtype=np.int32)
    it2it = np.zeros(upper, dtype=np.int32)
    pos = 0
    for gi in range(g):
        for j in range(int(blocks[gi])):
            if pos < upper:
                it2group[pos] = gi
                it2it[pos] = j
            pos += 1
    offsets = (np.cumsum(gs) - gs).astype(np.int32)
    total = np.asarray(blocks.sum(), dtype=np.int32)
    return GroupMetadata(gs, offsets, it2group, it2it, total)


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to("cpu").to(torch.float32)


def to_tf32(t: torch.Tensor, mode: str = "truncate") -> torch.Tensor:
    """float32 values reduced to TF32 (10 explicit mantissa bits), the operand precision of the
    tensor cores for float32 inputs.  "truncate" drops the low 13 bits; "nearest" rounds to
    nearest, ties away from zero (cvt.rna.tf32.f32)."""
    bits = _f32(t).contiguous().view(torch.int32)
    if mode == "nearest":
        bits = bits + 0x1000
    return (bits & ~0x1FFF).view(torch.float32)


def _group_ranges(group_sizes, m: int):
    gs = np.asarray(torch.as_tensor(group_sizes).cpu().numpy(), dtype=np.int64)
    start = 0
    for gi, s in enumerate(gs):
        s = int(max(s, 0))
        lo, hi = min(start, m), min(start + s, m)
        yield gi, lo, hi
        start += s


def ragged_dot(x: torch.Tensor, A: torch.Tensor, group_sizes, trans_rhs: bool = False,
               out_dtype: Optional[torch.dtype] = None, native_16bit: bool = False) -> torch.Tensor:
    """y[rows of g] = cast(f32(x[rows]) @ f32(A[g])); rows past the last group are zero.

    native_16bit=True hands the 16-bit operands straight to torch's CPU matmul (oneDNN: AMX /
    AVX512-BF16 with fp32 accumulation) instead of widening them first -- same semantics, used
    where the oracle is timed as the CPU baseline because it is several times faster."""
    m, k = x.shape
    n = A.shape[-1] if not trans_rhs else A.shape[-2]
    out_dtype = out_dtype or x.dtype
    if native_16bit:
        xc = x.detach().cpu()
        y16 = torch.zeros((m, n), dtype=x.dtype)
        for gi, lo, hi in _group_ranges(group_sizes, m):
            if hi > lo:
                w = A[gi].detach().cpu()
                y16[lo:hi] = xc[lo:hi] @ (w.T if trans_rhs else w)
        return y16.to(out_dtype)
    xf = _f32(x)
    y = torch.zeros((m, n), dtype=torch.float32)
    for gi, lo, hi in _group_ranges(group_sizes, m):
        if hi > lo:
            w = _f32(A[gi])
            y[lo:hi] = xf[lo:hi] @ (w.T if trans_rhs else w)
    return y.to(out_dtype)


def trans_ragged_dot(x: torch.Tensor, dout: torch.Tensor, group_sizes,
                     out_dtype: Optional[torch.dtype] = None, native_16bit: bool = False) -> torch.Tensor:
    """out[g] = cast(f32(x[rows of g])^T @ f32(dout[rows of g])); empty group -> zeros."""
    m, k = x.shape
    n = dout.shape[-1]
    g = int(torch.as_tensor(group_sizes).numel())
    out_dtype = out_dtype or x.dtype
    if native_16bit:
        xc, dc = x.detach().cpu(), dout.detach().cpu()
        out16 = torch.zeros((g, k, n), dtype=x.dtype)
        for gi, lo, hi in _group_ranges(group_sizes, m):
            if hi > lo:
                out16[gi] = xc[lo:hi].T @ dc[lo:hi]
        return out16.to(out_dtype)
    xf, df = _f32(x), _f32(dout)
    out = torch.zeros((g, k, n), dtype=torch.float32)
    for gi, lo, hi in _group_ranges(group_sizes, m):
        if hi > lo:
            out[gi] = xf[lo:hi].T @ df[lo:hi]
    return out.to(out_dtype)


def ragged_dot_vjp(x, A, group_sizes, dout, trans_rhs: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """(dlhs, drhs) exactly as the reference wires them (gpu_ragged_dot.py:399-402)."""
    dx = ragged_dot(dout, A, group_sizes, trans_rhs=not trans_rhs)
    dA = (trans_ragged_dot(x, dout, group_sizes) if not trans_rhs
          else trans_ragged_dot(dout, x, group_sizes))
    return dx, dA


def ragged_dot_permuted(x, A, group_sizes, in_rows=None, out_rows=None, y_rows=None,
                        trans_rhs: bool = False, out=None) -> torch.Tensor:
    """What a mixture-of-experts caller wraps around the reference's ragged_dot
    (gpu_ragged_dot.py:362-376): gather the token rows into group order, multiply, and put the
    result rows back: y[out_rows[r]] = (x[in_rows] . A)[r] for r < sum(group_sizes); other rows of
    y keep `out` (zeros by default).  Without out_rows it is ragged_dot on the gathered rows."""
    gs = torch.as_tensor(group_sizes).to(torch.int64)
    total = int(gs.sum())
    xs = x if in_rows is None else x[torch.as_tensor(in_rows).long()]
    ys = ragged_dot(xs, A, gs, trans_rhs=trans_rhs)
    if out_rows is None:
        return ys
    y_rows = ys.shape[0] if y_rows is None else y_rows
    y = torch.zeros((y_rows, ys.shape[1]), dtype=ys.dtype) if out is None else out.clone()
    y[torch.as_tensor(out_rows).long()[:total]] = ys[:total]
    return y


def ragged_dot_fp8(x: torch.Tensor, A: torch.Tensor, group_sizes, weight_scale=None,
                   group_to_weight=None) -> torch.Tensor:
    """The 8-bit extension (no counterpart in the reference): e4m3 operands, A stored [w, n, k];
    y[rows of group i] = bf16(scale[w] * (f32(x[rows]) @ f32(A[w])^T)), w = group_to_weight[i] or i.
    Products of e4m3 values are exact in fp32, so this is the same arithmetic as the kernel's."""
    m, k = x.shape
    n = A.shape[1]
    xf = _f32(x)
    y = torch.zeros((m, n), dtype=torch.float32)
    for gi, lo, hi in _group_ranges(group_sizes, m):
        if hi > lo:
            w = int(group_to_weight[gi]) if group_to_weight is not None else gi
            sc = float(weight_scale[w]) if weight_scale is not None else 1.0
            y[lo:hi] = (xf[lo:hi] @ _f32(A[w]).T) * sc
    return y.to(torch.bfloat16)


def ragged_dot_general_batched(mode: str, lhs: torch.Tensor, rhs: torch.Tensor, group_sizes) -> torch.Tensor:
    """jax.lax.ragged_dot_general with one batch dimension in canonical layouts (the dimension
    numbers of tests.py:31-36 with a leading batch dimension added):
      "ragged_m":     lhs [b,m,k], rhs [b,g,k,n], group_sizes [b,g] -> [b,m,n]
      "ragged_k":     lhs [b,m,k], rhs [b,m,n],   group_sizes [b,g] -> [g,b,k,n]
      "ragged_batch": lhs [b,m,k], rhs [b,k,n],   group_sizes [g]   -> [b,m,n], zero past sum(group_sizes)
    """
    b = lhs.shape[0]
    if mode == "ragged_m":
        return torch.stack([ragged_dot(lhs[i], rhs[i], group_sizes[i]) for i in range(b)])
    if mode == "ragged_k":
        return torch.stack([trans_ragged_dot(lhs[i], rhs[i], group_sizes[i]) for i in range(b)], dim=1)
    if mode == "ragged_batch":
        live = min(int(torch.as_tensor(group_sizes).sum()), b)
        out = torch.zeros((b, lhs.shape[1], rhs.shape[2]), dtype=torch.float32)
        for i in range(live):
            out[i] = _f32(lhs[i]) @ _f32(rhs[i])
        return out.to(lhs.dtype)
    raise ValueError(mode)


def rel_l2_err(a: torch.Tensor, b: torch.Tensor, axis=-1, mask=None) -> torch.Tensor:
    """err_fn of tests.py:74-79: ||a-b|| / max(||b||, 1e-7) along `axis`, zero where masked out."""
    a, b = _f32(a), _f32(b)
    dims = axis if isinstance(axis, (tuple, list)) else (axis,)
    err = torch.linalg.vector_norm(a - b, dim=dims) / torch.clamp(
        torch.linalg.vector_norm(b, dim=dims), min=1e-7)
    if mask is not None:
        mask = torch.as_tensor(mask).cpu()
        while mask.dim() < err.dim():
            mask = mask.unsqueeze(-1)
        err = torch.where(mask, err, torch.zeros_like(err))
    return err


def allclose_report(a: torch.Tensor, b: torch.Tensor, rtol: float, atol: float):
    """(ok, max violation ratio) for |a-b| <= atol + rtol*|b| elementwise."""
    a, b = _f32(a), _f32(b)
    viol = (a - b).abs() / (atol + rtol * b.abs())
    worst = float(viol.max()) if viol.numel() else 0.0
    return worst <= 1.0, worst


# ---------------------------------------------------------------- the reference's test generators
def reference_group_sizes(seed: int, g: int, target_m: int) -> np.ndarray:
    """generate_group_sizes of tests.py:51-57 with an integer seed in place of the jax key."""
    z = np.random.default_rng(seed).normal(size=(g,))
    p = np.exp(z - z.max())
    p = p / p.sum()
    gs = np.round(target_m * p).astype(np.int32)
    while gs.sum() != target_m:
        idx = int(np.argmax(gs))
        gs[idx] = max(gs[idx] + (target_m - gs.sum()), 0)
    return gs


def reference_normal(seed: int, shape, dtype: torch.dtype) -> torch.Tensor:
    """_normal of tests.py:60-62: float64 normals cast to the test dtype."""
    return torch.from_numpy(np.random.default_rng(seed).normal(size=shape)).to(dtype)
