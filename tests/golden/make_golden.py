"""Generates the golden fixtures in this directory by EXECUTING THE REFERENCE'S OWN CODE.

The reference (gpu_ragged_dot.py) imports jax + jax.experimental.pallas, which are not
installed and which would need a GPU for the Triton lowering.  This script installs a small
NumPy stand-in for the handful of jax / pallas entry points the reference calls (jnp array ops,
lax.fori_loop / dot_general, pl.pallas_call with BlockSpecs executed as a plain Python grid loop,
masked plgpu.load / store), imports the reference module from its own location and runs, on CPU:

  * _make_gmm_group_metadata           (gpu_ragged_dot.py:70-90)
  * _gpu_gmm_fwd  -> _gpu_gmm_kernel   (gpu_ragged_dot.py:93-228), plain and trans_rhs
  * _gpu_tgmm_fwd -> _gpu_tgmm_kernel  (gpu_ragged_dot.py:231-342)
  * _gpu_gmm_bwd                       (gpu_ragged_dot.py:383-402), the custom-VJP wiring

Inputs and the reference's outputs are stored in golden_*.npz (bf16 stored as uint16 bit
patterns).  Output buffers start as NaN, so elements the reference never writes stay NaN in the
fixture.  tests/test_oracle_golden.py checks the CPU oracle against these files; the GPU parity
tests check the CUDA path against the same files.

    python tests/golden/make_golden.py <path-to-reference-checkout>

Nothing from the reference is copied: it is imported and executed where it lies.
"""

from __future__ import annotations

import contextlib
import importlib.util
import os
import sys
import types
from typing import NamedTuple

import ml_dtypes
import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
BF16 = ml_dtypes.bfloat16


# ----------------------------------------------------------------------------------- stand-ins
class DS:
    """pl.ds(start, size)."""

    def __init__(self, start, size):
        self.start, self.size = int(start), int(size)


class Ref:
    """A block-shaped window into a full array.  offsets[d] is the window's origin along the
    base array's axis d; squeezed axes (block dimension None) are fixed at their offset."""

    def __init__(self, base, offsets, shape, squeezed):
        self.base, self.offsets, self.squeezed = base, list(offsets), list(squeezed)
        self.shape = tuple(shape)
        self.dtype = base.dtype
        self.ndim = len(self.shape)

    def _full_index(self, idx):
        if not isinstance(idx, tuple):
            idx = (idx,)
        idx = [i for i in idx if i is not Ellipsis]
        out, it = [], iter(idx)
        live = [d for d in range(self.base.ndim) if d not in self.squeezed]
        given = {}
        for d, i in zip(live, it):
            given[d] = i
        for d in range(self.base.ndim):
            if d in self.squeezed:
                out.append(self.offsets[d])
            elif d in given:
                i = given[d]
                if isinstance(i, DS):
                    out.append(DS(self.offsets[d] + i.start, i.size))
                else:
                    out.append(self.offsets[d] + int(i))
            else:
                out.append(DS(self.offsets[d], self.shape[live.index(d)]))
        return out

    def __getitem__(self, idx):
        return load(View(self, idx))

    def __array__(self, dtype=None, copy=None):
        a = load(View(self, ()))
        return a.astype(dtype) if dtype is not None else a

    @property
    def at(self):
        ref = self

        class _At:
            def __getitem__(self, idx):
                return View(ref, idx)

        return _At()


class View:
    def __init__(self, ref, idx):
        self.ref, self.idx = ref, idx


def _as_view(v):
    return v if isinstance(v, View) else View(v, ())


def _mesh(full, base_shape):
    """Index arrays (clipped into range) + an in-bounds mask for a list of int / DS indices."""
    axes, inb, shape = [], [], []
    for d, i in enumerate(full):
        if isinstance(i, DS):
            r = i.start + np.arange(i.size)
            axes.append(np.clip(r, 0, base_shape[d] - 1))
            inb.append((r >= 0) & (r < base_shape[d]))
            shape.append(i.size)
        else:
            axes.append(np.array([min(max(i, 0), base_shape[d] - 1)]))
            inb.append(np.array([0 <= i < base_shape[d]]))
    grids = np.ix_(*axes)
    ok = np.ones([len(a) for a in axes], dtype=bool)
    for d, m in enumerate(inb):
        sh = [1] * len(axes)
        sh[d] = len(m)
        ok = ok & m.reshape(sh)
    keep = [d for d, i in enumerate(full) if isinstance(i, DS)]
    return grids, ok, keep, tuple(shape)


def load(view, mask=None, other=None):
    view = _as_view(view)
    base = view.ref.base
    full = view.ref._full_index(view.idx)
    if base.ndim == 0:
        return base[()]
    grids, ok, keep, shape = _mesh(full, base.shape)
    vals = base[grids].reshape(shape) if keep else base[grids].reshape(())
    ok = ok.reshape(shape) if keep else ok.reshape(())
    if mask is not None:
        ok = ok & np.asarray(mask)
    if other is not None or mask is not None:
        vals = np.where(ok, vals, np.zeros((), base.dtype) if other is None else np.asarray(other, base.dtype))
    return vals


def store(view, value, mask=None):
    view = _as_view(view)
    base = view.ref.base
    full = view.ref._full_index(view.idx)
    grids, ok, keep, shape = _mesh(full, base.shape)
    ok = ok.reshape(shape)
    if mask is not None:
        ok = ok & np.asarray(mask)
    value = np.broadcast_to(np.asarray(value).astype(base.dtype), shape)
    idx = np.broadcast_arrays(*grids)
    flat_ok = ok.reshape(-1)
    sel = tuple(a.reshape(-1)[flat_ok] for a in idx)
    base[sel] = value.reshape(-1)[flat_ok]


class BlockSpec:
    def __init__(self, block_shape, index_map):
        self.block_shape, self.index_map = tuple(block_shape), index_map

    def ref(self, base, grid_idx):
        if base.ndim == 0:
            return Ref(base, [], (), [])
        blk = self.index_map(*grid_idx)
        offsets, shape, squeezed = [], [], []
        for d, (b, i) in enumerate(zip(self.block_shape, blk)):
            if b is None:
                offsets.append(int(i))
                squeezed.append(d)
            else:
                offsets.append(int(i) * b)
                shape.append(b)
        return Ref(base, offsets, shape, squeezed)


_program_id = []


def pallas_call(kernel, out_shape, grid, in_specs, out_specs, interpret=False, compiler_params=None, name=None):
    def run(*args):
        out = np.full(out_shape.shape, np.nan, dtype=out_shape.dtype)
        for gidx in np.ndindex(*[int(g) for g in grid]):
            _program_id[:] = list(gidx)
            refs = []
            for a, s in zip(args, in_specs):
                if isinstance(a, tuple):  # NamedTuple of arrays with a matching tuple of specs
                    refs.append(type(a)(*[si.ref(np.asarray(ai), gidx) for ai, si in zip(a, s)]))
                else:
                    refs.append(s.ref(np.asarray(a), gidx))
            kernel(*refs, out_specs.ref(out, gidx))
        return out

    return run


class ShapeDtypeStruct:
    def __init__(self, shape, dtype):
        self.shape, self.dtype = tuple(shape), np.dtype(dtype)


class CustomVJP:
    def __init__(self, fn, nondiff_argnames=()):
        self.fn = fn

    def defvjp(self, fwd, bwd):
        self.fwd, self.bwd = fwd, bwd

    def __call__(self, *a, **k):
        return self.fn(*a, **k)


def _dot_general(a, b, dimension_numbers, preferred_element_type=None):
    (ca, cb), _ = dimension_numbers
    af = np.asarray(a).astype(np.float32)
    bf = np.asarray(b).astype(np.float32)
    out = np.tensordot(af, bf, axes=(list(ca), list(cb)))
    return out.astype(preferred_element_type or a.dtype)


def _fori_loop(lo, hi, body, init):
    val = init
    for i in range(int(lo), int(hi)):
        val = body(i, val)
    return val


def _tree_map(f, tree):
    if isinstance(tree, tuple) and hasattr(tree, "_fields"):
        return type(tree)(*[f(x) for x in tree])
    return f(tree)


def install_stand_ins():
    jax = types.ModuleType("jax")
    jnp = types.ModuleType("jax.numpy")
    lax = types.ModuleType("jax.lax")
    exp = types.ModuleType("jax.experimental")
    pl = types.ModuleType("jax.experimental.pallas")
    plgpu = types.ModuleType("jax.experimental.pallas.triton")
    tree = types.ModuleType("jax.tree")

    for name in ("cumsum", "arange", "where", "sum", "clip", "zeros", "zeros_like", "array", "float32",
                 "int32", "maximum", "expand_dims"):
        setattr(jnp, name, getattr(np, name))
    jnp.bfloat16 = BF16
    jnp.dtype = np.dtype
    jnp.ndarray = np.ndarray

    jax.numpy = jnp
    jax.Array = np.ndarray
    jax.jit = lambda f=None, **kw: f if f is not None else (lambda g: g)
    jax.custom_vjp = CustomVJP
    jax.ShapeDtypeStruct = ShapeDtypeStruct
    jax.named_scope = lambda name: contextlib.nullcontext()
    tree.map = _tree_map
    jax.tree = tree
    lax.fori_loop = _fori_loop
    lax.dot_general = _dot_general
    jax.lax = lax

    pl.cdiv = lambda a, b: (a + b - 1) // b
    pl.next_power_of_2 = lambda x: 1 if x <= 1 else 1 << (int(x) - 1).bit_length()
    pl.BlockSpec = BlockSpec
    pl.pallas_call = pallas_call
    pl.program_id = lambda axis: np.int32(_program_id[axis])
    pl.ds = DS

    def when(cond):
        def deco(fn):
            if bool(cond):
                fn()
            return fn

        return deco

    pl.when = when
    plgpu.load = load
    plgpu.store = store
    plgpu.CompilerParams = lambda **kw: kw
    exp.pallas = pl
    pl.triton = plgpu
    jax.experimental = exp
    sys.modules.update({
        "jax": jax, "jax.numpy": jnp, "jax.lax": lax, "jax.experimental": exp,
        "jax.experimental.pallas": pl, "jax.experimental.pallas.triton": plgpu, "jax.tree": tree,
    })


def import_reference(ref_dir):
    install_stand_ins()
    spec = importlib.util.spec_from_file_location("reference_gpu_ragged_dot",
                                                  os.path.join(ref_dir, "gpu_ragged_dot.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


# ----------------------------------------------------------------------------------- fixtures
def group_sizes_like_reference_tests(seed, g, target_m):
    """generate_group_sizes of the reference's tests.py:51-57 (softmax of normals, fixed up)."""
    z = np.random.default_rng(seed).normal(size=(g,))
    p = np.exp(z - z.max())
    p /= p.sum()
    gs = np.round(target_m * p).astype(np.int32)
    while gs.sum() != target_m:
        idx = int(np.argmax(gs))
        gs[idx] = max(gs[idx] + (target_m - gs.sum()), 0)
    return gs


def bits(a):
    return np.asarray(a).astype(BF16).view(np.uint16)


METADATA_CASES = [
    ([5, 0, 12, 3, 0, 0, 9, 1], 32, 8),
    ([0, 0, 0, 0], 16, 8),
    ([128], 128, 128),
    ([127, 1, 128, 129, 0, 255], 640, 128),
    ([512, 0, 0, 512], 1024, 512),
    ([100, 37, 0, 300, 75], 600, 64),
    ([3] * 40, 128, 8),
    ([0, 0, 700, 0, 324], 1024, 128),
]

GEMM_CASES = [
    # name, m, k, n, g, fill_in, seed, random_inputs, block (m,k,n), chunk_m, explicit group sizes
    ("odd_shapes", 171, 58, 77, 8, 0.7, 0, True, (16, 32, 64), 8, None),
    ("aligned_g16", 128, 64, 64, 16, 1.0, 1, True, (64, 64, 64), 512, None),
    ("half_filled", 256, 64, 128, 8, 0.5, 0, True, (32, 16, 32), 512, None),
    ("all_ones", 171, 58, 77, 16, 0.7, 1, False, (64, 64, 16), 8, None),
    # groups of size zero at the start, in the middle, doubled and at the end: the reference's
    # zero-tile branch (gpu_ragged_dot.py:277-281) and its skipped programs (:113-114) write these
    ("empty_groups", 256, 64, 128, 8, 0.9, 2, True, (32, 32, 64), 64, [0, 57, 0, 0, 91, 1, 81, 0]),
    # the small benchmark configuration: m 512, k 256, n 384, 8 groups, multinomial(Dirichlet(1))
    # sizes with a forced empty group, A scaled by 1/sqrt(k).  Only the forward and the VJP of the
    # plain layout are stored (the file is the largest fixture as it is).
    ("baseline_small", 512, 256, 384, 8, 1.0, 3, True, (64, 64, 64), 512, "baseline_small"),
]


def baseline_small_group_sizes():
    """multinomial(512, Dirichlet(1)) over 8 groups with a forced empty group (seed 0): the same
    draw as gpu_ragged_dot_b200.workloads.group_sizes_small, restated so that this script needs
    nothing but NumPy and the reference."""
    rng = np.random.default_rng(0)
    gs = rng.multinomial(512, rng.dirichlet(np.ones(8))).astype(np.int32)
    if not (gs == 0).any():
        lo, hi = int(np.argmin(gs)), int(np.argmax(gs))
        gs[hi] += gs[lo]
        gs[lo] = 0
    return gs


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of rdyro/gpu_ragged_dot>")
    ref_dir = sys.argv[1]
    ref = import_reference(ref_dir)

    meta = {}
    for i, (gs, m, chunk) in enumerate(METADATA_CASES):
        md = ref._make_gmm_group_metadata(np.array(gs, dtype=np.int32), m, chunk)
        meta[f"c{i}_group_sizes"] = np.array(gs, dtype=np.int32)
        meta[f"c{i}_m_chunk"] = np.array([m, chunk], dtype=np.int32)
        meta[f"c{i}_group_offsets"] = np.asarray(md.group_offsets, dtype=np.int32)
        meta[f"c{i}_row_it2group"] = np.asarray(md.row_it2group, dtype=np.int32)
        meta[f"c{i}_row_it2it_in_group"] = np.asarray(md.row_it2it_in_group, dtype=np.int32)
        meta[f"c{i}_total_row_its"] = np.asarray(md.total_row_its, dtype=np.int32)
    np.savez_compressed(os.path.join(HERE, "golden_metadata.npz"), **meta)
    print("metadata cases:", len(METADATA_CASES))

    for name, m, k, n, g, fill, seed, rnd, (bm, bk, bn), chunk, explicit in GEMM_CASES:
        rng = np.random.default_rng(1000 + seed)
        small = explicit == "baseline_small"
        if rnd:
            x = rng.normal(size=(m, k)).astype(BF16)
            A = (rng.normal(size=(g, k, n)) * (k ** -0.5 if small else 1.0)).astype(BF16)
            dout = rng.normal(size=(m, n)).astype(BF16)
        else:
            x, A, dout = (np.ones(s, dtype=BF16) for s in ((m, k), (g, k, n), (m, n)))
        target_m = max(min(round(m * fill), m), 0)
        if small:
            gs = baseline_small_group_sizes()
        elif explicit is not None:
            gs = np.array(explicit, dtype=np.int32)
        else:
            gs = group_sizes_like_reference_tests(seed + 17, g, target_m)
        target_m = int(gs.sum())
        kw = dict(block_m=bm, block_k=bk, block_n=bn, chunk_m=chunk)
        y, _ = ref._gpu_gmm_fwd(x, A, gs, **kw)
        if small:
            bwd_args = (bm, bk, bn, False, False, None, np.float32, None, None, chunk)
            dx, dA, _ = ref._gpu_gmm_bwd(*bwd_args, (x, A, gs), dout)
            np.savez_compressed(
                os.path.join(HERE, f"golden_gemm_{name}.npz"),
                x=bits(x), A=bits(A), dout=bits(dout), group_sizes=gs,
                params=np.array([m, k, n, g, bm, bk, bn, chunk, target_m], dtype=np.int32),
                y=bits(y), dlhs=bits(dx), drhs=bits(dA))
            print(f"{name}: gs={gs.tolist()} (forward + VJP only)")
            continue
        At = np.ascontiguousarray(np.swapaxes(A, 1, 2))
        y_t, _ = ref._gpu_gmm_fwd(x, At, gs, trans_rhs=True, **kw)
        tg, _ = ref._gpu_tgmm_fwd(x, dout, gs, **kw)
        bwd_args = (bm, bk, bn, False, False, None, np.float32, None, None, chunk)
        dx, dA, dgs = ref._gpu_gmm_bwd(*bwd_args, (x, A, gs), dout)
        assert dgs is None
        bwd_args_t = (bm, bk, bn, True, False, None, np.float32, None, None, chunk)
        dx_t, dA_t, _ = ref._gpu_gmm_bwd(*bwd_args_t, (x, At, gs), dout)
        np.savez_compressed(
            os.path.join(HERE, f"golden_gemm_{name}.npz"),
            x=bits(x), A=bits(A), dout=bits(dout), group_sizes=gs,
            params=np.array([m, k, n, g, bm, bk, bn, chunk, target_m], dtype=np.int32),
            y=bits(y), y_trans_rhs=bits(y_t), tgmm=bits(tg), dlhs=bits(dx), drhs=bits(dA),
            dlhs_trans_rhs=bits(dx_t), drhs_trans_rhs=bits(dA_t),
        )
        written = int(np.isfinite(y.astype(np.float32)).all(axis=1).sum())
        print(f"{name}: gs={gs.tolist()} rows written by the reference: {written}/{m}")


if __name__ == "__main__":
    main()
