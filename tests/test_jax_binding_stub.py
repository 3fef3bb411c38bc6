"""The jax binding (gpu_ragged_dot_b200/jax_ffi.py) under a recording stand-in for jax.

jax is not installed where this library is developed, so the XLA custom calls themselves cannot
run here.  What can be checked without jax is everything the binding does around them: the
padding of k and n to 16-byte rows, the compute_dtype casts, the shapes it asks XLA for, and the
operand order of the two custom VJPs, which must be the reference's (gpu_ragged_dot.py:399-402
for gmm; the mathematically correct one for tgmm, whose reference version cannot run).  The
stand-in implements the few jax entry points the binding uses over NumPy and records every
``jax.ffi.ffi_call``.
"""

import importlib
import sys
import types

import ml_dtypes
import numpy as np
import pytest


class _CustomVJP:
    def __init__(self, fn, nondiff_argnames=()):
        self.fn, self.nondiff_argnames = fn, tuple(nondiff_argnames)
        self.fwd = self.bwd = None

    def defvjp(self, fwd, bwd):
        self.fwd, self.bwd = fwd, bwd

    def __call__(self, *a, **kw):
        return self.fn(*a, **kw)


class _Struct:
    def __init__(self, shape, dtype):
        self.shape, self.dtype = tuple(shape), np.dtype(dtype)


@pytest.fixture()
def binding(monkeypatch):
    calls = []
    jit_static = []
    jax = types.ModuleType("jax")
    jnp = types.ModuleType("jax.numpy")
    ffi = types.ModuleType("jax.ffi")
    jnp.dtype = np.dtype
    jnp.float32, jnp.int32, jnp.uint8 = np.float32, np.int32, np.uint8
    jnp.bfloat16, jnp.float16 = ml_dtypes.bfloat16, np.float16
    jnp.pad = np.pad
    jax.numpy = jnp
    jax.ShapeDtypeStruct = _Struct
    jax.custom_vjp = lambda fn=None, nondiff_argnames=(): _CustomVJP(fn, nondiff_argnames)

    def jit(fn=None, static_argnums=None):
        jit_static.append(list(static_argnums))
        return fn

    jax.jit = jit

    def ffi_call(name, results):
        def run(*args, **attrs):
            calls.append({"name": name, "args": args, "attrs": attrs,
                          "results": [(r.shape, r.dtype) for r in results]})
            return tuple(np.zeros(r.shape, dtype=r.dtype) for r in results)

        return run

    ffi.ffi_call = ffi_call
    jax.ffi = ffi
    for name, mod in (("jax", jax), ("jax.numpy", jnp), ("jax.ffi", ffi)):
        monkeypatch.setitem(sys.modules, name, mod)
    monkeypatch.delitem(sys.modules, "gpu_ragged_dot_b200.jax_ffi", raising=False)
    mod = importlib.import_module("gpu_ragged_dot_b200.jax_ffi")
    monkeypatch.setattr(mod, "_ensure_registered", lambda: None)  # no XLA shim library here
    yield mod, calls, jit_static
    sys.modules.pop("gpu_ragged_dot_b200.jax_ffi", None)


def _arrays(m, k, n, g, dtype=ml_dtypes.bfloat16, trans=False):
    x = np.ones((m, k), dtype=dtype)
    A = np.ones((g, n, k) if trans else (g, k, n), dtype=dtype)
    gs = np.full((g,), m // g, dtype=np.int32)
    return x, A, gs


def test_static_arguments_follow_the_reference(binding):
    mod, _, jit_static = binding
    # gmm: arguments 3..12 static, tgmm: 3..11 (gpu_ragged_dot.py:361,410)
    assert jit_static == [list(range(3, 13)), list(range(3, 12))]
    assert mod.gmm.nondiff_argnames == mod.NONDIFF_ARGNAMES + ("trans_rhs",)
    assert mod.tgmm.nondiff_argnames == mod.NONDIFF_ARGNAMES
    assert mod.ragged_dot is mod.gmm and mod.trans_ragged_dot is mod.tgmm


def test_reference_grid_shapes_are_padded_not_rejected(binding):
    mod, calls, _ = binding
    m, k, n, g = 171, 58, 77, 8  # the reference's own grid values (tests.py:95-96)
    x, A, gs = _arrays(m, k, n, g)
    y = mod.gmm(x, A, gs)
    assert y.shape == (m, n) and y.dtype == x.dtype
    c = calls[-1]
    assert c["name"] == "rd_gmm" and c["attrs"]["trans_rhs"] is False
    assert c["args"][0].shape == (m, 64) and c["args"][1].shape == (g, 64, 80)
    assert c["results"][0] == ((m, 80), np.dtype(ml_dtypes.bfloat16))
    assert c["results"][1][1] == np.dtype(np.uint8) and c["results"][1][0][0] >= 256
    # padding is with zeros: the padded operands still sum to the unpadded ones
    assert float(c["args"][0].astype(np.float32).sum()) == m * k
    xt, At, _ = _arrays(m, k, n, g, trans=True)
    y = mod.gmm(xt, At, gs, trans_rhs=True)
    assert y.shape == (m, n)
    assert calls[-1]["args"][1].shape == (g, 80, 64) and calls[-1]["attrs"]["trans_rhs"] is True
    out = mod.tgmm(x, np.ones((m, n), dtype=x.dtype), gs)
    assert out.shape == (g, k, n)
    assert calls[-1]["name"] == "rd_tgmm" and calls[-1]["results"][0][0] == (g, 64, 80)


def test_float32_rows_pad_to_four_elements(binding):
    mod, calls, _ = binding
    x, A, gs = _arrays(64, 58, 77, 4, dtype=np.float32)
    y = mod.gmm(x, A, gs)
    assert y.dtype == np.float32 and y.shape == (64, 77)
    assert calls[-1]["args"][0].shape == (64, 60) and calls[-1]["args"][1].shape == (4, 60, 80)


def test_compute_dtype_casts_operands_and_restores_the_input_type(binding):
    mod, calls, _ = binding
    x, A, gs = _arrays(64, 64, 64, 4)  # bfloat16 inputs
    y = mod.gmm(x, A, gs, compute_dtype=np.float32)
    assert calls[-1]["args"][0].dtype == np.float32 and calls[-1]["args"][1].dtype == np.float32
    assert calls[-1]["results"][0][1] == np.dtype(np.float32)
    assert y.dtype == x.dtype  # cast back, gpu_ragged_dot.py:149
    x32 = x.astype(np.float32)
    y = mod.gmm(x32, A, gs, compute_dtype=ml_dtypes.bfloat16)  # A may come in another type: it is cast too
    assert calls[-1]["args"][0].dtype == np.dtype(ml_dtypes.bfloat16) and y.dtype == np.float32
    with pytest.raises(NotImplementedError):
        mod.gmm(x, A, gs, interpret=True)
    with pytest.raises(NotImplementedError):
        mod.gmm(x, A, gs, acc_dtype=np.float16)


@pytest.mark.parametrize("trans_rhs", [False, True])
def test_gmm_vjp_operand_order(binding, trans_rhs):
    mod, calls, _ = binding
    m, k, n, g = 64, 32, 48, 4
    x, A, gs = _arrays(m, k, n, g, trans=trans_rhs)
    x = x * 2  # tell the operands apart by value
    do = np.full((m, n), 3, dtype=x.dtype)
    static = (64, 64, 64, trans_rhs, False, None, np.float32, None, None, 512)
    _, res = mod.gmm.fwd(x, A, gs, *static)
    del calls[:]
    dx, dA, dgs = mod.gmm.bwd(*static, res, do)
    assert dgs is None and dx.shape == x.shape and dA.shape == A.shape
    first, second = calls
    # dx = gmm(do, A, trans_rhs = not trans_rhs)
    assert first["name"] == "rd_gmm" and first["attrs"]["trans_rhs"] is (not trans_rhs)
    assert float(first["args"][0].astype(np.float32)[0, 0]) == 3.0 and first["args"][1].shape == A.shape
    # dA = tgmm(x, do) -> [g, k, n]   or, with trans_rhs, tgmm(do, x) -> [g, n, k]
    assert second["name"] == "rd_tgmm"
    lhs, rhs = (2.0, 3.0) if not trans_rhs else (3.0, 2.0)
    assert float(second["args"][0].astype(np.float32)[0, 0]) == lhs
    assert float(second["args"][1].astype(np.float32)[0, 0]) == rhs


def test_tgmm_vjp_operand_order(binding):
    mod, calls, _ = binding
    m, k, n, g = 64, 32, 48, 4
    x = np.full((m, k), 2, dtype=ml_dtypes.bfloat16)
    y = np.full((m, n), 5, dtype=ml_dtypes.bfloat16)
    gs = np.full((g,), m // g, dtype=np.int32)
    do = np.full((g, k, n), 3, dtype=x.dtype)
    static = (64, 64, 64, False, None, np.float32, None, None, 512)
    _, res = mod.tgmm.fwd(x, y, gs, *static)
    del calls[:]
    dx, dy, dgs = mod.tgmm.bwd(*static, res, do)
    assert dgs is None and dx.shape == x.shape and dy.shape == y.shape
    first, second = calls
    # dx_g = y_g do[g]^T: gmm(y, do, trans_rhs=True);  dy_g = x_g do[g]: gmm(x, do)
    assert first["name"] == "rd_gmm" and first["attrs"]["trans_rhs"] is True
    assert float(first["args"][0].astype(np.float32)[0, 0]) == 5.0
    assert second["name"] == "rd_gmm" and second["attrs"]["trans_rhs"] is False
    assert float(second["args"][0].astype(np.float32)[0, 0]) == 2.0
