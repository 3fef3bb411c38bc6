"""jax binding of the C ABI: ``ragged_dot`` / ``trans_ragged_dot`` as XLA custom calls with the
reference's signature and custom_vjp (gpu_ragged_dot.py:345-454).

Importing this module needs jax with ``jax.ffi``; the first call also needs the XLA-FFI shim
library (``librd_b200_xla.so``, built from csrc/xla_ffi_shim.cc against jaxlib's headers).
Neither is present in the image this library was developed in, so the custom calls have not run
there; the torch layer in ``ops.py`` drives the same entry points and carries the GPU tests, and
``tests/test_jax_binding_stub.py`` runs this file's wiring (padding, casts, the VJPs' operand
order) under a recording stand-in for jax.

Same behaviour as the torch layer: k and n that are not multiples of 16 bytes are zero-padded
(exact) before the call and the result is cut back; ``compute_dtype`` casts both operands before
the product and the result comes back in ``x.dtype`` (gpu_ragged_dot.py:116,145,149); float32 is
multiplied as TF32 with fp32 accumulation.
"""

from __future__ import annotations

import ctypes
import os
from functools import partial

import jax
import jax.numpy as jnp
import numpy as np

from . import _lib

_HERE = os.path.dirname(os.path.abspath(__file__))
_registered = False


def _ensure_registered() -> None:
    """Load the XLA-FFI shim and register its two handlers, once, at the first call."""
    global _registered
    if _registered:
        return
    xla = ctypes.CDLL(os.path.join(_HERE, "librd_b200_xla.so"))
    jax.ffi.register_ffi_target("rd_gmm", jax.ffi.pycapsule(xla.RdGmmFfi), platform="CUDA")
    jax.ffi.register_ffi_target("rd_tgmm", jax.ffi.pycapsule(xla.RdTgmmFfi), platform="CUDA")
    _registered = True


DEFAULT_BLOCK_M = DEFAULT_BLOCK_N = DEFAULT_BLOCK_K = 64
CHUNK_M = 512
NONDIFF_ARGNAMES = ("block_m", "block_k", "block_n", "interpret", "compute_dtype", "acc_dtype",
                    "num_warps", "num_stages", "chunk_m")


def _workspace_struct(m: int, g: int):
    nbytes = ctypes.c_size_t(0)
    _lib.check(_lib.load().rd_workspace_bytes(m, g, ctypes.byref(nbytes)), "rd_workspace_bytes")
    return jax.ShapeDtypeStruct((nbytes.value,), jnp.uint8)


_SUPPORTED = ("bfloat16", "float16", "float32")


def _check(x, interpret, compute_dtype, acc_dtype):
    if interpret:
        raise NotImplementedError("interpret=True: there is no CPU path")
    if compute_dtype is not None and jnp.dtype(compute_dtype).name not in _SUPPORTED:
        raise NotImplementedError("compute_dtype must be bfloat16, float16 or float32")
    if acc_dtype is not None and jnp.dtype(acc_dtype) != jnp.float32:
        raise NotImplementedError("acc_dtype must be float32")


def _pad_to(a, axis, mult):
    r = (-a.shape[axis]) % mult
    if r == 0:
        return a
    widths = [(0, 0)] * a.ndim
    widths[axis] = (0, r)
    return jnp.pad(a, widths)


def _gmm_call(x, A, group_sizes, trans_rhs, compute_dtype=None):
    assert A.ndim == 3 and x.ndim == 2 and A.shape[:1] == group_sizes.shape
    out_dtype = x.dtype
    cd = jnp.dtype(compute_dtype) if compute_dtype is not None else x.dtype
    x, A = x.astype(cd), A.astype(cd)
    m, g = x.shape[0], A.shape[0]
    n = A.shape[-1] if not trans_rhs else A.shape[-2]
    mult = 16 // cd.itemsize  # rows of k and of n elements must be multiples of 16 bytes
    xp = _pad_to(x, 1, mult)
    Ap = _pad_to(_pad_to(A, 1, mult), 2, mult)
    n_pad = Ap.shape[-1] if not trans_rhs else Ap.shape[-2]
    _ensure_registered()
    y, _ = jax.ffi.ffi_call(
        "rd_gmm", (jax.ShapeDtypeStruct((m, n_pad), cd), _workspace_struct(m, g)))(
        xp, Ap, group_sizes.astype(jnp.int32), trans_rhs=bool(trans_rhs), tile_n=np.int32(0))
    return y[:, :n].astype(out_dtype)


def _tgmm_call(x, y, group_sizes, compute_dtype=None):
    assert y.ndim == 2 and x.ndim == 2 and x.shape[0] == y.shape[0]
    out_dtype = x.dtype
    cd = jnp.dtype(compute_dtype) if compute_dtype is not None else x.dtype
    x, y = x.astype(cd), y.astype(cd)
    (m, k), n, g = x.shape, y.shape[-1], group_sizes.size
    mult = 16 // cd.itemsize
    xp, yp = _pad_to(x, 1, mult), _pad_to(y, 1, mult)
    _ensure_registered()
    out, _ = jax.ffi.ffi_call(
        "rd_tgmm", (jax.ShapeDtypeStruct((g, xp.shape[1], yp.shape[1]), cd), _workspace_struct(m, g)))(
        xp, yp, group_sizes.astype(jnp.int32), tile_n=np.int32(0))
    return out[:, :k, :n].astype(out_dtype)


@partial(jax.custom_vjp, nondiff_argnames=NONDIFF_ARGNAMES + ("trans_rhs",))
@partial(jax.jit, static_argnums=list(range(3, 13)))  # as the reference, gpu_ragged_dot.py:361
def gmm(x, A, group_sizes, block_m=DEFAULT_BLOCK_M, block_k=DEFAULT_BLOCK_K, block_n=DEFAULT_BLOCK_N,
        trans_rhs=False, interpret=False, compute_dtype=None, acc_dtype=jnp.float32, num_warps=None,
        num_stages=None, chunk_m=CHUNK_M):
    """jax.lax.ragged_dot: (m, k) x (g, k, n) -> (m, n)."""
    _check(x, interpret, compute_dtype, acc_dtype)
    return _gmm_call(x, A, group_sizes, trans_rhs, compute_dtype)


def _gmm_fwd(x, A, group_sizes, block_m, block_k, block_n, trans_rhs, interpret, compute_dtype,
             acc_dtype, num_warps, num_stages, chunk_m):
    _check(x, interpret, compute_dtype, acc_dtype)
    return _gmm_call(x, A, group_sizes, trans_rhs, compute_dtype), (x, A, group_sizes)


def _gmm_bwd(block_m, block_k, block_n, trans_rhs, interpret, compute_dtype, acc_dtype, num_warps,
             num_stages, chunk_m, res, do):
    x, A, group_sizes = res  # same wiring as gpu_ragged_dot.py:399-402
    dx = _gmm_call(do, A, group_sizes, not trans_rhs, compute_dtype)
    dA = (_tgmm_call(x, do, group_sizes, compute_dtype) if not trans_rhs
          else _tgmm_call(do, x, group_sizes, compute_dtype))
    return dx.astype(x.dtype), dA.astype(A.dtype), None


gmm.defvjp(_gmm_fwd, _gmm_bwd)
ragged_dot = gmm


@partial(jax.custom_vjp, nondiff_argnames=NONDIFF_ARGNAMES)
@partial(jax.jit, static_argnums=list(range(3, 12)))  # as the reference, gpu_ragged_dot.py:410
def tgmm(x, y, group_sizes, block_m=DEFAULT_BLOCK_M, block_k=DEFAULT_BLOCK_K, block_n=DEFAULT_BLOCK_N,
         interpret=False, compute_dtype=None, acc_dtype=jnp.float32, num_warps=None, num_stages=None,
         chunk_m=CHUNK_M):
    """Transposed ragged dot: (m, k) x (m, n) -> (g, k, n)."""
    _check(x, interpret, compute_dtype, acc_dtype)
    return _tgmm_call(x, y, group_sizes, compute_dtype)


def _tgmm_fwd(x, y, group_sizes, block_m, block_k, block_n, interpret, compute_dtype, acc_dtype,
              num_warps, num_stages, chunk_m):
    _check(x, interpret, compute_dtype, acc_dtype)
    return _tgmm_call(x, y, group_sizes, compute_dtype), (x, y, group_sizes)


def _tgmm_bwd(block_m, block_k, block_n, interpret, compute_dtype, acc_dtype, num_warps, num_stages,
              chunk_m, res, do):
    x, y, group_sizes = res  # out[g] = x_g^T y_g  =>  dx_g = y_g do[g]^T,  dy_g = x_g do[g]
    dx = _gmm_call(y, do, group_sizes, True, compute_dtype)
    dy = _gmm_call(x, do, group_sizes, False, compute_dtype)
    return dx.astype(x.dtype), dy.astype(y.dtype), None


tgmm.defvjp(_tgmm_fwd, _tgmm_bwd)
trans_ragged_dot = tgmm
