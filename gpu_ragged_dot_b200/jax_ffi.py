"""jax binding of the C ABI: ``ragged_dot`` / ``trans_ragged_dot`` as XLA custom calls with the
reference's signature and custom_vjp (gpu_ragged_dot.py:345-454).

Importing this module needs jax with ``jax.ffi`` and the XLA-FFI shim library
(``librd_b200_xla.so``, built from csrc/xla_ffi_shim.cc against jaxlib's headers).  Neither is
present in the image this library was developed in, so this file has not been executed there;
the torch layer in ``ops.py`` drives the same entry points and carries the tests.
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
_xla = ctypes.CDLL(os.path.join(_HERE, "librd_b200_xla.so"))
jax.ffi.register_ffi_target("rd_gmm", jax.ffi.pycapsule(_xla.RdGmmFfi), platform="CUDA")
jax.ffi.register_ffi_target("rd_tgmm", jax.ffi.pycapsule(_xla.RdTgmmFfi), platform="CUDA")

DEFAULT_BLOCK_M = DEFAULT_BLOCK_N = DEFAULT_BLOCK_K = 64
CHUNK_M = 512
NONDIFF_ARGNAMES = ("block_m", "block_k", "block_n", "interpret", "compute_dtype", "acc_dtype",
                    "num_warps", "num_stages", "chunk_m")


def _workspace_struct(m: int, g: int):
    nbytes = ctypes.c_size_t(0)
    _lib.check(_lib.load().rd_workspace_bytes(m, g, ctypes.byref(nbytes)), "rd_workspace_bytes")
    return jax.ShapeDtypeStruct((nbytes.value,), jnp.uint8)


def _check(x, interpret, compute_dtype, acc_dtype):
    if interpret:
        raise NotImplementedError("interpret=True: there is no CPU path")
    if compute_dtype is not None and jnp.dtype(compute_dtype) != x.dtype:
        raise NotImplementedError("compute_dtype must be None or the input dtype")
    if acc_dtype is not None and jnp.dtype(acc_dtype) != jnp.float32:
        raise NotImplementedError("acc_dtype must be float32")


def _gmm_call(x, A, group_sizes, trans_rhs):
    assert A.ndim == 3 and x.ndim == 2 and A.shape[:1] == group_sizes.shape
    m, g = x.shape[0], A.shape[0]
    n = A.shape[-1] if not trans_rhs else A.shape[-2]
    y, _ = jax.ffi.ffi_call(
        "rd_gmm", (jax.ShapeDtypeStruct((m, n), x.dtype), _workspace_struct(m, g)))(
        x, A, group_sizes.astype(jnp.int32), trans_rhs=bool(trans_rhs), tile_n=np.int32(0))
    return y


def _tgmm_call(x, y, group_sizes):
    assert y.ndim == 2 and x.ndim == 2 and x.shape[0] == y.shape[0]
    (m, k), n, g = x.shape, y.shape[-1], group_sizes.size
    out, _ = jax.ffi.ffi_call(
        "rd_tgmm", (jax.ShapeDtypeStruct((g, k, n), x.dtype), _workspace_struct(m, g)))(
        x, y, group_sizes.astype(jnp.int32), tile_n=np.int32(0))
    return out


@partial(jax.custom_vjp, nondiff_argnames=NONDIFF_ARGNAMES + ("trans_rhs",))
def gmm(x, A, group_sizes, block_m=DEFAULT_BLOCK_M, block_k=DEFAULT_BLOCK_K, block_n=DEFAULT_BLOCK_N,
        trans_rhs=False, interpret=False, compute_dtype=None, acc_dtype=jnp.float32, num_warps=None,
        num_stages=None, chunk_m=CHUNK_M):
    """jax.lax.ragged_dot: (m, k) x (g, k, n) -> (m, n)."""
    _check(x, interpret, compute_dtype, acc_dtype)
    return _gmm_call(x, A, group_sizes, trans_rhs)


def _gmm_fwd(x, A, group_sizes, block_m, block_k, block_n, trans_rhs, interpret, compute_dtype,
             acc_dtype, num_warps, num_stages, chunk_m):
    _check(x, interpret, compute_dtype, acc_dtype)
    return _gmm_call(x, A, group_sizes, trans_rhs), (x, A, group_sizes)


def _gmm_bwd(block_m, block_k, block_n, trans_rhs, interpret, compute_dtype, acc_dtype, num_warps,
             num_stages, chunk_m, res, do):
    x, A, group_sizes = res
    dx = _gmm_call(do, A, group_sizes, not trans_rhs)
    dA = _tgmm_call(x, do, group_sizes) if not trans_rhs else _tgmm_call(do, x, group_sizes)
    return dx, dA, None


gmm.defvjp(_gmm_fwd, _gmm_bwd)
ragged_dot = gmm


@partial(jax.custom_vjp, nondiff_argnames=NONDIFF_ARGNAMES)
def tgmm(x, y, group_sizes, block_m=DEFAULT_BLOCK_M, block_k=DEFAULT_BLOCK_K, block_n=DEFAULT_BLOCK_N,
         interpret=False, compute_dtype=None, acc_dtype=jnp.float32, num_warps=None, num_stages=None,
         chunk_m=CHUNK_M):
    """Transposed ragged dot: (m, k) x (m, n) -> (g, k, n)."""
    _check(x, interpret, compute_dtype, acc_dtype)
    return _tgmm_call(x, y, group_sizes)


def _tgmm_fwd(x, y, group_sizes, block_m, block_k, block_n, interpret, compute_dtype, acc_dtype,
              num_warps, num_stages, chunk_m):
    _check(x, interpret, compute_dtype, acc_dtype)
    return _tgmm_call(x, y, group_sizes), (x, y, group_sizes)


def _tgmm_bwd(block_m, block_k, block_n, interpret, compute_dtype, acc_dtype, num_warps, num_stages,
              chunk_m, res, do):
    x, y, group_sizes = res
    return _gmm_call(y, do, group_sizes, True), _gmm_call(x, do, group_sizes, False), None


tgmm.defvjp(_tgmm_fwd, _tgmm_bwd)
trans_ragged_dot = tgmm
