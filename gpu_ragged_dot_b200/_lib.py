"""ctypes binding of librd_b200.so (the C ABI declared in include/ragged_dot_b200.h).

There is no fallback: if the shared object is missing or does not export a symbol the header
declares, loading raises.  Build it with ``python -m gpu_ragged_dot_b200.build``.
"""

from __future__ import annotations

import ctypes
import os
import threading

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "librd_b200.so")

RD_OK = 0
RD_ERR_BAD_SHAPE, RD_ERR_BAD_DTYPE, RD_ERR_BAD_POINTER, RD_ERR_WORKSPACE, RD_ERR_BAD_CONFIG = 1, 2, 3, 4, 5
RD_ERR_TENSOR_MAP, RD_ERR_LAUNCH, RD_ERR_DRIVER, RD_ERR_DEVICE_WAIT, RD_ERR_TOO_LARGE = 6, 7, 8, 9, 10
RD_ERR_SCRATCH_SETUP = 11
RD_DTYPE_F16 = 0
RD_DTYPE_BF16 = 1
RD_DTYPE_F32 = 2
RD_CFG_NO_ZERO_TAIL = 1
RD_CFG_GROUP_BY_WEIGHT = 2

# Every symbol include/ragged_dot_b200.h declares, with its ctypes signature.
_c_int = ctypes.c_int
_c_void_p = ctypes.c_void_p
_c_size_t = ctypes.c_size_t


class TileCfg(ctypes.Structure):
    """Mirror of ``rd_tile_cfg``."""

    _fields_ = [("tile_n", ctypes.c_int32), ("max_ctas", ctypes.c_int32), ("cta_group", ctypes.c_int32),
                ("tile_m", ctypes.c_int32), ("flags", ctypes.c_int32), ("wait_limit_ms", ctypes.c_int32)]


class EpSend(ctypes.Structure):
    """Mirror of ``rd_ep_send``."""

    _fields_ = [("x_tokens", ctypes.c_void_p), ("send_index", ctypes.c_void_p), ("send_start", ctypes.c_void_p),
                ("dest_pos", ctypes.c_void_p), ("phase_done", ctypes.c_void_p),
                ("peer_base", ctypes.c_void_p), ("peer_flags", ctypes.c_void_p),
                ("row_bytes", ctypes.c_int32), ("top_k", ctypes.c_int32), ("world", ctypes.c_int32),
                ("rank", ctypes.c_int32), ("capacity_rows", ctypes.c_int32), ("sender_ctas", ctypes.c_int32)]


class EpStep(ctypes.Structure):
    """Mirror of ``rd_ep_step``."""

    _fields_ = [("routing", ctypes.c_void_p), ("tokens", ctypes.c_int32), ("top_k", ctypes.c_int32),
                ("num_experts", ctypes.c_int32), ("epoch", ctypes.c_int32),
                ("counts_scratch", ctypes.c_void_p), ("ticket", ctypes.c_void_p),
                ("peer_counts", ctypes.c_void_p), ("peer_count_flags", ctypes.c_void_p),
                ("counts_all", ctypes.c_void_p), ("count_flags", ctypes.c_void_p),
                ("dest_offset", ctypes.c_void_p), ("segment_sizes", ctypes.c_void_p), ("fill", ctypes.c_void_p),
                ("totals", ctypes.c_void_p), ("send_start", ctypes.c_void_p), ("list_fill", ctypes.c_void_p),
                ("plan_status", ctypes.c_void_p), ("dest_pos", ctypes.c_void_p), ("send_index", ctypes.c_void_p),
                ("own_buffer", ctypes.c_void_p), ("own_ready_flag", ctypes.c_void_p),
                ("wait_limit_ms", ctypes.c_int32)]


SIGNATURES = {
    "rd_version": (_c_int, []),
    "rd_status_string": (ctypes.c_char_p, [_c_int]),
    "rd_workspace_bytes": (_c_int, [_c_int, _c_int, ctypes.POINTER(_c_size_t)]),
    "rd_metadata": (
        _c_int,
        [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    ),
    "rd_gmm": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_size_t]
        + [_c_int] * 6
        + [ctypes.POINTER(TileCfg), _c_void_p],
    ),
    "rd_tgmm": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_size_t]
        + [_c_int] * 5
        + [ctypes.POINTER(TileCfg), _c_void_p],
    ),
    "rd_gmm_fp8": (
        _c_int,
        [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_size_t]
        + [_c_int] * 4
        + [ctypes.POINTER(TileCfg), _c_void_p],
    ),
    "rd_tgmm_strided": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_size_t]
        + [_c_int] * 6
        + [ctypes.POINTER(TileCfg), _c_void_p],
    ),
    "rd_ep_combine_pull": (_c_int, [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                                    _c_int, _c_int, _c_void_p, _c_int, _c_void_p]),
    "rd_gmm_indexed": (
        _c_int,
        [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_size_t]
        + [_c_int] * 6
        + [ctypes.POINTER(TileCfg), _c_void_p],
    ),
    "rd_ep_plan_ring": (_c_int, [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                 _c_void_p, _c_void_p, _c_void_p, _c_void_p]),
    "rd_ep_count_share": (_c_int, [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p,
                                   _c_void_p, _c_int, _c_void_p]),
    "rd_ep_plan_ring_when_counted": (_c_int, [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                                              _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                              _c_void_p, _c_int, _c_void_p]),
    "rd_ep_assign": (_c_int, [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p,
                              _c_void_p, _c_void_p, _c_void_p, _c_void_p]),
    "rd_ep_send_list": (_c_int, [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p,
                                 _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p]),
    "rd_gmm_ep_fused": (
        _c_int,
        [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_size_t]
        + [_c_int] * 6
        + [ctypes.POINTER(TileCfg), _c_void_p, _c_int, _c_int, ctypes.POINTER(EpSend), _c_void_p],
    ),
    "rd_gmm_indexed_when_ready": (
        _c_int,
        [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_size_t]
        + [_c_int] * 6
        + [ctypes.POINTER(TileCfg), _c_void_p, _c_int, _c_int, _c_void_p],
    ),
    "rd_gmm_permuted": (
        _c_int,
        [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
         _c_void_p, _c_void_p, _c_size_t]
        + [_c_int] * 6
        + [ctypes.POINTER(TileCfg), _c_void_p],
    ),
    "rd_tgmm_permuted": (
        _c_int,
        [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
         _c_size_t]
        + [_c_int] * 5
        + [ctypes.POINTER(TileCfg), _c_void_p],
    ),
    "rd_gather_rows": (_c_int, [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p]),
    "rd_ep_count": (_c_int, [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p]),
    "rd_ep_plan": (_c_int, [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                            _c_void_p]),
    "rd_ep_fused_forward": (
        _c_int,
        [ctypes.POINTER(EpStep), _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_size_t,
         _c_int, _c_int, _c_int, _c_int, ctypes.POINTER(TileCfg), _c_void_p, ctypes.POINTER(EpSend), _c_void_p],
    ),
    "rd_ep_dispatch": (
        _c_int,
        [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p,
         _c_int, _c_void_p, _c_void_p],
    ),
    "rd_device_status": (_c_int, [_c_void_p, _c_void_p]),
    "rd_gmm_static_scratch": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_void_p] + [_c_int] * 6 + [ctypes.POINTER(TileCfg), _c_void_p],
    ),
}

_lock = threading.Lock()
_lib = None


class RaggedDotError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code: int, text: str, where: str):
        super().__init__(f"{where}: {text} (status {code})")
        self.code = code


def load() -> ctypes.CDLL:
    """Load the library once and bind every declared symbol; raise if anything is missing."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: the CUDA library is not built. "
                "Run `python -m gpu_ragged_dot_b200.build` (needs nvcc with sm_100a support). "
                "There is no CPU or PyTorch fallback."
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is not exported
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
        return lib


def status_string(code: int) -> str:
    return load().rd_status_string(code).decode()


def check(code: int, where: str) -> None:
    if code != RD_OK:
        raise RaggedDotError(code, status_string(code), where)
