"""Host-side mirror of the reference's public interface (gpu_ragged_dot.py:345-454).

Same names (``gmm`` = ``ragged_dot``, ``tgmm`` = ``trans_ragged_dot``), same argument order,
same defaults and the same custom-VJP wiring, over torch CUDA tensors instead of jax arrays
(torch supplies device memory and streams; all arithmetic is in librd_b200.so).  The jax
binding of the same C ABI lives in ``jax_ffi.py``.

Differences from the reference, all deliberate:
  * ``block_m/block_k/block_n/num_warps/num_stages/chunk_m`` are accepted for drop-in
    compatibility but are hints only -- tiles come from the committed tile table
    (``tile_table.py``), which replaces the tune-jax search of tuning.py:49-58.
  * ``interpret=True`` raises: there is no CPU path.
  * float32 inputs are multiplied as TF32 on the tensor cores with fp32 accumulation and give
    float32 results (the precision the reference's Triton ``tl.dot`` uses for float32);
    ``precision="highest"`` (an extra keyword) runs three TF32 passes for nearly fp32 accuracy.
  * ``compute_dtype`` casts both operands before the product and the result comes back in
    ``x.dtype``, as in the reference (gpu_ragged_dot.py:116,145,149); the two inputs may differ in type.
  * rows past ``sum(group_sizes)`` are always zero, also when every group is empty (the
    reference leaves them unwritten in that case, gpu_ragged_dot.py:155-157).
  * the VJP of ``tgmm`` is the mathematically correct one; the reference's
    (gpu_ragged_dot.py:431-450) cannot run.
"""

from __future__ import annotations

import ctypes
import os
from typing import NamedTuple, Optional, Sequence

import torch

from . import _lib
from . import tile_table

__all__ = [
    "gmm",
    "tgmm",
    "ragged_dot",
    "trans_ragged_dot",
    "ragged_dot_general",
    "RaggedDotDimensionNumbers",
    "make_group_metadata",
    "GMMGroupLookupMetadata",
    "RaggedDotSizes",
    "BlockSizes",
]

DEFAULT_BLOCK_M = 64
DEFAULT_BLOCK_N = 64
DEFAULT_BLOCK_K = 64
CHUNK_M = 512


class RaggedDotSizes(NamedTuple):
    m: int
    k: int
    n: int
    g: int


class BlockSizes(NamedTuple):
    m: int
    k: int
    n: int


class GMMGroupLookupMetadata(NamedTuple):
    """Same five fields as the reference's tuple (gpu_ragged_dot.py:60-67), as int32 CUDA tensors."""

    group_sizes: torch.Tensor
    group_offsets: torch.Tensor
    row_it2group: torch.Tensor
    row_it2it_in_group: torch.Tensor
    total_row_its: torch.Tensor


_DTYPE_CODE = {torch.float16: _lib.RD_DTYPE_F16, torch.bfloat16: _lib.RD_DTYPE_BF16,
               torch.float32: _lib.RD_DTYPE_F32}


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(
            f"{name} must be a CUDA tensor: ragged_dot runs only on the GPU through librd_b200.so "
            "(no CPU fallback)"
        )


def _as_i32(group_sizes: torch.Tensor) -> torch.Tensor:
    _require_cuda(group_sizes, "group_sizes")
    if group_sizes.dim() != 1:
        raise AssertionError(f"group_sizes must be 1-D, got {group_sizes.dim()=}")
    if group_sizes.dtype != torch.int32:
        group_sizes = group_sizes.to(torch.int32)
    return group_sizes.contiguous()


def _dense16(t: torch.Tensor) -> torch.Tensor:
    t = t.contiguous()
    if t.data_ptr() % 16:
        t = t.clone()
    return t


def _pad_last(t: torch.Tensor, mult: int = 8) -> torch.Tensor:
    r = (-t.shape[-1]) % mult
    return torch.nn.functional.pad(t, (0, r)) if r else t


def _pad_last2(t: torch.Tensor, mult: int = 8) -> torch.Tensor:
    r1 = (-t.shape[-1]) % mult
    r2 = (-t.shape[-2]) % mult
    return torch.nn.functional.pad(t, (0, r1, 0, r2)) if (r1 or r2) else t


def _workspace(m: int, g: int, device: torch.device) -> torch.Tensor:
    lib = _lib.load()
    nbytes = ctypes.c_size_t(0)
    _lib.check(lib.rd_workspace_bytes(m, g, ctypes.byref(nbytes)), "rd_workspace_bytes")
    return torch.empty(max(nbytes.value, 256), dtype=torch.uint8, device=device)


def _cfg_ptr(cfg: Optional[_lib.TileCfg]):
    return ctypes.byref(cfg) if cfg is not None else None


def _check_status_enabled() -> bool:
    return os.environ.get("RD_CHECK_STATUS", "0") not in ("", "0")


def _maybe_check_status(workspace: torch.Tensor, where: str) -> None:
    """With RD_CHECK_STATUS=1 every GEMM call synchronises its stream and raises if a bounded wait
    expired inside the kernel (the output then has unwritten tiles).  Off by default: the check
    costs a device synchronisation per call."""
    if _check_status_enabled():
        code = device_status(workspace)
        if code != 0:
            raise _lib.RaggedDotError(code, _lib.status_string(code), where)


def make_group_metadata(group_sizes: torch.Tensor, m: int, chunk_m: int) -> GMMGroupLookupMetadata:
    """Device-side equivalent of ``_make_gmm_group_metadata`` (gpu_ragged_dot.py:70-90)."""
    lib = _lib.load()
    gs = _as_i32(group_sizes)
    g = gs.numel()
    u = (m + chunk_m - 1) // chunk_m + g
    dev = gs.device
    offsets = torch.empty(g, dtype=torch.int32, device=dev)
    it2group = torch.empty(u, dtype=torch.int32, device=dev)
    it2it = torch.empty(u, dtype=torch.int32, device=dev)
    total = torch.empty((), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = lib.rd_metadata(
            gs.data_ptr(), g, m, chunk_m, offsets.data_ptr(), it2group.data_ptr(), it2it.data_ptr(),
            total.data_ptr(), _stream_ptr(dev),
        )
    _lib.check(rc, "rd_metadata")
    return GMMGroupLookupMetadata(gs, offsets, it2group, it2it, total)


def gmm_forward(
    x: torch.Tensor,
    A: torch.Tensor,
    group_sizes: torch.Tensor,
    trans_rhs: bool = False,
    cfg: Optional[_lib.TileCfg] = None,
    out: Optional[torch.Tensor] = None,
    workspace: Optional[torch.Tensor] = None,
    group_to_weight: Optional[torch.Tensor] = None,
    ready: Optional[tuple] = None,
) -> torch.Tensor:
    """One call of ``rd_gmm``: y[m,n] = ragged x[m,k] . A[g,k,n] (or A[g,n,k] with trans_rhs).

    With ``group_to_weight`` (int32 [g], values in [0, A.shape[0])) it is ``rd_gmm_indexed``:
    group i multiplies by A[group_to_weight[i]] and g may differ from A.shape[0].
    With ``ready = (flags int32 tensor, groups_per_flag, epoch)`` it is
    ``rd_gmm_indexed_when_ready``: group i's rows are read once flags[i // groups_per_flag] >= epoch."""
    lib = _lib.load()
    _require_cuda(x, "x")
    _require_cuda(A, "A")
    assert A.dim() == 3 and x.dim() == 2, f"but {A.dim()=} {x.dim()=}"
    gs = _as_i32(group_sizes)
    if group_to_weight is None:
        assert A.shape[0] == gs.shape[0], f"{A.shape[0]=} != {gs.shape[0]=}"
        assert ready is None, "ready flags need group_to_weight (rd_gmm_indexed_when_ready)"
    else:
        group_to_weight = _as_i32(group_to_weight)
        assert group_to_weight.shape == gs.shape
    if x.dtype not in _DTYPE_CODE or A.dtype != x.dtype:
        raise NotImplementedError(f"inputs must both be float16, bfloat16 or float32, got {x.dtype} / {A.dtype}")
    m, k = x.shape
    g = gs.shape[0]
    n = A.shape[-1] if not trans_rhs else A.shape[-2]
    k_rhs = A.shape[-2] if not trans_rhs else A.shape[-1]
    assert k_rhs == k, f"contraction mismatch: x has k={k}, A has {k_rhs}"

    # TMA needs 16-byte row strides: pad k and n up to multiples of 16 bytes with zeros (exact).
    mult = 16 // x.element_size()
    xp = _dense16(_pad_last(x, mult))
    Ap = _dense16(_pad_last2(A, mult))
    kp = xp.shape[1]
    np_ = Ap.shape[-1] if not trans_rhs else Ap.shape[-2]
    padded_n = np_ != n
    if out is not None and not padded_n:
        assert out.shape == (m, n) and out.dtype == x.dtype and out.is_contiguous()
        y = out
    else:
        y = torch.empty((m, np_), dtype=x.dtype, device=x.device)
    ws = workspace if workspace is not None else _workspace(m, g, x.device)
    if cfg is None and x.dtype != torch.float32:  # the table's entries are for the 16-bit kernels
        cfg = tile_table.lookup("gmm_t" if trans_rhs else "gmm", m, kp, np_, g)
    with torch.cuda.device(x.device):
        if group_to_weight is None:
            rc = lib.rd_gmm(
                xp.data_ptr(), Ap.data_ptr(), gs.data_ptr(), y.data_ptr(), ws.data_ptr(), ws.numel(),
                m, kp, np_, g, int(bool(trans_rhs)), _DTYPE_CODE[x.dtype], _cfg_ptr(cfg),
                _stream_ptr(x.device),
            )
        elif ready is None:
            rc = lib.rd_gmm_indexed(
                xp.data_ptr(), Ap.data_ptr(), Ap.shape[0], gs.data_ptr(), group_to_weight.data_ptr(),
                y.data_ptr(), ws.data_ptr(), ws.numel(), m, kp, np_, g, int(bool(trans_rhs)),
                _DTYPE_CODE[x.dtype], _cfg_ptr(cfg), _stream_ptr(x.device),
            )
        else:
            flags, groups_per_flag, epoch = ready
            assert flags.dtype == torch.int32 and flags.is_cuda
            rc = lib.rd_gmm_indexed_when_ready(
                xp.data_ptr(), Ap.data_ptr(), Ap.shape[0], gs.data_ptr(), group_to_weight.data_ptr(),
                y.data_ptr(), ws.data_ptr(), ws.numel(), m, kp, np_, g, int(bool(trans_rhs)),
                _DTYPE_CODE[x.dtype], _cfg_ptr(cfg), flags.data_ptr(), int(groups_per_flag), int(epoch),
                _stream_ptr(x.device),
            )
    _lib.check(rc, "rd_gmm")
    _maybe_check_status(ws, "rd_gmm")
    if padded_n:
        y = y[:, :n].contiguous()
        if out is not None:
            out.copy_(y)
            y = out
    return y


def gmm_fp8_forward(x: torch.Tensor, A: torch.Tensor, group_sizes: torch.Tensor,
                    weight_scale: Optional[torch.Tensor] = None, group_to_weight: Optional[torch.Tensor] = None,
                    cfg: Optional[_lib.TileCfg] = None, out: Optional[torch.Tensor] = None,
                    workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``rd_gmm_fp8``: ragged x[m,k] . A[w]^T for e4m3 operands (``torch.float8_e4m3fn``), A stored
    ``[num_weights, n, k]``; fp32 accumulation, times ``weight_scale[w]`` (float32, optional), bf16
    result.  Forward only (an inference path): there is no 8-bit tgmm."""
    lib = _lib.load()
    _require_cuda(x, "x")
    _require_cuda(A, "A")
    f8 = torch.float8_e4m3fn
    if x.dtype != f8 or A.dtype != f8:
        raise NotImplementedError(f"inputs must both be float8_e4m3fn, got {x.dtype} / {A.dtype}")
    assert x.dim() == 2 and A.dim() == 3 and A.shape[2] == x.shape[1], "x [m,k], A [num_weights,n,k]"
    gs = _as_i32(group_sizes)
    g, (m, k), n = gs.numel(), x.shape, A.shape[1]
    if group_to_weight is None:
        assert A.shape[0] == g, f"{A.shape[0]=} != {g=}"
    else:
        group_to_weight = _as_i32(group_to_weight)
    if k % 16 or n % 8:
        raise NotImplementedError("8-bit inputs: k must be a multiple of 16 and n of 8")
    x, A = _dense16(x), _dense16(A)
    if weight_scale is not None:
        weight_scale = weight_scale.to(device=x.device, dtype=torch.float32).contiguous()
        assert weight_scale.numel() == A.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    assert out.shape == (m, n) and out.dtype == torch.bfloat16 and out.is_contiguous()
    ws = workspace if workspace is not None else _workspace(m, g, x.device)
    with torch.cuda.device(x.device):
        rc = lib.rd_gmm_fp8(x.data_ptr(), A.data_ptr(), A.shape[0], gs.data_ptr(),
                            group_to_weight.data_ptr() if group_to_weight is not None else None,
                            weight_scale.data_ptr() if weight_scale is not None else None,
                            out.data_ptr(), ws.data_ptr(), ws.numel(), m, k, n, g, _cfg_ptr(cfg),
                            _stream_ptr(x.device))
    _lib.check(rc, "rd_gmm_fp8")
    _maybe_check_status(ws, "rd_gmm_fp8")
    return out


def gather_rows(src: torch.Tensor, row_index: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dst[i] = src[row_index[i]] through ``rd_gather_rows`` (rows must be a multiple of 16 bytes)."""
    lib = _lib.load()
    _require_cuda(src, "src")
    idx = _as_i32(row_index)
    src = _dense16(src)
    assert src.dim() == 2
    rows_out, row_bytes = idx.numel(), src.shape[1] * src.element_size()
    dst = out if out is not None else torch.empty((rows_out, src.shape[1]), dtype=src.dtype, device=src.device)
    assert dst.is_contiguous() and dst.shape == (rows_out, src.shape[1]) and dst.dtype == src.dtype
    with torch.cuda.device(src.device):
        rc = lib.rd_gather_rows(src.data_ptr(), idx.data_ptr(), dst.data_ptr(), rows_out, src.shape[0],
                                row_bytes, _stream_ptr(src.device))
    _lib.check(rc, "rd_gather_rows")
    return dst


def ep_count(routing: torch.Tensor, num_experts: int) -> torch.Tensor:
    """counts[e] of a [tokens, top_k] int32 routing table (``rd_ep_count``)."""
    lib = _lib.load()
    r = _as_i32(routing.reshape(-1))
    counts = torch.empty(num_experts, dtype=torch.int32, device=r.device)
    with torch.cuda.device(r.device):
        rc = lib.rd_ep_count(r.data_ptr(), r.numel(), num_experts, counts.data_ptr(), _stream_ptr(r.device))
    _lib.check(rc, "rd_ep_count")
    return counts


def ep_plan(counts_all: torch.Tensor, rank: int):
    """(dest_offset[E], segment_sizes[W*El], fill[E], totals[1]) from counts_all[W, E] (``rd_ep_plan``)."""
    lib = _lib.load()
    assert counts_all.dim() == 2 and counts_all.dtype == torch.int32 and counts_all.is_contiguous()
    world, experts = counts_all.shape
    dev = counts_all.device
    dest_offset = torch.empty(experts, dtype=torch.int32, device=dev)
    segment_sizes = torch.empty(experts, dtype=torch.int32, device=dev)  # world * (experts / world)
    fill = torch.empty(experts, dtype=torch.int32, device=dev)
    totals = torch.empty(1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = lib.rd_ep_plan(counts_all.data_ptr(), world, experts, rank, dest_offset.data_ptr(),
                            segment_sizes.data_ptr(), fill.data_ptr(), totals.data_ptr(), _stream_ptr(dev))
    _lib.check(rc, "rd_ep_plan")
    return dest_offset, segment_sizes, fill, totals


def ep_dispatch(x: torch.Tensor, routing: torch.Tensor, num_experts: int, world: int,
                dest_offset: torch.Tensor, fill: torch.Tensor, peer_base: torch.Tensor,
                capacity_rows: int) -> torch.Tensor:
    """Copy every routed row of x into its owner's receive buffer (``rd_ep_dispatch``);
    peer_base is an int64 device tensor of `world` buffer addresses.  Returns dest_pos."""
    lib = _lib.load()
    _require_cuda(x, "x")
    x = _dense16(x)
    r = _as_i32(routing.reshape(-1))
    tokens, top_k = routing.shape
    assert peer_base.dtype == torch.int64 and peer_base.numel() == world and peer_base.is_cuda
    dest_pos = torch.empty(tokens * top_k, dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib.rd_ep_dispatch(x.data_ptr(), r.data_ptr(), tokens, top_k, x.shape[1] * x.element_size(),
                                num_experts, world, dest_offset.data_ptr(), fill.data_ptr(),
                                peer_base.data_ptr(), capacity_rows, dest_pos.data_ptr(),
                                _stream_ptr(x.device))
    _lib.check(rc, "rd_ep_dispatch")
    return dest_pos.view(tokens, top_k)


def ep_plan_ring(counts_all: torch.Tensor, rank: int, bufs: Optional[dict] = None) -> dict:
    """``rd_ep_plan_ring``: the plan of the fused exchange (receive buffer ordered by position
    q = (rank - source) mod W).  Returns / refills a dict with dest_offset[E], segment_sizes[E],
    fill[E], totals[1], phase_done[W], send_start[W+1], list_fill[W]."""
    lib = _lib.load()
    assert counts_all.dim() == 2 and counts_all.dtype == torch.int32 and counts_all.is_contiguous()
    world, experts = counts_all.shape
    dev = counts_all.device
    if bufs is None:
        bufs = {name: torch.empty(size, dtype=torch.int32, device=dev)
                for name, size in (("dest_offset", experts), ("segment_sizes", experts), ("fill", experts),
                                   ("totals", 1), ("phase_done", world), ("send_start", world + 1),
                                   ("list_fill", world))}
    with torch.cuda.device(dev):
        rc = lib.rd_ep_plan_ring(counts_all.data_ptr(), world, experts, rank, bufs["dest_offset"].data_ptr(),
                                 bufs["segment_sizes"].data_ptr(), bufs["fill"].data_ptr(),
                                 bufs["totals"].data_ptr(), bufs["phase_done"].data_ptr(),
                                 bufs["send_start"].data_ptr(), bufs["list_fill"].data_ptr(), _stream_ptr(dev))
    _lib.check(rc, "rd_ep_plan_ring")
    return bufs


def ep_count_share(routing: torch.Tensor, num_experts: int, scratch: torch.Tensor, world: int, rank: int,
                   peer_counts: torch.Tensor, peer_flags: torch.Tensor, epoch: int) -> None:
    """``rd_ep_count_share``: count the routing table and store the counts into row ``rank`` of every
    rank's counts_all, then ``epoch`` into every rank's count flag ``rank``.  ``scratch`` is an int32
    device tensor of num_experts + 1 zeros (the call leaves it zero); ``peer_counts`` / ``peer_flags``
    are int64 device tensors of `world` addresses."""
    lib = _lib.load()
    r = _as_i32(routing.reshape(-1))
    assert scratch.dtype == torch.int32 and scratch.numel() >= num_experts + 1 and scratch.is_cuda
    with torch.cuda.device(r.device):
        rc = lib.rd_ep_count_share(r.data_ptr(), r.numel(), num_experts, scratch.data_ptr(),
                                   scratch.data_ptr() + 4 * num_experts, world, rank, peer_counts.data_ptr(),
                                   peer_flags.data_ptr(), int(epoch), _stream_ptr(r.device))
    _lib.check(rc, "rd_ep_count_share")


def ep_plan_ring_when_counted(counts_all: torch.Tensor, count_flags: torch.Tensor, epoch: int, rank: int,
                              bufs: dict, workspace: torch.Tensor, wait_limit_ms: int = 0) -> dict:
    """``rd_ep_plan_ring_when_counted``: ``ep_plan_ring`` that first waits, on the device and bounded,
    for every source's counts of this epoch.  ``workspace`` holds the status word that reports an
    expired wait (any int32 device tensor; ``device_status`` reads it)."""
    lib = _lib.load()
    assert counts_all.dim() == 2 and counts_all.dtype == torch.int32 and counts_all.is_contiguous()
    world, experts = counts_all.shape
    dev = counts_all.device
    with torch.cuda.device(dev):
        rc = lib.rd_ep_plan_ring_when_counted(
            counts_all.data_ptr(), count_flags.data_ptr(), int(epoch), world, experts, rank,
            bufs["dest_offset"].data_ptr(), bufs["segment_sizes"].data_ptr(), bufs["fill"].data_ptr(),
            bufs["totals"].data_ptr(), bufs["phase_done"].data_ptr(), bufs["send_start"].data_ptr(),
            bufs["list_fill"].data_ptr(), workspace.data_ptr(), int(wait_limit_ms), _stream_ptr(dev))
    _lib.check(rc, "rd_ep_plan_ring_when_counted")
    return bufs


def ep_assign(routing: torch.Tensor, num_experts: int, world: int, rank: int, plan: dict, capacity_rows: int,
              dest_pos: torch.Tensor, send_index: torch.Tensor) -> None:
    """``rd_ep_assign``: positions at the owners (dest_pos) and the per-phase send lists."""
    lib = _lib.load()
    assert routing.dtype == torch.int32 and routing.is_contiguous() and routing.is_cuda
    entries = routing.numel()
    assert dest_pos.numel() >= entries and send_index.numel() >= entries
    with torch.cuda.device(routing.device):
        rc = lib.rd_ep_assign(routing.data_ptr(), entries, num_experts, world, rank, plan["dest_offset"].data_ptr(),
                              plan["fill"].data_ptr(), capacity_rows, dest_pos.data_ptr(),
                              plan["send_start"].data_ptr(), plan["list_fill"].data_ptr(), send_index.data_ptr(),
                              _stream_ptr(routing.device))
    _lib.check(rc, "rd_ep_assign")


def ep_send_list(x: torch.Tensor, top_k: int, send_index: torch.Tensor, plan: dict, phase: int, world: int,
                 dest_pos: torch.Tensor, dest_base: int, capacity_rows: int, dest_ready_flag: int, epoch: int) -> None:
    """``rd_ep_send_list``: copy one phase's rows with an ordinary kernel and raise the flag."""
    lib = _lib.load()
    assert x.is_contiguous() and x.is_cuda
    with torch.cuda.device(x.device):
        rc = lib.rd_ep_send_list(x.data_ptr(), top_k, x.shape[1] * x.element_size(), send_index.data_ptr(),
                                 plan["send_start"].data_ptr(), phase, world, send_index.numel(), dest_pos.data_ptr(),
                                 dest_base, capacity_rows, plan["phase_done"].data_ptr(), dest_ready_flag, epoch,
                                 _stream_ptr(x.device))
    _lib.check(rc, "rd_ep_send_list")


def gmm_ep_fused(recv: torch.Tensor, A: torch.Tensor, segment_sizes: torch.Tensor, group_to_weight: torch.Tensor,
                 out: torch.Tensor, workspace: torch.Tensor, flags: torch.Tensor, groups_per_flag: int, epoch: int,
                 send: "_lib.EpSend", cfg: Optional[_lib.TileCfg] = None) -> torch.Tensor:
    """``rd_gmm_ep_fused``: the flag-gated local ragged_dot over the receive buffer, with the last
    ``send.sender_ctas`` CTAs of the same launch sending this rank's rows to the other ranks."""
    lib = _lib.load()
    m, k = recv.shape
    g = segment_sizes.numel()
    n = A.shape[-1]
    assert recv.is_contiguous() and A.is_contiguous() and out.shape == (m, n) and out.is_contiguous()
    assert k % 8 == 0 and n % 8 == 0 and recv.dtype == A.dtype == out.dtype
    with torch.cuda.device(recv.device):
        rc = lib.rd_gmm_ep_fused(
            recv.data_ptr(), A.data_ptr(), A.shape[0], segment_sizes.data_ptr(), group_to_weight.data_ptr(),
            out.data_ptr(), workspace.data_ptr(), workspace.numel(), m, k, n, g, 0, _DTYPE_CODE[recv.dtype],
            _cfg_ptr(cfg), flags.data_ptr(), int(groups_per_flag), int(epoch), ctypes.byref(send),
            _stream_ptr(recv.device))
    _lib.check(rc, "rd_gmm_ep_fused")
    _maybe_check_status(workspace, "rd_gmm_ep_fused")
    return out


def ep_fused_forward(step: "_lib.EpStep", recv: torch.Tensor, A: torch.Tensor, group_to_weight: torch.Tensor,
                     out: torch.Tensor, workspace: torch.Tensor, capacity_rows: int, flags: torch.Tensor,
                     send: "_lib.EpSend", cfg: Optional[_lib.TileCfg] = None) -> torch.Tensor:
    """``rd_ep_fused_forward``: count + share, plan, assign, own-row copy and the fused send + GEMM
    kernel of one expert-parallel forward step, enqueued by one C call."""
    lib = _lib.load()
    k, n = recv.shape[1], A.shape[-1]
    with torch.cuda.device(recv.device):
        rc = lib.rd_ep_fused_forward(
            ctypes.byref(step), recv.data_ptr(), A.data_ptr(), A.shape[0], group_to_weight.data_ptr(),
            out.data_ptr(), workspace.data_ptr(), workspace.numel(), int(capacity_rows), k, n,
            _DTYPE_CODE[recv.dtype], _cfg_ptr(cfg), flags.data_ptr(), ctypes.byref(send), _stream_ptr(recv.device))
    _lib.check(rc, "rd_ep_fused_forward")
    _maybe_check_status(workspace, "rd_ep_fused_forward")
    return out


def tgmm_forward(
    x: torch.Tensor,
    y: torch.Tensor,
    group_sizes: torch.Tensor,
    cfg: Optional[_lib.TileCfg] = None,
    out: Optional[torch.Tensor] = None,
    workspace: Optional[torch.Tensor] = None,
    seg_count: int = 1,
) -> torch.Tensor:
    """One call of ``rd_tgmm``: out[g,k,n] = x_g^T . y_g over each group's rows.

    With ``seg_count > 1`` it is ``rd_tgmm_strided``: ``group_sizes`` has ``g * seg_count`` entries
    and block i sums the groups i, i + g, i + 2g, ... (the expert-parallel receive layout)."""
    lib = _lib.load()
    _require_cuda(x, "x")
    _require_cuda(y, "y")
    assert y.dim() == 2 and x.dim() == 2 and x.shape[0] == y.shape[0]
    gs = _as_i32(group_sizes)
    if x.dtype not in _DTYPE_CODE or y.dtype != x.dtype:
        raise NotImplementedError(f"inputs must both be float16, bfloat16 or float32, got {x.dtype} / {y.dtype}")
    (m, k), n = x.shape, y.shape[-1]
    assert seg_count >= 1 and gs.numel() % seg_count == 0
    g = gs.numel() // seg_count
    mult = 16 // x.element_size()
    xp = _dense16(_pad_last(x, mult))
    yp = _dense16(_pad_last(y, mult))
    kp, np_ = xp.shape[1], yp.shape[1]
    padded = (kp != k) or (np_ != n)
    if out is not None and not padded:
        assert out.shape == (g, k, n) and out.dtype == x.dtype and out.is_contiguous()
        res = out
    else:
        res = torch.empty((g, kp, np_), dtype=x.dtype, device=x.device)
    ws = workspace if workspace is not None else _workspace(m, gs.numel(), x.device)
    if cfg is None and seg_count == 1 and x.dtype != torch.float32:
        cfg = tile_table.lookup("tgmm", m, kp, np_, g)
    with torch.cuda.device(x.device):
        if seg_count == 1:
            rc = lib.rd_tgmm(
                xp.data_ptr(), yp.data_ptr(), gs.data_ptr(), res.data_ptr(), ws.data_ptr(), ws.numel(),
                m, kp, np_, g, _DTYPE_CODE[x.dtype], _cfg_ptr(cfg), _stream_ptr(x.device),
            )
        else:
            rc = lib.rd_tgmm_strided(
                xp.data_ptr(), yp.data_ptr(), gs.data_ptr(), res.data_ptr(), ws.data_ptr(), ws.numel(),
                m, kp, np_, g, int(seg_count), _DTYPE_CODE[x.dtype], _cfg_ptr(cfg), _stream_ptr(x.device),
            )
    _lib.check(rc, "rd_tgmm")
    _maybe_check_status(ws, "rd_tgmm")
    if padded:
        res = res[:, :k, :n].contiguous()
        if out is not None:
            out.copy_(res)
            res = out
    return res


def ep_combine_pull(routing: torch.Tensor, dest_pos: torch.Tensor, num_experts: int, world: int,
                    peer_base: torch.Tensor, capacity_rows: int, k: int, dtype: torch.dtype,
                    out: Optional[torch.Tensor] = None, max_blocks: int = 0) -> torch.Tensor:
    """``rd_ep_combine_pull``: out[t] = sum over the top_k slots of the gradient rows the owners
    hold at ``dest_pos``; ``peer_base`` is an int64 device tensor of `world` buffer addresses."""
    lib = _lib.load()
    tokens, top_k = routing.shape
    r = _as_i32(routing.reshape(-1))
    pos = _as_i32(dest_pos.reshape(-1))
    assert pos.numel() == tokens * top_k
    assert peer_base.dtype == torch.int64 and peer_base.numel() == world and peer_base.is_cuda
    if out is None:
        out = torch.empty((tokens, k), dtype=dtype, device=r.device)
    assert out.shape == (tokens, k) and out.dtype == dtype and out.is_contiguous()
    with torch.cuda.device(r.device):
        rc = lib.rd_ep_combine_pull(r.data_ptr(), pos.data_ptr(), tokens, top_k, k * out.element_size(),
                                    num_experts, world, peer_base.data_ptr(), capacity_rows,
                                    _DTYPE_CODE[dtype], out.data_ptr(), int(max_blocks), _stream_ptr(r.device))
    _lib.check(rc, "rd_ep_combine_pull")
    return out


def gmm_permuted_forward(
    x: torch.Tensor,
    A: torch.Tensor,
    group_sizes: torch.Tensor,
    in_rows: Optional[torch.Tensor] = None,
    out_rows: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    y_rows: Optional[int] = None,
    m: Optional[int] = None,
    trans_rhs: bool = False,
    cfg: Optional[_lib.TileCfg] = None,
    workspace: Optional[torch.Tensor] = None,
    group_to_weight: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """One call of ``rd_gmm_permuted``: for sorted row r < sum(group_sizes),
    ``y[out_rows[r]] = x[in_rows[r]] @ A[group of r]``, with the gather and the scatter done
    inside the GEMM kernel (TMA row gathers in the loader, indexed row stores in the epilogue).

    ``m`` is the number of sorted rows (default: len(in_rows), else len(out_rows), else x rows).
    With ``out_rows`` the result has ``y_rows`` rows (default m) and rows that no sorted row names
    keep the content of ``out`` (zeros when ``out`` is not given)."""
    lib = _lib.load()
    _require_cuda(x, "x")
    _require_cuda(A, "A")
    assert A.dim() == 3 and x.dim() == 2
    if x.dtype not in (torch.float16, torch.bfloat16) or A.dtype != x.dtype:
        raise NotImplementedError(f"inputs must both be float16 or bfloat16, got {x.dtype} / {A.dtype}")
    gs = _as_i32(group_sizes)
    g = gs.shape[0]
    if group_to_weight is None:
        assert A.shape[0] == g, f"{A.shape[0]=} != {g=}"
    else:
        group_to_weight = _as_i32(group_to_weight)
        assert group_to_weight.shape == gs.shape
    if in_rows is not None:
        in_rows = _as_i32(in_rows)
    if out_rows is not None:
        out_rows = _as_i32(out_rows)
    if m is None:
        m = in_rows.numel() if in_rows is not None else (out_rows.numel() if out_rows is not None else x.shape[0])
    assert in_rows is None or in_rows.numel() >= m
    assert out_rows is None or out_rows.numel() >= m
    x_rows, k = x.shape
    n = A.shape[-1] if not trans_rhs else A.shape[-2]
    k_rhs = A.shape[-2] if not trans_rhs else A.shape[-1]
    assert k_rhs == k, f"contraction mismatch: x has k={k}, A has {k_rhs}"
    if out_rows is None:
        y_rows = m
    elif y_rows is None:
        y_rows = out.shape[0] if out is not None else m

    xp = _dense16(_pad_last(x, 8))
    Ap = _dense16(_pad_last2(A, 8))
    kp = xp.shape[1]
    np_ = Ap.shape[-1] if not trans_rhs else Ap.shape[-2]
    padded_n = np_ != n
    if out is not None and not padded_n:
        assert out.shape == (y_rows, n) and out.dtype == x.dtype and out.is_contiguous()
        y = out
    elif out_rows is not None:
        y = torch.zeros((y_rows, np_), dtype=x.dtype, device=x.device)
        if out is not None:
            y[:, :n] = out
    else:
        y = torch.empty((y_rows, np_), dtype=x.dtype, device=x.device)
    ws = workspace if workspace is not None else _workspace(m, g, x.device)
    with torch.cuda.device(x.device):
        rc = lib.rd_gmm_permuted(
            xp.data_ptr(), x_rows, in_rows.data_ptr() if in_rows is not None else None,
            Ap.data_ptr(), Ap.shape[0], gs.data_ptr(),
            group_to_weight.data_ptr() if group_to_weight is not None else None,
            y.data_ptr(), y_rows, out_rows.data_ptr() if out_rows is not None else None,
            ws.data_ptr(), ws.numel(), m, kp, np_, g, int(bool(trans_rhs)), _DTYPE_CODE[x.dtype],
            _cfg_ptr(cfg), _stream_ptr(x.device),
        )
    _lib.check(rc, "rd_gmm_permuted")
    if padded_n:
        y = y[:, :n].contiguous()
        if out is not None:
            out.copy_(y)
            y = out
    return y


def tgmm_permuted_forward(
    x: torch.Tensor,
    y: torch.Tensor,
    group_sizes: torch.Tensor,
    x_rows_index: Optional[torch.Tensor] = None,
    y_rows_index: Optional[torch.Tensor] = None,
    m: Optional[int] = None,
    cfg: Optional[_lib.TileCfg] = None,
    out: Optional[torch.Tensor] = None,
    workspace: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """One call of ``rd_tgmm_permuted``: out[i] = x[x_rows_index[rows of group i]]^T .
    y[y_rows_index[rows of group i]], both gathers done by the kernel's loader."""
    lib = _lib.load()
    _require_cuda(x, "x")
    _require_cuda(y, "y")
    assert y.dim() == 2 and x.dim() == 2
    if x.dtype not in (torch.float16, torch.bfloat16) or y.dtype != x.dtype:
        raise NotImplementedError(f"inputs must both be float16 or bfloat16, got {x.dtype} / {y.dtype}")
    gs = _as_i32(group_sizes)
    g = gs.numel()
    if x_rows_index is not None:
        x_rows_index = _as_i32(x_rows_index)
    if y_rows_index is not None:
        y_rows_index = _as_i32(y_rows_index)
    if m is None:
        m = (x_rows_index.numel() if x_rows_index is not None
             else (y_rows_index.numel() if y_rows_index is not None else x.shape[0]))
    k, n = x.shape[1], y.shape[1]
    xp = _dense16(_pad_last(x, 8))
    yp = _dense16(_pad_last(y, 8))
    kp, np_ = xp.shape[1], yp.shape[1]
    padded = (kp != k) or (np_ != n)
    if out is not None and not padded:
        assert out.shape == (g, k, n) and out.dtype == x.dtype and out.is_contiguous()
        res = out
    else:
        res = torch.empty((g, kp, np_), dtype=x.dtype, device=x.device)
    ws = workspace if workspace is not None else _workspace(m, g, x.device)
    with torch.cuda.device(x.device):
        rc = lib.rd_tgmm_permuted(
            xp.data_ptr(), xp.shape[0], x_rows_index.data_ptr() if x_rows_index is not None else None,
            yp.data_ptr(), yp.shape[0], y_rows_index.data_ptr() if y_rows_index is not None else None,
            gs.data_ptr(), res.data_ptr(), ws.data_ptr(), ws.numel(), m, kp, np_, g,
            _DTYPE_CODE[x.dtype], _cfg_ptr(cfg), _stream_ptr(x.device),
        )
    _lib.check(rc, "rd_tgmm_permuted")
    if padded:
        res = res[:, :k, :n].contiguous()
        if out is not None:
            out.copy_(res)
            res = out
    return res


def _fused_permute_pays(m: int, g: int, scatter: bool) -> bool:
    """Measured on B200: the fused kernel (cp.async row gathers feeding 128-row tiles) beats
    gather_rows + the TMA-fed kernels only when it also saves the scatter pass over y and the
    groups are long enough to be compute-bound (Mixtral-like shapes: +5 %); on short groups and
    for gather-only calls the TMA-fed two-pass route is 2-6 % faster."""
    return scatter and g > 0 and m // g >= 512


def _gmm_permuted_two_pass(x, A, gs, in_rows, out_rows, y_rows, m, trans_rhs):
    xs = x if in_rows is None else gather_rows(x, in_rows[:m].clamp(0, x.shape[0] - 1))
    if xs.shape[0] != m:
        xs = xs[:m] if xs.shape[0] > m else torch.nn.functional.pad(xs, (0, 0, 0, m - xs.shape[0]))
    ys = gmm_forward(xs.contiguous(), A, gs, trans_rhs=trans_rhs)
    if out_rows is None:
        return ys
    # Only the rows below sum(group_sizes) have a destination; the others are parked on an extra
    # row that is dropped (no host read of group_sizes).
    live = torch.arange(m, device=x.device) < gs.sum()
    dest = torch.where(live & (out_rows[:m] >= 0) & (out_rows[:m] < y_rows), out_rows[:m].long(),
                       torch.full((), y_rows, dtype=torch.long, device=x.device))
    y = torch.zeros((y_rows + 1, ys.shape[1]), dtype=ys.dtype, device=x.device)
    y.index_copy_(0, dest, ys)
    return y[:y_rows]


class _GmmPermutedFn(torch.autograd.Function):
    """y = scatter(gmm(gather(x))) and its backward pass: dx_sorted = gmm(dy gathered by
    out_rows, A transposed), summed into x's rows; dA = tgmm(x gathered by in_rows, dy gathered
    by out_rows).  `fused` selects the permutation-fused kernels or gather_rows + the plain ones."""

    @staticmethod
    def forward(ctx, x, A, group_sizes, in_rows, out_rows, y_rows, m, trans_rhs, fused):
        ctx.save_for_backward(x, A, group_sizes, in_rows, out_rows)
        ctx.m, ctx.trans_rhs, ctx.fused = m, trans_rhs, fused
        g = group_sizes.numel()
        use_fused = fused if fused is not None else _fused_permute_pays(m, g, out_rows is not None)
        if use_fused:
            return gmm_permuted_forward(x, A, group_sizes, in_rows=in_rows, out_rows=out_rows, y_rows=y_rows,
                                        m=m, trans_rhs=trans_rhs)
        return _gmm_permuted_two_pass(x, A, _as_i32(group_sizes), in_rows, out_rows, y_rows, m, trans_rhs)

    @staticmethod
    def backward(ctx, dy):
        x, A, gs, in_rows, out_rows = ctx.saved_tensors
        m, trans_rhs, fused = ctx.m, ctx.trans_rhs, ctx.fused
        dy = dy.contiguous()
        dx = dA = None
        # Gather-only calls: the TMA-fed kernels after gather_rows are the faster route unless
        # the caller forces the fused kernels.
        use_fused = bool(fused)
        dys = None
        if not use_fused:
            dys = dy if out_rows is None else gather_rows(dy, out_rows[:m].clamp(0, dy.shape[0] - 1))
        if ctx.needs_input_grad[0]:
            if use_fused:
                dxs = gmm_permuted_forward(dy, A, gs, in_rows=out_rows, m=m, trans_rhs=not trans_rhs)
            else:
                dxs = gmm_forward(dys, A, gs, trans_rhs=not trans_rhs)
            if in_rows is None:
                dx = dxs[: x.shape[0]] if dxs.shape[0] >= x.shape[0] else torch.nn.functional.pad(
                    dxs, (0, 0, 0, x.shape[0] - dxs.shape[0]))
            else:  # a token row may feed several sorted rows (top-k routing): sum them in fp32
                idx = in_rows[:m].long().clamp_(0, x.shape[0] - 1)
                dx = torch.zeros(x.shape, dtype=torch.float32, device=x.device).index_add_(0, idx, dxs.float())
                dx = dx.to(x.dtype)
        if ctx.needs_input_grad[1]:
            if use_fused:
                if not trans_rhs:
                    dA = tgmm_permuted_forward(x, dy, gs, x_rows_index=in_rows, y_rows_index=out_rows, m=m)
                else:
                    dA = tgmm_permuted_forward(dy, x, gs, x_rows_index=out_rows, y_rows_index=in_rows, m=m)
            else:
                xs = x if in_rows is None else gather_rows(x, in_rows[:m].clamp(0, x.shape[0] - 1))
                dA = tgmm_forward(xs, dys, gs) if not trans_rhs else tgmm_forward(dys, xs, gs)
        return dx, dA, None, None, None, None, None, None, None


def ragged_dot_permuted(x, A, group_sizes, in_rows=None, out_rows=None, y_rows=None, m=None,
                        trans_rhs=False, fused=None):
    """``ragged_dot`` on un-sorted rows: ``y[out_rows[r]] = x[in_rows[r]] @ A[group of r]`` for the
    sorted rows r < sum(group_sizes), zeros elsewhere; differentiable in x and A.  This is what an
    MoE layer does around the reference's ``ragged_dot`` (gpu_ragged_dot.py:362) with
    ``x[sorted_token_idx]`` before and the inverse permutation after.

    ``fused=True`` runs the permutation-fused kernels (``rd_gmm_permuted`` / ``rd_tgmm_permuted``:
    the sorted copies never exist), ``False`` gathers rows first and calls the plain kernels,
    ``None`` picks by the measured rule in ``_fused_permute_pays``."""
    if m is None:
        m = in_rows.numel() if in_rows is not None else (out_rows.numel() if out_rows is not None else x.shape[0])
    if in_rows is not None:
        in_rows = _as_i32(in_rows)
    if out_rows is not None:
        out_rows = _as_i32(out_rows)
        if y_rows is None:
            y_rows = m
    return _GmmPermutedFn.apply(x, A, group_sizes, in_rows, out_rows, y_rows, m, trans_rhs, fused)


def _check_static_args(x, interpret, compute_dtype, acc_dtype):
    """Returns the torch dtype the product is computed in (None: the inputs' own)."""
    if interpret:
        raise NotImplementedError(
            "interpret=True is not supported: this build has no CPU path (CUDA sm_100a only)"
        )
    if acc_dtype is not None and _torch_dtype(acc_dtype) != torch.float32:
        raise NotImplementedError(f"acc_dtype={acc_dtype}: only float32 accumulation is implemented")
    if compute_dtype is None:
        return None
    cd = _torch_dtype(compute_dtype)
    if cd not in _DTYPE_CODE:
        raise NotImplementedError(f"compute_dtype={compute_dtype}: float16, bfloat16 or float32")
    return cd


def _check_precision(precision):
    if precision not in (None, "default", "highest"):
        raise NotImplementedError(f"precision={precision!r}: None / 'default' (one TF32 pass for float32) or 'highest'")


def _torch_dtype(d):
    if isinstance(d, torch.dtype):
        return d
    name = getattr(d, "name", None) or getattr(d, "__name__", None) or str(d)
    table = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16,
             "float64": torch.float64}
    if name in table:
        return table[name]
    raise NotImplementedError(f"unknown dtype {d!r}")


def _gmm_cast(x, A, group_sizes, trans_rhs, compute_dtype, precision):
    """The reference's cast -> dot -> cast (gpu_ragged_dot.py:116,145,149): both operands go to
    ``compute_dtype`` (default: x's type), the product is accumulated in fp32, the result comes
    back in x's type."""
    cd = compute_dtype or x.dtype
    if cd == torch.float32 and precision == "highest":
        y = _gmm_3xtf32(x.to(cd), A.to(cd), group_sizes, trans_rhs)
    else:
        y = gmm_forward(x.to(cd), A.to(cd), group_sizes, trans_rhs=trans_rhs)
    return y.to(x.dtype)


def _tgmm_cast(x, y, group_sizes, compute_dtype, precision):
    cd = compute_dtype or x.dtype
    if cd == torch.float32 and precision == "highest":
        out = _tgmm_3xtf32(x.to(cd), y.to(cd), group_sizes)
    else:
        out = tgmm_forward(x.to(cd), y.to(cd), group_sizes)
    return out.to(x.dtype)


def _split_tf32(t: torch.Tensor):
    """t = hi + lo exactly, hi holding the top 10 explicit mantissa bits rounded to nearest (a
    value the tensor cores read without loss) and lo the remainder."""
    bits = t.contiguous().view(torch.int32)
    hi = ((bits + 0x1000) & ~0x1FFF).view(torch.float32)
    hi = torch.where(torch.isfinite(hi), hi, t)  # rounding up the largest finite values would overflow
    return hi, t - hi


def _gmm_3xtf32(x, A, group_sizes, trans_rhs):
    """float32 product to nearly fp32 accuracy on the TF32 tensor cores: with x = xh + xl and
    A = Ah + Al (TF32 head + remainder), x.A ~ xh.Ah + xh.Al + xl.Ah; the dropped xl.Al term is
    2^-22 relative.  Three passes of the TF32 kernel, summed in fp32, small terms first."""
    xh, xl = _split_tf32(x)
    Ah, Al = _split_tf32(A)
    ws = _workspace(x.shape[0], _as_i32(group_sizes).numel(), x.device)
    y = gmm_forward(xl, Ah, group_sizes, trans_rhs=trans_rhs, workspace=ws)
    y += gmm_forward(xh, Al, group_sizes, trans_rhs=trans_rhs, workspace=ws)
    y += gmm_forward(xh, Ah, group_sizes, trans_rhs=trans_rhs, workspace=ws)
    return y


def _tgmm_3xtf32(x, y, group_sizes):
    xh, xl = _split_tf32(x)
    yh, yl = _split_tf32(y)
    ws = _workspace(x.shape[0], _as_i32(group_sizes).numel(), x.device)
    out = tgmm_forward(xl, yh, group_sizes, workspace=ws)
    out += tgmm_forward(xh, yl, group_sizes, workspace=ws)
    out += tgmm_forward(xh, yh, group_sizes, workspace=ws)
    return out


class _GmmFn(torch.autograd.Function):
    """custom_vjp of gmm: gpu_ragged_dot.py:383-405.  compute_dtype travels to the backward
    products as in the reference (its ``kw`` dict, :395-401)."""

    @staticmethod
    def forward(ctx, x, A, group_sizes, trans_rhs, compute_dtype, precision):
        ctx.trans_rhs, ctx.compute_dtype, ctx.precision = trans_rhs, compute_dtype, precision
        ctx.save_for_backward(x, A, group_sizes)  # residuals (x, A, group_sizes), reference :227
        return _gmm_cast(x, A, group_sizes, trans_rhs, compute_dtype, precision)

    @staticmethod
    def backward(ctx, do):
        x, A, group_sizes = ctx.saved_tensors
        cd, pr = ctx.compute_dtype, ctx.precision
        do = do.contiguous()
        dx = dA = None
        if ctx.needs_input_grad[0]:
            dx = _gmm_cast(do, A, group_sizes, not ctx.trans_rhs, cd, pr).to(x.dtype)
        if ctx.needs_input_grad[1]:
            dA = (
                _tgmm_cast(x, do, group_sizes, cd, pr)
                if not ctx.trans_rhs
                else _tgmm_cast(do, x, group_sizes, cd, pr)
            ).to(A.dtype)
        return dx, dA, None, None, None, None


class _TgmmFn(torch.autograd.Function):
    """VJP of tgmm.  out[g] = x_g^T y_g  =>  dx_g = y_g dout[g]^T,  dy_g = x_g dout[g]."""

    @staticmethod
    def forward(ctx, x, y, group_sizes, compute_dtype, precision):
        ctx.compute_dtype, ctx.precision = compute_dtype, precision
        ctx.save_for_backward(x, y, group_sizes)
        return _tgmm_cast(x, y, group_sizes, compute_dtype, precision)

    @staticmethod
    def backward(ctx, do):
        x, y, group_sizes = ctx.saved_tensors
        cd, pr = ctx.compute_dtype, ctx.precision
        do = do.contiguous()
        dx = dy = None
        if ctx.needs_input_grad[0]:
            dx = _gmm_cast(y, do, group_sizes, True, cd, pr).to(x.dtype)
        if ctx.needs_input_grad[1]:
            dy = _gmm_cast(x, do, group_sizes, False, cd, pr).to(y.dtype)
        return dx, dy, None, None, None


def gmm(
    x: torch.Tensor,  # [m, k]
    A: torch.Tensor,  # [g, k, n]
    group_sizes: torch.Tensor,  # [g]
    block_m: int = DEFAULT_BLOCK_M,
    block_k: int = DEFAULT_BLOCK_K,
    block_n: int = DEFAULT_BLOCK_N,
    trans_rhs: bool = False,
    interpret: bool = False,
    compute_dtype=None,
    acc_dtype=torch.float32,
    num_warps: Optional[int] = None,
    num_stages: Optional[int] = None,
    chunk_m: int = CHUNK_M,
    *,
    precision: Optional[str] = None,
) -> torch.Tensor:
    """Ragged dot corresponding to jax.lax.ragged_dot: (m, k) x (g, k, n) -> (m, n).

    Signature of the reference's ``gmm`` (gpu_ragged_dot.py:362-376) plus ``precision``:
    ``"highest"`` computes a float32 product to nearly fp32 accuracy (three TF32 passes); the
    default is one TF32 pass, the precision the reference's kernel and jax.lax.ragged_dot have
    for float32 on NVIDIA GPUs."""
    del block_m, block_k, block_n, num_warps, num_stages, chunk_m  # hints; the tile table decides
    cd = _check_static_args(x, interpret, compute_dtype, acc_dtype)
    _check_precision(precision)
    return _GmmFn.apply(x, A, group_sizes, bool(trans_rhs), cd, precision)


def tgmm(
    x: torch.Tensor,  # [m, k]
    y: torch.Tensor,  # [m, n]
    group_sizes: torch.Tensor,  # [g]
    block_m: int = DEFAULT_BLOCK_M,
    block_k: int = DEFAULT_BLOCK_K,
    block_n: int = DEFAULT_BLOCK_N,
    interpret: bool = False,
    compute_dtype=None,
    acc_dtype=torch.float32,
    num_warps: Optional[int] = None,
    num_stages: Optional[int] = None,
    chunk_m: int = CHUNK_M,
    *,
    precision: Optional[str] = None,
) -> torch.Tensor:
    """Transposed ragged dot: (m, k) x (m, n) -> (g, k, n).

    Signature of the reference's ``tgmm`` (gpu_ragged_dot.py:411-424) plus ``precision`` (see gmm)."""
    del block_m, block_k, block_n, num_warps, num_stages, chunk_m
    cd = _check_static_args(x, interpret, compute_dtype, acc_dtype)
    _check_precision(precision)
    return _TgmmFn.apply(x, y, group_sizes, cd, precision)


ragged_dot = gmm
trans_ragged_dot = tgmm


class RaggedDotDimensionNumbers(NamedTuple):
    """Same fields as ``jax.lax.RaggedDotDimensionNumbers``, the argument of the op the reference
    is tested against (tests.py:31-36): ``dot_dimension_numbers`` is
    ``((lhs_contracting, rhs_contracting), (lhs_batch, rhs_batch))``."""

    dot_dimension_numbers: tuple
    lhs_ragged_dimensions: Sequence[int]
    rhs_group_dimensions: Sequence[int]


def ragged_dot_general(lhs: torch.Tensor, rhs: torch.Tensor, group_sizes: torch.Tensor,
                       ragged_dot_dimension_numbers: RaggedDotDimensionNumbers, **kwargs) -> torch.Tensor:
    """``jax.lax.ragged_dot_general`` over the grouped GEMMs of this library.  The reference
    implements the first two modes without batch dimensions (its tests spell them as dimension
    numbers, tests.py:31-48); the third mode and one batch dimension are added here.

    With g groups, one contracting dimension and at most one batch dimension b on each side:

    * ragged non-contracting dimension -- lhs ``[m, k]`` / ``[b, m, k]`` ragged in m, rhs with one
      group dimension ``[g, k, n]`` (``[g, n, k]`` when its contracting dimension comes last), with a
      batch dimension in any position, group_sizes ``[g]`` / ``[b, g]``  ->  ``[m, n]`` / ``[b, m, n]``
      (``gmm`` per batch element);
    * ragged contracting dimension -- lhs ``[m, k]`` / ``[b, m, k]`` and rhs ``[m, n]`` / ``[b, m, n]``
      contracted over m, the ragged one, no rhs group dimension  ->  ``[g, k, n]`` / ``[g, b, k, n]``
      (``tgmm`` per batch element; the group dimension leads, as in jax);
    * ragged batch dimension -- lhs ``[b, m, k]``, rhs ``[b, k, n]``, group_sizes ``[g]`` partitioning
      b  ->  ``[b, m, n]``: every batch element is its own product, elements past
      ``sum(group_sizes)`` are zero (one ``gmm`` with b groups of m rows).

    Anything else (several contracting or batch dimensions, extra free dimensions, a group offset)
    raises ``NotImplementedError``.  ``kwargs`` are passed on (``block_*`` hints and so on)."""
    dn = ragged_dot_dimension_numbers
    (lhs_c, rhs_c), (lhs_b, rhs_b) = dn.dot_dimension_numbers
    lhs_c, rhs_c = [int(d) for d in lhs_c], [int(d) for d in rhs_c]
    lhs_b, rhs_b = [int(d) for d in lhs_b], [int(d) for d in rhs_b]
    ragged = [int(d) for d in dn.lhs_ragged_dimensions]
    groups = [int(d) for d in dn.rhs_group_dimensions]

    def bad(why):
        return NotImplementedError(
            f"ragged_dot_general: {why} (dimension numbers {dn}, shapes {tuple(lhs.shape)}, {tuple(rhs.shape)})")

    if len(lhs_c) != 1 or len(rhs_c) != 1 or len(ragged) != 1:
        raise bad("exactly one contracting and one ragged dimension are supported")
    if len(lhs_b) != len(rhs_b) or len(lhs_b) > 1:
        raise bad("at most one batch dimension on each side is supported")
    if len(groups) > 1:
        raise bad("at most one rhs group dimension")
    nb = len(lhs_b)
    if lhs.dim() != 2 + nb:
        raise bad("lhs must be [m, k] or [b, m, k] up to the order of its dimensions")
    if len(set(lhs_c + lhs_b)) != 1 + nb or len(set(rhs_c + rhs_b + groups)) != 1 + nb + len(groups):
        raise bad("a dimension is named twice")
    rg, lc = ragged[0], lhs_c[0]

    # ---- ragged batch dimension
    if nb == 1 and rg == lhs_b[0]:
        if groups or rhs.dim() != 3:
            raise bad("the ragged-batch mode takes an rhs [b, k, n] without a group dimension")
        m_dim = ({0, 1, 2} - {lhs_b[0], lc}).pop()
        n_dim = ({0, 1, 2} - {rhs_b[0], rhs_c[0]}).pop()
        x = lhs.permute(lhs_b[0], m_dim, lc).contiguous()          # [b, m, k]
        w = rhs.permute(rhs_b[0], rhs_c[0], n_dim).contiguous()    # [b, k, n]
        b, m, k = x.shape
        if w.shape[0] != b or w.shape[1] != k:
            raise bad("batch / contracting sizes of lhs and rhs differ")
        gs = _as_i32(group_sizes)
        live = torch.clamp(gs.sum(), max=b)                       # batch elements that belong to a group
        per_batch = torch.where(torch.arange(b, device=x.device) < live, m, 0).to(torch.int32)
        return gmm(x.reshape(b * m, k), w, per_batch, **kwargs).reshape(b, m, w.shape[2])

    # ---- ragged non-contracting dimension (gmm)
    if rg != lc and len(groups) == 1:
        if rhs.dim() != 3 + nb:
            raise bad("rhs must have a group, a contracting and a free dimension (and the batch dimension)")
        free = (set(range(rhs.dim())) - {groups[0], rhs_c[0]} - set(rhs_b)).pop()
        trans = rhs_c[0] > free  # rhs stored [.., n, k]: use the transposed-rhs kernel, no copy of the weights
        order = rhs_b + [groups[0]] + ([free, rhs_c[0]] if trans else [rhs_c[0], free])
        w = rhs.permute(*order)
        x = lhs.permute(*(lhs_b + [rg, lc]))
        if nb == 0:
            return gmm(x, w.contiguous(), group_sizes, trans_rhs=trans, **kwargs)
        gs = group_sizes
        if gs.dim() != 2 or gs.shape[0] != x.shape[0] or w.shape[0] != x.shape[0]:
            raise bad("with a batch dimension group_sizes must be [b, g] and the batch sizes must agree")
        return torch.stack([gmm(x[i].contiguous(), w[i].contiguous(), gs[i], trans_rhs=trans, **kwargs)
                            for i in range(x.shape[0])])

    # ---- ragged contracting dimension (tgmm)
    if rg == lc and not groups:
        if rhs.dim() != 2 + nb:
            raise bad("rhs must be [m, n] or [b, m, n] up to the order of its dimensions")
        k_dim = (set(range(lhs.dim())) - {lc} - set(lhs_b)).pop()
        n_dim = (set(range(rhs.dim())) - {rhs_c[0]} - set(rhs_b)).pop()
        x = lhs.permute(*(lhs_b + [lc, k_dim]))
        y = rhs.permute(*(rhs_b + [rhs_c[0], n_dim]))
        if nb == 0:
            return tgmm(x.contiguous(), y.contiguous(), group_sizes, **kwargs)
        gs = group_sizes
        if gs.dim() != 2 or gs.shape[0] != x.shape[0] or y.shape[0] != x.shape[0]:
            raise bad("with a batch dimension group_sizes must be [b, g] and the batch sizes must agree")
        return torch.stack([tgmm(x[i].contiguous(), y[i].contiguous(), gs[i], **kwargs)
                            for i in range(x.shape[0])], dim=1)  # [g, b, k, n]
    raise bad("unsupported combination of ragged, group and contracting dimensions")


def device_status(workspace: torch.Tensor) -> int:
    """Synchronise and return the status the kernels left in ``workspace`` (0 = ok)."""
    lib = _lib.load()
    with torch.cuda.device(workspace.device):
        return lib.rd_device_status(workspace.data_ptr(), _stream_ptr(workspace.device))
