"""``ragged_dot`` (forward and the custom_vjp backward) for operands that live in pinned HOST memory.

The reference's ``ragged_dot`` takes device arrays (gpu_ragged_dot.py:362-380) and its backward
is ``_gpu_gmm_bwd`` (gpu_ragged_dot.py:383-402).  A caller whose activations and expert weights
sit in host memory pays for the PCIe copies around those calls; done naively (copy everything in,
compute, copy everything out, one stream) the two directions of the link are never busy at the
same time and the GPU idles for the whole step.

``HostRaggedDot`` runs the same three GEMMs through the same C ABI (``rd_gmm`` / ``rd_tgmm``), but
expert chunk by expert chunk on three streams:

    copy-in stream :  A[c], x rows of c, dout rows of c          (host -> device)
    compute stream :  y_c = gmm, dlhs_c = gmm(trans_rhs), drhs_c = tgmm    (waits for copy-in c)
    copy-out stream:  y rows, dlhs rows, drhs[c]                  (device -> host, waits for compute c)

so chunk c+1 arrives while chunk c is multiplied and chunk c-1 leaves.  Groups are independent
GEMMs, hence a chunk of experts with its row range is a complete ``ragged_dot`` problem of its own
and the results are those of one call over all groups.  ``group_sizes`` is a host array here (the
caller holds host buffers), which is what lets the host cut the row ranges.

The device buffers are owned by the object and reused by every call; nothing is allocated per
call.  Results are in the host buffers once the current stream (which is made to wait for the last
copy-out) or the device has been synchronised.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import ops

__all__ = ["HostRaggedDot", "plan_chunks"]


def plan_chunks(sizes: List[int], experts_per_chunk: int) -> List[Tuple[int, int, int, int]]:
    """Cut ``g = len(sizes)`` experts into consecutive chunks of ``experts_per_chunk`` (the last one
    may be shorter): (first expert, end expert, first row, end row) per chunk, in order.  The row
    ranges tile ``[0, sum(sizes))`` without gaps because the rows are sorted by expert."""
    if experts_per_chunk < 1:
        raise ValueError("experts_per_chunk must be at least 1")
    out, row = [], 0
    for e0 in range(0, len(sizes), experts_per_chunk):
        e1 = min(len(sizes), e0 + experts_per_chunk)
        rows = sum(sizes[e0:e1])
        out.append((e0, e1, row, row + rows))
        row += rows
    return out


class HostRaggedDot:
    """Pipelined host-buffer ``ragged_dot`` for one problem shape ``(m, k, n, g)``.

    ``chunk_bytes`` bounds the weight bytes of one chunk (at least one expert per chunk): small
    chunks start the pipeline sooner, large chunks launch fewer kernels.  ``trans_rhs`` has the
    reference's meaning: the weights are ``[g, n, k]``."""

    def __init__(self, m: int, k: int, n: int, g: int, dtype: torch.dtype = torch.bfloat16,
                 device="cuda", backward: bool = True, trans_rhs: bool = False,
                 chunk_bytes: int = 128 << 20):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("HostRaggedDot needs a CUDA device (no CPU path)")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        esz = torch.empty((), dtype=dtype).element_size()
        if (k * esz) % 16 or (n * esz) % 16:
            raise ValueError(f"k and n must make 16-byte rows (multiples of {16 // esz}), got {k=} {n=}")
        self.m, self.k, self.n, self.g = int(m), int(k), int(n), int(g)
        self.dtype, self.backward, self.trans_rhs = dtype, bool(backward), bool(trans_rhs)
        self.experts_per_chunk = max(1, int(chunk_bytes) // max(1, k * n * esz))
        dev = self.device
        a_shape = (g, n, k) if trans_rhs else (g, k, n)
        self.d_x = torch.empty((m, k), dtype=dtype, device=dev)
        self.d_A = torch.empty(a_shape, dtype=dtype, device=dev)
        self.d_gs = torch.empty((g,), dtype=torch.int32, device=dev)
        self.d_y = torch.empty((m, n), dtype=dtype, device=dev)
        if self.backward:
            self.d_dout = torch.empty((m, n), dtype=dtype, device=dev)
            self.d_dx = torch.empty((m, k), dtype=dtype, device=dev)
            self.d_dA = torch.empty(a_shape, dtype=dtype, device=dev)
        self.workspace = ops._workspace(m, min(g, self.experts_per_chunk), dev)
        self.s_in = torch.cuda.Stream(dev)
        self.s_compute = torch.cuda.Stream(dev)
        self.s_out = torch.cuda.Stream(dev)
        self._inputs_free: Optional[torch.cuda.Event] = None   # previous call's last GEMM
        self._outputs_free: Optional[torch.cuda.Event] = None  # previous call's last copy-out

    # ------------------------------------------------------------------ helpers
    def chunks(self, sizes: List[int]) -> List[Tuple[int, int, int, int]]:
        return plan_chunks(sizes, self.experts_per_chunk)

    def _check_host(self, t: torch.Tensor, shape, name: str, dtype=None) -> None:
        if t.is_cuda:
            raise ValueError(f"{name} must be a host tensor (use ragged_dot for device tensors)")
        if tuple(t.shape) != tuple(shape) or t.dtype != (dtype or self.dtype) or not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous {tuple(shape)} {dtype or self.dtype}, got "
                             f"{tuple(t.shape)} {t.dtype}")
        if not t.is_pinned():
            raise ValueError(f"{name} must be pinned host memory (asynchronous copies need it)")

    # ------------------------------------------------------------------ the call
    def __call__(self, x: torch.Tensor, A: torch.Tensor, group_sizes: torch.Tensor,
                 dout: Optional[torch.Tensor] = None, y: Optional[torch.Tensor] = None,
                 dlhs: Optional[torch.Tensor] = None, drhs: Optional[torch.Tensor] = None):
        """Enqueue one step.  ``x[m,k]``, ``A`` and ``dout[m,n]`` are pinned host tensors,
        ``group_sizes[g]`` a host int32 tensor with ``sum <= m``; ``y``, ``dlhs``, ``drhs`` are
        pinned host outputs (allocated when missing).  Returns ``y`` for a forward-only object,
        else ``(y, dlhs, drhs)``.  Rows at and past ``sum(group_sizes)`` of ``y`` and ``dlhs`` are
        zero, as are the ``drhs`` blocks of empty groups."""
        m, k, n, g = self.m, self.k, self.n, self.g
        a_shape = tuple(self.d_A.shape)
        self._check_host(x, (m, k), "x")
        self._check_host(A, a_shape, "A")
        if group_sizes.is_cuda or group_sizes.dtype != torch.int32 or tuple(group_sizes.shape) != (g,):
            raise ValueError(f"group_sizes must be a host int32 tensor of shape ({g},)")
        sizes = [int(v) for v in group_sizes.tolist()]
        if min(sizes, default=0) < 0 or sum(sizes) > m:
            raise ValueError("group_sizes must be non-negative and sum to at most m")
        pin = lambda shape: torch.empty(shape, dtype=self.dtype).pin_memory()  # noqa: E731
        y = pin((m, n)) if y is None else y
        self._check_host(y, (m, n), "y")
        if self.backward:
            if dout is None:
                raise ValueError("this object was built with backward=True: pass dout")
            self._check_host(dout, (m, n), "dout")
            dlhs = pin((m, k)) if dlhs is None else dlhs
            drhs = pin(a_shape) if drhs is None else drhs
            self._check_host(dlhs, (m, k), "dlhs")
            self._check_host(drhs, a_shape, "drhs")

        s_in, s_cmp, s_out = self.s_in, self.s_compute, self.s_out
        # The device buffers are shared with the previous call: its GEMMs must have consumed the
        # inputs before they are overwritten, its copies-out must have read the outputs before
        # the first GEMM of this call writes them.
        if self._inputs_free is not None:
            s_in.wait_event(self._inputs_free)
        if self._outputs_free is not None:
            s_cmp.wait_event(self._outputs_free)

        with torch.cuda.stream(s_in):
            self.d_gs.copy_(group_sizes, non_blocking=True)
        total = 0
        for (e0, e1, r0, r1) in self.chunks(sizes):
            total = r1
            arrived = torch.cuda.Event()
            with torch.cuda.stream(s_in):
                self.d_A[e0:e1].copy_(A[e0:e1], non_blocking=True)
                if r1 > r0:
                    self.d_x[r0:r1].copy_(x[r0:r1], non_blocking=True)
                    if self.backward:
                        self.d_dout[r0:r1].copy_(dout[r0:r1], non_blocking=True)
                arrived.record(s_in)
            done = torch.cuda.Event()
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(arrived)
                gs_c = self.d_gs[e0:e1]
                if r1 > r0:
                    ops.gmm_forward(self.d_x[r0:r1], self.d_A[e0:e1], gs_c, trans_rhs=self.trans_rhs,
                                    out=self.d_y[r0:r1], workspace=self.workspace)
                    if self.backward:
                        ops.gmm_forward(self.d_dout[r0:r1], self.d_A[e0:e1], gs_c,
                                        trans_rhs=not self.trans_rhs, out=self.d_dx[r0:r1],
                                        workspace=self.workspace)
                        if self.trans_rhs:  # drhs is [g, n, k]: roles of x and dout swap
                            ops.tgmm_forward(self.d_dout[r0:r1], self.d_x[r0:r1], gs_c,
                                             out=self.d_dA[e0:e1], workspace=self.workspace)
                        else:
                            ops.tgmm_forward(self.d_x[r0:r1], self.d_dout[r0:r1], gs_c,
                                             out=self.d_dA[e0:e1], workspace=self.workspace)
                elif self.backward:
                    self.d_dA[e0:e1].zero_()
                done.record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                if r1 > r0:
                    y[r0:r1].copy_(self.d_y[r0:r1], non_blocking=True)
                    if self.backward:
                        dlhs[r0:r1].copy_(self.d_dx[r0:r1], non_blocking=True)
                if self.backward:
                    drhs[e0:e1].copy_(self.d_dA[e0:e1], non_blocking=True)
            self._inputs_free = done
        if total < m:  # rows no group owns: zero, like the device op (host memory, host memset)
            y[total:].zero_()
            if self.backward:
                dlhs[total:].zero_()
        self._outputs_free = torch.cuda.Event()
        self._outputs_free.record(s_out)
        torch.cuda.current_stream(self.device).wait_event(self._outputs_free)
        return (y, dlhs, drhs) if self.backward else y
