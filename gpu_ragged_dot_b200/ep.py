"""Expert-parallel ragged_dot: experts sharded g/W per GPU, token rows exchanged with an NCCL
all-to-all, then the local ragged_dot.  One process per GPU (torch.distributed).

The reference has no multi-device code; this is the sharding its hot path admits: groups are
independent GEMMs, so the only exchange is rows travelling to the rank that owns their expert.

Per step, on each rank (T tokens, top_k routing, E experts, El = E / W per rank):
  1. plan      sort the T*top_k (token, expert) pairs by expert; per-expert counts; exchange the
               counts (all-to-all of int32 [W, El]); read the 2*W split sizes on the host.
  2. permute   gather the token rows into expert order (rd_gather_rows).
  3. exchange  all_to_all_single of the rows (split sizes from the plan).  Rows land in this
               GPU's own memory, ordered (source rank, local expert).
  4. compute   rd_gmm_indexed over the W*El received segments; segment (s, e) multiplies by
               local expert e's weights.  No re-sort after the exchange.

`plan_dispatch` and `exchange_rows` use only torch + torch.distributed and run on any backend
(the CPU tests drive them over gloo); `ExpertParallelRaggedDot` adds the CUDA steps.

A second dispatch mode, ``dispatch="p2p"``, has no host round trip at all: the counts are
all-gathered (NCCL, E int32 per rank), `rd_ep_plan` turns them into write offsets on the device,
and `rd_ep_dispatch` stores every row directly into the owner's receive buffer through peer
memory (torch symmetric memory supplies the peer addresses and the cross-rank barrier).  The
receive buffer has a fixed capacity (every row of every rank could land on one rank), the
local GEMM gets that capacity as its static row bound and the true segment sizes on the device.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class DispatchPlan:
    token_index: torch.Tensor       # [T*top_k] source token of every sorted row (int32)
    send_splits: List[int]          # rows this rank sends to each rank
    recv_splits: List[int]          # rows this rank receives from each rank
    segment_sizes: torch.Tensor     # [W*El] int32: rows of (source rank s, local expert e), s-major
    segment_to_expert: torch.Tensor  # [W*El] int32: local expert of each segment
    rows_received: int


def plan_dispatch(routing: torch.Tensor, num_experts: int, group: Optional[dist.ProcessGroup] = None) -> DispatchPlan:
    """routing: [T, top_k] expert ids.  Expert e lives on rank e // (num_experts // world)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    assert num_experts % world == 0, "experts must divide evenly over ranks"
    local = num_experts // world
    top_k = routing.shape[1]
    flat = routing.reshape(-1).to(torch.int64)
    _, order = torch.sort(flat, stable=True)
    token_index = (order // top_k).to(torch.int32)
    counts = torch.bincount(flat, minlength=num_experts).to(torch.int32)  # [E]
    if world > 1:
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=group)  # [W, El]: from each source rank
    else:
        recv_counts = counts
    both = torch.stack([counts.view(world, local).sum(1), recv_counts.view(world, local).sum(1)]).cpu()
    send_splits, recv_splits = both[0].tolist(), both[1].tolist()
    seg2e = torch.arange(local, dtype=torch.int32, device=routing.device).repeat(world)
    return DispatchPlan(token_index, send_splits, recv_splits, recv_counts.contiguous(), seg2e,
                        int(sum(recv_splits)))


def exchange_rows(rows_sorted: torch.Tensor, plan: DispatchPlan, group: Optional[dist.ProcessGroup] = None,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """all-to-all of expert-sorted rows; returns [rows_received, k] ordered (source, expert)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if out is None:
        out = torch.empty((plan.rows_received, rows_sorted.shape[1]), dtype=rows_sorted.dtype,
                          device=rows_sorted.device)
    if world == 1:
        out.copy_(rows_sorted)
        return out
    dist.all_to_all_single(out, rows_sorted, output_split_sizes=plan.recv_splits,
                           input_split_sizes=plan.send_splits, group=group)
    return out


class ExpertParallelRaggedDot:
    """Holds this rank's experts' weights and runs the four steps above on its GPU."""

    def __init__(self, num_experts: int, k: int, n: int, device: torch.device, seed: int = 0,
                 dtype: torch.dtype = torch.bfloat16, group: Optional[dist.ProcessGroup] = None,
                 dispatch: str = "nccl", capacity_rows: Optional[int] = None,
                 own_blocks: int = 0, side_blocks: int = 0, sender_ctas: int = 0):
        from . import workloads

        assert dispatch in ("nccl", "p2p", "overlap", "fused")
        self.dispatch, self.capacity_rows, self._p2p = dispatch, capacity_rows, None
        self._ov, self._epoch = None, 0
        # overlap mode: grid caps of the phase kernels (0 = library default), phase 0 / the others
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        self.own_blocks, self.side_blocks = own_blocks or 8 * sms, side_blocks
        self.dtype = dtype
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        # fused mode: CTAs of the GEMM grid that send instead of multiplying.  Measured: 16 sender
        # CTAs move 600 GB/s per GPU at 2 and at 8 ranks; 8 are too few (220 GB/s), 24 are slower
        # again at 8 ranks (480 GB/s) and take more SMs from the GEMM.
        self.sender_ctas = sender_ctas or 16
        assert num_experts % self.world == 0
        self.num_experts, self.local_experts = num_experts, num_experts // self.world
        self.k, self.n, self.device = k, n, device
        self.weights = workloads.normal_tensor((self.local_experts, k, n), k ** -0.5, seed, device, dtype)
        self._events = []
        self._host = None

    def reset_timers(self):
        self._events = []

    def timers_ms(self, steps: int):
        torch.cuda.synchronize(self.device)
        tot = {"permute": 0.0, "a2a": 0.0, "gemm": 0.0}
        for e in self._events:
            tot["permute"] += e[0].elapsed_time(e[1])
            tot["a2a"] += e[1].elapsed_time(e[2])
            # overlap mode: exchange and GEMM both start when the plan is done and run together
            tot["gemm"] += (e[1] if self.dispatch in ("overlap", "fused") else e[2]).elapsed_time(e[3])
        if self.dispatch in ("overlap", "fused"):  # when the GEMM could start: own rows copied
            tot["own_rows"] = sum(e[1].elapsed_time(e[4]) for e in self._events)
        return {k: v / max(steps, 1) for k, v in tot.items()}

    # ------------------------------------------------------------------ peer-store dispatch
    def _p2p_setup(self, capacity_rows: int):
        """Allocate the receive buffer in symmetric memory and fetch every rank's address."""
        import torch.distributed._symmetric_memory as symm_mem

        buf = symm_mem.empty((capacity_rows, self.k), dtype=self.dtype, device=self.device)
        if self.world > 1:
            hdl = symm_mem.rendezvous(buf, self.group if self.group is not None else dist.group.WORLD)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
        else:
            hdl, ptrs = None, [buf.data_ptr()]
        self._p2p = {
            "buf": buf, "hdl": hdl, "capacity": capacity_rows,
            "peer_base": torch.tensor(ptrs, dtype=torch.int64, device=self.device),
            "counts_all": torch.empty((self.world, self.num_experts), dtype=torch.int32, device=self.device),
            "y": torch.empty((capacity_rows, self.n), dtype=self.dtype, device=self.device),
            "seg2e": torch.arange(self.local_experts, dtype=torch.int32, device=self.device).repeat(self.world),
        }

    def forward_p2p(self, x_tokens: torch.Tensor, routing: torch.Tensor, timed: bool = False):
        """Dispatch by peer stores + local ragged_dot, fully stream-ordered (no host sync).

        Returns (y [capacity, n], segment_sizes [W*El], dest_pos [T, top_k], totals [1]); only the
        first totals[0] rows of y are defined; dest_pos says where on its owner each row went."""
        from . import _lib, ops

        tokens, top_k = routing.shape
        if self._p2p is None:
            cap = self.capacity_rows or tokens * top_k * self.world
            self._p2p_setup(cap)
        st = self._p2p
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if timed else None
        if timed:
            ev[0].record()
        routing = routing.to(torch.int32)
        counts = ops.ep_count(routing, self.num_experts)
        if self.world > 1:
            # Also the "receive buffers are free again" barrier: it cannot complete before every
            # rank has finished the GEMM of its previous step (stream order on each rank).
            dist.all_gather_into_tensor(st["counts_all"].view(-1), counts, group=self.group)
        else:
            st["counts_all"].copy_(counts.view(1, -1))
        dest_offset, seg_sizes, fill, totals = ops.ep_plan(st["counts_all"], self.rank)
        if timed:
            ev[1].record()
        dest_pos = ops.ep_dispatch(x_tokens, routing, self.num_experts, self.world, dest_offset, fill,
                                   st["peer_base"], st["capacity"])
        if self.world > 1:
            st["hdl"].barrier(channel=0)  # every rank's rows have landed everywhere
        if timed:
            ev[2].record()
        cfg = _lib.TileCfg(0, 0, 0, 0, _lib.RD_CFG_NO_ZERO_TAIL)
        y = ops.gmm_forward(st["buf"], self.weights, seg_sizes, group_to_weight=st["seg2e"], cfg=cfg,
                            out=st["y"])
        if timed:
            ev[3].record()
            self._events.append(ev)
        return y, seg_sizes, dest_pos, totals

    # ------------------------------------------------------------------ overlapped exchange + GEMM
    def _overlap_setup(self, capacity_rows: int):
        """Receive buffer and ready flags in symmetric memory, persistent plan buffers, side stream."""
        import torch.distributed._symmetric_memory as symm_mem
        from . import ops

        dev = self.device
        buf = symm_mem.empty((capacity_rows, self.k), dtype=self.dtype, device=dev)
        flags = symm_mem.empty((max(self.world, 4),), dtype=torch.int32, device=dev)
        flags.zero_()
        if self.world > 1:
            grp = self.group if self.group is not None else dist.group.WORLD
            hb = symm_mem.rendezvous(buf, grp)
            hf = symm_mem.rendezvous(flags, grp)
            buf_ptrs, flag_ptrs = [int(p) for p in hb.buffer_ptrs], [int(p) for p in hf.buffer_ptrs]
            torch.cuda.synchronize(dev)
            hf.barrier(channel=0)  # every rank's flags are zero before anyone stores an epoch
            torch.cuda.synchronize(dev)
        else:
            hb = hf = None
            buf_ptrs, flag_ptrs = [buf.data_ptr()], [flags.data_ptr()]
        E, W = self.num_experts, self.world
        self._ov = {
            "buf": buf, "flags": flags, "handles": (hb, hf), "capacity": capacity_rows,
            "buf_ptrs": buf_ptrs, "flag_ptrs": flag_ptrs,
            "counts_all": torch.empty((W, E), dtype=torch.int32, device=dev),
            "plan": {name: torch.empty(size, dtype=torch.int32, device=dev)
                     for name, size in (("dest_offset", E), ("segment_sizes", E), ("fill", E), ("totals", 1),
                                        ("phase_done", W), ("send_start", W + 1), ("list_fill", W))},
            "y": torch.empty((capacity_rows, self.n), dtype=self.dtype, device=dev),
            "ws": ops._workspace(capacity_rows, E, dev),
            "seg2e": torch.arange(self.local_experts, dtype=torch.int32, device=dev).repeat(W),
            "side": torch.cuda.Stream(device=dev, priority=-1),
            "ev_plan": torch.cuda.Event(), "ev_done": torch.cuda.Event(),
        }

    def forward_overlap(self, x_tokens: torch.Tensor, routing: torch.Tensor, timed: bool = False):
        """Exchange and local ragged_dot running together: after the plan, the W dispatch phases go
        out on a side stream (phase p sends to rank+p and raises flag p there) while the GEMM,
        launched at once on the main stream, multiplies position q as soon as flag q is up.

        Returns (y [capacity, n], segment_sizes [W*El] in position order, dest_pos [T, top_k], totals)."""
        from . import _lib, ops

        tokens, top_k = routing.shape
        if self._ov is None:
            self._overlap_setup(self.capacity_rows or tokens * top_k * self.world)
        st = self._ov
        self._epoch += 1
        epoch, W = self._epoch, self.world
        main = torch.cuda.current_stream(self.device)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if timed else None
        if timed:
            ev[0].record()
        routing = routing.to(torch.int32).contiguous()
        x_tokens = x_tokens.contiguous()
        counts = ops.ep_count(routing, self.num_experts)
        if W > 1:
            # Also the "receive buffers are free again" barrier (see forward_p2p).
            dist.all_gather_into_tensor(st["counts_all"].view(-1), counts, group=self.group)
        else:
            st["counts_all"].copy_(counts.view(1, -1))
        plan = ops.ep_plan_ring(st["counts_all"], self.rank, st["plan"])
        dest_pos = torch.empty(tokens * top_k, dtype=torch.int32, device=self.device)
        if timed:
            ev[1].record()
        def phase(p):
            d = (self.rank + p) % W
            ops.ep_dispatch_phase(x_tokens, routing, self.num_experts, W, self.rank, p, plan,
                                  st["buf_ptrs"][d], st["capacity"], dest_pos, st["flag_ptrs"][d] + 4 * p, epoch,
                                  max_blocks=self.own_blocks if p == 0 else self.side_blocks)

        # Phase 0 (this rank's own rows, a local copy) runs alone and first, on the main stream:
        # the GEMM behind it never waits for a kernel of its own GPU, and the copy is not slowed
        # down by the NVLink phases (measured: 0.15 ms next to them, 0.05 ms alone).
        phase(0)
        if timed:
            ev.append(torch.cuda.Event(enable_timing=True))
            ev[4].record()
        st["ev_plan"].record(main)
        side = st["side"]
        side.wait_event(st["ev_plan"])
        # Phases to the other ranks go out on the side stream while the GEMM runs; the local
        # GEMM never waits for them -- it waits for the other GPUs' phases.
        with torch.cuda.stream(side):
            for p in range(1, W):
                phase(p)
            if timed:
                ev[2].record(side)
            st["ev_done"].record(side)
        cfg = _lib.TileCfg(0, 0, 1, 0, _lib.RD_CFG_NO_ZERO_TAIL)
        y = ops.gmm_forward(st["buf"], self.weights, plan["segment_sizes"], group_to_weight=st["seg2e"],
                            cfg=cfg, out=st["y"], workspace=st["ws"],
                            ready=(st["flags"], self.local_experts, epoch))
        if timed:
            ev[3].record()
        # The step is over on this rank when its own sends are, too.
        main.wait_event(st["ev_done"])
        if timed:
            self._events.append(ev)
        return y, plan["segment_sizes"], dest_pos.view(tokens, top_k), plan["totals"]

    def forward_fused(self, x_tokens: torch.Tensor, routing: torch.Tensor, timed: bool = False):
        """Exchange and local ragged_dot in ONE kernel launch: after count / all-gather / plan /
        assign and a copy of this rank's own rows, ``rd_gmm_ep_fused`` runs the flag-gated GEMM on
        most CTAs while ``sender_ctas`` CTAs of the same grid push the rows of phases 1..W-1 to
        their owners and raise the owners' flags.  Same return values as ``forward_overlap``."""
        from . import _lib, ops

        tokens, top_k = routing.shape
        if self._ov is None:
            self._overlap_setup(self.capacity_rows or tokens * top_k * self.world)
        st = self._ov
        self._epoch += 1
        epoch, W = self._epoch, self.world
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)] if timed else None
        if timed:
            ev[0].record()
        routing = routing.to(torch.int32).contiguous()
        x_tokens = x_tokens.contiguous()
        counts = ops.ep_count(routing, self.num_experts)
        if W > 1:
            dist.all_gather_into_tensor(st["counts_all"].view(-1), counts, group=self.group)
        else:
            st["counts_all"].copy_(counts.view(1, -1))
        plan = ops.ep_plan_ring(st["counts_all"], self.rank, st["plan"])
        entries = tokens * top_k
        dest_pos = torch.empty(entries, dtype=torch.int32, device=self.device)
        send_index = torch.empty(entries, dtype=torch.int32, device=self.device)
        ops.ep_assign(routing, self.num_experts, W, self.rank, plan, st["capacity"], dest_pos, send_index)
        if timed:
            ev[1].record()
        # own rows: a local copy, alone on the GPU, in front of the fused launch
        ops.ep_send_list(x_tokens, top_k, send_index, plan, 0, W, dest_pos, st["buf_ptrs"][self.rank],
                         st["capacity"], st["flag_ptrs"][self.rank], epoch)
        if timed:
            ev[4].record()
            ev[2].record()
        if "send" not in st:
            st["send_arrays"] = (torch.tensor(st["buf_ptrs"], dtype=torch.int64, device=self.device),
                                 torch.tensor(st["flag_ptrs"], dtype=torch.int64, device=self.device))
            st["send"] = _lib.EpSend()
            st["send"].peer_base = st["send_arrays"][0].data_ptr()
            st["send"].peer_flags = st["send_arrays"][1].data_ptr()
        send = st["send"]
        send.x_tokens, send.send_index = x_tokens.data_ptr(), send_index.data_ptr()
        send.send_start, send.dest_pos = plan["send_start"].data_ptr(), dest_pos.data_ptr()
        send.phase_done = plan["phase_done"].data_ptr()
        send.row_bytes, send.top_k = x_tokens.shape[1] * x_tokens.element_size(), top_k
        send.world, send.rank, send.capacity_rows = W, self.rank, st["capacity"]
        send.sender_ctas = self.sender_ctas if W > 1 else 1
        cfg = _lib.TileCfg(0, 0, 1, 0, _lib.RD_CFG_NO_ZERO_TAIL)
        y = ops.gmm_ep_fused(st["buf"], self.weights, plan["segment_sizes"], st["seg2e"], st["y"], st["ws"],
                             st["flags"], self.local_experts, epoch, send, cfg=cfg)
        if timed:
            ev[3].record()
            self._events.append(ev)
        return y, plan["segment_sizes"], dest_pos.view(tokens, top_k), plan["totals"]

    def forward(self, x_tokens: torch.Tensor, routing: torch.Tensor, timed: bool = False):
        """Returns (y [rows_received, n], plan).  y's rows are ordered (source rank, local expert)."""
        from . import ops

        if self.dispatch == "p2p":
            return self.forward_p2p(x_tokens, routing, timed=timed)
        if self.dispatch == "overlap":
            return self.forward_overlap(x_tokens, routing, timed=timed)
        if self.dispatch == "fused":
            return self.forward_fused(x_tokens, routing, timed=timed)

        plan = plan_dispatch(routing, self.num_experts, self.group)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if timed else None
        if timed:
            ev[0].record()
        rows_sorted = ops.gather_rows(x_tokens, plan.token_index)
        if timed:
            ev[1].record()
        received = exchange_rows(rows_sorted, plan, self.group)
        if timed:
            ev[2].record()
        y = ops.gmm_forward(received, self.weights, plan.segment_sizes, group_to_weight=plan.segment_to_expert)
        if timed:
            ev[3].record()
            self._events.append(ev)
        return y, plan

    # ------------------------------------------------------------------ host-resident tokens
    def forward_host(self, x_host: torch.Tensor, routing_host: torch.Tensor, y_host: torch.Tensor) -> int:
        """One step for a caller whose tokens, routing and result live in pinned host memory.

        The copy-in goes to one of two device slots on a copy stream, so the tokens of step i+1
        cross PCIe while step i is exchanged, multiplied and copied out (on a third stream); the
        step itself is ``forward`` on the current stream.  Copies ``min(len(y_host), rows of y)``
        rows of the result into ``y_host`` and returns that count.  ``wait_host_outputs`` orders
        the current stream after the last copy-out."""
        for name, t in (("x_host", x_host), ("routing_host", routing_host), ("y_host", y_host)):
            if t.is_cuda or not t.is_pinned():
                raise ValueError(f"{name} must be a pinned host tensor")
        if routing_host.dtype != torch.int32:
            raise ValueError("routing_host must be int32")
        dev = self.device
        if self._host is None:
            self._host = {
                "x": [torch.empty(x_host.shape, dtype=x_host.dtype, device=dev) for _ in range(2)],
                "r": [torch.empty(routing_host.shape, dtype=torch.int32, device=dev) for _ in range(2)],
                "s_in": torch.cuda.Stream(dev), "s_out": torch.cuda.Stream(dev),
                "read": [None, None],  # the step that last read slot i has finished
                "out": None,           # the last copy-out has finished
                "step": 0,
            }
        h = self._host
        slot = h["step"] & 1
        h["step"] += 1
        s_in, s_out = h["s_in"], h["s_out"]
        cur = torch.cuda.current_stream(dev)
        arrived = torch.cuda.Event()
        with torch.cuda.stream(s_in):
            if h["read"][slot] is not None:
                s_in.wait_event(h["read"][slot])
            h["x"][slot].copy_(x_host, non_blocking=True)
            h["r"][slot].copy_(routing_host, non_blocking=True)
            arrived.record(s_in)
        cur.wait_event(arrived)
        if h["out"] is not None:  # the result buffer of the previous step is still being copied out
            cur.wait_event(h["out"])
        y = self.forward(h["x"][slot], h["r"][slot])[0]
        done = torch.cuda.Event()
        done.record(cur)
        h["read"][slot] = done
        rows = min(y_host.shape[0], y.shape[0])
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            y_host[:rows].copy_(y[:rows], non_blocking=True)
            y.record_stream(s_out)
            h["out"] = torch.cuda.Event()
            h["out"].record(s_out)
        return rows

    def wait_host_outputs(self) -> None:
        """Make the current stream wait for the last ``forward_host`` copy-out."""
        if self._host is not None and self._host["out"] is not None:
            torch.cuda.current_stream(self.device).wait_event(self._host["out"])
