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

The backward pass (``backward``) mirrors the reference's custom_vjp wiring (gpu_ragged_dot.py:399-402)
on the sharded layout: dlhs = the transposed grouped GEMM over the received rows on the owner,
brought back to the tokens' ranks by the reverse exchange (summed over the top_k copies of a
token); drhs = tgmm over the received rows, summed per local expert over the source ranks.

A second dispatch mode, ``dispatch="p2p"``, has no host round trip at all: the counts are
all-gathered (NCCL, E int32 per rank), `rd_ep_plan` turns them into write offsets on the device,
and `rd_ep_dispatch` stores every row directly into the owner's receive buffer through peer
memory (torch symmetric memory supplies the peer addresses and the cross-rank barrier).  The
receive buffer has a fixed capacity (every row of every rank could land on one rank), the
local GEMM gets that capacity as its static row bound and the true segment sizes on the device.

The third mode, ``dispatch="fused"``, runs the exchange inside the GEMM launch (sender CTAs of the
same grid), see ``forward_fused``.
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
                 dispatch: str = "nccl", capacity_rows: Optional[int] = None, sender_ctas: int = 0,
                 pull_sms: int = 0, count_exchange: str = "peer"):
        from . import workloads

        assert dispatch in ("nccl", "p2p", "fused")
        self.dispatch, self.capacity_rows, self._p2p = dispatch, capacity_rows, None
        self._ring, self._epoch = None, 0
        self._saved = None  # what the last forward left for backward
        self.dtype = dtype
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        # fused mode: CTAs of the GEMM grid that send instead of multiplying.  Measured: 16 sender
        # CTAs move 600 GB/s per GPU at 2 and at 8 ranks; 8 are too few (220 GB/s), 24 are slower
        # again at 8 ranks (480 GB/s) and take more SMs from the GEMM.
        self.sender_ctas = sender_ctas or 16
        # backward: SMs the drhs product leaves free for the return exchange that runs beside it
        # (0: the exchange runs after drhs, on all SMs)
        self.pull_sms = pull_sms or (16 if self.world <= 2 else 24)
        # fused mode: how the per-expert counts cross ranks: "peer" = stored by the count kernel
        # itself into every rank's table (rd_ep_count_share), "nccl" = an all-gather
        assert count_exchange in ("peer", "nccl")
        self.count_exchange = count_exchange
        assert num_experts % self.world == 0
        self.num_experts, self.local_experts = num_experts, num_experts // self.world
        self.k, self.n, self.device = k, n, device
        self.weights = workloads.normal_tensor((self.local_experts, k, n), k ** -0.5, seed, device, dtype)
        self._events = []
        self._bwd_events = []
        self._grad = None
        self._host = None

    def reset_timers(self):
        self._events = []
        self._bwd_events = []

    def device_status(self) -> int:
        """Synchronises and returns the status word of the kernels of the last step (0 = ok; non-zero
        means a bounded wait expired inside a kernel and the result has unwritten rows)."""
        from . import ops

        for st in (self._ring, self._grad):
            if st is not None and ops.device_status(st["ws"]) != 0:
                return ops.device_status(st["ws"])
        if self._ring is not None and self._ring["share"] is not None:
            return ops.device_status(self._ring["share"]["status"])
        return 0

    def timers_ms(self, steps: int):
        torch.cuda.synchronize(self.device)
        tot = {"permute": 0.0, "a2a": 0.0, "gemm": 0.0}
        for e in self._events:
            tot["permute"] += e[0].elapsed_time(e[1])
            tot["a2a"] += e[1].elapsed_time(e[2])
            # fused mode: exchange and GEMM both start when the plan is done and run together
            tot["gemm"] += (e[1] if self.dispatch == "fused" else e[2]).elapsed_time(e[3])
        if self.dispatch == "fused":  # when the GEMM could start: own rows copied
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
        cfg = _lib.TileCfg(0, 0, 0, 0, _lib.RD_CFG_NO_ZERO_TAIL | self._order_flag(tokens, top_k))
        y = ops.gmm_forward(st["buf"], self.weights, seg_sizes, group_to_weight=st["seg2e"], cfg=cfg,
                            out=st["y"])
        if timed:
            ev[3].record()
            self._events.append(ev)
        self._saved = {"recv": st["buf"], "seg": seg_sizes, "seg2e": st["seg2e"], "dest_pos": dest_pos,
                       "routing": routing, "capacity": st["capacity"]}
        return y, seg_sizes, dest_pos, totals

    # ------------------------------------------------------------------ exchange inside the GEMM launch
    def _ring_setup(self, capacity_rows: int):
        """Receive buffer and ready flags in symmetric memory, persistent plan buffers."""
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
        share = None
        if W > 1 and self.count_exchange == "peer":
            # two counts_all tables (by epoch parity) and the count flags, addressable by every rank
            tables = symm_mem.empty((2, W, E), dtype=torch.int32, device=dev)
            cflags = symm_mem.empty((max(W, 4),), dtype=torch.int32, device=dev)
            tables.zero_()
            cflags.zero_()
            ht, hc = symm_mem.rendezvous(tables, grp), symm_mem.rendezvous(cflags, grp)
            torch.cuda.synchronize(dev)
            hc.barrier(channel=0)
            torch.cuda.synchronize(dev)
            tptr = [int(p) for p in ht.buffer_ptrs]
            share = {"tables": tables, "flags": cflags, "handles": (ht, hc),
                     "scratch": torch.zeros(E + 1, dtype=torch.int32, device=dev),
                     # set by the plan kernel if its wait for the counts expired (the GEMM's own
                     # status word is reset by the GEMM call that follows the plan)
                     "status": torch.zeros(4, dtype=torch.int32, device=dev),
                     "peer_counts": [torch.tensor([p + par * W * E * 4 for p in tptr], dtype=torch.int64, device=dev)
                                     for par in (0, 1)],
                     "peer_flags": torch.tensor([int(p) for p in hc.buffer_ptrs], dtype=torch.int64, device=dev)}
        self._ring = {
            "share": share,
            "buf": buf, "flags": flags, "handles": (hb, hf), "capacity": capacity_rows,
            "buf_ptrs": buf_ptrs, "flag_ptrs": flag_ptrs,
            "counts_all": torch.empty((W, E), dtype=torch.int32, device=dev),
            "plan": {name: torch.empty(size, dtype=torch.int32, device=dev)
                     for name, size in (("dest_offset", E), ("segment_sizes", E), ("fill", E), ("totals", 1),
                                        ("phase_done", W), ("send_start", W + 1), ("list_fill", W))},
            "y": torch.empty((capacity_rows, self.n), dtype=self.dtype, device=dev),
            "ws": ops._workspace(capacity_rows, E, dev),
            "seg2e": torch.arange(self.local_experts, dtype=torch.int32, device=dev).repeat(W),
        }

    def forward_fused(self, x_tokens: torch.Tensor, routing: torch.Tensor, timed: bool = False):
        """Exchange and local ragged_dot in ONE kernel launch: after count / all-gather / plan /
        assign and a copy of this rank's own rows, ``rd_gmm_ep_fused`` runs the flag-gated GEMM on
        most CTAs while ``sender_ctas`` CTAs of the same grid push the rows of phases 1..W-1 to
        their owners and raise the owners' flags.  The senders are CTAs of the same launch as the
        CTAs that wait for other GPUs' senders, resident before them by construction, so no rank's
        progress depends on a separately launched kernel finding room on a busy GPU.

        Returns (y [capacity, n], segment_sizes [W*El] in position order, dest_pos [T, top_k], totals).
        y, segment_sizes and totals are buffers of the layer that the next forward overwrites;
        dest_pos stays valid until the step after the next."""
        from . import _lib, ops

        tokens, top_k = routing.shape
        if self._ring is None:
            self._ring_setup(self.capacity_rows or tokens * top_k * self.world)
        st = self._ring
        self._epoch += 1
        epoch, W = self._epoch, self.world
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)] if timed else None
        if timed:
            ev[0].record()
        routing = routing.to(torch.int32).contiguous()
        x_tokens = x_tokens.contiguous()
        entries = tokens * top_k
        if st["share"] is not None and not timed:
            return self._forward_fused_one_call(st, x_tokens, routing, tokens, top_k, epoch)
        if st["share"] is not None:
            # counts cross ranks inside the count kernel; the plan kernel waits for them
            sh = st["share"]
            ops.ep_count_share(routing, self.num_experts, sh["scratch"], W, self.rank,
                               sh["peer_counts"][epoch & 1], sh["peer_flags"], epoch)
            plan = ops.ep_plan_ring_when_counted(sh["tables"][epoch & 1], sh["flags"], epoch, self.rank,
                                                 st["plan"], sh["status"])
        else:
            counts = ops.ep_count(routing, self.num_experts)
            if W > 1:
                dist.all_gather_into_tensor(st["counts_all"].view(-1), counts, group=self.group)
            else:
                st["counts_all"].copy_(counts.view(1, -1))
            plan = ops.ep_plan_ring(st["counts_all"], self.rank, st["plan"])
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
        send = self._send_struct(st, x_tokens, send_index, dest_pos, plan, top_k)
        cfg = _lib.TileCfg(0, 0, 1, 0, _lib.RD_CFG_NO_ZERO_TAIL | self._order_flag(tokens, top_k))
        y = ops.gmm_ep_fused(st["buf"], self.weights, plan["segment_sizes"], st["seg2e"], st["y"], st["ws"],
                             st["flags"], self.local_experts, epoch, send, cfg=cfg)
        if timed:
            ev[3].record()
            self._events.append(ev)
        self._saved = {"recv": st["buf"], "seg": plan["segment_sizes"], "seg2e": st["seg2e"],
                       "dest_pos": dest_pos, "routing": routing, "capacity": st["capacity"]}
        return y, plan["segment_sizes"], dest_pos.view(tokens, top_k), plan["totals"]

    def _order_flag(self, tokens: int, top_k: int) -> int:
        """Small steps (a decode batch: a few rows per expert and source) are bound by the weights'
        way out of HBM, and an expert's W segments lie far apart in the receive buffer: take the
        segments expert by expert (RD_CFG_GROUP_BY_WEIGHT) so each weight matrix is read once.
        Large steps keep the row order, which is the order the rows arrive in."""
        from . import _lib

        return _lib.RD_CFG_GROUP_BY_WEIGHT if tokens * top_k <= 4096 else 0

    def _send_struct(self, st, x_tokens, send_index, dest_pos, plan, top_k):
        from . import _lib

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
        send.world, send.rank, send.capacity_rows = self.world, self.rank, st["capacity"]
        # a decode-sized step has a few hundred rows to send: four sender CTAs (60 copying warps) are
        # plenty, and the multiplying CTAs are what such a step is short of
        small = x_tokens.shape[0] * top_k <= 4096
        send.sender_ctas = (min(self.sender_ctas, 4) if small else self.sender_ctas) if self.world > 1 else 1
        return send

    def _forward_fused_one_call(self, st, x_tokens, routing, tokens, top_k, epoch):
        """The fused forward through ``rd_ep_fused_forward``: the five launches of the step from one
        C call, with persistent position / send-list buffers (two sets, taken in turn, so the
        dest_pos a step returns stays valid until the step after the next)."""
        from . import _lib, ops

        sh, plan, par = st["share"], st["plan"], epoch & 1
        entries = tokens * top_k
        key = (entries, par)
        if key not in st.setdefault("pos", {}):
            st["pos"][key] = (torch.empty(entries, dtype=torch.int32, device=self.device),
                              torch.empty(entries, dtype=torch.int32, device=self.device))
        dest_pos, send_index = st["pos"][key]
        send = self._send_struct(st, x_tokens, send_index, dest_pos, plan, top_k)
        if "step" not in st:
            step = _lib.EpStep()
            step.num_experts = self.num_experts
            step.counts_scratch = sh["scratch"].data_ptr()
            step.ticket = sh["scratch"].data_ptr() + 4 * self.num_experts
            step.peer_count_flags = sh["peer_flags"].data_ptr()
            step.count_flags = sh["flags"].data_ptr()
            for name in ("dest_offset", "segment_sizes", "fill", "totals", "send_start", "list_fill"):
                setattr(step, name, plan[name].data_ptr())
            step.plan_status = sh["status"].data_ptr()
            step.own_buffer = st["buf_ptrs"][self.rank]
            step.own_ready_flag = st["flag_ptrs"][self.rank]
            step.wait_limit_ms = 0
            st["step"] = step
            st["cfg"] = _lib.TileCfg(0, 0, 1, 0, _lib.RD_CFG_NO_ZERO_TAIL)
        st["cfg"].flags = _lib.RD_CFG_NO_ZERO_TAIL | self._order_flag(tokens, top_k)
        step = st["step"]
        step.routing, step.tokens, step.top_k, step.epoch = routing.data_ptr(), tokens, top_k, epoch
        step.peer_counts = sh["peer_counts"][par].data_ptr()
        step.counts_all = sh["tables"][par].data_ptr()
        step.dest_pos, step.send_index = dest_pos.data_ptr(), send_index.data_ptr()
        ops.ep_fused_forward(step, st["buf"], self.weights, st["seg2e"], st["y"], st["ws"], st["capacity"],
                             st["flags"], send, st["cfg"])
        self._saved = {"recv": st["buf"], "seg": plan["segment_sizes"], "seg2e": st["seg2e"],
                       "dest_pos": dest_pos, "routing": routing, "capacity": st["capacity"]}
        return st["y"], plan["segment_sizes"], dest_pos.view(tokens, top_k), plan["totals"]

    def forward(self, x_tokens: torch.Tensor, routing: torch.Tensor, timed: bool = False):
        """Returns (y [rows_received, n], plan).  y's rows are ordered (source rank, local expert)."""
        from . import ops

        if self._grad is not None and self.world > 1:
            self._grad["pulled"] = True  # this step's count exchange orders the gradient buffers
        if self.dispatch == "p2p":
            return self.forward_p2p(x_tokens, routing, timed=timed)
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
        self._saved = {"recv": received, "plan": plan, "tokens": x_tokens.shape[0]}
        return y, plan

    # ------------------------------------------------------------------ backward
    def _grad_setup(self, capacity_rows: int):
        """Buffer of gradient rows (dlhs over the received layout) in symmetric memory, so the
        ranks the rows came from can pull them back."""
        import torch.distributed._symmetric_memory as symm_mem
        from . import ops

        dev = self.device
        buf = symm_mem.empty((capacity_rows, self.k), dtype=self.dtype, device=dev)
        if self.world > 1:
            hdl = symm_mem.rendezvous(buf, self.group if self.group is not None else dist.group.WORLD)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
        else:
            hdl, ptrs = None, [buf.data_ptr()]
        self._grad = {"buf": buf, "hdl": hdl, "capacity": capacity_rows,
                      "peer_base": torch.tensor(ptrs, dtype=torch.int64, device=dev),
                      "ws": ops._workspace(capacity_rows, self.num_experts, dev),
                      "ws_tgmm": ops._workspace(capacity_rows, self.num_experts, dev),
                      "side": torch.cuda.Stream(device=dev), "ev_dlhs": torch.cuda.Event(),
                      "ev_pull": torch.cuda.Event(), "pulled": True}

    def backward(self, dy: torch.Tensor, timed: bool = False):
        """VJP of the last ``forward`` with the reference's wiring (gpu_ragged_dot.py:399-402) on the
        sharded layout.  ``dy`` is the cotangent of the y that forward returned, same rows.

        Returns (dx_tokens [T, k], dW [local experts, k, n]):
          dlhs  rows = rd_gmm_indexed(dy, W, trans_rhs) over the received segments, on the owner;
                they go back to the tokens' ranks and the top_k copies of a token are summed
                (p2p / fused: ``rd_ep_combine_pull`` reads them from the owners' buffers after a
                cross-rank barrier; nccl: the reverse all-to-all, then an index_add);
          drhs  = rd_tgmm_strided over the received rows: local expert j sums its W segments.
        Stream-ordered; in the p2p / fused modes nothing is read on the host."""
        from . import _lib, ops

        sv = self._saved
        if sv is None:
            raise RuntimeError("backward needs a forward first")
        W, El = self.world, self.local_experts
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if timed else None
        if timed:
            ev[0].record()
        cfg = _lib.TileCfg(0, 0, 0, 0, _lib.RD_CFG_NO_ZERO_TAIL)
        if self.dispatch == "nccl":
            plan, recv = sv["plan"], sv["recv"]
            dy = dy[: recv.shape[0]].contiguous()
            d_recv = ops.gmm_forward(dy, self.weights, plan.segment_sizes, trans_rhs=True,
                                     group_to_weight=plan.segment_to_expert, cfg=cfg)
            if timed:
                ev[1].record()
            dW = ops.tgmm_forward(recv, dy, plan.segment_sizes, seg_count=W)
            if timed:
                ev[2].record()
            d_sorted = torch.empty((sum(plan.send_splits), self.k), dtype=self.dtype, device=self.device)
            if W > 1:
                dist.all_to_all_single(d_sorted, d_recv, output_split_sizes=plan.send_splits,
                                       input_split_sizes=plan.recv_splits, group=self.group)
            else:
                d_sorted.copy_(d_recv)
            dx = torch.zeros((sv["tokens"], self.k), dtype=torch.float32, device=self.device)
            dx.index_add_(0, plan.token_index.long(), d_sorted.float())
            dx = dx.to(self.dtype)
            if timed:
                ev[3].record()
                self._bwd_events.append(ev)
            return dx, dW
        cap = sv["capacity"]
        if getattr(self, "_grad", None) is None:
            self._grad_setup(cap)
        gr = self._grad
        assert dy.shape == (cap, self.n) and dy.is_contiguous()
        main = torch.cuda.current_stream(self.device)
        side = gr["side"]
        if not gr["pulled"] and gr["hdl"] is not None:
            gr["hdl"].barrier(channel=1)  # two backward calls in a row: the last pull has finished everywhere
        ops.gmm_forward(dy, self.weights, sv["seg"], trans_rhs=True, group_to_weight=sv["seg2e"], cfg=cfg,
                        out=gr["buf"], workspace=gr["ws"])
        if timed:
            ev[1].record()
        tokens = sv["routing"].shape[0]
        dx = torch.empty((tokens, self.k), dtype=self.dtype, device=self.device)
        overlap = W > 1 and self.pull_sms > 0
        if overlap:
            # The return exchange runs on a side stream under the drhs product, which leaves
            # `pull_sms` SMs free for it.  Neither kernel waits for the other on the device: the
            # barrier and the pull only need those SMs, drhs needs nothing remote.
            gr["ev_dlhs"].record(main)
            side.wait_event(gr["ev_dlhs"])
            with torch.cuda.stream(side):
                gr["hdl"].barrier(channel=0)  # every owner's gradient rows are complete
                ops.ep_combine_pull(sv["routing"], sv["dest_pos"], self.num_experts, W, gr["peer_base"], cap,
                                    self.k, self.dtype, out=dx, max_blocks=8 * self.pull_sms)
                gr["ev_pull"].record(side)
            sms = torch.cuda.get_device_properties(self.device).multi_processor_count
            tcfg = _lib.TileCfg(0, max(sms - self.pull_sms, 1), 0, 0, 0)
            dW = ops.tgmm_forward(sv["recv"], dy, sv["seg"], seg_count=W, workspace=gr["ws_tgmm"], cfg=tcfg)
            if timed:
                ev[2].record()
            main.wait_event(gr["ev_pull"])
        else:
            # drhs is local work: it runs while the other ranks finish their dlhs
            dW = ops.tgmm_forward(sv["recv"], dy, sv["seg"], seg_count=W, workspace=gr["ws_tgmm"])
            if timed:
                ev[2].record()
            if gr["hdl"] is not None:
                gr["hdl"].barrier(channel=0)  # every owner's gradient rows are complete
            ops.ep_combine_pull(sv["routing"], sv["dest_pos"], self.num_experts, W, gr["peer_base"], cap,
                                self.k, self.dtype, out=dx)
        gr["pulled"] = False
        if timed:
            ev[3].record()
            self._bwd_events.append(ev)
        return dx, dW

    def backward_timers_ms(self, steps: int):
        torch.cuda.synchronize(self.device)
        # with the return exchange running under drhs, the third span is only what sticks out
        names = ("dlhs_gemm", "drhs_tgmm", "return_exchange_and_combine")
        tot = dict.fromkeys(names, 0.0)
        for e in self._bwd_events:
            for i, nm in enumerate(names):
                tot[nm] += e[i].elapsed_time(e[i + 1])
        return {k: v / max(steps, 1) for k, v in tot.items()}

    # ------------------------------------------------------------------ host-resident tokens
    def forward_host(self, x_host: torch.Tensor, routing_host: torch.Tensor, y_host: torch.Tensor,
                     rows_host: Optional[torch.Tensor] = None) -> int:
        """One step for a caller whose tokens, routing and result live in pinned host memory.

        The copy-in goes to one of two device slots on a copy stream, so the tokens of step i+1
        cross PCIe while step i is exchanged, multiplied and copied out (on a third stream); the
        step itself is ``forward`` on the current stream.  Copies ``min(len(y_host), rows of y)``
        rows of the result into ``y_host`` and returns that count, an upper bound: in the p2p and
        fused modes y has the receive buffer's capacity and only the rows this rank received are
        defined.  ``rows_host`` (pinned int32 [1]) receives that number of defined rows with the
        result, i.e. it is valid once the copy-out has finished.  ``wait_host_outputs`` orders the
        current stream after the last copy-out."""
        for name, t in (("x_host", x_host), ("routing_host", routing_host), ("y_host", y_host)):
            if t.is_cuda or not t.is_pinned():
                raise ValueError(f"{name} must be a pinned host tensor")
        if routing_host.dtype != torch.int32:
            raise ValueError("routing_host must be int32")
        if rows_host is not None and (rows_host.is_cuda or not rows_host.is_pinned()
                                      or rows_host.dtype != torch.int32 or rows_host.numel() < 1):
            raise ValueError("rows_host must be a pinned int32 host tensor with one element")
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
        res = self.forward(h["x"][slot], h["r"][slot])
        y = res[0]
        done = torch.cuda.Event()
        done.record(cur)
        h["read"][slot] = done
        h["last_slot"] = slot
        rows = min(y_host.shape[0], y.shape[0])
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            y_host[:rows].copy_(y[:rows], non_blocking=True)
            y.record_stream(s_out)
            if rows_host is not None:
                if self.dispatch == "nccl":
                    rows_host[0] = res[1].rows_received
                else:
                    rows_host[:1].copy_(res[3][:1], non_blocking=True)
                    res[3].record_stream(s_out)
            h["out"] = torch.cuda.Event()
            h["out"].record(s_out)
        return rows

    def backward_host(self, dy_host: torch.Tensor, rows: int, dx_host: torch.Tensor,
                      dW_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``backward`` for a caller whose cotangent and token gradients live in pinned host memory:
        the first ``rows`` rows of ``dy_host`` (the rows this rank received in the last forward; see
        ``forward_host``'s ``rows_host``) are copied in on the copy-in stream, dx leaves on the
        copy-out stream.  The weight gradient stays where the weights are, on the device, and is
        returned; it is also copied to ``dW_host`` if that is given.  Rows of the device-side
        cotangent past ``rows`` are not read by the kernels (they lie outside every segment)."""
        for name, t in (("dy_host", dy_host), ("dx_host", dx_host), ("dW_host", dW_host)):
            if t is not None and (t.is_cuda or not t.is_pinned()):
                raise ValueError(f"{name} must be a pinned host tensor")
        if self._host is None or self._saved is None:
            raise RuntimeError("backward_host needs a forward_host first")
        h, dev = self._host, self.device
        full_rows = self._saved["recv"].shape[0]
        if h.get("dy") is None or h["dy"].shape[0] != full_rows:
            h["dy"] = torch.empty((full_rows, self.n), dtype=self.dtype, device=dev)
            h["dy_read"] = None
        rows = min(int(rows), full_rows, dy_host.shape[0])
        cur = torch.cuda.current_stream(dev)
        arrived = torch.cuda.Event()
        with torch.cuda.stream(h["s_in"]):
            if h["dy_read"] is not None:
                h["s_in"].wait_event(h["dy_read"])
            h["dy"][:rows].copy_(dy_host[:rows], non_blocking=True)
            arrived.record(h["s_in"])
        cur.wait_event(arrived)
        dx, dW = self.backward(h["dy"])
        done = torch.cuda.Event()
        done.record(cur)
        h["dy_read"] = done
        # the backward pass still reads the routing table of the slot the forward used: the slot
        # may be refilled only after it
        h["read"][h["last_slot"]] = done
        with torch.cuda.stream(h["s_out"]):
            h["s_out"].wait_event(done)
            dx_host.copy_(dx, non_blocking=True)
            dx.record_stream(h["s_out"])
            if dW_host is not None:
                dW_host.copy_(dW, non_blocking=True)
                dW.record_stream(h["s_out"])
            h["out"] = torch.cuda.Event()
            h["out"].record(h["s_out"])
        return dW

    def wait_host_outputs(self) -> None:
        """Make the current stream wait for the last ``forward_host`` / ``backward_host`` copy-out."""
        if self._host is not None and self._host["out"] is not None:
            torch.cuda.current_stream(self.device).wait_event(self._host["out"])
