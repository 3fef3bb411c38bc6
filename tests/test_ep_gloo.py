"""Expert-parallel host logic over gloo (world_size 2, CPU): the dispatch plan, the row
exchange and the (source, expert) segment bookkeeping, checked against a single-process
routing oracle.  The local GEMM is done by the CPU oracle here: what is under test is the
sharding, not the kernel."""

import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from gpu_ragged_dot_b200 import ep, workloads
    from oracle import ragged_dot_oracle as oracle

    E, k, n, T, top_k = 8, 16, 24, 40, 2
    local = E // world
    x = workloads.normal_tensor((T, k), 1.0, 1000 + rank, "cpu")
    routing = torch.from_numpy(workloads.topk_routing(T, E, top_k, seed=3000 + rank))
    weights = workloads.normal_tensor((E, k, n), k ** -0.5, 7, "cpu")  # same on every rank
    plan = ep.plan_dispatch(routing, E)
    rows_sorted = x[plan.token_index.long()]
    got = ep.exchange_rows(rows_sorted, plan)
    # local compute with the oracle, segment (s, e) -> local expert e
    seg_w = weights[rank * local:(rank + 1) * local][plan.segment_to_expert.long()]
    y = oracle.ragged_dot(got, seg_w, plan.segment_sizes)
    torch.save({"x": x, "routing": routing, "received": got, "y": y, "seg": plan.segment_sizes,
                "send": plan.send_splits, "recv": plan.recv_splits}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_dispatch_two_ranks(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    from gpu_ragged_dot_b200 import workloads

    E, k, n, top_k = 8, 16, 24, 2
    local = E // world
    weights = workloads.normal_tensor((E, k, n), k ** -0.5, 7, "cpu")
    for dst in range(world):
        # routing oracle: what rank `dst` must hold, in (source, expert, token order) order
        want_rows, want_seg = [], []
        for src in range(world):
            x, routing = res[src]["x"], res[src]["routing"]
            flat = routing.reshape(-1)
            for e in range(dst * local, (dst + 1) * local):
                idx = (flat == e).nonzero().flatten() // top_k
                want_rows.append(x[idx])
                want_seg.append(len(idx))
        want_rows = torch.cat(want_rows)
        assert res[dst]["seg"].tolist() == want_seg
        assert torch.equal(res[dst]["received"], want_rows)
        assert sum(res[dst]["recv"]) == want_rows.shape[0]
        # results: every received row times its expert's weights
        off = 0
        for si, cnt in enumerate(want_seg):
            e = dst * local + si % local
            ref = (want_rows[off:off + cnt].float() @ weights[e].float()).to(torch.bfloat16)
            assert torch.allclose(res[dst]["y"][off:off + cnt].float(), ref.float(), rtol=2e-2, atol=2e-2)
            off += cnt
    # conservation: rows sent == rows received overall
    assert sum(sum(r["send"]) for r in res) == sum(sum(r["recv"]) for r in res) == 2 * 40 * top_k
