"""Offline tile sweep: regenerates entries of ``tile_table.json`` for given shapes.

The replacement for the reference's run-time tune-jax search (tuning.py:49-58): instead of
searching block sizes at every process start, candidates are timed once on a B200 and the winner
per (op, k, n, g, m range) is committed.

    python -m gpu_ragged_dot_b200.tune --shape 8192,4096,14336,8 [--shape m,k,n,g ...]
                                       [--group-sizes uniform|dirichlet] [--write]

For each shape it times ``gmm`` (fwd), ``gmm_t`` (the dlhs call: trans_rhs with k and n swapped)
and ``tgmm`` for every kernel configuration, candidates interleaved in random order inside one
process (GPUs here are power-capped, so only same-process comparisons are meaningful), and prints
the table; ``--write`` merges the winners into ``tile_table.json``.
"""

from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import time

import numpy as np
import torch

from . import _lib, ops, tile_table, workloads

# (tile_n, cta_group, tile_m)
CANDIDATES = [(256, 1, 128), (256, 1, 256), (256, 2, 128), (256, 2, 256), (128, 1, 128), (64, 1, 128)]


def _time(fn, reps):
    time.sleep(0.1)
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def sweep_shape(m, k, n, g, group_sizes, dev, rounds=3, reps=20):
    x, A, dout = workloads.make_inputs(workloads.Shape("tune", m, k, n, g), dev)
    gs = torch.from_numpy(group_sizes.astype(np.int32)).to(dev)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    dx = torch.empty((m, k), dtype=torch.bfloat16, device=dev)
    dA = torch.empty_like(A)
    ws = ops._workspace(m, g, dev)
    calls = {
        "gmm": lambda cfg: ops.gmm_forward(x, A, gs, cfg=cfg, out=y, workspace=ws),
        "gmm_t": lambda cfg: ops.gmm_forward(dout, A, gs, trans_rhs=True, cfg=cfg, out=dx, workspace=ws),
        "tgmm": lambda cfg: ops.tgmm_forward(x, dout, gs, cfg=cfg, out=dA, workspace=ws),
    }
    results = {}
    rng = random.Random(0)
    for _ in range(rounds):
        # narrow tiles never win on wide outputs; skip them there to keep the sweep short
        jobs = [(op, c) for op in calls for c in CANDIDATES if not (c[0] < 256 and min(k, n) > 4096)]
        rng.shuffle(jobs)
        for op, c in jobs:
            cfg = _lib.TileCfg(c[0], 0, c[1], c[2], 0)
            try:
                ms = _time(lambda: calls[op](cfg), reps)
            except _lib.RaggedDotError:
                continue
            results.setdefault((op, c), []).append(ms)
    best = {}
    for op in calls:
        rows = sorted(((statistics.median(v), c) for (o, c), v in results.items() if o == op))
        best[op] = rows
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", action="append", required=True, help="m,k,n,g")
    ap.add_argument("--group-sizes", default="dirichlet", choices=["uniform", "dirichlet"])
    ap.add_argument("--write", action="store_true")
    args = ap.parse_args()
    _lib.load()
    dev = torch.device("cuda", 0)
    new_entries = []
    for spec in args.shape:
        m, k, n, g = (int(v) for v in spec.split(","))
        if args.group_sizes == "uniform":
            gs = np.full(g, m // g)
            gs[-1] += m - gs.sum()
        else:
            rng = np.random.default_rng(0)
            gs = rng.multinomial(m, rng.dirichlet(2.0 * np.ones(g)))
        best = sweep_shape(m, k, n, g, gs, dev)
        flops = 2.0 * m * k * n
        for op, rows in best.items():
            print(f"shape m={m} k={k} n={n} g={g}  op={op}")
            for ms, (tn, cg, tm) in rows:
                print(f"    tile_n={tn:3d} cta_group={cg} tile_m={tm:3d}: {ms:.4f} ms  {flops / ms / 1e9:7.1f} TFLOP/s")
            ms, (tn, cg, tm) = rows[0]
            kk, nn = (n, k) if op == "gmm_t" else (k, n)
            new_entries.append({"op": op, "k": kk, "n": nn, "g": g, "m_min": max(1, m // 2), "m_max": m * 2,
                                "tile_n": tn, "max_ctas": 0, "cta_group": cg, "tile_m": tm,
                                "note": f"swept at m={m}: {ms:.4f} ms"})
    if args.write:
        path = tile_table._TABLE_PATH
        with open(path) as f:
            table = json.load(f)
        keep = [e for e in table["entries"]
                if not any(e["op"] == n_["op"] and e["k"] == n_["k"] and e["n"] == n_["n"] and e["g"] == n_["g"]
                           and e.get("m_min", 0) <= n_["m_max"] and n_["m_min"] <= e.get("m_max", 1 << 62)
                           for n_ in new_entries)]
        table["entries"] = keep + new_entries
        with open(path, "w") as f:
            json.dump(table, f, indent=1)
        print(f"wrote {len(new_entries)} entries to {os.path.relpath(path)}")


if __name__ == "__main__":
    main()
