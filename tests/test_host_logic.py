"""Host-side logic that needs no GPU: workload generators, tile table, static-argument
handling and the refusal to run on CPU tensors."""

import numpy as np
import pytest
import torch

import gpu_ragged_dot_b200 as rd
from gpu_ragged_dot_b200 import ops, tile_table, workloads


def test_group_size_generators():
    gs = workloads.group_sizes_small(0)
    assert gs.sum() == 512 and gs.size == 8 and (gs == 0).any() and gs.dtype == np.int32
    gs = workloads.group_sizes_mixtral(0)
    assert gs.sum() == 8192 and gs.size == 8 and gs.min() > 0
    r = workloads.group_sizes_mixtral_ragged(0)
    assert r.sum() == 8192 and (r[:-1] % 128 != 0).all()
    d = workloads.group_sizes_deepseek(0)
    assert d.sum() == 32768 and d.size == 256
    assert 0.05 < (d == 0).mean() < 0.45 and d.max() > 5 * d.mean()
    # same seed, same sizes
    assert np.array_equal(workloads.group_sizes_deepseek(0), d)


def test_topk_routing_is_distinct_and_uniform():
    r = workloads.topk_routing(512, 64, 4, seed=1)
    assert r.shape == (512, 4) and r.min() >= 0 and r.max() < 64
    assert all(len(set(row)) == 4 for row in r.tolist())
    gs = workloads.group_sizes_from_routing(r, 64)
    assert gs.sum() == 2048 and gs.size == 64


def test_normal_tensor_is_seeded():
    a = workloads.normal_tensor((64, 32), 0.5, 3, "cpu")
    b = workloads.normal_tensor((64, 32), 0.5, 3, "cpu")
    assert torch.equal(a, b) and a.dtype == torch.bfloat16
    assert 0.4 < float(a.float().std()) < 0.6


def test_tile_table_lookup(tmp_path, monkeypatch):
    assert tile_table.lookup("gmm", 1, 8, 8, 1) is None or True  # default table loads
    p = tmp_path / "t.json"
    p.write_text('{"entries": [{"op": "gmm", "k": 4096, "n": 1536, "g": 64, "m_max": 512, "tile_n": 128}]}')
    monkeypatch.setenv("RD_TILE_TABLE", str(p))
    monkeypatch.setattr(tile_table, "_entries", None)
    hit = tile_table.lookup("gmm", 256, 4096, 1536, 64)
    assert hit is not None and hit.tile_n == 128 and hit.max_ctas == 0
    assert tile_table.lookup("gmm", 1024, 4096, 1536, 64) is None
    assert tile_table.lookup("tgmm", 256, 4096, 1536, 64) is None
    monkeypatch.setattr(tile_table, "_entries", None)


def test_reference_signature_is_kept():
    import inspect

    sig = inspect.signature(rd.gmm)
    # the reference's thirteen parameters, in its order; anything added is keyword-only
    assert list(sig.parameters)[:13] == [
        "x", "A", "group_sizes", "block_m", "block_k", "block_n", "trans_rhs", "interpret",
        "compute_dtype", "acc_dtype", "num_warps", "num_stages", "chunk_m"]
    assert all(p.kind is inspect.Parameter.KEYWORD_ONLY for p in list(sig.parameters.values())[13:])
    assert sig.parameters["block_m"].default == 64 and sig.parameters["chunk_m"].default == 512
    sig = inspect.signature(rd.tgmm)
    assert list(sig.parameters)[:12] == [
        "x", "y", "group_sizes", "block_m", "block_k", "block_n", "interpret", "compute_dtype",
        "acc_dtype", "num_warps", "num_stages", "chunk_m"]
    assert all(p.kind is inspect.Parameter.KEYWORD_ONLY for p in list(sig.parameters.values())[12:])
    assert rd.ragged_dot is rd.gmm and rd.trans_ragged_dot is rd.tgmm


def test_cpu_tensors_are_refused():
    x = torch.zeros(8, 8, dtype=torch.bfloat16)
    A = torch.zeros(1, 8, 8, dtype=torch.bfloat16)
    gs = torch.tensor([8], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        rd.gmm(x, A, gs)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        rd.tgmm(x, x, gs)
    with pytest.raises(NotImplementedError):
        rd.gmm(x, A, gs, interpret=True)
    with pytest.raises(NotImplementedError):
        rd.gmm(x, A, gs, compute_dtype=torch.float64)  # float16, bfloat16 or float32 only
    with pytest.raises(NotImplementedError):
        rd.gmm(x, A, gs, acc_dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        rd.gmm(x, A, gs, precision="fastest")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        rd.gmm(x, A, gs, compute_dtype=torch.float32)  # accepted, and then there is no CPU path
    assert ops._torch_dtype("float32") is torch.float32


def test_host_pipeline_chunk_plan():
    """Chunks of experts for the host-buffer pipeline: consecutive, covering every expert once, row
    ranges back to back, empty experts and empty chunks included."""
    from gpu_ragged_dot_b200.host_pipeline import plan_chunks

    sizes = [5, 0, 12, 3, 0, 0, 9, 1]
    assert plan_chunks(sizes, 1) == [(i, i + 1, sum(sizes[:i]), sum(sizes[:i + 1])) for i in range(8)]
    assert plan_chunks(sizes, 3) == [(0, 3, 0, 17), (3, 6, 17, 20), (6, 8, 20, 30)]
    assert plan_chunks(sizes, 100) == [(0, 8, 0, 30)]
    assert plan_chunks([0, 0, 0], 2) == [(0, 2, 0, 0), (2, 3, 0, 0)]
    assert plan_chunks([], 4) == []
    with pytest.raises(ValueError):
        plan_chunks(sizes, 0)


def test_ragged_dot_general_dimension_numbers():
    """Dimension numbers the op does not cover are refused before any device work; the two it
    covers reach gmm / tgmm (which then refuse CPU tensors: there is no CPU path)."""
    x, A, y = torch.zeros(8, 4), torch.zeros(2, 4, 6), torch.zeros(8, 6)
    gs = torch.tensor([3, 5], dtype=torch.int32)
    DN = rd.RaggedDotDimensionNumbers
    gmm_dn = DN((([1], [1]), ([], [])), [0], [0])       # tests.py:31-33 of the reference
    tgmm_dn = DN((([0], [0]), ([], [])), [0], [])       # tests.py:34-36
    for dn, rhs in ((gmm_dn, A), (tgmm_dn, y), (DN((([1], [2]), ([], [])), [0], [0]), A.transpose(1, 2))):
        with pytest.raises(RuntimeError, match="no CPU fallback"):
            rd.ragged_dot_general(x, rhs, gs, dn)
    for dn, rhs in ((DN((([1], [1]), ([0], [0])), [0], [0]), A),   # a batch dimension on a 2-D lhs
                    (DN((([1, 0], [1, 0]), ([], [])), [0], [0]), A),  # two contracting dimensions
                    (DN((([1], [1]), ([], [])), [1], [0]), A),     # ragged in the contracting dim of a 3-D rhs
                    (DN((([0], [0]), ([], [])), [0], [0]), y),     # group dimension on a 2-D rhs
                    (gmm_dn, y)):                                  # gmm numbers, 2-D rhs
        with pytest.raises(NotImplementedError):
            rd.ragged_dot_general(x, rhs, gs, dn)


def test_ragged_dot_general_batched_modes_reach_the_kernels():
    """One batch dimension and the ragged-batch mode are routed to gmm / tgmm (which refuse CPU
    tensors); malformed batched calls are refused first."""
    DN = rd.RaggedDotDimensionNumbers
    b, m, k, n, g = 2, 8, 4, 6, 3
    lhs, w, y = torch.zeros(b, m, k), torch.zeros(b, g, k, n), torch.zeros(b, m, n)
    gs2 = torch.tensor([[3, 5, 0], [8, 0, 0]], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        rd.ragged_dot_general(lhs, w, gs2, DN((([2], [2]), ([0], [0])), [1], [1]))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        rd.ragged_dot_general(lhs, y, gs2, DN((([1], [1]), ([0], [0])), [1], []))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        rd.ragged_dot_general(lhs, torch.zeros(b, k, n), torch.tensor([1, 1], dtype=torch.int32),
                              DN((([2], [1]), ([0], [0])), [0], []))
    with pytest.raises(NotImplementedError):  # group_sizes must carry the batch dimension
        rd.ragged_dot_general(lhs, w, gs2[0], DN((([2], [2]), ([0], [0])), [1], [1]))
    with pytest.raises(NotImplementedError):  # ragged batch with a group dimension on rhs
        rd.ragged_dot_general(lhs, w, gs2[0], DN((([2], [2]), ([0], [0])), [0], [1]))
