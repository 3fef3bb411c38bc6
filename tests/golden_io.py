"""Loader for the fixtures tests/golden/make_golden.py wrote (bf16 stored as uint16 bits)."""

import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
BF16_KEYS = ("x", "A", "dout", "y", "y_trans_rhs", "tgmm", "dlhs", "drhs", "dlhs_trans_rhs", "drhs_trans_rhs")


def bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.astype(np.int16)).view(torch.bfloat16)


def gemm_cases():
    out = []
    for path in sorted(glob.glob(os.path.join(GOLDEN_DIR, "golden_gemm_*.npz"))):
        z = np.load(path)
        case = {k: bf16(z[k]) for k in BF16_KEYS if k in z.files}  # the largest case stores a subset
        case["group_sizes"] = torch.from_numpy(z["group_sizes"].astype(np.int32))
        m, k, n, g, bm, bk, bn, chunk, target_m = (int(v) for v in z["params"])
        case.update(m=m, k=k, n=n, g=g, target_m=target_m, name=os.path.basename(path)[12:-4])
        out.append(case)
    return out


def metadata_cases():
    z = np.load(os.path.join(GOLDEN_DIR, "golden_metadata.npz"))
    n = len([k for k in z.files if k.endswith("_group_sizes")])
    return [{f: z[f"c{i}_{f}"] for f in ("group_sizes", "m_chunk", "group_offsets", "row_it2group",
                                          "row_it2it_in_group", "total_row_its")} for i in range(n)]
