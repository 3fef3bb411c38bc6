"""B200-native (sm_100a) ragged dot: drop-in for rdyro/gpu_ragged_dot's ``ragged_dot`` /
``trans_ragged_dot`` backed by hand-written CUDA (TMA + tcgen05) behind a C ABI."""

from .host_pipeline import HostRaggedDot  # noqa: F401
from .ops import (  # noqa: F401
    CHUNK_M,
    DEFAULT_BLOCK_K,
    DEFAULT_BLOCK_M,
    DEFAULT_BLOCK_N,
    BlockSizes,
    GMMGroupLookupMetadata,
    RaggedDotDimensionNumbers,
    RaggedDotSizes,
    gmm,
    gmm_forward,
    gmm_fp8_forward,
    make_group_metadata,
    ragged_dot,
    ragged_dot_general,
    ragged_dot_permuted,
    tgmm,
    tgmm_forward,
    trans_ragged_dot,
)

__all__ = ["gmm", "tgmm", "ragged_dot", "trans_ragged_dot", "ragged_dot_permuted", "HostRaggedDot", "gmm_fp8_forward",
           "ragged_dot_general", "RaggedDotDimensionNumbers"]
