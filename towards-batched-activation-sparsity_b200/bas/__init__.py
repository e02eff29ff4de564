"""ctypes binding of libbas, the sm_100a implementation of the batch-shared block-sparse
activation GEMM and its mask selection.

Loading is strict: if ``libbas.so`` has not been built, importing :mod:`bas` raises.  There
is no CPU or PyTorch fallback anywhere in this package.
"""

from .abi import (  # noqa: F401
    BasError,
    BLOCK_K,
    MAX_BATCH,
    SCORE_ENERGY,
    SCORE_NORM,
    TILE_N,
    lib,
    lib_path,
    launch_count,
)
