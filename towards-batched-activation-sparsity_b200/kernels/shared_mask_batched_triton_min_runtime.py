"""Drop-in for the reference module ``kernels/shared_mask_batched_triton_min_runtime.py``.

Same names, argument meaning and error behaviour as the reference's host wrappers, so that
``scripts/bench_perstep_actual_kernel_speedup.py``, ``scripts/profile_kernel_configs.py`` and the
end-to-end decode scripts run against it unchanged; the work is done by libbas (hand-written
sm_100a CUDA) instead of Triton kernels.  Differences a caller can observe:

* ``num_split_k`` and the ``tile_*`` arguments are accepted and ignored: the split of the active
  blocks over the GPU is chosen inside the library (column ranges per CTA or per cluster), and
  the result does not depend on it beyond fp32 rounding.
* The tensor returned by ``_get_prepacked_weight_block_major`` is an opaque uint8 buffer in
  libbas's tile-major layout, not the reference's ``[K/64, 64, N]`` view.  No caller reads it.
* float16 or bfloat16 (x, weight and out alike).  There is no CPU path: CPU tensors raise
  ``ValueError``.
"""

from __future__ import annotations

from types import SimpleNamespace
from typing import Optional

import torch

from bas import ops as _ops
from bas.abi import BLOCK_K as _BLOCK_K

# kernels/shared_mask_batched_triton_min_runtime.py:17 — the reference reads an environment
# override; the block size of this implementation is fixed.
INDEX_BLOCK_META_SIZE = _BLOCK_K

# The tuner (scripts/profile_kernel_configs.py:70-83, 135-146) enumerates tile configurations and
# reads ``.best_config`` of the autotuned bitmap kernel.  There is one configuration here.
_PREPACK_AUTOTUNE_CONFIGS = [SimpleNamespace(kwargs={"BLOCK_B": 16, "BLOCK_N": 128}, num_warps=4, num_stages=3)]
prepacked_block_sparse_gemm_bitmap_preload_batched_kernel = SimpleNamespace(best_config=_PREPACK_AUTOTUNE_CONFIGS[0])


def _build_active_k_bitmap(active_blocks: torch.Tensor, total_k_blocks: int, device) -> torch.Tensor:
    """uint8 [total_k_blocks], 1 at the active ids (reference :1056-1061)."""
    return _ops.build_bitmap(active_blocks, int(total_k_blocks), device)


def _get_prepacked_weight_block_major(weight: torch.Tensor, block_k: int, cache_prefix: str = "gemm") -> torch.Tensor:
    """Warm (or hit) the packed-weight cache (reference :3133-3163)."""
    return _ops.get_packed_weight(weight, int(block_k), cache_prefix)


def _views(x: torch.Tensor, out: torch.Tensor):
    bsz, seqlen, m_dim = x.shape
    n_dim = out.shape[-1]
    bt = bsz * seqlen
    x2d = x.view(bt, m_dim)
    y2d = out.view(bt, n_dim)
    if not x2d.is_contiguous():
        x2d = x2d.contiguous()
    if y2d.stride(-1) != 1:
        raise ValueError("out must have unit stride along its last dimension")
    return x2d, y2d


def _ids32(active_blocks: torch.Tensor) -> torch.Tensor:
    if active_blocks.dtype != torch.int32:
        active_blocks = active_blocks.to(dtype=torch.int32)
    if not active_blocks.is_contiguous():
        active_blocks = active_blocks.contiguous()
    return active_blocks


def _prepacked_block_sparse_gemm_from_active_blocks_splitk(
    x: torch.Tensor,
    weight: torch.Tensor,
    active_blocks: torch.Tensor,
    out: torch.Tensor,
    cache_prefix: str = "gemm_1d_sk",
    num_split_k: Optional[int] = None,
    tile_b: Optional[int] = None,
    tile_n: Optional[int] = None,
    tile_warps: Optional[int] = None,
    tile_stages: Optional[int] = None,
) -> None:
    """Index-list family (reference :1350-1454): out = x[:, active blocks] . W[:, active blocks]^T."""
    if int(active_blocks.numel()) <= 0:
        out.zero_()
        return
    packed = _ops.get_packed_weight(weight, _BLOCK_K, cache_prefix)
    x2d, y2d = _views(x, out)
    _ops.gemm(x2d, packed, y2d, ids=_ids32(active_blocks))


def _prepacked_block_sparse_gemm_from_active_blocks_bitmap_preload(
    x: torch.Tensor,
    weight: torch.Tensor,
    active_blocks: torch.Tensor,
    out: torch.Tensor,
    cache_prefix: str = "gemm_bpl",
    total_k_blocks: Optional[int] = None,
    prebuilt_bitmap: Optional[torch.Tensor] = None,
) -> None:
    """Bitmap family (reference :1064-1138).  As in the reference, when a bitmap is passed it, not
    the id list, decides which blocks are summed (:847); the id list only answers "is it empty"."""
    if int(active_blocks.numel()) <= 0:
        out.zero_()
        return
    packed = _ops.get_packed_weight(weight, _BLOCK_K, cache_prefix)
    x2d, y2d = _views(x, out)
    if prebuilt_bitmap is not None:
        nb = (x.shape[-1] + _BLOCK_K - 1) // _BLOCK_K
        if total_k_blocks is not None and int(total_k_blocks) != nb:
            raise ValueError(f"total_k_blocks={total_k_blocks} does not match K={x.shape[-1]}")
        if int(prebuilt_bitmap.numel()) != nb:
            raise ValueError(f"bitmap has {prebuilt_bitmap.numel()} entries, expected {nb}")
        # the id list and the byte map agree in every caller: its length sizes the launch
        _ops.gemm(x2d, packed, y2d, bitmap=prebuilt_bitmap, k_host=min(int(active_blocks.numel()), nb))
    else:
        _ops.gemm(x2d, packed, y2d, ids=_ids32(active_blocks))


def _prepacked_block_sparse_gemm_from_active_blocks_bitmap_preload_splitk(
    x: torch.Tensor,
    weight: torch.Tensor,
    active_blocks: torch.Tensor,
    out: torch.Tensor,
    cache_prefix: str = "gemm_bpl_sk",
    total_k_blocks: Optional[int] = None,
    prebuilt_bitmap: Optional[torch.Tensor] = None,
    num_split_k: Optional[int] = None,
    tile_b: Optional[int] = None,
    tile_n: Optional[int] = None,
    tile_warps: Optional[int] = None,
    tile_stages: Optional[int] = None,
) -> None:
    """Bitmap family with split-K (reference :1235-1347); same computation as the call above."""
    _prepacked_block_sparse_gemm_from_active_blocks_bitmap_preload(
        x, weight, active_blocks, out, cache_prefix=cache_prefix,
        total_k_blocks=total_k_blocks, prebuilt_bitmap=prebuilt_bitmap)


def _prepacked_block_sparse_gemm_from_active_blocks(
    x: torch.Tensor,
    weight: torch.Tensor,
    active_blocks: torch.Tensor,
    out: torch.Tensor,
    cache_prefix: str = "gemm",
    proj_tag: str = "",
    sort_active_blocks: bool = True,
    use_run_compressed: bool = True,
    active_blocks_limit: Optional[int] = None,
) -> None:
    """Generic 1-D entry of the decode scripts (reference :3166-3344).  Sorting and run compression
    only reorder the same sum, so they are accepted and ignored; ``active_blocks_limit`` keeps the
    first entries of the list (:3178, :3190-3191)."""
    num_blocks = int(active_blocks.numel()) if active_blocks_limit is None else int(active_blocks_limit)
    if num_blocks <= 0:
        out.zero_()
        return
    ids = _ids32(active_blocks)
    if int(ids.numel()) > num_blocks:
        ids = ids[:num_blocks].contiguous()
    packed = _ops.get_packed_weight(weight, _BLOCK_K, cache_prefix)
    x2d, y2d = _views(x, out)
    _ops.gemm(x2d, packed, y2d, ids=ids)
