"""Generate the golden vectors under tests/golden/ from the reference's own Python code.

Run where the reference checkout is available (it needs no GPU):

    python tests/golden/make_golden.py --reference /path/to/reference

The inputs are seeded and come from oracle/bas_oracle.py, so only the reference's OUTPUTS
are stored (ids, bitmaps, small output matrices).  What is recorded, and from where:

* selection_norm    scripts/bench_roundrobin_e2e_decode.py  _select_active_blocks (also with its
                    block_score_scale and block_prior arguments)
* selection_energy  scripts/bench_alpaca_energy_budget_e2e.py  _block_energy, _topk_active,
                    _energy_budget_active
* bitmap            kernels/shared_mask_batched_triton_min_runtime.py  _build_active_k_bitmap
* prepack           same file, _get_prepacked_weight_block_major
* gemm_triton       same file, the split-K wrappers (index-list and bitmap families) run by the
                    Triton interpreter on CPU tensors
* gemm_torch        F.linear(x * blockmask, W) in float16 on CPU, the construction at
                    scripts/bench_alpaca_uniform_online_topk_e2e.py:596-603
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import types
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from oracle import bas_oracle as O  # noqa: E402

SELECT_CASES = [
    # (batch, K, density, dist, seed)
    (16, 4096, 0.5, "normal", 0),          # single masked linear, 32 of 64 blocks
    (2, 11008, 0.197, "laplace", 1),       # down_proj shapes at the thesis sparsities
    (16, 11008, 0.362, "laplace", 2),
    (64, 11008, 0.48, "laplace", 3),
    (1, 4096, 0.25, "normal", 4),
    (8, 4096, 0.05, "normal", 5),
    (32, 4096, 0.95, "normal", 6),
    (3, 200, 0.5, "normal", 7),            # ragged K: trailing 8 channels never scored
    (5, 64, 1.0, "laplace", 8),            # one block
    (4, 640, 0.01, "normal", 9),           # rounds to zero -> keeps one block
] + [(16, 11008, 0.36, "laplace", 100 + s) for s in range(11)]   # per-step online selection

BUDGET_KEEPS = [0.5, 0.9, 0.99]
N_WEIGHTED = 10                # the first cases are also recorded with channel weights / a block prior
PRIOR_ALPHA, PRIOR_EPS = 0.5, 0.05

GEMM_CASES = [
    # (batch, K, N, n_keep, dist, seed, split_k)
    (2, 256, 128, 2, "laplace", 20, 2),
    (4, 512, 256, 5, "normal", 21, 2),
    (16, 1024, 128, 7, "normal", 22, 4),
    (16, 704, 192, 6, "laplace", 23, 2),
    (3, 200, 96, 3, "normal", 24, 2),      # ragged K and N
    (33, 512, 128, 4, "normal", 25, 2),
]


def _stub_matplotlib() -> None:
    """The energy-budget script imports matplotlib at module top; give it an inert stand-in."""
    if "matplotlib" in sys.modules:
        return
    m = types.ModuleType("matplotlib")
    m.use = lambda *a, **k: None
    p = types.ModuleType("matplotlib.pyplot")
    t = types.ModuleType("matplotlib.ticker")
    m.pyplot, m.ticker = p, t
    sys.modules.update({"matplotlib": m, "matplotlib.pyplot": p, "matplotlib.ticker": t})


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    args = ap.parse_args()
    ref = Path(args.reference).resolve()
    sys.path.insert(0, str(ref))
    sys.path.insert(0, str(ref / "scripts"))
    _stub_matplotlib()

    import torch
    import torch.nn.functional as F
    import kernels.shared_mask_batched_triton_min_runtime as K
    import bench_roundrobin_e2e_decode as RR
    import bench_alpaca_energy_budget_e2e as EB

    out: dict[str, np.ndarray] = {}
    meta: dict[str, list] = {"select": [], "gemm": [], "prepack": [], "bitmap": []}

    # ---- selection ----
    for ci, (b, k, density, dist, seed) in enumerate(SELECT_CASES):
        x = O.make_activations(b, k, seed, dist)
        x3 = torch.from_numpy(x).reshape(b, 1, k)
        nb = k // 64
        ids_norm = RR._select_active_blocks(x3, density, 64).numpy()
        energy = EB._block_energy(x3, 64, nb)
        ids_energy = EB._topk_active(energy, density).numpy()
        out[f"select{ci}_norm_ids"] = ids_norm.astype(np.int32)
        out[f"select{ci}_energy_ids"] = ids_energy.astype(np.int32)
        out[f"select{ci}_energy_f32"] = energy.numpy().astype(np.float32)
        for keep in BUDGET_KEEPS:
            ids_b = EB._energy_budget_active(energy, keep).numpy()
            out[f"select{ci}_budget{int(round(keep * 100))}_ids"] = ids_b.astype(np.int32)
        if ci < N_WEIGHTED:
            # the optional channel weights and block prior of _select_active_blocks
            scale = torch.from_numpy(O.make_channel_scale(k, seed))
            prior = torch.from_numpy(O.make_block_prior(nb, seed))
            out[f"select{ci}_scale_ids"] = RR._select_active_blocks(
                x3, density, 64, block_score_scale=scale).numpy().astype(np.int32)
            out[f"select{ci}_prior_ids"] = RR._select_active_blocks(
                x3, density, 64, block_prior=prior, prior_alpha=PRIOR_ALPHA, prior_eps=PRIOR_EPS).numpy().astype(np.int32)
            out[f"select{ci}_scale_prior_ids"] = RR._select_active_blocks(
                x3, density, 64, block_prior=prior, prior_alpha=1.0, prior_eps=0.1,
                block_score_scale=scale).numpy().astype(np.int32)
        meta["select"].append(dict(batch=b, k=k, density=density, dist=dist, seed=seed))

    # ---- bitmap ----
    for bi, (nb, n_keep, seed) in enumerate([(64, 32, 0), (172, 62, 1), (172, 0, 2), (7, 7, 3)]):
        ids = O.random_active_blocks(nb, n_keep, seed)
        bm = K._build_active_k_bitmap(torch.from_numpy(ids), nb, "cpu").numpy()
        out[f"bitmap{bi}"] = bm.astype(np.uint8)
        meta["bitmap"].append(dict(nb=nb, n_keep=n_keep, seed=seed))

    # ---- prepack ----
    for pi, (n, k, seed) in enumerate([(8, 130, 30), (96, 200, 31), (128, 256, 32)]):
        w = O.make_weight(n, k, seed)
        wp = K._get_prepacked_weight_block_major(torch.from_numpy(w), 64, cache_prefix=f"golden{pi}")
        out[f"prepack{pi}"] = wp.numpy().astype(np.float16)
        meta["prepack"].append(dict(n=n, k=k, seed=seed))

    # ---- contraction ----
    for gi, (b, k, n, n_keep, dist, seed, split_k) in enumerate(GEMM_CASES):
        nb = (k + 63) // 64
        x = O.make_activations(b, k, seed, dist)
        w = O.make_weight(n, k, seed, std=0.05)
        ids = O.random_active_blocks(nb, n_keep, seed)
        tx = torch.from_numpy(x).reshape(b, 1, k)
        tw = torch.from_numpy(w)
        tids = torch.from_numpy(ids)
        y_list = torch.zeros(b, 1, n, dtype=torch.float16)
        K._prepacked_block_sparse_gemm_from_active_blocks_splitk(
            tx, tw, tids, y_list, cache_prefix=f"golden_l{gi}", num_split_k=split_k,
            tile_b=16, tile_n=64, tile_warps=2, tile_stages=2)
        y_bitmap = torch.zeros(b, 1, n, dtype=torch.float16)
        K._prepacked_block_sparse_gemm_from_active_blocks_bitmap_preload_splitk(
            tx, tw, tids, y_bitmap, cache_prefix=f"golden_b{gi}", total_k_blocks=nb,
            prebuilt_bitmap=K._build_active_k_bitmap(tids, nb, "cpu"), num_split_k=split_k,
            tile_b=16, tile_n=64, tile_warps=2, tile_stages=2)
        mask = torch.from_numpy(O.block_mask(ids, k)).to(torch.float16)
        y_torch = F.linear(tx * mask, tw)
        out[f"gemm{gi}_triton_list"] = y_list.numpy().reshape(b, n)
        out[f"gemm{gi}_triton_bitmap"] = y_bitmap.numpy().reshape(b, n)
        out[f"gemm{gi}_torch_f16"] = y_torch.numpy().reshape(b, n)
        meta["gemm"].append(dict(batch=b, k=k, n=n, n_keep=n_keep, dist=dist, seed=seed, split_k=split_k))
        print(f"gemm case {gi} done", flush=True)

    np.savez_compressed(HERE / "reference_outputs.npz", **out)
    meta["versions"] = dict(torch=torch.__version__, numpy=np.__version__)
    (HERE / "reference_outputs.json").write_text(json.dumps(meta, indent=1) + "\n")
    print("wrote", HERE / "reference_outputs.npz", sum(v.nbytes for v in out.values()), "bytes raw")


if __name__ == "__main__":
    main()
