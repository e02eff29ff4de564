"""CPU oracle for the batch-shared block-sparse activation GEMM and its mask selection.

TEST INFRASTRUCTURE ONLY.  This file is a numpy restatement of the reference
algorithm; it exists so that the CUDA path can be checked against it.  Nothing
in the product package imports it: only the tests, the smoke check and the
benchmark's CPU-baseline leg do.  The product fails loudly when its CUDA
library is missing; it never falls back to this code.

Parity status: pinned.  ``tests/golden/`` holds outputs of the reference's own
Python functions (imported and run on CPU, see ``tests/golden/make_golden.py``)
and this oracle is checked against every one of them in ``tests/test_oracle.py``.

Reference sites restated here (paths relative to the reference project):

* block scores and top-k       scripts/bench_roundrobin_e2e_decode.py:90-113
* energy score / top-k / budget scripts/bench_alpaca_energy_budget_e2e.py:43-62
* bitmap                        kernels/shared_mask_batched_triton_min_runtime.py:1056-1061
* block-major weight prepack    kernels/shared_mask_batched_triton_min_runtime.py:3133-3163
* the contraction itself        kernels/shared_mask_batched_triton_min_runtime.py:684-733
  (and its semantic form ``F.linear(x * blockmask, W)`` at
  scripts/bench_alpaca_uniform_online_topk_e2e.py:596-603)

Numerical conventions
---------------------
Scores are evaluated in float64 from the exact float16 inputs.  A float16
square is exact in float32, and 64 of them summed in float64 lose nothing for
any realistic dynamic range, so the float64 score is the value that every
float32 evaluation order of the reference approximates.  Ties (exactly equal
scores) go to the lower block index.  The contraction's golden value is the
float64 product rounded once; the device accumulates in float32, and the test
tolerance (2e-3 * max|ref|) covers the difference.
"""

from __future__ import annotations

import numpy as np

BLOCK_K = 64            # channels per activation block (INDEX_BLOCK_META_SIZE)
TILE_N = 128            # widest column sub-tile one kernel pass handles
SCORE_NORM = 0          # mean over batch of per-block L2 norm
SCORE_ENERGY = 1        # mean over batch of per-block squared L2 norm


# --------------------------------------------------------------------------
# seeded synthetic inputs (the distributions the benchmark configurations name)
# --------------------------------------------------------------------------

def make_activations(batch: int, k: int, seed: int, dist: str = "normal") -> np.ndarray:
    """float16 [batch, k] activations, N(0,1) or Laplace(0,1), from a seeded PCG64 stream."""
    rng = np.random.Generator(np.random.PCG64(seed))
    if dist == "normal":
        x = rng.standard_normal((batch, k), dtype=np.float32)
    elif dist == "laplace":
        u = rng.random((batch, k), dtype=np.float32) - np.float32(0.5)
        x = -np.sign(u) * np.log1p(-2.0 * np.abs(u).astype(np.float64))
        x = x.astype(np.float32)
    else:
        raise ValueError(f"unknown distribution {dist!r}")
    return x.astype(np.float16)


def make_weight(n: int, k: int, seed: int, std: float = 0.02) -> np.ndarray:
    """float16 [n, k] weight in nn.Linear layout, N(0, std^2)."""
    rng = np.random.Generator(np.random.PCG64(seed + 7_000_003))
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(std)
    return w.astype(np.float16)


def random_active_blocks(nb: int, n_keep: int, seed: int) -> np.ndarray:
    """Sorted int32 ids of ``n_keep`` distinct blocks out of ``nb`` (a random mask, as the
    kernel benchmark draws one: scripts/bench_perstep_actual_kernel_speedup.py:84-87)."""
    rng = np.random.Generator(np.random.PCG64(seed + 11))
    return np.sort(rng.permutation(nb)[:n_keep]).astype(np.int32)


# --------------------------------------------------------------------------
# selection
# --------------------------------------------------------------------------

def n_keep_from_density(density: float, nb: int, min_keep: int = 1) -> int:
    """max(min_keep, min(nb, int(round(density * nb)))) with Python's half-to-even round
    (scripts/bench_roundrobin_e2e_decode.py:102, bench_alpaca_energy_budget_e2e.py:61)."""
    return max(int(min_keep), min(int(nb), int(round(float(density) * int(nb)))))


def block_scores(x: np.ndarray, kind: int = SCORE_NORM, block_k: int = BLOCK_K) -> np.ndarray:
    """float64 [nb] batch-shared block scores.

    kind SCORE_NORM   : mean_b sqrt(sum_i x[b, 64j+i]^2)   (bench_roundrobin_e2e_decode.py:103-105)
    kind SCORE_ENERGY : mean_b      sum_i x[b, 64j+i]^2    (bench_alpaca_energy_budget_e2e.py:43-46)
    Channels past nb*block_k are never scored (``d_eff``).
    """
    x2 = np.asarray(x).reshape(-1, x.shape[-1])
    nb = x2.shape[1] // block_k
    xb = x2[:, : nb * block_k].astype(np.float64).reshape(x2.shape[0], nb, block_k)
    e = np.zeros((x2.shape[0], nb), dtype=np.float64)
    for i in range(block_k):                     # fixed order; exact for realistic ranges
        e += xb[:, :, i] * xb[:, :, i]
    if kind == SCORE_NORM:
        e = np.sqrt(e)
    elif kind != SCORE_ENERGY:
        raise ValueError(f"unknown score kind {kind}")
    s = np.zeros(nb, dtype=np.float64)
    for b in range(x2.shape[0]):                 # batch reduced in row order
        s += e[b]
    return s / float(x2.shape[0])


def descending_order(scores: np.ndarray) -> np.ndarray:
    """Block ids from the largest score to the smallest; equal scores go to the lower id and a NaN
    ranks above everything, +inf included (the order of ``torch.topk`` and of a descending
    ``torch.sort``), all NaNs alike.  A total order whatever the scores hold."""
    s = np.asarray(scores, dtype=np.float64)
    nan = np.isnan(s)
    clean = np.where(nan, np.inf, s)
    return np.lexsort((np.arange(s.size), -clean, ~nan))   # NaNs first, then by -score, then by index


def topk_ids(scores: np.ndarray, n_keep: int) -> np.ndarray:
    """Ascending int32 ids of the ``n_keep`` largest scores; equal scores go to the lower id
    (``torch.topk(score, k).indices.sort()`` at bench_roundrobin_e2e_decode.py:113)."""
    return np.sort(descending_order(scores)[: int(n_keep)]).astype(np.int32)


def make_channel_scale(k: int, seed: int) -> np.ndarray:
    """Seeded float32 [k] positive per-channel weights, the stand-in for the squared column norms of
    a weight that the reference passes as ``block_score_scale``."""
    rng = np.random.default_rng(seed + 7_000_003)
    return rng.uniform(0.25, 4.0, size=int(k)).astype(np.float32)


def make_block_prior(nb: int, seed: int) -> np.ndarray:
    """Seeded float32 [nb] in [0, 1): the stand-in for a per-block activation frequency
    (``block_prior``)."""
    rng = np.random.default_rng(seed + 9_000_011)
    return rng.uniform(0.0, 1.0, size=int(nb)).astype(np.float32)


def prior_multiplier(prior: np.ndarray, alpha: float = 1.0, eps: float = 0.1) -> np.ndarray:
    """float32 [nb]: ``clamp(prior + eps, min=1e-6) ** alpha`` evaluated in float32, the factor the
    reference multiplies the scores by (scripts/bench_roundrobin_e2e_decode.py:109-112)."""
    p32 = np.asarray(prior, dtype=np.float32) + np.float32(eps)
    p32 = np.maximum(p32, np.float32(1e-6))
    return np.power(p32, np.float32(alpha)).astype(np.float32)


def weighted_block_scores(x: np.ndarray, chan_scale: np.ndarray | None, block_mult: np.ndarray | None,
                          kind: int = SCORE_NORM, block_k: int = BLOCK_K) -> np.ndarray:
    """float64 [nb] scores with the reference's two optional modifiers
    (scripts/bench_roundrobin_e2e_decode.py:104-112).  With ``chan_scale`` the score is
    mean_b sum_i x[b,i]^2 * chan_scale[i] whatever ``kind`` says; ``block_mult`` (see
    prior_multiplier) then multiplies the batch mean."""
    if chan_scale is None:
        s = block_scores(x, kind, block_k)
    else:
        x2 = np.asarray(x).reshape(-1, x.shape[-1])
        nb = x2.shape[1] // block_k
        xb = x2[:, : nb * block_k].astype(np.float64).reshape(x2.shape[0], nb, block_k)
        sc = np.asarray(chan_scale, dtype=np.float32)[: nb * block_k].astype(np.float64).reshape(nb, block_k)
        e = np.zeros((x2.shape[0], nb), dtype=np.float64)
        for i in range(block_k):
            e += (xb[:, :, i] * xb[:, :, i]) * sc[None, :, i]
        s = np.zeros(nb, dtype=np.float64)
        for b in range(x2.shape[0]):
            s += e[b]
        s = s / float(x2.shape[0])
    if block_mult is not None:
        s = s * np.asarray(block_mult, dtype=np.float32).astype(np.float64)
    return s


def select_active_blocks(x: np.ndarray, density: float, kind: int = SCORE_NORM,
                         block_k: int = BLOCK_K, block_prior: np.ndarray | None = None,
                         prior_alpha: float = 1.0, prior_eps: float = 0.1,
                         block_score_scale: np.ndarray | None = None) -> np.ndarray:
    """Scores + uniform top-k, the per-step batch-shared mask (``_select_active_blocks``,
    scripts/bench_roundrobin_e2e_decode.py:90-113), with its optional channel weights and block
    prior.  Like the reference, a prior whose length is not the block count is ignored."""
    nb = np.asarray(x).shape[-1] // block_k
    mult = None
    if block_prior is not None and int(np.asarray(block_prior).size) == nb:
        mult = prior_multiplier(block_prior, prior_alpha, prior_eps)
    s = weighted_block_scores(x, block_score_scale, mult, kind, block_k)
    return topk_ids(s, n_keep_from_density(density, s.size))


def energy_budget_ids(energy: np.ndarray, energy_keep: float, min_keep: int = 1) -> np.ndarray:
    """Smallest prefix of the descending energies whose sum reaches ``energy_keep`` of the
    total (``_energy_budget_active``, bench_alpaca_energy_budget_e2e.py:49-56): ascending ids."""
    e = np.asarray(energy, dtype=np.float64)
    order = descending_order(e)
    with np.errstate(invalid="ignore"):
        cum = np.cumsum(e[order])
        thresh = float(energy_keep) * float(cum[-1])
    if np.isnan(thresh):                       # not a number in the energies: every block is kept
        k = int(e.size)
    else:
        k = int(np.searchsorted(cum, thresh, side="left")) + 1
    k = max(int(min_keep), min(int(e.size), k))
    return np.sort(order[:k]).astype(np.int32)


def build_bitmap(ids: np.ndarray, nb: int) -> np.ndarray:
    """uint8 [nb], 1 at active ids (``_build_active_k_bitmap``)."""
    bm = np.zeros(int(nb), dtype=np.uint8)
    if np.asarray(ids).size:
        bm[np.asarray(ids, dtype=np.int64)] = 1
    return bm


# --------------------------------------------------------------------------
# weight layouts
# --------------------------------------------------------------------------

def pack_weight_block_major(w: np.ndarray, block_k: int = BLOCK_K) -> np.ndarray:
    """The reference's packed layout: Wp[j, i, n] = W[n, 64j+i], zero rows past K
    (``_get_prepacked_weight_block_major``).  Shape [nb, block_k, N]."""
    n, k = w.shape
    nb = (k + block_k - 1) // block_k
    wt = np.zeros((nb * block_k, n), dtype=w.dtype)
    wt[:k] = w.T
    return np.ascontiguousarray(wt.reshape(nb, block_k, n))


def pack_weight_blocks(w: np.ndarray) -> np.ndarray:
    """The device library's private layout, bit for bit.

    Shape [nb, npad, 64] float16 with npad = N rounded up to a multiple of 8: entry (j, n) holds
    the 64 channels W[n, 64j : 64j+64] (zero outside W) as one 128-byte row, and the row's eight
    16-byte chunks are stored at chunk position ``q ^ (n % 8)`` (the 128-byte shared-memory
    swizzle).  Any range of output columns of a block is thus one contiguous chunk that a plain
    bulk copy lands bank-conflict-free and tensor-core-ready.
    """
    n, k = w.shape
    nb = (k + BLOCK_K - 1) // BLOCK_K
    npad = (n + 7) // 8 * 8
    wp = np.zeros((npad, nb * BLOCK_K), dtype=np.float16)
    wp[:n, :k] = w
    t = wp.reshape(npad, nb, 8, 8).transpose(1, 0, 2, 3)             # [nb, n, q, e]
    out = np.empty_like(t)
    r = np.arange(npad)
    for q in range(8):
        out[:, r, q ^ (r % 8), :] = t[:, r, q, :]
    return np.ascontiguousarray(out.reshape(nb, npad, BLOCK_K))


# --------------------------------------------------------------------------
# the contraction
# --------------------------------------------------------------------------

def block_mask(ids: np.ndarray, k: int, block_k: int = BLOCK_K) -> np.ndarray:
    """float32 [k] channel mask: 1 on the channels of the active blocks."""
    nb = (k + block_k - 1) // block_k
    m = np.repeat(build_bitmap(ids, nb).astype(np.float32), block_k)
    return m[:k]


def masked_gemm(x: np.ndarray, w: np.ndarray, ids: np.ndarray, block_k: int = BLOCK_K) -> np.ndarray:
    """Golden float32 [B, N]: (x * blockmask) @ W^T evaluated in float64, rounded once.

    Equals sum over active blocks j of X[:, 64j:64j+64] @ W[:, 64j:64j+64]^T, the sum the
    reference kernels form in float32 (kernels ...:712-730)."""
    x2 = np.asarray(x).reshape(-1, x.shape[-1])
    m = block_mask(ids, x2.shape[1], block_k).astype(np.float64)
    y = (x2.astype(np.float64) * m) @ np.asarray(w).astype(np.float64).T
    return y.astype(np.float32)


def masked_gemm_blocks_f32(x: np.ndarray, w: np.ndarray, ids: np.ndarray,
                           block_k: int = BLOCK_K) -> np.ndarray:
    """float32 [B, N] formed block by block in float32, in list order, as the reference's
    index-list kernel does; used to bound the effect of summation order."""
    x2 = np.asarray(x).reshape(-1, x.shape[-1]).astype(np.float32)
    wf = np.asarray(w).astype(np.float32)
    acc = np.zeros((x2.shape[0], wf.shape[0]), dtype=np.float32)
    for j in np.asarray(ids, dtype=np.int64):
        lo, hi = j * block_k, min((j + 1) * block_k, x2.shape[1])
        acc += x2[:, lo:hi] @ wf[:, lo:hi].T
    return acc


def masked_linear_torch_cpu(x, w, ids, block_k: int = BLOCK_K):
    """The reference's CPU-runnable formulation ``F.linear(x * blockmask, W)`` on torch CPU
    tensors of the input dtype (scripts/bench_alpaca_uniform_online_topk_e2e.py:596-603).
    This is the leg the benchmark times as the CPU baseline."""
    import torch
    import torch.nn.functional as F

    k = x.shape[-1]
    nb = (k + block_k - 1) // block_k
    bm = torch.zeros(nb, dtype=x.dtype)
    if len(ids):
        bm[torch.as_tensor(np.asarray(ids, dtype=np.int64))] = 1
    mask = bm.repeat_interleave(block_k)[:k]
    return F.linear(x * mask, w)


def select_active_blocks_torch_cpu(x3, density: float, kind: int = SCORE_NORM,
                                   block_k: int = BLOCK_K):
    """The reference's selection written with the same torch ops in float32 on CPU
    (bench_roundrobin_e2e_decode.py:99-113; bench_alpaca_energy_budget_e2e.py:43-46,59-62);
    timed with the CPU baseline, and a cross-check on the float64 restatement above."""
    import torch

    d_in = x3.shape[-1]
    nb = d_in // block_k
    n_keep = n_keep_from_density(density, nb)
    xb = x3[..., : nb * block_k].float().reshape(-1, nb, block_k)
    if kind == SCORE_NORM:
        score = xb.norm(dim=2).mean(dim=0)
    else:
        score = xb.pow(2).sum(dim=2).mean(dim=0)
    return torch.topk(score, k=n_keep).indices.sort()[0].to(torch.int32)


def round_to_bf16(a: np.ndarray) -> np.ndarray:
    """fp32 array whose every value is exactly representable in bfloat16 (round to nearest even on
    the upper 16 bits): the oracle's stand-in for a bf16 tensor, numpy having no such dtype."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def max_err_ratio(y: np.ndarray, ref: np.ndarray) -> float:
    """max|y - ref| / max|ref|, the quantity the parity rule bounds by 2e-3."""
    ref = np.asarray(ref, dtype=np.float64)
    d = np.abs(np.asarray(y, dtype=np.float64) - ref).max() if ref.size else 0.0
    return float(d / max(np.abs(ref).max() if ref.size else 0.0, 1e-30))
