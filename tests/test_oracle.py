"""The CPU oracle against the golden vectors recorded from the reference's own code."""

import numpy as np
import pytest

from oracle import bas_oracle as O


def _gap(scores, ids):
    """Relative gap between the weakest kept and the strongest dropped score."""
    keep = np.zeros(scores.size, bool)
    keep[ids] = True
    if keep.all():
        return float("inf")
    lo, hi = scores[keep].min(), scores[~keep].max()
    return float((lo - hi) / max(abs(lo), 1e-300))


def test_selection_norm_matches_reference(golden):
    data, meta = golden
    for ci, c in enumerate(meta["select"]):
        x = O.make_activations(c["batch"], c["k"], c["seed"], c["dist"])
        s = O.block_scores(x, O.SCORE_NORM)
        ids = O.topk_ids(s, O.n_keep_from_density(c["density"], s.size))
        ref = data[f"select{ci}_norm_ids"]
        assert ids.dtype == np.int32
        assert np.array_equal(ids, ref), f"case {ci} {c}: threshold gap {_gap(s, ids):.3e}"


def test_selection_energy_matches_reference(golden):
    data, meta = golden
    for ci, c in enumerate(meta["select"]):
        x = O.make_activations(c["batch"], c["k"], c["seed"], c["dist"])
        s = O.block_scores(x, O.SCORE_ENERGY)
        ids = O.topk_ids(s, O.n_keep_from_density(c["density"], s.size))
        assert np.array_equal(ids, data[f"select{ci}_energy_ids"]), f"case {ci}: gap {_gap(s, ids):.3e}"
        # the float64 score is what the reference's float32 evaluation approximates
        np.testing.assert_allclose(s, data[f"select{ci}_energy_f32"].astype(np.float64), rtol=2e-6)


def test_selection_budget_matches_reference(golden):
    data, meta = golden
    for ci, c in enumerate(meta["select"]):
        x = O.make_activations(c["batch"], c["k"], c["seed"], c["dist"])
        s = O.block_scores(x, O.SCORE_ENERGY)
        for keep in (0.5, 0.9, 0.99):
            ids = O.energy_budget_ids(s, keep)
            ref = data[f"select{ci}_budget{int(round(keep * 100))}_ids"]
            assert np.array_equal(ids, ref), f"case {ci} keep {keep}: {ids.size} vs {ref.size}"


def test_weighted_selection_matches_reference(golden):
    """_select_active_blocks with block_score_scale and / or block_prior
    (scripts/bench_roundrobin_e2e_decode.py:104-112), recorded from the reference."""
    data, meta = golden
    n_cases = 0
    for ci, c in enumerate(meta["select"]):
        if f"select{ci}_scale_ids" not in data:
            continue
        x = O.make_activations(c["batch"], c["k"], c["seed"], c["dist"])
        scale = O.make_channel_scale(c["k"], c["seed"])
        prior = O.make_block_prior(c["k"] // 64, c["seed"])
        assert np.array_equal(O.select_active_blocks(x, c["density"], block_score_scale=scale),
                              data[f"select{ci}_scale_ids"]), ci
        assert np.array_equal(O.select_active_blocks(x, c["density"], block_prior=prior, prior_alpha=0.5,
                                                     prior_eps=0.05), data[f"select{ci}_prior_ids"]), ci
        assert np.array_equal(O.select_active_blocks(x, c["density"], block_prior=prior, block_score_scale=scale),
                              data[f"select{ci}_scale_prior_ids"]), ci
        n_cases += 1
    assert n_cases == 10


def test_prior_multiplier_follows_the_reference_formula():
    """clamp(prior + eps, min=1e-6) ** alpha in float32
    (scripts/bench_roundrobin_e2e_decode.py:109-112), against the same expression in torch on CPU."""
    import torch

    prior = O.make_block_prior(172, 5)
    prior[:3] = [-1.0, 0.0, -0.05]                    # the clamp's branch
    for alpha, eps in ((1.0, 0.1), (0.5, 0.05), (2.0, 0.0)):
        want = torch.clamp(torch.from_numpy(prior) + float(eps), min=1e-6).pow(float(alpha)).numpy()
        got = O.prior_multiplier(prior, alpha, eps)
        assert got.dtype == np.float32
        np.testing.assert_allclose(got, want, rtol=3e-7, atol=0)


def test_prior_of_wrong_length_is_ignored():
    x = O.make_activations(4, 640, 3, "normal")
    assert np.array_equal(O.select_active_blocks(x, 0.5, block_prior=np.ones(7, np.float32)),
                          O.select_active_blocks(x, 0.5))


def test_norm_and_energy_select_different_sets(golden):
    data, _ = golden
    assert not np.array_equal(data["select0_norm_ids"], data["select0_energy_ids"])


def test_n_keep_rule():
    assert O.n_keep_from_density(0.5, 64) == 32
    assert O.n_keep_from_density(0.36, 172) == 62
    assert O.n_keep_from_density(0.0, 64) == 1          # never empty
    assert O.n_keep_from_density(1.5, 64) == 64
    assert O.n_keep_from_density(2.5 / 64, 64) == 2     # half-to-even
    assert O.n_keep_from_density(3.5 / 64, 64) == 4


def test_topk_ties_go_to_lower_index():
    s = np.array([1.0, 3.0, 3.0, 0.5, 3.0])
    assert O.topk_ids(s, 2).tolist() == [1, 2]
    assert O.topk_ids(np.zeros(6), 3).tolist() == [0, 1, 2]


def test_bitmap_matches_reference(golden):
    data, meta = golden
    for bi, c in enumerate(meta["bitmap"]):
        ids = O.random_active_blocks(c["nb"], c["n_keep"], c["seed"])
        assert np.array_equal(O.build_bitmap(ids, c["nb"]), data[f"bitmap{bi}"])


def test_prepack_matches_reference(golden):
    data, meta = golden
    for pi, c in enumerate(meta["prepack"]):
        w = O.make_weight(c["n"], c["k"], c["seed"])
        assert np.array_equal(O.pack_weight_block_major(w), data[f"prepack{pi}"])


def test_private_layout_is_a_permutation_of_the_reference_layout():
    w = O.make_weight(203, 200, 5)
    blocks = O.pack_weight_blocks(w)                  # [nb, npad, 64] swizzled
    nb, npad = blocks.shape[:2]
    assert (nb, npad) == (4, 208)
    ref = O.pack_weight_block_major(w)                # [nb, 64, N] (the reference's layout)
    r = np.arange(npad)
    for q in range(8):
        chunk = blocks.reshape(nb, npad, 8, 8)[:, r, q ^ (r % 8), :]      # logical chunk q: [nb, npad, 8]
        want = ref[:, 8 * q:8 * q + 8, :].transpose(0, 2, 1)              # [nb, N, 8]
        assert np.array_equal(chunk[:, :203], want)
        assert not chunk[:, 203:].any()


def test_contraction_matches_reference_kernels(golden):
    data, meta = golden
    for gi, c in enumerate(meta["gemm"]):
        nb = (c["k"] + 63) // 64
        x = O.make_activations(c["batch"], c["k"], c["seed"], c["dist"])
        w = O.make_weight(c["n"], c["k"], c["seed"], std=0.05)
        ids = O.random_active_blocks(nb, c["n_keep"], c["seed"])
        ref = O.masked_gemm(x, w, ids)
        for name in ("triton_list", "triton_bitmap", "torch_f16"):
            y = data[f"gemm{gi}_{name}"]
            assert y.dtype == np.float16 and y.shape == ref.shape
            assert O.max_err_ratio(y, ref) <= 2e-3, (gi, name)
        assert O.max_err_ratio(O.masked_gemm_blocks_f32(x, w, ids), ref) <= 1e-5


def test_contraction_edge_cases():
    x = O.make_activations(3, 256, 1)
    w = O.make_weight(16, 256, 1)
    assert not O.masked_gemm(x, w, np.zeros(0, np.int32)).any()          # empty mask -> zeros
    full = O.masked_gemm(x, w, np.arange(4, dtype=np.int32))
    np.testing.assert_allclose(full, x.astype(np.float64) @ w.astype(np.float64).T, rtol=1e-6)
    a = O.masked_gemm(x, w, np.array([3, 0], np.int32))                   # order does not matter
    b = O.masked_gemm(x, w, np.array([0, 3], np.int32))
    assert np.array_equal(a, b)


def test_torch_cpu_legs_agree_with_oracle():
    torch = pytest.importorskip("torch")
    x = O.make_activations(16, 4096, 0)
    w = O.make_weight(512, 4096, 0)
    ids = O.select_active_blocks(x, 0.5, O.SCORE_NORM)
    t_ids = O.select_active_blocks_torch_cpu(torch.from_numpy(x).reshape(16, 1, 4096), 0.5, O.SCORE_NORM)
    assert np.array_equal(ids, t_ids.numpy())
    y = O.masked_linear_torch_cpu(torch.from_numpy(x), torch.from_numpy(w), ids).numpy()
    assert O.max_err_ratio(y, O.masked_gemm(x, w, ids)) <= 2e-3


def test_bf16_rounding_matches_torch():
    """The oracle's bf16 stand-in (fp32 values rounded to nearest even on 16 bits) against torch's
    own float32 -> bfloat16 conversion."""
    import torch

    rng = np.random.default_rng(3)
    a = np.concatenate([rng.standard_normal(5000).astype(np.float32) * 10.0 ** rng.integers(-6, 6, 5000),
                        np.array([0.0, -0.0, 1.0, 1.00390625, 1.005859375, 3.0e38, 1e-40], np.float32)])
    want = torch.from_numpy(a).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(O.round_to_bf16(a), want)


def test_nan_and_inf_scores_rank_like_torch_topk():
    """Not-a-number ranks above +inf (torch.topk, torch.sort descending), equal scores to the lower id:
    the order is total, so exactly n_keep ids come back whatever the activations hold."""
    torch = pytest.importorskip("torch")
    s = np.array([1.0, np.nan, np.inf, 0.5, np.nan, -np.inf, 2.0, np.inf], np.float64)
    order = O.descending_order(s)
    assert order.tolist() == [1, 4, 2, 7, 6, 0, 3, 5]
    for n_keep in range(1, 9):
        ids = O.topk_ids(s, n_keep)
        assert ids.size == n_keep and np.array_equal(ids, np.sort(order[:n_keep]))
        # torch agrees on WHICH scores are kept (its order among equal scores is unspecified)
        tk = torch.topk(torch.from_numpy(s), n_keep).values.numpy()
        np.testing.assert_array_equal(np.sort(np.nan_to_num(tk, nan=1e300)), np.sort(np.nan_to_num(s[ids], nan=1e300)))
    x = O.make_activations(4, 512, seed=3)
    x[1, 70] = np.nan
    x[2, 200] = np.inf
    assert O.select_active_blocks(x, 0.25, O.SCORE_NORM).tolist() == [1, 3]
    # a total that is not a number keeps every block; an infinite one keeps the infinite block
    assert O.energy_budget_ids(np.array([1.0, np.nan, 3.0]), 0.5).tolist() == [0, 1, 2]
    assert O.energy_budget_ids(np.array([1.0, np.inf, 3.0]), 0.5).tolist() == [1]
