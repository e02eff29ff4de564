"""GPU test of the model hook layer (bas.hooks) on a synthetic two-layer module with Llama-2-7B's
projection shapes: the call pattern of the reference's patchers
(scripts/bench_roundrobin_e2e_decode.py:287-512, scripts/bench_alpaca_energy_budget_e2e.py:65-123)
without the model's weights.  Every patched projection is checked against the oracle."""

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import bas_oracle as O  # noqa: E402

TOL = 2e-3
PROJ_SHAPES = {"q_proj": (4096, 4096), "k_proj": (4096, 4096), "v_proj": (4096, 4096), "o_proj": (4096, 4096),
               "gate_proj": (11008, 4096), "up_proj": (11008, 4096), "down_proj": (4096, 11008)}


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def _no_grad():
    with torch.no_grad():       # decode: the projections' weights are parameters
        yield


def _toy_model(dev, layers=2, seed=0):
    """model.model.layers[i].self_attn.{q,k,v,o}_proj and .mlp.{gate,up,down}_proj as bias-free nn.Linear."""
    nn = torch.nn

    class Holder(nn.Module):
        pass

    model, inner = Holder(), Holder()
    inner.layers = nn.ModuleList()
    for li in range(layers):
        layer, attn, mlp = Holder(), Holder(), Holder()
        for pi, (name, (n, k)) in enumerate(PROJ_SHAPES.items()):
            lin = nn.Linear(k, n, bias=False, device=dev, dtype=torch.float16)
            with torch.no_grad():
                lin.weight.copy_(torch.from_numpy(O.make_weight(n, k, seed=seed + 10 * li + pi)).to(dev))
            setattr(attn if name in ("q_proj", "k_proj", "v_proj", "o_proj") else mlp, name, lin)
        layer.self_attn, layer.mlp = attn, mlp
        inner.layers.append(layer)
    model.model = inner
    return model


def _input(dev, b, k, seed, seq=1):
    x = O.make_activations(b * seq, k, seed=seed, dist="laplace" if k == 11008 else "normal")
    return x, torch.from_numpy(x).to(dev).reshape(b, seq, k)


def test_patch_sparse_matches_oracle_and_restores(dev):
    from bas import hooks

    model = _toy_model(dev)
    alloc = {str(li): {p: d for p, d in zip(hooks.PROJS, (0.5, 0.36, 0.25, 1.0, 0.36, 0.6, 0.36))} for li in range(2)}
    sweep_new = {s: {"0.4": {"mask": "bitmap", "K": 4, "tile": [16, 64, 4, 3]}} for s in ("qkvo", "gate_up", "down")}
    sweep_old = {s: {"0.4": {"best_kern": "naive", "best_K": 1, "best_tile": None}} for s in ("qkvo", "gate_up", "down")}
    for sweep in (sweep_new, sweep_old, None):          # both lookup schemas, or none
        originals, stats = hooks.patch_sparse(model, alloc, sweep)
        for li in range(2):
            for proj in hooks.PROJS:
                mod = hooks.get_module(model, li, proj)
                n, k = PROJ_SHAPES[proj]
                x, tx = _input(dev, 16, k, seed=100 + li)
                y = mod(tx)
                assert y.shape == (16, 1, n)
                w = mod.weight.detach().cpu().numpy()
                density = alloc[str(li)][proj]
                if density >= 1.0:
                    ref = x.astype(np.float32) @ w.astype(np.float32).T
                else:
                    ref = O.masked_gemm(x, w, O.select_active_blocks(x, density, O.SCORE_NORM))
                assert O.max_err_ratio(y.reshape(16, n).cpu().numpy(), ref) <= TOL, (li, proj)
        # prefill (several positions) stays dense
        mod = hooks.get_module(model, 0, "q_proj")
        x, tx = _input(dev, 2, 4096, seed=7, seq=5)
        y = mod(tx)
        ref = x.astype(np.float32) @ mod.weight.detach().cpu().numpy().astype(np.float32).T
        assert O.max_err_ratio(y.reshape(10, 4096).cpu().numpy(), ref) <= TOL
        assert stats["dense_calls"] >= 3 and stats["sparse_calls"] == 12
        hooks.restore(originals)
        x, tx = _input(dev, 4, 4096, seed=9)
        assert torch.equal(mod(tx), torch.nn.functional.linear(tx, mod.weight))


def test_patch_sparse_schedules_priors_weight_scores_and_mask_reuse(dev):
    from bas import hooks

    model = _toy_model(dev, layers=1)
    alloc = {"0": {p: 0.36 for p in hooks.PROJS}}
    nb = 4096 // 64
    prior = torch.from_numpy(O.make_block_prior(nb, seed=3)).to(dev)
    schedule = {(0, "q_proj"): [1.0, 0.5, 0.25]}
    originals, stats = hooks.patch_sparse(model, alloc, None, block_priors={(0, "k_proj"): prior}, prior_alpha=0.7, prior_eps=0.2,
                                          weight_aware_score=True, step_density_alloc=schedule, reuse_masks=False)
    q, kproj = hooks.get_module(model, 0, "q_proj"), hooks.get_module(model, 0, "k_proj")
    wq, wk = q.weight.detach().cpu().numpy(), kproj.weight.detach().cpu().numpy()
    scale_q = (q.weight.detach().float().pow(2).sum(dim=0)).cpu().numpy()
    scale_k = (kproj.weight.detach().float().pow(2).sum(dim=0)).cpu().numpy()
    # decode calls walk the schedule from index 1 and wrap: 0.5, 0.25, 0.5, ...
    for step, density in enumerate((0.5, 0.25, 0.5)):
        x, tx = _input(dev, 8, 4096, seed=20 + step)
        ids = O.select_active_blocks(x, density, O.SCORE_NORM, block_score_scale=scale_q)
        assert O.max_err_ratio(q(tx).reshape(8, 4096).cpu().numpy(), O.masked_gemm(x, wq, ids)) <= TOL, step
    x, tx = _input(dev, 8, 4096, seed=30)
    ids = O.select_active_blocks(x, 0.36, O.SCORE_NORM, block_prior=prior.cpu().numpy(), prior_alpha=0.7, prior_eps=0.2,
                                 block_score_scale=scale_k)
    assert O.max_err_ratio(kproj(tx).reshape(8, 4096).cpu().numpy(), O.masked_gemm(x, wk, ids)) <= TOL
    hooks.restore(originals)
    # mask reuse: the first decode call's mask serves every later call of the cell
    originals, stats = hooks.patch_sparse(model, alloc, None, reuse_masks=True)
    x0, tx0 = _input(dev, 8, 4096, seed=40)
    ids0 = O.select_active_blocks(x0, 0.36, O.SCORE_NORM)
    q(tx0)
    x1, tx1 = _input(dev, 8, 4096, seed=41)
    y1 = q(tx1)
    assert O.max_err_ratio(y1.reshape(8, 4096).cpu().numpy(), O.masked_gemm(x1, wq, ids0)) <= TOL
    assert np.array_equal(stats["mask_cache"][(0, "q_proj")].cpu().numpy(), ids0)
    hooks.restore(originals)


@pytest.mark.parametrize("mode,value,min_sparse", [("energy", 0.9, 0.0), ("energy", 0.999, 0.3), ("uniform", 0.6, 0.0),
                                                   ("uniform", 0.1, 0.3)])
def test_patch_adaptive_matches_oracle(dev, mode, value, min_sparse):
    from bas import hooks

    model = _toy_model(dev, layers=1, seed=5)
    originals, stats = hooks.patch_adaptive(model, None, mode, value, min_sparse_sparsity=min_sparse)
    for proj in ("q_proj", "down_proj", "gate_proj"):
        mod = hooks.get_module(model, 0, proj)
        n, k = PROJ_SHAPES[proj]
        nb = k // 64
        x, tx = _input(dev, 16, k, seed=50)
        y = mod(tx.reshape(16, k))                      # 2-D input form
        assert y.shape == (16, n)
        energy = O.block_scores(x, O.SCORE_ENERGY)
        ids = O.energy_budget_ids(energy, value) if mode == "energy" else O.topk_ids(energy, O.n_keep_from_density(1.0 - value, nb))
        dense = (1.0 - float(ids.size) / float(nb)) < float(min_sparse)
        if dense:
            ids = np.arange(nb, dtype=np.int32)
        w = mod.weight.detach().cpu().numpy()
        assert O.max_err_ratio(y.cpu().numpy(), O.masked_gemm(x, w, ids)) <= TOL, proj
        cell = hooks.read_stats(stats)[(0, proj)]
        assert cell["kept"] == ids.size and cell["total_k"] == nb and cell["dense_fallback_calls"] == int(dense and ids.size == nb and min_sparse > 0)
    hooks.restore(originals)
