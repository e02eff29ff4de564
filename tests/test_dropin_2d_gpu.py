"""The drop-in module's 2-D wrappers (the reference's names and argument meaning,
kernels/shared_mask_batched_triton_min_runtime.py:3411-3495, 3498-4009) against the CPU oracle and - where the
reference's own module is at hand (baseline/_ref, filled by baseline/fill_ref.py) - against the reference's Triton
kernels run on the same GPU with the same inputs."""

import importlib.util
import os
from pathlib import Path

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import bas_oracle as O  # noqa: E402

TOL = 2e-3
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)


@pytest.fixture(scope="module")
def dropin():
    import kernels.shared_mask_batched_triton_min_runtime as m
    return m


@pytest.fixture(scope="module")
def reference():
    path = ROOT / "baseline" / "_ref" / "kernels" / "shared_mask_batched_triton_min_runtime.py"
    if not path.exists():
        pytest.skip("baseline/_ref is not filled")
    for key, val in (("TEAL_EXP_ENABLE_SPLIT_K_1D", "0"), ("TEAL_EXP_USE_RUN_COMPRESSED_METADATA", "0")):
        os.environ.setdefault(key, val)
    try:
        spec = importlib.util.spec_from_file_location("reference_triton_kernels_2d", path)
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
    except Exception as exc:                      # no Triton for this GPU, or the like
        pytest.skip(f"the reference module does not import here: {exc}")
    return ref


def _inputs(dev, batch, k, n, k_keep, n_keep, seed):
    x_h = O.make_activations(batch, k, seed=seed, dist="laplace")
    w_h = O.make_weight(n, k, seed=seed + 1)
    k_ids = O.random_active_blocks(k // 64, k_keep, seed=seed + 2)
    n_ids = O.random_active_blocks((n + 63) // 64, n_keep, seed=seed + 3)
    x = torch.from_numpy(x_h).to(dev).reshape(batch, 1, k)
    w = torch.from_numpy(w_h).to(dev)
    return x, w, torch.from_numpy(k_ids).to(dev), torch.from_numpy(n_ids).to(dev), O.masked_gemm(x_h, w_h, k_ids), n_ids


@pytest.mark.parametrize("batch,k,n,k_keep,n_keep", [(16, 4096, 11008, 23, 62), (2, 4096, 4096, 13, 5), (64, 11008, 4096, 83, 64)])
def test_dense_and_compact_forms(dev, dropin, batch, k, n, k_keep, n_keep):
    x, w, k_ids, n_ids, ref, n_np = _inputs(dev, batch, k, n, k_keep, n_keep, seed=batch + n)
    scale = np.abs(ref).max()
    listed = np.zeros(n, bool)
    for o in n_np:
        listed[o * 64:(o + 1) * 64] = True
    # dense form, zero-filled
    out = torch.full((batch, 1, n), 7.0, dtype=torch.float16, device=dev)
    comp, ids = dropin._prepacked_block_sparse_gemm_2d_from_active_blocks(x, w, k_ids, n_ids, out, zero_fill_out=True)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy().reshape(batch, n)
    assert comp is None and np.array_equal(ids.cpu().numpy(), n_np)
    assert np.abs(got[:, listed] - ref[:, listed]).max() <= TOL * scale and not np.any(got[:, ~listed])
    # dense form, the other columns kept
    out.fill_(7.0)
    dropin._prepacked_block_sparse_gemm_2d_bitmap_from_active_blocks(x, w, k_ids, n_ids, out)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy().reshape(batch, n)
    assert np.abs(got[:, listed] - ref[:, listed]).max() <= TOL * scale and np.all(got[:, ~listed] == 7.0)
    # compact form, and its scatter
    comp, ids = dropin._prepacked_block_sparse_gemm_2d_compact_from_active_blocks(x, w, k_ids, n_ids)
    torch.cuda.synchronize()
    assert tuple(comp.shape) == (batch, 1, n_keep * 64)
    gc = comp.float().cpu().numpy().reshape(batch, -1)
    for q, o in enumerate(n_np):
        assert np.abs(gc[:, q * 64:(q + 1) * 64] - ref[:, o * 64:(o + 1) * 64]).max() <= TOL * scale
    dense = torch.zeros((batch, 1, n), dtype=torch.float16, device=dev)
    dropin._scatter_compact_to_dense_output(comp, ids, 64, dense)
    gd = dense.float().cpu().numpy().reshape(batch, n)
    assert np.array_equal(gd[:, listed], gc) and not np.any(gd[:, ~listed])


def test_compact_input_wrapper_and_the_chain(dev, dropin):
    batch, hidden, inter = 16, 4096, 11008
    x, wu, k_ids, mid_ids, up_ref, mid_np = _inputs(dev, batch, hidden, inter, 23, 62, seed=300)
    wd_h = O.make_weight(hidden, inter, seed=310)
    wd = torch.from_numpy(wd_h).to(dev)
    comp, ids = dropin._prepacked_block_sparse_gemm_2d_compact_from_active_blocks(x, wu, k_ids, mid_ids)
    y = torch.full((batch, 1, hidden), float("nan"), dtype=torch.float16, device=dev)
    dropin._prepacked_block_sparse_gemm_from_compact_input_blocks(comp, wd, ids, y)
    torch.cuda.synchronize()
    mid_dev = comp.float().cpu().numpy().reshape(batch, -1)
    full = np.zeros((batch, inter), np.float16)
    for q, o in enumerate(mid_np):
        full[:, o * 64:(o + 1) * 64] = mid_dev[:, q * 64:(q + 1) * 64]
    assert O.max_err_ratio(y.float().cpu().numpy().reshape(batch, hidden), O.masked_gemm(full, wd_h, mid_np)) <= TOL


def test_empty_sets(dev, dropin):
    x, w, k_ids, n_ids, _, _ = _inputs(dev, 4, 1024, 512, 4, 3, seed=9)
    out = torch.full((4, 1, 512), 3.0, dtype=torch.float16, device=dev)
    comp, ids = dropin._prepacked_block_sparse_gemm_2d_from_active_blocks(x, w, k_ids[:0], n_ids, out)
    assert comp is None and ids.numel() == 0 and not bool(out.any())
    out.fill_(3.0)
    comp, ids = dropin._prepacked_block_sparse_gemm_2d_from_active_blocks(x, w, k_ids, n_ids[:0], out)
    assert comp is None and ids.numel() == 0 and not bool(out.any())
    comp, ids = dropin._prepacked_block_sparse_gemm_2d_compact_from_active_blocks(x, w, k_ids, n_ids[:0])
    assert tuple(comp.shape) == (4, 1, 0) and ids.numel() == 0


@pytest.mark.parametrize("batch,k,n,k_keep,n_keep", [(16, 4096, 11008, 23, 62), (4, 4096, 4096, 32, 16)])
def test_against_the_reference_kernels(dev, dropin, reference, batch, k, n, k_keep, n_keep):
    """Same inputs through the reference's Triton 2-D wrappers and through the drop-in's."""
    x, w, k_ids, n_ids, ref, n_np = _inputs(dev, batch, k, n, k_keep, n_keep, seed=batch + k + n)
    out_r = torch.zeros((batch, 1, n), dtype=torch.float16, device=dev)
    out_d = torch.zeros((batch, 1, n), dtype=torch.float16, device=dev)
    try:
        reference._prepacked_block_sparse_gemm_2d_from_active_blocks(x, w, k_ids, n_ids, out_r, zero_fill_out=True)
        comp_r, ids_r = reference._prepacked_block_sparse_gemm_2d_compact_from_active_blocks(x, w, k_ids, n_ids)
        torch.cuda.synchronize()
    except Exception as exc:
        pytest.skip(f"the reference's kernels do not run here: {type(exc).__name__}: {exc}"[:300])
    dropin._prepacked_block_sparse_gemm_2d_from_active_blocks(x, w, k_ids, n_ids, out_d, zero_fill_out=True)
    comp_d, ids_d = dropin._prepacked_block_sparse_gemm_2d_compact_from_active_blocks(x, w, k_ids, n_ids)
    torch.cuda.synchronize()
    scale = float(np.abs(ref).max())
    assert float((out_r.float() - out_d.float()).abs().max()) <= TOL * scale
    assert np.array_equal(ids_r.cpu().numpy(), ids_d.cpu().numpy())
    # The reference passes the compact tensor's width to its kernel as the output width (:3969-4009 hand
    # out_compact to the generic wrapper, which takes n_dim from out.shape[-1], :3515), so its kernel masks every
    # output block whose own columns lie past that width and returns zeros there.  The drop-in computes them.
    # Blocks that lie inside agree; for the others the reference's zeros are confirmed, and the drop-in is checked
    # against the oracle.
    width = n_keep * 64
    cr, cd = comp_r.float().cpu().numpy().reshape(batch, -1), comp_d.float().cpu().numpy().reshape(batch, -1)
    inside = 0
    for q, o in enumerate(n_np):
        sl = slice(q * 64, (q + 1) * 64)
        assert np.abs(cd[:, sl] - ref[:, o * 64:(o + 1) * 64]).max() <= TOL * scale
        if (o + 1) * 64 <= width:
            assert np.abs(cr[:, sl] - cd[:, sl]).max() <= TOL * scale
            inside += 1
        elif o * 64 >= width:
            assert not np.any(cr[:, sl])
    assert inside > 0
