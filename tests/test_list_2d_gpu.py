"""GPU parity of output-block sparsity and compact operands in the list kernel - the reference's 2-D kernels
(kernels/shared_mask_batched_triton_min_runtime.py:2289-2386: only the listed 64-column output blocks are
computed, the other columns of Y stay as they were), their compact output (:2473-2558) and the compact-input
contraction that consumes it (:3411-3467) - against the CPU oracle's masked product."""

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import bas_oracle as O  # noqa: E402

TOL = 2e-3   # max|y - ref| / max|ref|
TOL_BF16 = 2.0 ** -7


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)


def _ops():
    from bas import ops
    return ops


def _case(dev, batch, k, n, k_keep, n_blocks, seed, dtype=torch.float16, shuffle=False):
    rng = np.random.default_rng(seed)
    x_h = O.make_activations(batch, k, seed=seed, dist="laplace")
    w_h = O.make_weight(n, k, seed=seed + 1)
    k_ids = O.random_active_blocks((k + 63) // 64, k_keep, seed=seed + 2)
    nbn = (n + 63) // 64
    n_ids = np.sort(rng.choice(nbn, size=n_blocks, replace=False)).astype(np.int32)
    if shuffle:
        rng.shuffle(n_ids)
    x = torch.from_numpy(x_h).to(dev).to(dtype)
    w = torch.from_numpy(w_h).to(dev).to(dtype)
    ref = O.masked_gemm(x.float().cpu().numpy(), w.float().cpu().numpy(), k_ids)
    return x, w, k_ids, n_ids, ref


@pytest.mark.parametrize("batch,k,n,k_keep,n_blocks,shuffle", [
    (16, 4096, 11008, 23, 60, False), (16, 4096, 11008, 23, 172, False), (16, 4096, 11008, 23, 160, True),
    (2, 1024, 4096, 5, 1, False), (64, 2048, 4096, 12, 33, True), (7, 704, 200, 4, 3, False),
    (16, 704, 200, 11, 4, True), (33, 1024, 64, 16, 1, False)])
def test_listed_output_blocks_only(dev, batch, k, n, k_keep, n_blocks, shuffle):
    ops = _ops()
    x, w, k_ids, n_ids, ref = _case(dev, batch, k, n, k_keep, n_blocks, seed=batch + k + n + n_blocks, shuffle=shuffle)
    out = torch.full((batch, n), float("nan"), dtype=torch.float16, device=dev)
    comp = torch.full((batch, n_blocks * 64), float("nan"), dtype=torch.float16, device=dev)
    ids_t, nid_t = torch.from_numpy(k_ids).to(dev), torch.from_numpy(n_ids).to(dev)
    pk = ops.pack_weight(w)
    lst = ops.GemmList([{"x": x, "packed": pk, "out": out, "ids": ids_t, "n_ids": nid_t},
                        {"x": x, "packed": pk, "out": comp, "ids": ids_t, "n_ids": nid_t, "out_compact": True, "n": n}])
    for _ in range(2):
        out.fill_(float("nan"))
        comp.fill_(float("nan"))
        lst.run()
        torch.cuda.synchronize()
        assert lst.read_status() == 0
        got, gotc = out.float().cpu().numpy(), comp.float().cpu().numpy()
        listed = np.zeros(n, bool)
        scale = np.abs(ref).max()
        for q, o in enumerate(n_ids):
            c0, c1 = o * 64, min(o * 64 + 64, n)
            listed[c0:c1] = True
            assert np.abs(got[:, c0:c1] - ref[:, c0:c1]).max() <= TOL * scale
            assert np.abs(gotc[:, q * 64:q * 64 + (c1 - c0)] - ref[:, c0:c1]).max() <= TOL * scale
            assert np.isnan(gotc[:, q * 64 + (c1 - c0):(q + 1) * 64]).all()      # past the real width: not written
        assert np.isnan(got[:, ~listed]).all()                                    # the other columns: left alone
    lst.close()


def test_compact_input_equals_full_input(dev):
    ops = _ops()
    batch, k, n, k_keep = 16, 11008, 4096, 62
    x, w, k_ids, _, ref = _case(dev, batch, k, n, k_keep, 1, seed=5)
    xc = torch.cat([x[:, j * 64:(j + 1) * 64] for j in k_ids], dim=1).contiguous()
    assert xc.shape == (batch, k_keep * 64)
    out = torch.full((batch, n), float("nan"), dtype=torch.float16, device=dev)
    lst = ops.GemmList([{"x": xc, "packed": ops.pack_weight(w), "out": out, "ids": torch.from_numpy(k_ids).to(dev),
                         "x_compact": True, "k": k}])
    lst.run()
    torch.cuda.synchronize()
    assert lst.read_status() == 0
    lst.close()
    assert O.max_err_ratio(out.float().cpu().numpy(), ref) <= TOL


def test_compact_chain_gate_up_into_down(dev):
    """gate/up compute only the intermediate blocks that down's mask keeps and write them side by side; down
    reads that compact activation (one launch, down waits for the call before it)."""
    ops = _ops()
    batch, hidden, inter = 16, 4096, 11008
    x_h = O.make_activations(batch, hidden, seed=40)
    wu_h = O.make_weight(inter, hidden, seed=41, std=1.0 / np.sqrt(64 * 23))
    wd_h = O.make_weight(hidden, inter, seed=42, std=1.0 / np.sqrt(64 * 62))
    k_ids = O.random_active_blocks(hidden // 64, 23, seed=43)
    mid_ids = O.random_active_blocks(inter // 64, 62, seed=44)        # down's input mask = up's output blocks
    x = torch.from_numpy(x_h).to(dev)
    wu, wd = torch.from_numpy(wu_h).to(dev), torch.from_numpy(wd_h).to(dev)
    mid = torch.full((batch, 62 * 64), float("nan"), dtype=torch.float16, device=dev)
    y = torch.full((batch, hidden), float("nan"), dtype=torch.float16, device=dev)
    kid_t, mid_t = torch.from_numpy(k_ids).to(dev), torch.from_numpy(mid_ids).to(dev)
    lst = ops.GemmList([
        {"x": x, "packed": ops.pack_weight(wu), "out": mid, "ids": kid_t, "n_ids": mid_t, "out_compact": True, "n": inter},
        {"x": mid, "packed": ops.pack_weight(wd), "out": y, "ids": mid_t, "x_compact": True, "k": inter, "depends_on": 0}])
    g = torch.cuda.CUDAGraph()
    for run in range(3):
        mid.fill_(float("nan"))
        y.fill_(float("nan"))
        if run == 0:
            lst.run()
        else:
            if run == 1:
                with torch.cuda.graph(g):
                    lst.run()
            g.replay()
        torch.cuda.synchronize()
        assert lst.read_status() == 0
        up_ref = O.masked_gemm(x_h, wu_h, k_ids)
        mid_dev = mid.float().cpu().numpy()
        for q, o in enumerate(mid_ids):
            assert np.abs(mid_dev[:, q * 64:(q + 1) * 64] - up_ref[:, o * 64:(o + 1) * 64]).max() <= TOL * np.abs(up_ref).max()
        full = np.zeros((batch, inter), np.float32)                 # the device's own intermediate, scattered
        for q, o in enumerate(mid_ids):
            full[:, o * 64:(o + 1) * 64] = mid_dev[:, q * 64:(q + 1) * 64]
        assert O.max_err_ratio(y.float().cpu().numpy(), O.masked_gemm(full.astype(np.float16), wd_h, mid_ids)) <= TOL
    lst.close()


def test_mask_from_an_entry_and_listed_output_blocks(dev):
    ops = _ops()
    from bas import abi
    batch, k, n, keep = 16, 4096, 4096, 23
    x, w, _, n_ids, _ = _case(dev, batch, k, n, keep, 20, seed=77)
    out = torch.full((batch, n), float("nan"), dtype=torch.float16, device=dev)
    ids_out = torch.full((keep,), -1, dtype=torch.int32, device=dev)
    lst = ops.GemmList([{"select": x, "n_keep": keep, "score_kind": abi.SCORE_NORM},
                        {"x": x, "packed": ops.pack_weight(w), "out": out, "mask_from": 0, "ids_out": ids_out,
                         "n_ids": torch.from_numpy(n_ids).to(dev)}])
    lst.run()
    torch.cuda.synchronize()
    assert lst.read_status() == 0
    lst.close()
    k_ids = O.topk_ids(O.block_scores(x.cpu().numpy(), O.SCORE_NORM), keep)
    assert np.array_equal(ids_out.cpu().numpy(), k_ids)
    ref = O.masked_gemm(x.float().cpu().numpy(), w.float().cpu().numpy(), k_ids)
    got = out.float().cpu().numpy()
    for o in n_ids:
        assert np.abs(got[:, o * 64:(o + 1) * 64] - ref[:, o * 64:(o + 1) * 64]).max() <= TOL * np.abs(ref).max()


def test_bf16(dev):
    ops = _ops()
    x, w, k_ids, n_ids, ref = _case(dev, 16, 2048, 1024, 12, 7, seed=91, dtype=torch.bfloat16)
    out = torch.full((16, 7 * 64), float("nan"), dtype=torch.bfloat16, device=dev)
    lst = ops.GemmList([{"x": x, "packed": ops.pack_weight(w), "out": out, "ids": torch.from_numpy(k_ids).to(dev),
                         "n_ids": torch.from_numpy(n_ids).to(dev), "out_compact": True, "n": 1024}])
    lst.run()
    torch.cuda.synchronize()
    assert lst.read_status() == 0
    lst.close()
    got = out.float().cpu().numpy()
    for q, o in enumerate(n_ids):
        assert np.abs(got[:, q * 64:(q + 1) * 64] - ref[:, o * 64:(o + 1) * 64]).max() <= TOL_BF16 * np.abs(ref).max()


def test_bad_output_block_id_is_reported(dev):
    ops = _ops()
    from bas import abi
    x, w, k_ids, _, ref = _case(dev, 16, 1024, 512, 6, 1, seed=3)
    out = torch.full((16, 512), float("nan"), dtype=torch.float16, device=dev)
    n_ids = torch.tensor([1, 99, 3], dtype=torch.int32, device=dev)       # 99: not a block of this output
    lst = ops.GemmList([{"x": x, "packed": ops.pack_weight(w), "out": out, "ids": torch.from_numpy(k_ids).to(dev), "n_ids": n_ids}])
    lst.run()
    torch.cuda.synchronize()
    assert lst.read_status() == abi.DEV_BAD_BLOCK_ID
    lst.close()
    got = out.float().cpu().numpy()
    for o in (1, 3):
        assert np.abs(got[:, o * 64:(o + 1) * 64] - ref[:, o * 64:(o + 1) * 64]).max() <= TOL * np.abs(ref).max()
    assert np.isnan(got[:, 0:64]).all() and np.isnan(got[:, 128:192]).all()


def test_argument_checks(dev):
    ops = _ops()
    from bas import abi
    x = torch.zeros(16, 1024, dtype=torch.float16, device=dev)
    pk = ops.pack_weight(torch.zeros(512, 1024, dtype=torch.float16, device=dev))
    out = torch.zeros(16, 512, dtype=torch.float16, device=dev)
    ids = torch.arange(4, dtype=torch.int32, device=dev)
    nid = torch.arange(3, dtype=torch.int32, device=dev)
    base = {"x": x, "packed": pk, "out": out, "ids": ids}
    with pytest.raises(abi.BasError):                       # more blocks than the output has
        ops.GemmList([dict(base, n_ids=torch.arange(9, dtype=torch.int32, device=dev))])
    with pytest.raises(abi.BasError):                       # compact output without a block list
        ops.GemmList([dict(base, out_compact=True)])
    with pytest.raises((abi.BasError, ValueError)):         # a compact output needs n_host * 64 columns
        ops.GemmList([dict(base, n_ids=nid, out_compact=True, out=out[:, :128], n=512)])
    with pytest.raises(abi.BasError):                       # compact X goes with an id list
        ops.GemmList([dict(base, ids=None, bitmap=torch.ones(16, dtype=torch.uint8, device=dev), x_compact=True)])
    with pytest.raises((abi.BasError, ValueError)):         # compact X narrower than its blocks
        ops.GemmList([dict(base, x=x[:, :128], x_compact=True, k=1024)])
    with pytest.raises(abi.BasError):                       # clusters
        ops.GemmList([dict(base, n_ids=nid)], cluster=2)
