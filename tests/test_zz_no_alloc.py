"""The allocation-free selection entry point against the regular one.

Collected last on purpose (file name): a run that stops at the first failure has then already run
every other test.  Some hosts give all device memory to their own pool or forbid allocation calls
once serving has started; for them libbas offers ``bas_select_topk_noalloc``, whose scratch is a
fixed array inside the library.  It must return exactly what ``bas_select_topk`` returns, call
after call, although every call reuses (and finds the leftovers in) the same scratch.
"""

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import bas_oracle as O  # noqa: E402


def test_noalloc_selection_matches_regular_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bas import abi, ops

    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row, different shapes and score kinds, so the second finds the first's leftovers
    for call, (b, k, n_keep, kind) in enumerate([(16, 11008, 62, O.SCORE_ENERGY), (5, 4096, 20, O.SCORE_NORM)]):
        x = torch.from_numpy(O.make_activations(b, k, seed=900 + call, dist="laplace")).to(dev)
        nb = k // 64
        want_bm = torch.full((nb,), 9, dtype=torch.uint8, device=dev)
        want_sc = torch.zeros(nb, dtype=torch.float64, device=dev)
        want_ids, want_cnt = ops.select_topk(x, n_keep, kind, bitmap_out=want_bm, scores_out=want_sc)
        want_ids = want_ids.clone()
        want_cnt = want_cnt.clone()

        ids = torch.full((nb,), -1, dtype=torch.int32, device=dev)
        cnt = torch.full((1,), -1, dtype=torch.int32, device=dev)
        bm = torch.full((nb,), 7, dtype=torch.uint8, device=dev)
        sc = torch.zeros(nb, dtype=torch.float64, device=dev)
        abi.check(abi.lib.bas_select_topk_noalloc(x.data_ptr(), x.stride(0), b, k, n_keep, kind, ids.data_ptr(),
                                                  cnt.data_ptr(), bm.data_ptr(), sc.data_ptr(), stream),
                  "bas_select_topk_noalloc")
        torch.cuda.synchronize()
        assert int(cnt.item()) == int(want_cnt.item()) == n_keep
        assert torch.equal(ids[:n_keep], want_ids[:n_keep])            # bit-exact, as everywhere for ids
        assert torch.equal(bm, want_bm)
        assert torch.equal(sc, want_sc)                                # same kernel, same order: same bits
        assert np.array_equal(ids[:n_keep].cpu().numpy(), O.topk_ids(O.block_scores(x.cpu().numpy(), kind), n_keep))

    # sizes beyond the fixed scratch are refused, not truncated
    big = torch.zeros(1, 64 * 1025, dtype=torch.float16, device=dev)
    st = abi.lib.bas_select_topk_noalloc(big.data_ptr(), big.stride(0), 1, 64 * 1025, 1, 0, ids.data_ptr(),
                                         cnt.data_ptr(), None, None, stream)
    assert st == 6                                                     # BAS_ERR_TOO_LARGE


def test_noalloc_calls_back_to_back_on_one_stream_and_bfloat16():
    """Two calls enqueued on one stream with no synchronisation between them (different K, so the
    second finds the first's scores in the shared scratch), then a bfloat16 call: each against the
    regular entry point.  Calls of one stream are ordered, so they may share the array."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bas import abi, ops

    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream().cuda_stream
    cases = [(16, 11008, 62, O.SCORE_ENERGY, torch.float16), (64, 2048, 7, O.SCORE_NORM, torch.float16),
             (8, 4096, 23, O.SCORE_ENERGY, torch.bfloat16)]
    xs, got = [], []
    for call, (b, k, n_keep, kind, dt) in enumerate(cases):
        x = torch.from_numpy(O.make_activations(b, k, seed=950 + call, dist="laplace")).to(dev).to(dt)
        ids = torch.full((k // 64,), -1, dtype=torch.int32, device=dev)
        cnt = torch.full((1,), -1, dtype=torch.int32, device=dev)
        xs.append(x)
        got.append((ids, cnt))
    torch.cuda.synchronize()
    for (b, k, n_keep, kind, dt), x, (ids, cnt) in zip(cases, xs, got):      # enqueued back to back
        flags = kind | (256 if dt == torch.bfloat16 else 0)                   # BAS_SCORE_BF16
        abi.check(abi.lib.bas_select_topk_noalloc(x.data_ptr(), x.stride(0), b, k, n_keep, flags, ids.data_ptr(),
                                                  cnt.data_ptr(), None, None, stream), "bas_select_topk_noalloc")
    torch.cuda.synchronize()
    for (b, k, n_keep, kind, dt), x, (ids, cnt) in zip(cases, xs, got):
        want_ids, want_cnt = ops.select_topk(x, n_keep, kind)
        torch.cuda.synchronize()
        assert int(cnt.item()) == n_keep == int(want_cnt.item())
        assert torch.equal(ids[:n_keep], want_ids[:n_keep])
    # more rows than the selection kernel takes: refused before anything is enqueued
    tall = torch.zeros(1025, 64, dtype=torch.float16, device=dev)
    st = abi.lib.bas_select_topk_noalloc(tall.data_ptr(), tall.stride(0), 1025, 64, 1, 0, got[0][0].data_ptr(),
                                         got[0][1].data_ptr(), None, None, stream)
    assert st == 2                                                     # BAS_ERR_UNSUPPORTED
