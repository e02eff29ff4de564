"""The reference's two kernel-benchmark scripts run UNMODIFIED against the drop-in module
(scripts/profile_kernel_configs.py, scripts/bench_perstep_actual_kernel_speedup.py), from the copies
that baseline/fill_ref.py puts under the git-ignored baseline/_ref/.  Skipped where that folder
has not been filled."""

import json
from pathlib import Path

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def test_reference_scripts_run_unmodified_against_the_drop_in(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    if not (REF / "scripts" / "bench_perstep_actual_kernel_speedup.py").exists():
        pytest.skip("baseline/_ref is not filled (python baseline/fill_ref.py)")
    from bas import launch_count, refscripts

    before = launch_count()
    res = refscripts.run_thesis_protocol(REF, tmp_path, batch_sizes=(16,), warmup=3, iterations=10, repeats=1,
                                         bench_warmup=5, bench_iters=20, bench_repeats=1)
    assert launch_count() > before + 100, "the scripts did not reach this library's kernels"
    rows = res["rows"]
    assert [r["batch_size"] for r in rows] == [16]
    assert rows[0]["n_group_steps"] == 55 and rows[0]["kernel_speedup"] > 0.5
    table = json.loads((Path(res["lookup_dir"]) / "llama2_kernel_best_sweep_B16.json").read_text())
    assert set(table) == {"qkvo", "gate_up", "down"}
    for shape in table.values():
        for cell in shape.values():
            assert cell["mask"] in ("dense", "naive", "bitmap") and cell["sparse_ms"] > 0
