"""CPU-side checks: the C ABI library loads and exports what include/bas.h declares, the pure
host functions answer without a GPU, and the host layer refuses CPU tensors (no fallback)."""

import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (ROOT / "include" / "bas.h").read_text()
    return sorted(set(re.findall(r"BAS_API[^;(]*?\b(bas_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from bas import abi as L

    declared = _declared_symbols()
    assert len(declared) >= 18
    for name in declared:
        assert hasattr(L.lib, name), f"libbas.so does not export {name}"
    assert sorted(L.EXPORTED) == [d for d in declared if d in L.EXPORTED]
    missing_in_binding = [d for d in declared if d not in L.EXPORTED]
    assert not missing_in_binding, f"ctypes binding lacks {missing_in_binding}"


def test_flag_constants_match_the_header():
    """The Python binding's flag values are the header's: a drifted constant would silently turn a
    caller's promise into another flag."""
    from bas import abi as L

    text = (ROOT / "include" / "bas.h").read_text()
    defines = {m.group(1): int(m.group(2)) for m in re.finditer(r"#define\s+(BAS_[A-Z_0-9]+)\s+(\d+)\b", text)}
    enums = {m.group(1): int(m.group(2)) for m in re.finditer(r"\b(BAS_SCORE_[A-Z_0-9]+)\s*=\s*(\d+)", text)}
    assert defines["BAS_GEMM_IDS_STABLE"] == L.IDS_STABLE
    assert defines["BAS_GEMM_X_STABLE"] == L.X_STABLE
    assert defines["BAS_GEMM_NEXT_INDEPENDENT"] == L.NEXT_INDEPENDENT
    assert defines["BAS_GEMM_BF16"] == L.GEMM_BF16
    assert enums["BAS_SCORE_NORM"] == L.SCORE_NORM and enums["BAS_SCORE_ENERGY"] == L.SCORE_ENERGY
    assert enums["BAS_SCORE_BF16"] == L.SCORE_BF16
    assert enums["BAS_SCORE_INPUTS_STABLE"] == L.SCORE_INPUTS_STABLE
    # flag bits the library does not know are refused, not ignored
    dummy = ctypes.c_void_p(4096)
    st = L.lib.bas_gemm_ex(dummy, 64, dummy, dummy, None, 1, None, 2, 64, 128, dummy, 128, dummy, 1 << 30, 1 << 27, None)
    assert st == 1


def test_host_only_entry_points():
    from bas import abi as L

    assert L.lib.bas_status_string(0) == b"ok"
    assert b"workspace" in L.lib.bas_status_string(3)
    assert L.lib.bas_packed_weight_bytes(4096, 11008) == 172 * 4096 * 128   # = the fp16 weight size
    assert L.lib.bas_packed_weight_bytes(99, 200) == 4 * 104 * 128          # K to whole blocks, N to 8
    assert L.lib.bas_packed_weight_bytes(0, 64) == 0
    assert L.lib.bas_gemm_workspace_bytes(16, 4096) >= 4
    assert L.lib.bas_select_workspace_bytes(11008) >= 256 + 172 * 8
    assert L.launch_count() >= 0


def test_argument_checks_need_no_gpu():
    from bas import abi as L

    st = L.lib.bas_gemm(None, 64, None, None, None, 0, None, 1, 64, 128, None, 128, None, 0, None)
    assert st == 1
    # batch beyond the kernels' limit
    dummy = ctypes.c_void_p(4096)
    st = L.lib.bas_gemm(dummy, 64, dummy, dummy, None, 1, None, 65, 64, 128, dummy, 128, dummy, 1 << 30, None)
    assert st == 2
    # K not a multiple of 8 cannot be bulk-copied
    st = L.lib.bas_gemm(dummy, 72, dummy, dummy, None, 1, None, 2, 68, 128, dummy, 128, dummy, 1 << 30, None)
    assert st == 1
    with pytest.raises(L.BasError):
        L.check(3, "x")


def test_no_cpu_fallback():
    torch = pytest.importorskip("torch")
    from bas import ops
    import kernels.shared_mask_batched_triton_min_runtime as K

    x = torch.zeros(2, 1, 128, dtype=torch.float16)
    w = torch.zeros(128, 128, dtype=torch.float16)
    out = torch.zeros(2, 1, 128, dtype=torch.float16)
    ids = torch.tensor([0], dtype=torch.int32)
    with pytest.raises(ValueError):
        K._prepacked_block_sparse_gemm_from_active_blocks_splitk(x, w, ids, out)
    with pytest.raises(ValueError):
        ops.select_topk(x.view(2, 128), 1)
    # empty active set: zero fill, as the reference does, needs no kernel
    out.fill_(1)
    K._prepacked_block_sparse_gemm_from_active_blocks_splitk(x, w, ids[:0], out)
    assert not out.any()


def test_drop_in_module_surface():
    import inspect
    import kernels.shared_mask_batched_triton_min_runtime as K

    assert K.INDEX_BLOCK_META_SIZE == 64
    sig = inspect.signature(K._prepacked_block_sparse_gemm_from_active_blocks_bitmap_preload_splitk)
    assert list(sig.parameters) == ["x", "weight", "active_blocks", "out", "cache_prefix", "total_k_blocks",
                                    "prebuilt_bitmap", "num_split_k", "tile_b", "tile_n", "tile_warps", "tile_stages"]
    sig = inspect.signature(K._prepacked_block_sparse_gemm_from_active_blocks_splitk)
    assert list(sig.parameters) == ["x", "weight", "active_blocks", "out", "cache_prefix", "num_split_k",
                                    "tile_b", "tile_n", "tile_warps", "tile_stages"]
    sig = inspect.signature(K._prepacked_block_sparse_gemm_from_active_blocks)
    assert list(sig.parameters) == ["x", "weight", "active_blocks", "out", "cache_prefix", "proj_tag",
                                    "sort_active_blocks", "use_run_compressed", "active_blocks_limit"]
    cfg = K.prepacked_block_sparse_gemm_bitmap_preload_batched_kernel.best_config
    assert cfg.kwargs["BLOCK_B"] and cfg.kwargs["BLOCK_N"] and cfg.num_warps and cfg.num_stages
    assert K._PREPACK_AUTOTUNE_CONFIGS


def test_column_split_matches_kernel_rules():
    """The column split used by the kernels: ranges of whole 8-column units tile the padded width."""
    def begin(r, units, ranges):
        return r * units // ranges * 8

    for n, ranges in [(4096, 148), (11008, 148), (4096, 37), (4096, 74), (96, 12), (8, 1), (24000, 148)]:
        units = (n + 7) // 8
        ranges = min(ranges, units)
        edges = [begin(r, units, ranges) for r in range(ranges + 1)]
        assert edges[0] == 0 and edges[-1] == units * 8
        widths = np.diff(edges)
        assert (widths > 0).all() and widths.max() - widths.min() <= 8 and (widths % 8 == 0).all()


def test_struct_layouts_match_the_header(tmp_path):
    """The ctypes structures of the binding against what a C compiler makes of include/bas.h: sizes and the
    offset of every field (a list of calls is passed as an array of these)."""
    import shutil
    import subprocess

    from bas import abi as L

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    structs = {"bas_list_call": L.ListCall, "bas_step_call": L.StepCall}
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "bas.h"', "int main(void) {"]
    for cname, st in structs.items():
        lines.append(f'  printf("{cname} size %zu\\n", sizeof({cname}));')
        for field, _ in st._fields_:
            lines.append(f'  printf("{cname} {field} %zu\\n", offsetof({cname}, {field}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.check_call([gcc, "-std=c11", "-I", str(ROOT / "include"), str(src), "-o", str(exe)])
    out = subprocess.check_output([str(exe)], text=True)
    seen = 0
    for row in out.splitlines():
        cname, field, value = row.split()
        st = structs[cname]
        want = ctypes.sizeof(st) if field == "size" else getattr(st, field).offset
        assert int(value) == want, row
        seen += 1
    assert seen == sum(len(st._fields_) + 1 for st in structs.values())
