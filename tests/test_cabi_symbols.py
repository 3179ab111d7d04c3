"""The shared library builds, loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

from tests.conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "minfer_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(minf_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    names = _declared_symbols()
    for must in ("minf_convert_vertical_slash_indexes", "minf_vs_estimate", "minf_vs_build_plan",
                 "minf_sparse_attention_fwd", "minf_block_sparse_build_plan", "minf_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(built_lib)
    missing = [n for n in _declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing


def test_python_binding_covers_header(built_lib):
    from minference_b200 import _cabi

    assert sorted(_cabi.SIGNATURES) == _declared_symbols()
    lib = _cabi.lib()
    assert lib.minf_version().decode().startswith("minfer_b200")


def test_host_side_argument_checks(built_lib):
    """Entry points reject bad arguments before touching the device (safe without a GPU)."""
    from minference_b200 import _cabi

    lib = _cabi.lib()
    assert lib.minf_plan_bytes(1, 32, 131072, 1000, 6096) > 0
    assert lib.minf_plan_bytes(0, 32, 131072, 1000, 6096) == 0
    rc = lib.minf_convert_vertical_slash_indexes(None, None, None, 1, 1, 64, 1, 1, None, None, None, None, None, None)
    assert rc == -1 and b"null" in lib.minf_last_error()
    import ctypes as C
    st = (C.c_int64 * 3)(1, 1, 128)
    one = C.c_void_p(16)
    rc = lib.minf_sparse_attention_fwd(one, one, one, one, st, st, st, st, 1, 4, 2, 128, 64, 0.1,
                                       None, None, one, None, 1, 1, one, None)
    assert rc == -3 and b"head_dim" in lib.minf_last_error()


def test_no_cpu_path():
    import pytest
    import torch

    from minference_b200 import _cabi
    from minference_b200.ops.pit_sparse_flash_attention_v2 import vertical_slash_sparse_attention

    q = torch.zeros(1, 1, 64, 128, dtype=torch.bfloat16)
    idx = torch.zeros(1, 1, 1, dtype=torch.int32)
    with pytest.raises(_cabi.MInferB200Error):
        vertical_slash_sparse_attention(q, q, q, idx, idx)
