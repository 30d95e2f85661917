"""The C-ABI library loads without a GPU and exports every symbol include/xattn_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from xattn_b200 import _lib, build
    build.build()
    return _lib.load()


def _declared():
    text = open(os.path.join(ROOT, "include", "xattn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(xattn_b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from xattn_b200 import _lib
    names = _declared()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names


def test_host_only_entry_points(lib):
    assert lib.xattn_b200_version() >= 100
    assert lib.xattn_b200_error_string(0) == b"ok"
    assert b"argument" in lib.xattn_b200_error_string(1)
    for L, want in ((1000, 2048), (4096, 4096), (16384, 16384), (32768, 8192), (62208, 4096), (131072, 2048)):
        assert lib.xattn_b200_default_chunk_size(L) == want      # Xattention.py:322-331
    out = (ctypes.c_int * 8)()
    assert lib.xattn_b200_estimate_geometry(1024, 5000, 2048, 16, 128, out) == 0
    assert list(out) == [2048, 6144, 16, 48, 1, 3, 16, 32]
    assert lib.xattn_b200_estimate_geometry(5000, 1024, 2048, 16, 128, out) != 0   # k chunks < q chunks
    assert lib.xattn_b200_estimate_workspace_bytes(1, 32, 131072, 131072, 16, 128, 2048) > (1 << 30)
    assert lib.xattn_b200_estimate_workspace_bytes(1, 32, 4096, 4096, 3, 128, 2048) == 0       # bad stride


def test_ops_refuse_cpu_tensors():
    import torch
    from xattn_b200 import Xattention_prefill
    from xattn_b200._lib import XattnB200Error
    q = torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16)
    with pytest.raises(XattnB200Error):
        Xattention_prefill(q, q, q, stride=16)


def test_reference_import_path():
    from xattn.src.Xattention import Xattention_prefill, xattn_estimate  # noqa: F401
    from xattn.src.utils import find_blocks_chunked  # noqa: F401
