"""The C ABI: the shared library builds for sm_100a, loads without a GPU and exports every
function that include/logo_b200.h declares; nothing is computed here."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "logo_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(?:int|size_t)\s+(logo_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for required in ("logo_select_rows", "logo_sq_attn_fwd", "logo_sq_attn_bwd", "logo_swa_fwd", "logo_swa_bwd",
                     "logo_fuse_fwd", "logo_fuse_bwd", "logo_decode_attn", "logo_cache_append", "logo_last_error",
                     "logo_version"):
        assert required in names


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(str(lib_path))
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_python_binding_covers_the_header(lib_path):
    from logo_b200 import _lib

    assert set(_lib.exported_symbols()) == set(declared_functions())
    lib = _lib.load()
    assert lib.logo_version() >= 100


def test_argument_validation_needs_no_gpu(lib_path):
    """Bad arguments are rejected on the host before any CUDA call."""
    from logo_b200 import _lib

    lib = _lib.load()
    # head_dim 64 is not implemented
    rc = lib.logo_sq_attn_fwd(None, None, None, None, None, None, None, None, None, None, None, 1, 16, 2, 1, 64, 0.1,
                              0, None, None)
    assert rc == 3 and "head_dim" in _lib.last_error()
    # hq not a multiple of h
    rc = lib.logo_swa_fwd(None, None, None, None, None, None, None, None, 1, 16, 3, 2, 128, 128, 0.1, None, None)
    assert rc == 1
    rc = lib.logo_swa_fwd(None, None, None, None, None, None, None, None, 1, 0, 2, 2, 128, 0, 0.1, None, None)
    assert rc == 1 and "window" in _lib.last_error()
    assert lib.logo_select_workspace_bytes(32768) >= 16 * 12
    assert lib.logo_decode_workspace_bytes(4, 16, 4096) > 0
    with pytest.raises(RuntimeError):
        _lib.check(rc, "logo_swa_fwd")


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from logo_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "liblogo_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_cpu_tensors_are_rejected(lib_path):
    import torch
    from logo_b200 import ops

    q = torch.zeros(1, 8, 2, 128, dtype=torch.bfloat16)
    sel = torch.ones(1, 8, dtype=torch.bool)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.sq_full_attn(q, q, q, sel, cu_seqlens=torch.tensor([0, 8], dtype=torch.int32))
    # the reference's own argument checks come first (selected_full_attn.py:516-522)
    with pytest.raises(AssertionError, match="cu_seqlens"):
        ops.sq_full_attn(q, q, q, sel)
    with pytest.raises(AssertionError, match="B=1"):
        ops.sq_full_attn(q.expand(2, -1, -1, -1), q.expand(2, -1, -1, -1), q.expand(2, -1, -1, -1),
                         sel.expand(2, -1), cu_seqlens=torch.tensor([0, 8]))
