"""The C-ABI library builds, loads, and exports every symbol include/sgl_b200.h declares (no GPU needed)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "sgl_b200.h")


def _declared():
    txt = open(HEADER).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    decls = {}
    for m in re.finditer(r"\b(?:int64_t|int|size_t|const char\*)\s+(sgl_\w+)\s*\(([^;]*?)\)\s*;", txt, flags=re.S):
        args = m.group(2).strip()
        n = 0 if args in ("", "void") else len([a for a in args.split(",") if a.strip()])
        decls[m.group(1)] = n
    return decls


@pytest.fixture(scope="module")
def lib_path():
    import importlib.util
    spec = importlib.util.spec_from_file_location("sgl_build", os.path.join(ROOT, "starrygl-framework_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build()


def test_header_declares_entry_points():
    d = _declared()
    assert len(d) >= 25
    for must in ("sgl_tcsr_build", "sgl_sample_layer", "sgl_unique_pairs", "sgl_build_csc", "sgl_gather_rows",
                 "sgl_cache_gather", "sgl_route_pack", "sgl_route_unpack", "sgl_seeds_in_window"):
        assert must in d


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(lib_path)
    for name in _declared():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    lib.sgl_build_info.restype = ctypes.c_char_p
    assert b"sm_100a" in lib.sgl_build_info()


def test_ctypes_signatures_match_header(lib_path):
    from starrygl import _C
    d = _declared()
    assert set(_C._SIGNATURES) == set(d), set(_C._SIGNATURES) ^ set(d)
    for name, (_, args) in _C._SIGNATURES.items():
        assert len(args) == d[name], (name, len(args), d[name])


def test_argument_errors_need_no_gpu(lib_path):
    """Host-side validation happens before any CUDA call, so these paths run on a machine without a GPU."""
    from starrygl import _C
    L = _C.lib()
    assert L.sgl_radix_sort_ws_bytes(4096) > 0 and L.sgl_tcsr_build_ws_bytes(10, 100) > 0
    rc = L.sgl_sample_layer(None, None, None, None, 10, None, None, 4, None, 0, 0, 0, -1, 0, 0, 0, None, None, None, None,
                            None, None, None, None, None, 0, None)
    assert rc == -1 and b"fanout" in L.sgl_last_error()
    rc = L.sgl_sample_layer(None, None, None, None, 10, None, None, 4, None, 513, 1, 0, -1, 0, 0, 0, None, None, None, None,
                            None, None, None, None, None, 0, None)
    assert rc == -5 and b"uniform fanout" in L.sgl_last_error()
    rc = L.sgl_unique_pairs(None, None, 4, None, None, None, 0, None, 40, 40, 0, None, None, None, None, None, None, None,
                            0, None)
    assert rc == -5
    rc = L.sgl_gather_rows(None, 4, 6, 6, None, None, 0, 3, None, None, 6, None, None, 0, None, None)
    assert rc == -5   # rows must be multiples of 4 bytes


def test_cpu_tensors_are_refused():
    import torch
    from starrygl import _C, ops
    with pytest.raises(_C.SglError):
        _C.ptr(torch.zeros(4))
    with pytest.raises(_C.SglError):
        ops.gather_rows(torch.zeros(4, 4), torch.zeros(2, dtype=torch.int64))


def test_missing_library_fails_loudly(monkeypatch):
    from starrygl import _C
    monkeypatch.setattr(_C, "_lib", None)
    monkeypatch.setattr(_C, "LIB_PATH", "/nonexistent/libsgl_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _C.lib()
