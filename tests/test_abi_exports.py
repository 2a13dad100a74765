"""The C-ABI library builds for sm_100a, loads, and exports every symbol that
include/b200tp.h declares.  No compute call is made (CPU only)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib_path():
    import __graft_entry__ as entry
    entry.build()
    path = os.path.join(ROOT, "nano-vllm_b200", "lib", "libb200tp.so")
    assert os.path.exists(path)
    return path


def declared_functions():
    text = open(os.path.join(ROOT, "include", "b200tp.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_path():
    names = declared_functions()
    for must in ("b2_ctx_create", "b2_symm_export", "b2_symm_import", "b2_ctx_destroy", "b2_status", "b2_gemm", "b2_rowpar_fused",
                 "b2_rmsnorm", "b2_add_rmsnorm", "b2_store_kvcache", "b2_embed", "b2_lm_head"):
        assert must in names


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(lib_path)
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in include/b200tp.h but not exported: {missing}"


def test_binding_covers_every_declared_symbol(lib_path, pkg):
    from nanovllm_b200 import _abi
    assert sorted(_abi.EXPORTED) == declared_functions()
    assert _abi.launch_count() >= 0


def test_argument_errors_without_a_gpu(lib_path, pkg):
    """Entry points validate their arguments before touching CUDA."""
    from nanovllm_b200 import _abi
    lib = _abi.lib
    assert lib.b2_store_kvcache(None, 128, None, 128, None, None, None, 0, 128, None) == _abi.OK      # empty input is a no-op
    assert lib.b2_store_kvcache(None, 128, None, 128, None, None, None, 4, 128, None) == _abi.ERR_ARG  # null pointers
    assert lib.b2_store_kvcache(None, 128, None, 128, None, None, None, 4, 100, None) == _abi.ERR_ARG  # D not a multiple of 8
    assert lib.b2_rmsnorm(None, 128, None, 1e-6, 0, 128, None, 128, None) == _abi.OK
    assert lib.b2_rmsnorm(None, 128, None, 1e-6, 3, 127, None, 128, None) == _abi.ERR_ARG
    assert lib.b2_gemm(None, None, 8, None, 8, None, None, 8, 1, 8, 8, None) == _abi.ERR_ARG           # no context
    assert lib.b2_ctx_destroy(None) == _abi.ERR_ARG
