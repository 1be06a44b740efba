"""The C-ABI library loads without a GPU and exports exactly what the header declares."""
import ctypes as C
import os

from ksearch_b200 import _lib


def test_library_exports_every_header_symbol():
    lib = _lib.load()
    names = _lib.header_symbols()
    assert len(names) >= 39
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ksearch_cuda.h but not exported"


def test_python_signatures_cover_header():
    assert sorted(_lib.SIGNATURES) == _lib.header_symbols()


def test_no_torch_or_python_dependency():
    import subprocess
    out = subprocess.run(["ldd", _lib.LIB_PATH], capture_output=True, text=True).stdout
    assert "torch" not in out and "python" not in out


def test_context_creation_fails_loudly_without_gpu():
    """No CPU fallback: without a usable sm_100 device ks_ctx_create returns NULL and says why.
    (On a GPU box this test creates and destroys a context instead.)"""
    lib = _lib.load()
    h = lib.ks_ctx_create(0, 0)
    if h:
        assert lib.ks_ctx_sm_count(h) > 0
        lib.ks_ctx_destroy(h)
    else:
        msg = lib.ks_last_error(None).decode()
        assert msg, "a failed create must leave a message"


def test_size_helpers_need_no_gpu():
    lib = _lib.load()
    assert lib.ks_sdpa_tmp_floats(1, 8, 256, 16) == 8 * 16 * 258
    assert lib.ks_sdpa_tmp_floats(4, 8, 256, 1) == 0
    assert lib.ks_buf_size(None) == 0
