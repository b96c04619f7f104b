"""The C-ABI library loads on a machine without a GPU and exports exactly what include/ivab.h
declares.  No compute entry point is called here."""

import ctypes
import os
import re

import iva_b200
from iva_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "ivab.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ivab_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared()
    for must in ("ivab_kv_gather", "ivab_kv_scatter", "ivab_paged_append", "ivab_paged_gather",
                 "ivab_paged_decode_attn", "ivab_decode_workspace_bytes", "ivab_decode_status", "ivab_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(built_library)
    for name in _declared():
        assert hasattr(lib, name), f"{name} declared in include/ivab.h but not exported"


def test_python_binding_covers_the_header(built_library):
    assert sorted(_lib.SIGNATURES) == _declared()
    lib = iva_b200.load_library()
    assert lib.ivab_version() >= 110
    assert lib.ivab_last_error() is not None


def test_argument_validation_needs_no_gpu(built_library):
    """Pure host-side checks: they return an error code before touching the device."""
    lib = iva_b200.load_library()
    rc = lib.ivab_kv_gather(None, None, None, 7, 7, 1, 1, 1, 32, 1, 0, 0, 0, 0, 0, 0, None, None)
    assert rc == _lib.ERR_INVALID and b"dtype" in lib.ivab_last_error()
    rc = lib.ivab_kv_gather(None, None, None, _lib.F16, _lib.F16, 1, 1, 1, 12, 1, 0, 0, 0, 0, 0, 0, None, None)
    assert rc == _lib.ERR_UNSUPPORTED                      # 24-byte rows are not 16-byte multiples
    rc = lib.ivab_kv_gather(None, None, None, _lib.F16, _lib.F16, 1, 1, 1, 64, 1, 64, 64, 64, 64, 64, 64, None, None)
    assert rc == _lib.ERR_INVALID and b"null" in lib.ivab_last_error()
    n = ctypes.c_size_t(0)
    assert lib.ivab_decode_workspace_bytes(64, 32, 32, 128, ctypes.byref(n)) == 0 and n.value > 0
    assert lib.ivab_decode_workspace_bytes(64, 32, 5, 128, ctypes.byref(n)) == _lib.ERR_INVALID


def test_plain_c_client_binds_and_validates(built_library, tmp_path):
    """tests/abi_client.c is C99: it includes include/ivab.h, binds the library with dlopen the way a
    foreign-function layer would, and checks the host-side argument validation.  No GPU needed."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc") or shutil.which("cc")
    assert gcc, "a C compiler is part of the toolchain this library is built with"
    exe = str(tmp_path / "abi_client")
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "abi_client.c"), "-o", exe, "-ldl"], check=True)
    res = subprocess.run([exe, built_library], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and "abi client ok" in res.stdout, res.stdout + res.stderr


def test_workspace_size_follows_the_head_grouping(built_library):
    """Head ratios above 8 are served as equal groups of at most 8 query heads, each numbered like a
    KV head of its own: 32 query / 2 KV heads (ratio 16 = 2 x 8) plans -- and sizes its workspace --
    like 32 / 4.  Host-side arithmetic only."""
    lib = iva_b200.load_library()

    def need(b, hq, hkv, d):
        n = ctypes.c_size_t(0)
        assert lib.ivab_decode_workspace_bytes(b, hq, hkv, d, ctypes.byref(n)) == 0
        return n.value

    assert need(8, 32, 2, 128) == need(8, 32, 4, 128)        # 16 -> 2 groups of 8
    assert need(8, 24, 2, 128) == need(8, 24, 4, 128)        # 12 -> 2 groups of 6
    assert need(8, 64, 1, 128) == need(8, 64, 8, 128)        # multi-query, 64 -> 8 groups of 8
    assert need(8, 18, 2, 64) == need(8, 18, 6, 64)          # 9 -> 3 groups of 3
