"""ctypes binding of ``libivab.so`` (declared in ``include/ivab.h``).

The library is the only implementation of the operators in this package.  If it is
missing or cannot be loaded, every operator raises ``RuntimeError`` -- there is no
PyTorch or CPU fallback.
"""

from __future__ import annotations

import ctypes
import os
import threading
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

PKG_DIR = os.path.dirname(os.path.abspath(__file__))

OK = 0
ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_WORKSPACE, ERR_DEVICE = -1, -2, -3, -4, -5
F32, F16, BF16, F8E4M3 = 0, 1, 2, 3
STATUS_WAIT_TIMEOUT, STATUS_BAD_PAGE, STATUS_BAD_CTX_LEN, STATUS_BAD_SLOT, STATUS_WORKSPACE_OVERFLOW = 1, 2, 4, 8, 16
OUT_TOKEN_MAJOR, OUT_HEAD_MAJOR = 0, 1

# name -> (restype, argtypes); one entry per declaration in include/ivab.h
SIGNATURES = {
    "ivab_last_error": (c_char_p, []),
    "ivab_version": (c_int, []),
    "ivab_launch_count": (c_int64, []),
    "ivab_kv_gather": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int] + [c_int64] * 11 + [c_void_p, c_void_p]),
    "ivab_kv_gather_rows": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int] + [c_int64] * 11 + [c_void_p, c_void_p]),
    "ivab_compact_indices": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "ivab_kv_scatter": (c_int, [c_void_p, c_void_p, c_void_p, c_int] + [c_int64] * 11 + [c_void_p, c_void_p]),
    "ivab_paged_append": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int64,
                                  c_int64, c_int] + [c_int64] * 5 + [c_void_p, c_void_p]),
    "ivab_paged_append_fp8": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int64,
                                      c_int64, c_int, c_float, c_float] + [c_int64] * 5 + [c_void_p, c_void_p]),
    "ivab_paged_gather": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                  c_int, c_int] + [c_int64] * 6 + [c_void_p, c_void_p]),
    "ivab_decode_workspace_bytes": (c_int, [c_int64, c_int64, c_int64, c_int64, POINTER(c_size_t)]),
    "ivab_paged_decode_attn": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64,
                                       c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p,
                                       c_int, c_int] + [c_int64] * 7 + [c_float, c_void_p, c_size_t, c_void_p]),
    "ivab_paged_decode_attn_noalloc": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64,
                                               c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p,
                                               c_int, c_int] + [c_int64] * 7 + [c_float, c_void_p, c_void_p]),
    "ivab_paged_decode_attn_fp8": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64,
                                           c_float, c_float, c_void_p, c_int64, c_void_p, c_void_p, c_int64,
                                           c_void_p, c_int64, c_int64, c_void_p, c_int, c_int] + [c_int64] * 7 +
                                   [c_float, c_void_p, c_size_t, c_void_p]),
    "ivab_paged_decode_step": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                                       c_int64, c_int64, c_int, c_float, c_float, c_void_p, c_int64, c_void_p, c_void_p,
                                       c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int, c_int] + [c_int64] * 7 +
                               [c_float, c_void_p, c_size_t, c_void_p]),
    "ivab_paged_decode_step_allgather": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                                                 c_int64, c_int64, c_int, c_float, c_float, c_void_p, c_int64, c_void_p, c_void_p,
                                                 c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int] + [c_int64] * 7 +
                                         [c_float, c_void_p, c_size_t,
                                          c_void_p, c_int64, POINTER(c_void_p), c_int, c_int, c_int, c_int64, c_void_p, c_void_p,
                                          c_int64, c_void_p]),
    "ivab_peer_allgather": (c_int, [c_void_p, c_int64, POINTER(c_void_p), c_int, c_int, c_int, c_int64, c_void_p, c_void_p,
                                    c_int64, c_void_p]),
    "ivab_decode_status": (c_int, [c_void_p, POINTER(c_int32), c_void_p]),
    "ivab_selftest_bounded_wait": (c_int, [c_void_p, c_int64, c_void_p]),
}


class IvabError(RuntimeError):
    """A call into libivab.so returned an error code."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libivab error {code}: {message}")
        self.code = code


_lock = threading.Lock()
_lib = None


def lib_path() -> str:
    return os.environ.get("IVAB_LIBRARY", os.path.join(PKG_DIR, "libivab.so"))


def load_library() -> ctypes.CDLL:
    """Load the shared library once; raise loudly if it is not there."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} not found: the CUDA extension is not built (run `python iva1.0_b200/build.py`). "
                "This package has no fallback implementation."
            )
        lib = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)   # AttributeError if the library does not export it
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc: int) -> None:
    """Turn a return code into the exception the reference's operators would raise:
    invalid arguments -> ValueError, everything else -> IvabError (a RuntimeError)."""
    if rc == OK:
        return
    msg = load_library().ivab_last_error().decode("utf-8", "replace")
    if rc in (ERR_INVALID, ERR_UNSUPPORTED):
        raise ValueError(f"libivab: {msg}")
    raise IvabError(rc, msg)


def dtype_code(dtype) -> int:
    import torch

    try:
        return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.float8_e4m3fn: F8E4M3}[dtype]
    except KeyError:
        raise ValueError(f"unsupported KV dtype {dtype}; supported: float32, float16, bfloat16, float8_e4m3fn") from None


def stream_ptr(device) -> int:
    import torch

    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "iva_b200 operators run on CUDA tensors only (got a tensor on "
                f"{t.device}); there is no CPU implementation in this package"
            )


def require_device_readable(*tensors) -> None:
    """CUDA tensors, or pinned host tensors (page-locked memory is mapped into the device's address space under
    unified addressing, so a kernel can read it in place over the bus)."""
    for t in tensors:
        if t is not None and not t.is_cuda and not t.is_pinned():
            raise RuntimeError(
                "iva_b200 operators read CUDA tensors or pinned host tensors only (got pageable memory on "
                f"{t.device}); there is no CPU implementation in this package"
            )


def status_message(status: int) -> str:
    names = []
    for bit, name in ((1, "a bounded in-kernel wait timed out"), (2, "block-table entry out of range"),
                      (4, "context length out of range"), (8, "slot index out of range"),
                      (16, "workspace overflow")):
        if status & bit:
            names.append(name)
    return ", ".join(names) or "ok"
