"""ctypes binding of ``liblogo_b200.so`` (the C ABI declared in ``include/logo_b200.h``).

There is no fallback: if the shared library is missing or a call fails, an exception is
raised. Build the library with ``python -m logo_b200.build``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_size_t, c_uint32, c_void_p
from pathlib import Path
from typing import Optional

import os

# LOGO_B200_LIB points at another build of the same library (e.g. one compiled with extra diagnostics)
LIB_PATH = Path(os.environ.get("LOGO_B200_LIB") or (Path(__file__).resolve().parent / "liblogo_b200.so"))

DTYPE_BF16, DTYPE_F32, DTYPE_F16, DTYPE_BOOL = 0, 1, 2, 3

DEVICE_STATUS_TEXT = {
    0: "ok",
    1: "a bounded barrier wait expired inside a kernel (results invalid)",
    2: "an index derived from q_idx / cu_seqlens was out of range",
    3: "the prefix-scan look-back gave up",
}

# name -> (restype, argtypes); mirrors include/logo_b200.h one to one
_SIGNATURES = {
    "logo_version": (c_int, []),
    "logo_last_error": (c_int, [c_char_p, c_int]),
    "logo_select_workspace_bytes": (c_size_t, [c_int]),
    "logo_select_rows": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "logo_select_rows_static": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "logo_sq_attn_fwd": (c_int, [c_void_p] * 11 + [c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
                                                   c_void_p]),
    "logo_swa_fwd": (c_int, [c_void_p] * 8 + [c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]),
    "logo_attn_bwd_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "logo_set_backward_mode": (c_int, [c_int, c_int]),
    "logo_get_backward_mode": (c_int, [c_int]),
    "logo_sq_attn_bwd": (c_int, [c_void_p] * 16 + [c_size_t, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                                   c_void_p]),
    "logo_swa_bwd": (c_int, [c_void_p] * 13 + [c_size_t, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                               c_void_p]),
    "logo_fuse_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
                              c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "logo_fuse_bwd_workspace_bytes": (c_size_t, [c_int]),
    "logo_fuse_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int,
                              c_void_p, c_size_t, c_void_p]),
    "logo_rmsnorm_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_float, c_void_p]),
    "logo_silu_mul": (c_int, [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p]),
    "logo_rope": (c_int, [c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                          c_void_p]),
    "logo_proj_rope": (c_int, [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                               c_int, c_int, c_void_p, c_void_p]),
    "logo_cache_append": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_longlong, c_void_p,
                                  c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                  c_int, c_void_p, c_void_p]),
    "logo_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "logo_decode_attn": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                 c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                 c_int, c_float, c_void_p, c_size_t, c_void_p, c_void_p]),
    "logo_shift_labels": (c_int, [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p]),
    "logo_ce_rows": (c_int, [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_float, c_int, c_int, c_int,
                             c_void_p, c_void_p]),
    "logo_profile_enable": (c_int, [c_int]),
    "logo_profile_reserve": (c_int, [c_int]),
    "logo_profile_read": (c_int, [c_void_p, c_void_p, c_int]),
    "logo_umma_selftest": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32,
                                   c_void_p, c_void_p]),
}

_lib: Optional[ctypes.CDLL] = None


def exported_symbols():
    """Names every build of the library must export (used by the CPU-only ABI test)."""
    return sorted(_SIGNATURES)


def load() -> ctypes.CDLL:
    """Load the shared library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA library has not been built. "
            "Run `python -m logo_b200.build` (needs nvcc); there is no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name, None)
        if fn is None:
            raise RuntimeError(f"{LIB_PATH} does not export `{name}`; rebuild it with `python -m logo_b200.build`")
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    buf = ctypes.create_string_buffer(512)
    load().logo_last_error(buf, 512)
    return buf.value.decode(errors="replace")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed (code {rc}): {last_error()}")


def ptr(t) -> Optional[int]:
    """Device pointer of a tensor (None stays NULL)."""
    return None if t is None else t.data_ptr()


def torch_dtype_code(dtype) -> int:
    import torch

    table = {torch.bfloat16: DTYPE_BF16, torch.float32: DTYPE_F32, torch.float16: DTYPE_F16, torch.bool: DTYPE_BOOL}
    if dtype not in table:
        raise TypeError(f"unsupported dtype {dtype}")
    return table[dtype]


def on_device(t):
    """Context manager that makes the device of tensor ``t`` current for the enclosed C-ABI calls.

    The library launches on, and keys its per-device caches by, the calling thread's current
    device; a tensor on ``cuda:1`` while ``cuda:0`` is current would otherwise hand the library a
    stream of another device."""
    import torch

    return torch.cuda.device(t.device)


def current_stream_ptr(device) -> int:
    import torch

    return torch.cuda.current_stream(device).cuda_stream
