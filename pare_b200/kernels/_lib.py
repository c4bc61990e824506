"""ctypes binding of libpare_b200.so — the only bridge between Python and the CUDA code.

The library is loaded lazily and exactly once.  There is no alternative backend: if the
shared object is missing, :func:`lib` raises, and every wrapper that needs a kernel fails
with it.  Signatures mirror ``include/pare_b200.h`` one to one.
"""

from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libpare_b200.so"

F16, BF16, F32 = 0, 1, 2
PRODUCER_RMSNORM, PRODUCER_SILU_MUL = 1, 2
_DTYPE_CODE = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}

_lock = threading.Lock()
_lib: C.CDLL | None = None

_vp, _i, _i64, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t

# name -> (restype, argtypes); kept in the order of the header
SIGNATURES: dict[str, tuple] = {
    "pare_version": (_i, []),
    "pare_status_string": (C.c_char_p, [_i]),
    "pare_w4a16_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "pare_w4a16_forward": (_i, [_vp, _i, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64,
                                _i, _i, _i, _i, _vp, _sz, _vp]),
    "pare_w4a16_prepared_bytes": (_sz, [_i, _i]),
    "pare_w4a16_prepare": (_i, [_vp, _i, _i64, _vp, _vp, _i, _i, _vp, _vp]),
    "pare_w4a16_forward_prepared": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i64,
                                         _i, _i, _i, _i, _vp, _sz, _vp]),
    "pare_w4a16_forward_produced": (_i, [_i, _vp, _vp, _vp, _vp, _i64, C.c_float, _i,
                                         _vp, _vp, _vp, _vp, _vp, _vp, _i64,
                                         _i, _i, _i, _i, _vp, _sz, _vp]),
    "pare_kivi_append": (_i, [_vp, _vp, _i, _i64, _i64, _i64, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp,
                              _i, _i, _i, _i, _i, _i, _i, _vp]),
    "pare_kivi_dequant": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i,
                               _vp, _vp, _i, _i64, _i64, _i64, _vp]),
    "pare_kivi_attn_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "pare_kivi_decode_attn": (_i, [_vp, _i, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i,
                                   _vp, _vp, _i64, _i64, _i64, _i,
                                   _vp, _vp, _i64, _i64, _vp,
                                   _vp, _i64, _i64, _vp, C.c_float,
                                   _i, _i, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "pare_prefill_attn": (_i, [_vp, _vp, _vp, _vp, _i, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                               _i, _i, _i, _i, _i, _i, C.c_float, _i, _vp]),
    "pare_rmsnorm_residual": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, C.c_float, _i, _vp]),
    "pare_silu_mul": (_i, [_vp, _vp, _vp, _i, _i, _i64, _i, _vp]),
    "pare_rope": (_i, [_vp, _i64, _i64, _i64, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "pare_peer_buffer_create": (_i, [_sz, C.POINTER(C.c_void_p), C.c_char_p]),
    "pare_peer_buffer_open": (_i, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "pare_peer_buffer_close": (_i, [_vp]),
    "pare_peer_buffer_destroy": (_i, [_vp]),
    "pare_peer_status": (_i, [_vp, _vp]),
    "pare_peer_allreduce": (_i, [_vp, _i64, _vp, _i64, _i, _i, _i, _i, _i, C.POINTER(C.c_void_p), _sz, _vp]),
    "pare_w4a16_forward_prepared_allreduce": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i64,
                                                   _i, _i, _i, _i, _vp, _sz, _i, _i, C.POINTER(C.c_void_p), _sz, _vp]),
    "pare_w4a16_forward_produced_allreduce": (_i, [_i, _vp, _vp, _vp, _vp, _i64, C.c_float, _i,
                                                   _vp, _vp, _vp, _vp, _vp, _vp, _i64,
                                                   _i, _i, _i, _i, _vp, _sz, _i, _i, C.POINTER(C.c_void_p), _sz, _vp]),
    "pare_workspace_status": (_i, [_vp, _vp]),
    "pare_selftest_bounded_wait": (_i, [_vp, C.c_uint, _vp]),
    "pare_w4a16_static_status": (_i, [_vp]),
    "pare_w4a16_static_scratch_bytes": (_sz, []),
    "pare_w4a16_forward_static": (_i, [_vp, _i, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64,
                                       _i, _i, _i, _i, _vp]),
}


class KernelLibraryError(RuntimeError):
    """The CUDA library is missing, failed to load, or a call returned an error status."""


def lib() -> C.CDLL:
    """Return the loaded library, loading it on first use."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not LIB_PATH.exists():
                    raise KernelLibraryError(
                        f"{LIB_PATH} not found — build it with `python -m pare_b200.build` "
                        "(there is no fallback implementation)"
                    )
                handle = C.CDLL(str(LIB_PATH))
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(handle, name)
                    fn.restype = res
                    fn.argtypes = args
                _lib = handle
    return _lib


def available() -> bool:
    """True when the library file exists and a CUDA device is visible."""
    return LIB_PATH.exists() and torch.cuda.is_available()


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelLibraryError(f"dtype {dtype} is not supported by libpare_b200") from None


def check(status: int, what: str) -> None:
    if status != 0:
        msg = lib().pare_status_string(status).decode()
        raise KernelLibraryError(f"{what} failed: {msg} (status {status})")


def ptr(t: torch.Tensor | None) -> int | None:
    """Device address of a tensor (None stays None → NULL)."""
    return None if t is None else t.data_ptr()


def current_stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


# One zero-initialised workspace per device and stream; the kernels leave it zero-consistent.
_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def workspace_status(device: torch.device) -> int:
    """Status word of the current stream's workspace on ``device``: 0, or the time-out code if a bounded wait inside a
    kernel gave up since the last read.  Synchronises the stream and clears the word; 0 if no workspace exists yet."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None:
        return 0
    return lib().pare_workspace_status(buf.data_ptr(), current_stream(device))


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-filled scratch buffer of at least ``nbytes`` for the current stream of ``device``."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        size = max(nbytes, 8 << 20)
        buf = torch.zeros(size, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf
