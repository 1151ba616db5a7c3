"""ctypes binding of ``lib/libcpb.so`` (the sm_100a kernels and the C++ runtime).

The library has a plain C ABI: every launcher takes raw device pointers, sizes and a CUDA stream
and returns 0 or a negative error code whose text is available from ``cpb_last_error``.  Python
passes ``tensor.data_ptr()`` and ``torch.cuda.current_stream().cuda_stream``.

On a machine with a GPU a missing or unloadable library is a hard error: the CUDA ops never fall
back to PyTorch silently.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_long, c_void_p
from pathlib import Path
from typing import Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libcpb.so"


class NativeError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    """Load (once) and return the native library."""
    global _LIB
    if _LIB is None:
        if not _LIB_PATH.exists():
            if os.environ.get("CPB_NO_AUTOBUILD", "0") == "1":
                raise NativeError(f"{_LIB_PATH} is missing; run `python -m context_parallelism_b200._build`")
            from . import _build
            _build.build()
        # libnccl / libcudart are provided by the already-imported torch; load with global symbols visible
        _LIB = ctypes.CDLL(str(_LIB_PATH), mode=ctypes.RTLD_GLOBAL)
        _LIB.cpb_last_error.restype = c_char_p
    return _LIB


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = lib().cpb_last_error().decode(errors="replace")
        raise NativeError(f"{what} failed (code {rc}): {msg}")


def stream_ptr(device=None) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0) if t is None else c_void_p(t.data_ptr())


LAUNCHES = [0]          # number of kernel launchers invoked (each launches exactly one of our kernels)
_FN_CACHE = {}
_PROFILE = None         # name -> list of (start event, end event) while a per-kernel device timing is being taken


def call(name: str, *args) -> None:
    """Invoke ``cpb_<name>`` with already-converted ctypes arguments and raise on error."""
    fn = _FN_CACHE.get(name)
    if fn is None:
        fn = getattr(lib(), "cpb_" + name)
        fn.restype = c_int
        _FN_CACHE[name] = fn
    LAUNCHES[0] += 1
    if _PROFILE is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = fn(*args)
        e1.record()
        _PROFILE.setdefault(name, []).append((e0, e1))
    else:
        rc = fn(*args)
    if rc != 0:
        check(rc, name)


def profile_start() -> None:
    """Start timing every launcher call with a pair of CUDA events on the stream it is issued to (diagnostics:
    device time per kernel name without a profiler; for the cross-rank barrier kernels this is the time spent
    waiting for the slowest peer)."""
    global _PROFILE
    _PROFILE = {}


def profile_stop():
    """Stop timing; returns ``{name: (calls, total_ms)}`` after one device synchronisation."""
    global _PROFILE
    prof, _PROFILE = _PROFILE, None
    torch.cuda.synchronize()
    return {k: (len(v), sum(a.elapsed_time(b) for a, b in v)) for k, v in (prof or {}).items()}


# --------------------------------------------------------------------------- kernel status words
_STATUS_CODES = {1: "mbarrier wait timed out", 2: "peer/readiness flag wait timed out", 3: "index out of range"}


class KernelStatus:
    """A 4-int device word ``[code, site, block, aux]`` kernels report bounded-wait expiry and
    bounds-check failures into; the host turns a non-zero code into an exception."""

    def __init__(self, device):
        self.buf = torch.zeros(4, dtype=torch.int32, device=device)

    def ptr(self) -> c_void_p:
        return c_void_p(self.buf.data_ptr())

    def check(self, what: str = "kernel") -> None:
        code, site, block, aux = self.buf.tolist()
        if code != 0:
            self.buf.zero_()
            raise NativeError(f"{what}: {_STATUS_CODES.get(code, 'error %d' % code)} "
                              f"(site {site}, block {block}, aux {aux})")


_status_cache = {}


def status_for(device) -> KernelStatus:
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    st = _status_cache.get(key)
    if st is None:
        st = _status_cache[key] = KernelStatus(torch.device("cuda", key))
    return st


def f(x) -> c_float:
    return c_float(float(x))


def i(x) -> c_int:
    return c_int(int(x))


def l(x) -> c_long:
    return c_long(int(x))
