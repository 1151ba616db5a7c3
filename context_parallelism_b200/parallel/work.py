"""Asynchronous work handle with a deadline (``csrc/runtime/work.cpp``): a CUDA event recorded after a piece of
stream work plus a wall-clock limit watched by a background thread, so the host waits by polling a state word instead
of blocking inside the driver, and a step that never finishes becomes an exception instead of a hang.  Mirrors the
reference's ``Work`` (process_group/CpuSync_fixed.hpp:89-187: ``wait`` / ``streamWait`` / ``query``) and supplies the
time-out watcher it left commented out (process_group/processGroupNCCL.cpp:719-744)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native as nv

PENDING, DONE, TIMED_OUT, ERROR = 0, 1, 2, 3


class StepTimeout(RuntimeError):
    pass


class Work:
    def __init__(self, device: Optional[torch.device], timeout_s: float, stream: Optional[torch.cuda.Stream] = None):
        """Records an event on ``stream`` (default: the current stream of ``device``); ``device=None`` makes a
        host-only handle that its owner completes with :meth:`complete`."""
        lib = nv.lib()
        h = ctypes.c_void_p()
        if device is not None and device.type == "cuda":
            s = stream.cuda_stream if stream is not None else torch.cuda.current_stream(device).cuda_stream
            nv.check(lib.cpb_work_create(ctypes.c_void_p(s), 1, ctypes.c_double(timeout_s), ctypes.byref(h)), "work_create")
        else:
            nv.check(lib.cpb_work_create(ctypes.c_void_p(0), 0, ctypes.c_double(timeout_s), ctypes.byref(h)), "work_create")
        self._h = h

    def query(self) -> int:
        return int(nv.lib().cpb_work_query(self._h))

    def complete(self) -> None:
        nv.lib().cpb_work_complete(self._h)

    def stream_wait(self, stream: torch.cuda.Stream) -> None:
        nv.check(nv.lib().cpb_work_stream_wait(self._h, ctypes.c_void_p(stream.cuda_stream)), "work_stream_wait")

    def wait(self, poll_s: float = 2e-4) -> int:
        """Block the host (polling) until done, timed out or failed; returns the final state."""
        return int(nv.lib().cpb_work_wait(self._h, ctypes.c_double(poll_s)))

    def close(self) -> None:
        if self._h is not None:
            nv.lib().cpb_work_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def wait_for_stream(device: torch.device, timeout_s: float, what: str = "step") -> None:
    """Host-side wait for everything queued on the current stream of ``device``, bounded by ``timeout_s``."""
    w = Work(device, timeout_s)
    try:
        st = w.wait()
    finally:
        w.close()
    if st == TIMED_OUT:
        raise StepTimeout(f"{what} did not finish within {timeout_s:.0f} s (CP_WATCHDOG_S); a rank or a collective is stuck")
    if st == ERROR:
        raise nv.NativeError(f"{what}: CUDA reported an error while waiting")
