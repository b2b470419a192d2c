"""ctypes view of ``liberedu_cuda.so`` (the ``eredu_*`` C ABI of the sm_100a kernels).

The library is built in-tree by :mod:`eredu_b200.build`. On a machine with a GPU a missing library
is an error, never a silent fallback: ``lib()`` raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p, POINTER
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "liberedu_cuda.so"
_lib = None

P, I, F, L = c_void_p, c_int, c_float, c_longlong

_SIGNATURES = {
    # name: (restype, [argtypes])
    "eredu_gemm_pick_split": (I, [I, I, I, I]),
    "eredu_gemm_bf16": (I, [P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, I, P, P, I, F, I, P, I, P]),
    "eredu_attn_prefill": (I, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P]),
    "eredu_attn_decode": (I, [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P]),
    "eredu_peer_send": (I, [P, I, I, P, L, P, I, P, P]),
    "eredu_peer_recv": (I, [P, I, I, P, L, P, I, P, P]),
    "eredu_attn_prefill_tc": (I, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, P, P]),
    "eredu_attn_decode_scratch_elems": (None, [I, I, I, I, I, POINTER(L), POINTER(L)]),
    "eredu_attn_decode_rope": (I, [P, I, P, P, P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, F, F, F, P]),
    "eredu_rmsnorm": (I, [P, P, P, P, P, I, I, F, F, P]),
    "eredu_rope_kv": (I, [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, F, F, P]),
    "eredu_embedding": (I, [P, P, P, I, I, I, I, F, P, P]),
    "eredu_silu_mul": (I, [P, P, I, I, I, F, P]),
    "eredu_decode_advance": (I, [P, P, P, P, P, P, I, P, P, I, P, I, I, P]),
    "eredu_sampler_row_bytes": (I, []),
    "eredu_launch_count": (L, []),
    "eredu_selftest_bounded_wait": (I, [P, L, P]),
    "eredu_sample": (I, [P, P, I, P, P, I, P, P, I, I, P]),
    "eredu_spec_verify": (I, [P, P, P, P, P, I, I, I, P]),
}


def available() -> bool:
    return _LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: run `python -m eredu_b200.build` (needs nvcc) before using CUDA tensors"
            )
        handle = ctypes.CDLL(str(_LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            try:
                fn = getattr(handle, name)
            except AttributeError:
                continue
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def register(name: str, restype, argtypes) -> None:
    """Declare another exported symbol (used by modules that own their kernels' signatures)."""
    _SIGNATURES[name] = (restype, argtypes)
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype = restype
        fn.argtypes = argtypes


def launch_count() -> int:
    """Kernel launches issued so far by this library's launchers (graph replays are not counted)."""
    return int(lib().eredu_launch_count())


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_status: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word where kernels record a bounded-wait timeout (0 = ok)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


STATUS_NAMES = {
    0: "ok",
    1: "TMA stage never landed",
    2: "shared-memory stage never released",
    3: "accumulator never committed",
    4: "peer flag never arrived",
    5: "bad argument",
}


def check_status(device: torch.device) -> None:
    """Synchronising read of the status word; raises if a kernel gave up on a wait."""
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        raise RuntimeError(f"eredu kernel reported status {code}: {STATUS_NAMES.get(code, 'unknown')}")


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with code {code}")


class Completion:
    """An exact completion of the work submitted to a stream so far (``ExecutionBackend::Completion``,
    eredu-core/src/execution.rs): a CUDA event plus an asynchronous copy of the device's status word taken at the same
    point of the stream. ``is_ready`` polls without blocking; ``wait`` blocks and turns a recorded bounded-wait timeout
    into an exception, so an error surfaces at the completion of the step that raised it and not at some later check.
    On CPU the work is already done when the object is made."""

    def __init__(self, device=None, stream=None):
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self._event = None
        self._status = None
        self._done = self.device.type != "cuda"
        if not self._done:
            s = stream or torch.cuda.current_stream(self.device)
            with torch.cuda.stream(s):
                self._status = torch.empty(1, dtype=torch.int32).pin_memory()
                self._status.copy_(status_word(self.device), non_blocking=True)
                self._event = torch.cuda.Event()
                self._event.record(s)

    def is_ready(self) -> bool:
        return self._done or self._event.query()

    def wait(self, timeout_s: float | None = None) -> None:
        """Blocks until the recorded point is reached (``timeout_s``: poll with that limit and raise TimeoutError)."""
        if self._done:
            return
        if timeout_s is None:
            self._event.synchronize()
        else:
            import time

            t0 = time.monotonic()
            while not self._event.query():
                if time.monotonic() - t0 > timeout_s:
                    raise TimeoutError(f"device work did not complete within {timeout_s} s")
                time.sleep(0.0002)
        self._done = True
        code = int(self._status[0])
        if code != 0:
            status_word(self.device).zero_()
            raise RuntimeError(f"eredu kernel reported status {code}: {STATUS_NAMES.get(code, 'unknown')}")
