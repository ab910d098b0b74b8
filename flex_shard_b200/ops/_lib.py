"""Loader for the native sm_100a library (``flex_shard_b200/lib/libfsb200.so``).

The library exposes a C ABI; Python passes raw device pointers and the current
CUDA stream. On a machine with a GPU a missing library is an error (the ops do
not fall back to PyTorch silently); on a CPU-only machine ``available()`` is
False and callers use their CPU reference paths.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libfsb200.so"
_lib = None
_lock = threading.Lock()
_status: dict[int, torch.Tensor] = {}

STATUS_NAMES = {
    0: "ok",
    1: "bad argument",
    2: "TMA descriptor encode failed",
    3: "kernel launch failed",
    16: "timeout waiting for a TMA stage",
    17: "timeout waiting for a free stage",
    18: "timeout waiting for a TMEM accumulator",
    19: "timeout waiting for a free TMEM accumulator",
    32: "timeout waiting for a peer signal",
    64: "size beyond the supported maximum",
}


class NativeError(RuntimeError):
    pass


_launches = 0  # native kernel launches issued through this package


def count_launch(n: int = 1) -> None:
    global _launches
    _launches += n


def launch_count() -> int:
    return _launches


def lib_path() -> Path:
    return _LIB_PATH


def load(required: bool = True):
    """Return the ctypes handle of the native library, building it if asked by env."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not _LIB_PATH.exists() and os.environ.get("FSB200_BUILD_ON_IMPORT", "0") == "1":
            from ..csrc.build import build

            build()
        if not _LIB_PATH.exists():
            if required:
                raise NativeError(
                    f"native library {_LIB_PATH} is missing; run "
                    "`python -m flex_shard_b200.csrc.build`"
                )
            return None
        _lib = ctypes.CDLL(str(_LIB_PATH))
        _declare(_lib)
    return _lib


def available() -> bool:
    """True when CUDA kernels can run: a GPU is visible and the library loads."""
    if not torch.cuda.is_available():
        return False
    return load(required=True) is not None


def _declare(lib) -> None:
    c = ctypes
    vp, i32, i64, f32 = c.c_void_p, c.c_int, c.c_longlong, c.c_float
    sigs = {
        "fsb_gemm_bf16": [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, i32, i32, i32, i32,
                          f32, f32, i32, i64, i64, vp, i32, vp, i32, vp],
        "fsb_rmsnorm_fwd": [vp, vp, vp, vp, vp, vp, i64, i32, f32, vp],
        "fsb_rmsnorm_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i64, i32, vp],
        "fsb_rope": [vp, vp, i64, i32, i32, i32, i64, i32, vp],
        "fsb_swiglu_fwd": [vp, vp, i64, i32, vp],
        "fsb_swiglu_bwd": [vp, vp, vp, i64, i32, vp],
        "fsb_cross_entropy": [vp, vp, vp, i64, i32, i64, f32, i64, vp],
        "fsb_adamw": [vp, vp, vp, vp, vp, i64, i32, i32, f32, f32, f32, f32, f32, i32, f32, vp],
        "fsb_cast_scale": [vp, vp, i64, i32, f32, i32, vp],
        "fsb_segment_op": [vp, i32, i32, vp],
        "fsb_segment_op_host": [vp, i32, i32, vp],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = args
        fn.restype = c.c_int


def declare(name: str, argtypes) -> None:
    """Register the signature of a symbol added by a later source file."""
    fn = getattr(load(), name)
    fn.argtypes = argtypes
    fn.restype = ctypes.c_int


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


STATUS_INTS = 8     # [0] code; a failed peer wait also leaves [1],[2] flag address, [3] epoch, [4] peer, [5] value seen


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 record the kernels write an error code to when a bounded wait runs out (element 0;
    a failed wait on a peer's flag adds which flag, epoch and peer in the following elements)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(STATUS_INTS, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


# (first flag address, bytes of flags, name) of every live symmetric region: turns the address in a failure
# record into "which wait"
_flag_ranges: list = []


def register_flag_range(base: int, nbytes: int, name, slot_bytes: int) -> None:
    _flag_ranges.append((base, nbytes, name, slot_bytes))
    del _flag_ranges[:-4096]


def _describe(rec) -> str:
    code = int(rec[0])
    text = f"device-side failure: {STATUS_NAMES.get(code, code)} (code {code})"
    addr = (int(rec[1]) & 0xFFFFFFFF) | ((int(rec[2]) & 0xFFFFFFFF) << 32)
    if code == 32 and addr:
        where = f"flag at {addr:#x}"
        for base, nbytes, name, slot_bytes in reversed(_flag_ranges):
            if base <= addr < base + nbytes:
                where = f"{name() if callable(name) else name}, flag slot {(addr - base) // slot_bytes}"
                break
        text += (f": waited for epoch {int(rec[3]) & 0xFFFFFFFF} from group rank {int(rec[4])} on {where}, "
                 f"last value seen {int(rec[5]) & 0xFFFFFFFF}")
    return text


def check_status(device=None) -> None:
    """Synchronise and raise if any kernel on ``device`` reported a failed wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    t = status_word(dev)
    rec = t.tolist()
    if rec[0] != 0:
        t.zero_()
        raise NativeError(_describe(rec))
    for hook in _check_hooks:
        hook()


_polls: dict[int, tuple] = {}
_check_hooks: list = []      # extra debug checks run by check_status (e.g. guard bytes behind symmetric regions)


def poll_status(device=None) -> None:
    """Non-blocking status check for once-per-step call sites (optimizer steps).

    Raises if the copy of the status word that the *previous* call enqueued has landed and shows a
    failed wait, then enqueues a new device -> pinned-host copy behind the work queued so far on the
    current stream.  A failure is therefore reported one call late at most, and the host never waits
    for the GPU.  Does nothing when no kernel of this process has asked for the status word yet."""
    if not torch.cuda.is_available() or torch.cuda.is_current_stream_capturing():
        return      # event queries and pinned allocations are not allowed inside a stream capture
    idx = (torch.cuda.current_device() if device is None or device.index is None else device.index)
    word = _status.get(idx)
    if word is None:
        return
    prev = _polls.get(idx)
    if prev is not None:
        host, ev = prev
        if not ev.query():
            return          # the previous copy has not landed yet: look again at the next call
        rec = host.tolist()
        if rec[0] != 0:
            word.zero_()
            _polls.pop(idx, None)
            raise NativeError(_describe(rec))
    else:
        host = torch.zeros(STATUS_INTS, dtype=torch.int32).pin_memory()
    host.copy_(word, non_blocking=True)
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(idx))
    _polls[idx] = (host, ev)


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what}: {STATUS_NAMES.get(rc, rc)} (code {rc})")
