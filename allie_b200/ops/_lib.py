"""ctypes binding to the in-tree native libraries.

``cuda()`` returns the sm_100a kernel library and raises if it is missing:
on a GPU machine there is no silent fallback to library kernels.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p
from pathlib import Path

import torch

_LIB_DIR = Path(__file__).resolve().parent.parent / "lib"
_cuda_lib = None
_host_lib = None
LAUNCHES = 0   # kernels of this package launched so far (counted by the Python entry points)


def count_launches(n: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n


class NativeLibraryMissing(RuntimeError):
    pass


def cuda() -> ctypes.CDLL:
    global _cuda_lib
    if _cuda_lib is None:
        path = _LIB_DIR / "liballie_b200.so"
        if not path.exists():
            raise NativeLibraryMissing(
                f"{path} not built; run `python -m allie_b200.build` (needs nvcc)")
        _cuda_lib = ctypes.CDLL(str(path))
    return _cuda_lib


def host() -> ctypes.CDLL:
    global _host_lib
    if _host_lib is None:
        path = _LIB_DIR / "liballie_host.so"
        if not path.exists():
            from .. import build
            build.build_host()
        _host_lib = ctypes.CDLL(str(path))
    return _host_lib


def have_cuda_lib() -> bool:
    return (_LIB_DIR / "liballie_b200.so").exists()


class GemmEpilogue(ctypes.Structure):
    _fields_ = [
        ("out", c_void_p), ("ldo", c_longlong), ("out_fp32", c_int), ("accumulate", c_int),
        ("bias", c_void_p), ("act", c_int), ("aux", c_void_p), ("ldaux", c_longlong),
        ("resid", c_void_p), ("ldr", c_longlong),
        ("drop_seed", c_ulonglong), ("drop_stream", c_uint), ("drop_thr16", c_uint),
        ("alpha", c_float), ("m_limit", c_void_p), ("k_limit", c_void_p), ("pdl", c_int),
        ("aux_grad", c_int),
    ]


class GroupedGemm(ctypes.Structure):
    """``AbGroupedGemm`` of ``csrc/gemm_grouped.cuh``."""
    _fields_ = [
        ("groups", c_int), ("cap", c_int), ("mode", c_int), ("rows", c_void_p), ("tile_ready", c_void_p),
        ("ret", c_void_p), ("peers", c_void_p * 8), ("flags", c_void_p * 8), ("phase", c_int),
        ("epoch", c_uint), ("rank", c_int), ("world", c_int), ("ticket", c_void_p),
    ]


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def stream_ptr() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_status: dict[int, torch.Tensor] = {}


def status_word() -> torch.Tensor:
    """Per-device int32 the kernels write a nonzero code into when a bounded
    wait ran out.  Checked by :func:`check_status` (one D2H read)."""
    dev = torch.cuda.current_device()
    if dev not in _status:
        _status[dev] = torch.zeros(16, dtype=torch.int32, device=f"cuda:{dev}")
    return _status[dev]


STATUS_NAMES = {
    1: "timeout waiting for a TMA stage", 2: "timeout waiting for a free smem stage",
    3: "timeout waiting for an accumulator", 4: "timeout waiting for accumulator drain",
    5: "timeout waiting for a peer GPU", 6: "timeout (misc)", 7: "bad argument",
}


def check_status() -> None:
    code = int(status_word()[0].item())
    if code != 0:
        status_word().zero_()
        raise RuntimeError(f"allie_b200 kernel status {code}: {STATUS_NAMES.get(code, '?')}")


def dropout_thr16(p: float) -> int:
    t = p * 65536.0
    if t <= 0:
        return 0
    return min(65535, int(t + 0.5))
