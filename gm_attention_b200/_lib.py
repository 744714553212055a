"""ctypes binding of ``libgmb200.so`` (declarations: ``include/gm_b200.h``).

The library is the only compute path of this package.  :func:`lib` raises a
``RuntimeError`` when the shared object is absent or fails to load; nothing
falls back to PyTorch or to a CPU implementation.
"""

from __future__ import annotations

import collections
import ctypes
import functools
from pathlib import Path
from typing import Any

import torch

LIBRARY = Path(__file__).resolve().parent / "libgmb200.so"
ABI_VERSION = 3

GM_F32, GM_F64, GM_BF16 = 0, 1, 2
_DTYPES = {torch.float32: GM_F32, torch.float64: GM_F64, torch.bfloat16: GM_BF16}

_P, _I, _L, _D = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_double

#: name -> argument ctypes, in the order of include/gm_b200.h
SIGNATURES: dict[str, list[Any]] = {
    "gm_softmax_forward": [_P] * 8 + [_L, _L, _I, _I, _I, _I, _D, _L, _I, _I, _P, _P],
    "gm_softmax_backward": [_P] * 10 + [_L, _L, _I, _I, _I, _I, _D, _L, _I, _P, _P, _P],
    "gm_conv_forward": [_P] * 10 + [_L, _L, _I, _I, _I, _I, _I, _I, _P, _P],
    "gm_conv_backward": [_P] * 11 + [_L, _L, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P],
    "gm_attention_forward": [_P] * 9 + [_L, _L, _L, _I, _I, _I, _I, _D, _I, _P, _P, _P],
    "gm_geometry_count": [_P, _L, _P, _P, _D, _P, _P],
    "gm_geometry_fill": [_P, _P, _P, _L, _P, _P, _D, _P, _I, _I] + [_P] * 10,
    "gm_attention_backward": [_P] * 12 + [_L, _L, _L, _I, _I, _I, _I, _D, _I, _P, _P, _P, _P, _P],
    "gm_lattice_attention_forward": [_P] * 8 + [_I, _P, _I, _I, _I, _L, _I, _I, _I, _I, _I, _D, _I, _P, _P, _P],
    "gm_lattice_attention_forward_tc": [_P] * 8 + [_I, _P, _I, _I, _I, _L, _I, _I, _I, _I, _I, _D, _P, _P, _P],
    "gm_lattice_attention_backward_tc": [_P] * 11 + [_I] + [_P] * 5 + [_I, _P, _I, _I, _I, _L, _I, _I, _I, _I, _I, _D, _P, _P, _P, _P, _P],
    "gm_lattice_attention_backward_tc_passes": [_P] * 11 + [_I] + [_P] * 5 + [_I, _P, _I, _I, _I, _L, _I, _I, _I, _I, _I, _D, _P, _P, _P, _P, _I, _P],
    "gm_lattice_attention_backward": [_P] * 11 + [_I] + [_P] * 5 + [_I, _P, _I, _I, _I, _L, _I, _I, _I, _I, _I, _D, _I, _P, _P, _P, _P, _P],
    "gm_factored_forward": [_P] * 11 + [_L, _L, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "gm_factored_aggregate": [_P, _P, _P, _L, _L, _I, _I, _P, _P],
    "gm_factored_backward": [_P] * 15 + [_L, _L, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P],
    "gm_pairs_forward": [_P] * 8 + [_L, _I, _I, _I, _I, _I, _P],
    "gm_pairs_backward": [_P] * 11 + [_L, _I, _I, _I, _I, _I, _P],
    "gm_lattice_attention_tc_wait_expired": [_P],
    "gm_lattice_attention_forward_tc4": [_P] * 8 + [_I, _P, _I, _I, _I, _L, _I, _I, _I, _I, _I, _D, _P, _P, _P],
    "gm_lattice_attention_backward_tc4_passes": [_P] * 11 + [_I] + [_P] * 5 + [_I, _P, _I, _I, _I, _L, _I, _I, _I, _I, _I, _D, _P, _P, _P, _P, _I, _P],
    "gm_lattice_attention_tc4_wait_expired": [_P],
    "gm_halo_unique_id": [_P],
    "gm_halo_comm_create": [_P, _I, _I, _P],
    "gm_halo_comm_destroy": [_P],
    "gm_halo_comm_error": [_P, _P],
    "gm_halo_exchange": [_P, _I, _P, _P, _P, _P, _P],
    "gm_halo_accumulate": [_P, _P, _L, _L, _L, _L, _I, _P],
    "gm_halo_move": [_I, _P, _I, _L, _L, _L, _P, _I, _P],
    "gm_lattice_conv_apply": [_P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "gm_lattice_conv_table_grad": [_P, _P, _P, _I, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "gm_peer_alloc": [_L, _P, _P],
    "gm_peer_free": [_P],
    "gm_peer_open": [_P, _P],
    "gm_peer_close": [_P],
    "gm_peer_send": [_P, _I, _L, _L, _L, _P, _P, _P, _P, ctypes.c_uint32, _P],
    "gm_peer_land": [_P, _I, _L, _L, _L, _P, _I, _I, _P, _P, _P, ctypes.c_uint32, _P],
    "gm_peer_send_many": [_I, _P, _I, _L, _P, _L, _P, _P, _P, _P, _P, _P],
    "gm_peer_land_many": [_I, _P, _I, _L, _P, _L, _P, _I, _I, _P, _P, _P, _P, _P],
    "gm_peer_error": [_P],
    "gm_attention_backward_static": [_P] * 12 + [_L, _L, _L, _I, _I, _I, _I, _D, _I, _P, _P, _P, _P],
}
#: entry points that return a size instead of a status
SIZE_QUERIES: dict[str, list[Any]] = {
    "gm_attention_backward_scratch_bytes": [_L, _L, _I, _I],
    "gm_attention_backward_static_capacity": [],
}


@functools.cache
def lib() -> ctypes.CDLL:
    """Load the shared library once and declare every entry point."""
    if not LIBRARY.exists():
        raise RuntimeError(
            f"{LIBRARY} is missing: build it with `python -m gm_attention_b200.build` "
            "(this package has no CPU or PyTorch fallback)"
        )
    handle = ctypes.CDLL(str(LIBRARY))
    handle.gm_abi_version.restype = ctypes.c_int
    handle.gm_last_error.restype = ctypes.c_char_p
    if handle.gm_abi_version() != ABI_VERSION:
        raise RuntimeError(f"{LIBRARY} has ABI {handle.gm_abi_version()}, this package expects {ABI_VERSION}: rebuild it")
    for name, argtypes in SIGNATURES.items():
        fn = getattr(handle, name)
        fn.argtypes = argtypes
        fn.restype = ctypes.c_int
    for name, argtypes in SIZE_QUERIES.items():
        fn = getattr(handle, name)
        fn.argtypes = argtypes
        fn.restype = ctypes.c_int64
    return handle


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise RuntimeError(f"unsupported dtype {dtype}") from None


def ptr(tensor: torch.Tensor | None) -> int | None:
    """Device address of a tensor's first element (``None`` for an absent or empty tensor)."""
    if tensor is None or tensor.numel() == 0:
        return None
    return tensor.data_ptr()


def stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


#: calls made per entry point (for callers that report how many kernels they launched)
CALLS: collections.Counter = collections.Counter()


def call(name: str, *args: Any) -> None:
    """Invoke an entry point; a non-zero status becomes ``RuntimeError`` with the library's message."""
    handle = lib()
    CALLS[name] += 1
    status = getattr(handle, name)(*args)
    if status != 0:
        message = handle.gm_last_error().decode(errors="replace")
        raise RuntimeError(f"{name} failed ({status}): {message}")


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    """All tensors on one CUDA device; that device is returned."""
    device = tensors[0].device
    if device.type != "cuda":
        raise RuntimeError("gm_attention_b200 runs on CUDA tensors only (there is no CPU path)")
    for t in tensors:
        if t.device != device:
            raise RuntimeError("every tensor must live on the same device")
    return device
