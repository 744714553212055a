"""The C-ABI library loads on a machine without a GPU and exports every entry
point that include/gm_b200.h declares (no compute call is made here)."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent


def declared_symbols() -> list[str]:
    text = (REPO / "include" / "gm_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gm_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def library():
    from gm_attention_b200 import build

    return ctypes.CDLL(str(build.build()))


def test_header_declares_the_boundary():
    names = declared_symbols()
    for required in ("gm_softmax_forward", "gm_softmax_backward", "gm_conv_forward", "gm_conv_backward", "gm_attention_forward",
                     "gm_attention_backward"):
        assert required in names


def test_library_exports_every_declared_symbol(library):
    missing = [name for name in declared_symbols() if not hasattr(library, name)]
    assert not missing, f"declared in include/gm_b200.h but not exported: {missing}"


def test_python_binding_covers_every_declared_symbol(library):
    from gm_attention_b200 import _lib

    bound = set(_lib.SIGNATURES) | set(_lib.SIZE_QUERIES) | {"gm_abi_version", "gm_last_error"}
    assert set(declared_symbols()) == bound


def test_abi_version_and_error_string(library):
    from gm_attention_b200 import _lib

    library.gm_abi_version.restype = ctypes.c_int
    assert library.gm_abi_version() == _lib.ABI_VERSION
    library.gm_last_error.restype = ctypes.c_char_p
    assert isinstance(library.gm_last_error(), bytes)


def test_bad_arguments_are_refused_without_a_gpu(library):
    """Argument validation happens before any CUDA call: status -1 / -2 and a message."""
    fn = library.gm_softmax_forward
    fn.restype = ctypes.c_int
    P, I, L, D = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_double
    fn.argtypes = [P] * 8 + [L, L, I, I, I, I, D, L, I, I, P, P]
    status = fn(None, None, None, None, None, None, None, None, 4, 4, 8, 1, 1, 99, 1.0, 1, 0, 0, None, None)
    assert status == -1
    library.gm_last_error.restype = ctypes.c_char_p
    assert b"heads" in library.gm_last_error()
    status = fn(None, None, None, None, None, None, None, None, 4, 4, 8, 1, 1, 2, 1.0, 1, 0, 7, None, None)
    assert status == -2


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from gm_attention_b200 import _lib

    monkeypatch.setattr(_lib, "LIBRARY", tmp_path / "libgmb200.so")
    _lib.lib.cache_clear()
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()
    _lib.lib.cache_clear()


def test_cpu_tensors_are_refused():
    import torch

    from gm_attention_b200.nn.ext import AttentionExtension

    q = torch.zeros(2, 2)
    e = torch.zeros(0)
    with pytest.raises(RuntimeError):
        AttentionExtension().softmax_forward(q, q, torch.zeros(1, 1, 2), torch.zeros(1), torch.zeros(1, dtype=torch.uint8),
                                             torch.tensor([[0, 2, 0, 0, 1]]), torch.tensor([0, 1, 1]), torch.tensor([0]), 1, 1.0, 1)
