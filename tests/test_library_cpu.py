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


def test_tensor_core_layouts_and_row_cost():
    """Host-side gates of the tensor-core lattice kernels: head layouts they are instantiated for (complex
    frequencies must be the orders 1 .. n) and the per-row cost model that balances the latitude bands."""
    import torch

    from gm_attention_b200.attention import tensor_core_layout_supported
    from gm_attention_b200.parallel import balanced_cuts, tensor_core_row_cost

    row = lambda n, a, off: (n, a, off, 0, 1 if n == 0 else 2)
    assert tensor_core_layout_supported((row(0, 16, 0), row(1, 16, 64), row(2, 16, 192)))      # headline
    assert tensor_core_layout_supported((row(0, 8, 0), row(1, 8, 32), row(2, 8, 96), row(3, 8, 160)))
    assert tensor_core_layout_supported((row(1, 6, 0), row(2, 6, 12)))                           # no scalar block
    assert not tensor_core_layout_supported((row(0, 16, 0), row(1, 16, 64), row(3, 16, 192)))  # orders 1, 3
    assert not tensor_core_layout_supported((row(0, 16, 0), row(2, 16, 64)))                    # order 2 alone
    assert not tensor_core_layout_supported((row(0, 16, 0), row(1, 16, 64), row(2, 8, 192)))   # two multiplicities
    assert not tensor_core_layout_supported((row(0, 32, 0), row(1, 16, 128)))                   # scalar block too wide
    # a whole-row polar window costs more per ROW but far less per EDGE than a narrow equatorial one
    counts = torch.tensor([[0, 512, 512, 512, 0], [7, 7, 7, 7, 7]])
    polar, equator = tensor_core_row_cost(counts)
    assert polar > equator
    assert polar / (3 * 512) < 0.3 * equator / (5 * 7)
    cuts = balanced_cuts([polar] * 4 + [equator] * 120 + [polar] * 4, 4)
    assert cuts[0] == 0 and cuts[-1] == 128 and cuts == sorted(cuts) and len(set(cuts)) == 5


def header_prototypes() -> dict[str, list[str]]:
    """name -> parameter declarations of every prototype in include/gm_b200.h."""
    text = (REPO / "include" / "gm_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for name, params in re.findall(r"\b(gm_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", text):
        params = " ".join(params.split())
        out[name] = [] if params in ("", "void") else [x.strip() for x in params.split(",")]
    return out


def test_header_compiles_as_c(tmp_path):
    """include/gm_b200.h is a C header: a C99 translation unit that includes it and takes the address of an entry
    point compiles with gcc (no C++ leaks into the boundary)."""
    import subprocess

    src = tmp_path / "use_header.c"
    src.write_text('#include "gm_b200.h"\n'
                   "typedef int (*forward_fn)(const void*, const void*, const void*, const void*, const void*, const uint8_t*, const int64_t*,\n"
                   "                          const int64_t*, const int64_t*, int64_t, int64_t, int64_t, int, int, int, int, double, int, void*, void*, void*);\n"
                   "forward_fn pick(void) { return &gm_attention_forward; }\n"
                   "int version(void) { return gm_abi_version() + GM_OK; }\n")
    done = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", str(REPO / "include"), "-c", str(src), "-o", str(tmp_path / "use_header.o")],
                          capture_output=True, text=True)
    assert done.returncode == 0, done.stderr


def test_ctypes_signatures_match_the_header():
    """The hand-written ctypes argument lists have the arity and the kinds (pointer / int / int64 / uint32 / double) of the
    header's prototypes: a mismatch would otherwise pass garbage silently."""
    from gm_attention_b200 import _lib

    protos = header_prototypes()
    kinds = {ctypes.c_void_p: "pointer", ctypes.c_int: "int", ctypes.c_int64: "int64", ctypes.c_double: "double", ctypes.c_uint32: "uint32"}

    def kind_of(decl: str) -> str:
        if "*" in decl:
            return "pointer"
        base = decl.rsplit(" ", 1)[0].replace("const ", "").strip()
        return {"int": "int", "int64_t": "int64", "double": "double", "uint32_t": "uint32"}[base]

    for name, argtypes in {**_lib.SIGNATURES, **_lib.SIZE_QUERIES}.items():
        assert name in protos, name
        want = [kind_of(d) for d in protos[name]]
        assert [kinds[a] for a in argtypes] == want, f"{name}: ctypes {[kinds[a] for a in argtypes]} vs header {want}"


def test_tensor_core_entry_table_layout():
    """The padded entry table of the tensor-core lattice kernels: runs keep their order, padding carries bias -inf,
    the bias is pre-multiplied by log2(e), and the packed words hold (entry x | entry x - 1) in bf16."""
    import numpy as np
    import torch

    from gm_attention_b200.attention import TC_PAD_AFTER, TC_PAD_BEFORE, tensor_core_entries, tensor_core_entry_words

    rng = np.random.default_rng(0)
    for norders in (2, 3):
        win_cnt = np.array([[0, 3, 2], [5, 0, 1]], np.int32)
        win_off = np.array([[0, 0, 3], [5, 0, 10]], np.int32)
        entries = rng.standard_normal((11, 8)).astype(np.float32)
        entries[4, 2 * norders] = -np.inf  # a masked pair inside a window
        table, off = tensor_core_entries(entries, win_cnt, win_off, norders)
        assert table.shape[1] == tensor_core_entry_words(norders) and (table.shape[1] // 4) % 2 == 1 and off.shape == win_off.shape
        assert table.shape[0] == int((win_cnt[win_cnt > 0] + TC_PAD_BEFORE + TC_PAD_AFTER).sum()) + 1
        bf16 = lambda x: torch.from_numpy(np.ascontiguousarray(x)).bfloat16().view(torch.int16).numpy().astype(np.uint16).astype(np.uint32)
        words = lambda x: np.ascontiguousarray(x).view(np.uint32)
        for (i, c), cnt in np.ndenumerate(win_cnt):
            if cnt == 0:
                continue
            o, src = int(off[i, c]), int(win_off[i, c])
            run = table[o:o + cnt]
            assert np.array_equal(run[:, 0:4], entries[src:src + cnt, 0:4])
            assert np.array_equal(run[:, 8], entries[src:src + cnt, 2 * norders] * np.float32(1.4426950408889634))
            before, after = table[o - TC_PAD_BEFORE:o], table[o + cnt:o + cnt + TC_PAD_AFTER]
            assert np.isneginf(before[:, 8]).all() and np.isneginf(after[:, 8]).all()
            assert not before[:, 0:4].any() and not after[:, 0:4].any() and not words(before[:, 4:8]).any()
            assert np.array_equal(words(run[:, 4:8]) & 0xFFFF, bf16(entries[src:src + cnt, 0:4]))
            previous = np.vstack([np.zeros((1, 4), np.float32), entries[src:src + cnt - 1, 0:4]])
            assert np.array_equal(words(run[:, 4:8]) >> 16, bf16(previous))
            if norders == 3:
                assert np.array_equal(run[:, 9:11], entries[src:src + cnt, 4:6])
                assert np.array_equal(words(run[:, 12:14]) & 0xFFFF, bf16(entries[src:src + cnt, 4:6]))
        assert not table[:, 11].any() and not table[:, 14:].any()
