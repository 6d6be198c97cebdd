"""CPU checks of the boundary: the shared library builds, loads without a GPU and exports
every symbol the public headers declare; the ctypes table matches the header."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include", "gigaslop_b200")


def declared_symbols():
    names = set()
    for base, _, files in os.walk(INC):
        for f in files:
            if not f.endswith(".h"):
                continue
            text = open(os.path.join(base, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            text = re.sub(r"//[^\n]*", "", text)
            names |= set(re.findall(r"\b(gsb200_[a-z0-9_]+)\s*\(", text))
    return names


@pytest.fixture(scope="module")
def handle():
    from gigaslop_b200 import build, _lib
    build.build()
    return ctypes.CDLL(_lib.LIB_PATH)


def test_library_exports_every_declared_symbol(handle):
    syms = declared_symbols()
    assert len(syms) >= 12
    missing = [s for s in sorted(syms) if not hasattr(handle, s)]
    assert not missing, f"declared in include/ but not exported: {missing}"


def test_ctypes_table_covers_the_header():
    from gigaslop_b200 import _lib
    assert set(_lib.SIGNATURES) == declared_symbols()


def test_version_string_and_no_cpu_fallback(handle):
    import torch
    import gigaslop_b200 as g
    assert b"sm_100a" in g.lib().gsb200_version()
    with pytest.raises(RuntimeError):
        g.quantize_tensor(torch.zeros(4, 16))
    with pytest.raises(RuntimeError):
        g.gemm_i8_i32(torch.zeros(4, 16, dtype=torch.int8), torch.zeros(8, 16, dtype=torch.int8))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from gigaslop_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()
