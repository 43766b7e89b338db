"""The C-ABI library loads on a machine without a GPU and exports every symbol the public
headers declare. No compute entry point is called here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tessera_sm100_\w+|tsr[A-Z]\w+|tessera_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    missing = []
    for header in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not header.endswith(".h"):
            continue
        names = _declared(header)
        assert names, f"{header} declares nothing"
        for name in names:
            if not hasattr(lib, name):
                missing.append(f"{header}:{name}")
    assert not missing, missing


def test_ctypes_table_covers_the_op_header(lib):
    from tessera_b200 import _lib
    declared = set(_declared("tessera_sm100.h"))
    bound = set(_lib.exported_symbols())
    assert declared <= bound, sorted(declared - bound)


def test_version_and_error_strings(lib):
    assert b"sm_100a" in lib.tessera_sm100_version()
    assert isinstance(lib.tessera_sm100_last_error(), bytes)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from tessera_b200 import _lib
    monkeypatch.setenv("TESSERA_SM100_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_lib, "_LIB", None)
    with pytest.raises(_lib.BackendError):
        _lib.load()


def test_device_count_is_reported_without_a_gpu(lib):
    n = ctypes.c_int(-1)
    assert lib.tessera_sm100_device_count(ctypes.byref(n)) == 0
    assert n.value >= 0
