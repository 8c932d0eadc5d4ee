"""CPU: the C-ABI library loads and exports every symbol include/flint_b200.h declares (no compute calls)."""
import os
import re

import pytest

from flint_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "flint_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fb_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_all_bound():
    assert _declared() == sorted(_lib.EXPORTED_SYMBOLS)


def test_library_exports_every_symbol():
    if not os.path.exists(_lib.LIB_PATH):
        from flint_b200.csrc import build
        build.build()
    lib = _lib.load()
    for name in _declared():
        assert hasattr(lib, name), name


def test_stream_bytes_is_host_only_arithmetic():
    lib = _lib.load()
    assert lib.fb_stream_bytes(16, 2560, 0) == 16 * (1280 + 40)       # 4 tiles of 4 rows: nibbles + 20 bf16 scales per row
    assert lib.fb_stream_bytes(3, 14336, 1) == 4 * (7168 + 448)        # tiles of 2 rows: 3 rows occupy 2 tiles
    assert lib.fb_stream_bytes(5, 640, 0) == 16 * (320 + 10)           # 5 groups: one tile of 16 rows
    assert lib.fb_stream_bytes(4, 1376, 0) == 0          # not a multiple of the group


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError):
        _lib.load()
