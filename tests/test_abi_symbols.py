"""The C-ABI library loads on a CPU-only box and exports every symbol include/lbk.h declares
(no compute calls here)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def header_functions():
    text = (ROOT / "include" / "lbk.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(lbk_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


@pytest.fixture(scope="module")
def lib():
    from lemonade_burn_b200 import build, _lib
    build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    names = header_functions()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/lbk.h but not exported"


def test_binding_table_matches_header():
    from lemonade_burn_b200 import _lib
    assert sorted(n for n, _, _ in _lib.SYMBOLS) == header_functions()


def test_layout_helpers_and_errors_without_gpu(lib):
    assert lib.lbk_abi_version() == 1
    for cols, want in [(0, 0), (1, 128), (128, 128), (129, 256), (300, 384), (2560, 2560), (6912, 6912)]:
        assert lib.lbk_padded_cols(cols) == want
        assert lib.lbk_row_bytes(cols) == want // 4
    import torch
    if not torch.cuda.is_available():
        h = ctypes.c_void_p()
        st = lib.lbk_init(0, ctypes.byref(h))
        assert st != 0 and not h.value
        assert b"CUDA" in lib.lbk_last_error() or b"device" in lib.lbk_last_error()


def test_header_is_plain_c_and_a_c_program_links(lib, tmp_path):
    """The boundary is a C ABI: include/lbk.h compiles as C99 with -pedantic (no C++ in the signatures), and
    a C program (tests/abi_c_client.c) links against liblbk.so and gets status codes and messages."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    inc = ROOT / "include"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-fsyntax-only", "-x", "c", str(inc / "lbk.h")], check=True)
    libdir = ROOT / "lemonade_burn_b200"
    exe = tmp_path / "abi_c_client"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", f"-I{inc}", "-o", str(exe), str(ROOT / "tests" / "abi_c_client.c"),
                    f"-L{libdir}", "-llbk", f"-Wl,-rpath,{libdir}"], check=True)
    res = subprocess.run([str(exe)], stdout=subprocess.PIPE, text=True, timeout=120)
    assert res.returncode == 0 and "C client ok" in res.stdout, res.stdout


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    """No fallback: a missing liblbk.so must raise, not route anywhere else."""
    from lemonade_burn_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "liblbk.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()


def test_product_never_imports_the_oracle():
    for p in (ROOT / "lemonade_burn_b200").rglob("*"):
        if p.suffix in (".py", ".cu", ".cuh", ".h", ".hpp", ".cpp"):
            text = p.read_text()
            assert "oracle" not in text.replace("# oracle", ""), f"{p} mentions the oracle"
