"""The C-ABI library must load without a GPU and export every function declared in include/*.h;
the ctypes binding must declare every one of them too. No compute call is made here."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    names = []
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names += re.findall(r"^\s*(?:const\s+)?[A-Za-z_][\w\s\*]*?\b(cgpt_\w+)\s*\(", text, flags=re.M)
    return sorted(set(names))


def test_header_declares_functions():
    names = declared_functions()
    assert "cgpt_rmsnorm_backward" in names and "cgpt_adamw_step" in names and len(names) >= 15


def test_library_exports_every_declared_symbol():
    lib_path = ROOT / "cgpt_b200" / "libcgpt_b200.so"
    assert lib_path.exists(), "build with `python -m cgpt_b200.build`"
    lib = ctypes.CDLL(str(lib_path))
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"
    lib.cgpt_b200_version.restype = ctypes.c_char_p
    assert b"sm_100a" in lib.cgpt_b200_version()


def test_ctypes_binding_covers_header():
    from cgpt_b200 import _lib
    missing = [n for n in declared_functions() if n not in _lib.SIGNATURES]
    assert not missing, f"no ctypes signature for: {missing}"
