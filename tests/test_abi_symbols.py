"""The C-ABI library loads and exports every symbol include/tkv.h declares (no GPU)."""
import ctypes as C
import os
import re

import pytest

from tempura_b200 import _build, _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    _build.build()
    return _native.lib()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "tkv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tkv_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    names = declared_functions()
    assert len(names) > 50
    assert sorted(_native.SIGNATURES) == names


def test_library_exports_every_declared_symbol(L):
    raw = C.CDLL(_build.LIB_PATH)
    for name in declared_functions():
        assert hasattr(raw, name), name


def test_version_and_error_text(L):
    assert b"sm_100a" in L.tkv_version()
    buf = C.create_string_buffer(64)
    L.tkv_last_error(buf, 64)          # no crash with an empty message


def test_struct_layout_matches_header():
    # sizes implied by the POD definitions in include/tkv.h on LP64
    assert C.sizeof(_native.TkvPool) == 72
    assert C.sizeof(_native.TkvBatch) == 48
    assert C.sizeof(_native.TkvShard) == 24
    assert C.sizeof(_native.TkvPairing) == 32
    assert C.sizeof(_native.TkvStats) == 80
    assert C.sizeof(_native.TkvTransfer) == 40


def test_header_is_plain_c99_and_ctypes_structs_have_the_compilers_sizes(tmp_path):
    """include/tkv.h compiles as C99 (it is the boundary a cgo / Rust FFI / ctypes binding reads), and every struct the
    ctypes binding declares has the size the C compiler gives it."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    assert gcc, "gcc not found"
    names = sorted(n for n in dir(_native) if n.startswith("Tkv") and isinstance(getattr(_native, n), type)
                   and issubclass(getattr(_native, n), C.Structure))
    assert len(names) >= 15
    src = tmp_path / "sizes.c"
    body = "\n".join(f'    printf("{n} %zu\\n", sizeof({n}));' for n in names)
    src.write_text(f'#include <stdio.h>\n#include "tkv.h"\nint main(void) {{\n{body}\n    return 0;\n}}\n')
    exe = tmp_path / "sizes"
    proc = subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(ROOT, "include"), "-o", str(exe), str(src)],
                          capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    out = subprocess.run([str(exe)], capture_output=True, text=True).stdout
    sizes = dict(line.split() for line in out.strip().splitlines())
    for n in names:
        assert int(sizes[n]) == C.sizeof(getattr(_native, n)), n
