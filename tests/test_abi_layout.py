"""The ctypes mirror of the C ABI (``ops/native.py``) against the header itself: a small
program compiled with the host compiler prints ``sizeof`` / ``offsetof`` of every struct
member, and the Python structures must agree."""

import ctypes
import os
import shutil
import subprocess

import pytest

from flashoptim_b200.ops import native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "flashoptim_b200", "csrc", "fo_api.h")

STRUCTS = {
    "FoSeg": native.FoSeg,
    "FoAdamHyper": native.FoAdamHyper,
    "FoMomentumHyper": native.FoMomentumHyper,
    "FoCommArgs": native.FoCommArgs,
}


@pytest.mark.skipif(shutil.which("g++") is None, reason="no host C++ compiler")
def test_ctypes_structures_match_the_header(tmp_path):
    lines = ['#include <cstdio>', '#include <cstddef>', f'#include "{HEADER}"', "int main() {"]
    for name, cls in STRUCTS.items():
        lines.append(f'  std::printf("{name} size %zu\\n", sizeof({name}));')
        for field, _ in cls._fields_:
            lines.append(f'  std::printf("{name} {field} %zu\\n", offsetof({name}, {field}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.cpp"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["g++", "-std=c++17", str(src), "-o", str(exe)], check=True, capture_output=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    want = {}
    for line in out.splitlines():
        name, field, value = line.split()
        want[(name, field)] = int(value)
    for name, cls in STRUCTS.items():
        assert ctypes.sizeof(cls) == want[(name, "size")], name
        for field, _ in cls._fields_:
            assert getattr(cls, field).offset == want[(name, field)], (name, field)
    # every member of the header is mirrored (a member missing in Python would shift nothing
    # before it but shrink the structure)
    assert ctypes.sizeof(native.FoSeg) == 64


def _declared_functions():
    import re

    decls = {}
    for header in ("fo_api.h", "fo_noalloc.h"):
        text = open(os.path.join(ROOT, "flashoptim_b200", "csrc", header)).read()
        text = re.sub(r"//[^\n]*", "", text)
        for m in re.finditer(r"\b(?:int|void)\s+(fo_\w+)\s*\(([^)]*)\)\s*;", text):
            args = m.group(2).strip()
            decls[m.group(1)] = 0 if args in ("", "void") else args.count(",") + 1
    return decls


def test_every_exported_function_is_declared_with_the_right_arity():
    try:
        lib = native.load()
    except Exception as e:  # library not built on this machine
        pytest.skip(f"native library unavailable: {e}")
    decls = _declared_functions()
    assert len(decls) >= 15
    checked = 0
    for name, n_args in decls.items():
        fn = getattr(lib, name)  # AttributeError: declared in the header but not exported
        if fn.argtypes is not None:
            assert len(fn.argtypes) == n_args, name
            checked += 1
    assert checked >= 12
