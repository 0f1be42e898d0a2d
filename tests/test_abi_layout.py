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
