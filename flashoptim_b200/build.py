"""In-tree build of ``libflashoptim_b200.so`` (hand-written sm_100a CUDA, C ABI).

``python -m flashoptim_b200.build`` compiles every ``csrc/*.cu`` with nvcc for
``sm_100a`` and links one shared library next to the package.  The library has
no PyTorch dependency: Python passes raw device pointers and the current CUDA
stream through :mod:`ctypes` (see :mod:`flashoptim_b200.ops.native`).  A stamp
file holding a hash of sources and flags makes repeated calls free.
"""

from __future__ import annotations

import contextlib
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
SRC_DIR = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "_lib"
LIB_PATH = LIB_DIR / "libflashoptim_b200.so"
STAMP_PATH = LIB_DIR / "build.stamp"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
]


def find_nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc")
    if cand:
        return cand
    p = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc"
    return str(p) if p.exists() else None


def _sources() -> list[Path]:
    return sorted(SRC_DIR.glob("*.cu"))


def source_hash(extra_flags: tuple[str, ...] = ()) -> str:
    h = hashlib.sha256()
    for f in sorted(SRC_DIR.iterdir()):
        if f.suffix in (".cu", ".cuh", ".h"):
            h.update(f.name.encode())
            h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS + list(extra_flags)).encode())
    return h.hexdigest()


def is_current(extra_flags: tuple[str, ...] = ()) -> bool:
    return (
        LIB_PATH.exists()
        and STAMP_PATH.exists()
        and STAMP_PATH.read_text().strip() == source_hash(extra_flags)
    )


@contextlib.contextmanager
def _build_lock(lock_dir: Path):
    """Exclusive inter-process lock: under torchrun every rank may find the library stale at
    the same moment, and only one of them may run nvcc into the shared object directory."""
    lock_dir.mkdir(parents=True, exist_ok=True)
    with open(lock_dir / ".build.lock", "w") as fh:
        try:
            import fcntl

            fcntl.flock(fh, fcntl.LOCK_EX)
        except ImportError:  # no fcntl: single-process builds only
            pass
        yield


def build(
    force: bool = False,
    verbose: bool = False,
    extra_flags: tuple[str, ...] = (),
    out_path: Path | None = None,
) -> Path:
    """Compile and link the library; returns its path.

    ``extra_flags`` (e.g. ``-DFO_UNROLL=4``) and ``out_path`` exist for tuning
    builds; the default build writes ``_lib/libflashoptim_b200.so``.
    """
    default_target = out_path is None
    out = LIB_PATH if default_target else Path(out_path)
    if default_target and not force and is_current(extra_flags):
        return out
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError(
            "nvcc not found: cannot build libflashoptim_b200.so "
            "(set NVCC or CUDA_HOME, or ship a prebuilt _lib/)"
        )
    with _build_lock(out.parent):
        # another process may have finished the same build while this one waited
        if default_target and not force and is_current(extra_flags):
            return out
        return _build_locked(nvcc, out, default_target, verbose, extra_flags)


def _build_locked(nvcc: str, out: Path, default_target: bool, verbose: bool, extra_flags: tuple[str, ...]) -> Path:
    obj_dir = out.parent / ("obj_" + out.stem)
    obj_dir.mkdir(parents=True, exist_ok=True)

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-I", str(SRC_DIR), "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(_sources()) or 1)) as ex:
        objs = list(ex.map(compile_one, _sources()))
    # link beside the target and rename into place: a process that dlopens the library at this
    # moment sees the old file or the new one, never a half-written one; the stamp comes last
    fd, tmp = tempfile.mkstemp(prefix=out.stem + ".", suffix=".so.tmp", dir=str(out.parent))
    os.close(fd)
    try:
        link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp] + [str(o) for o in objs]
        if verbose:
            print(" ".join(link), flush=True)
        r = subprocess.run(link, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.chmod(tmp, 0o755)
        os.replace(tmp, out)
    finally:
        if os.path.exists(tmp):
            os.unlink(tmp)
    if default_target:
        stamp_tmp = STAMP_PATH.with_suffix(".stamp.tmp")
        stamp_tmp.write_text(source_hash(extra_flags))
        os.replace(stamp_tmp, STAMP_PATH)
    return out


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True)
    print(f"built {path}")
