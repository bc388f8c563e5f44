"""In-tree native builds: the sm_100a kernel library (nvcc) and the C++ accountant (g++/pybind11).

Artefacts are written next to their sources so they travel with a snapshot of the tree.  A
build is skipped when the artefact is newer than every source; ``force=True`` rebuilds.
"""
from __future__ import annotations

import contextlib
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
CSRC = PKG / "ops" / "csrc"
KERNEL_LIB = PKG / "ops" / "libopaque_b200.so"
ACC_SRC = PKG / "accounting" / "csrc"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]
# Approximate division / exp / tanh are fine in the GEMM epilogues and activation kernels.  The translation unit that draws
# the DP noise and applies the optimizer is compiled WITHOUT them: its logarithm, sine / cosine, square roots and divisions
# are the IEEE-accurate ones.
FAST_MATH = "--use_fast_math"
EXACT_MATH_SOURCES = {"dp_update.cu"}
OBJ_DIR = CSRC / "build"


def _find(tool: str, extra: list[str]) -> str | None:
    hit = shutil.which(tool)
    if hit:
        return hit
    for p in extra:
        if os.path.exists(p):
            return p
    return None


@contextlib.contextmanager
def _build_lock(target: Path):
    """Exclusive advisory lock beside ``target`` (held across one compile); a no-op where ``fcntl`` is missing."""
    try:
        import fcntl
    except ImportError:          # pragma: no cover
        yield
        return
    lock_path = target.with_name("." + target.name + ".lock")
    with open(lock_path, "w") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources)


def _flags_for(src: Path) -> list[str]:
    return list(NVCC_FLAGS) + ([] if src.name in EXACT_MATH_SOURCES else [FAST_MATH])


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``.cu`` under ``ops/csrc`` (one object each, rebuilt only when stale) and link one shared library
    for sm_100a."""
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    deps = sources + headers
    if not force and not _stale(KERNEL_LIB, deps):
        return KERNEL_LIB
    nvcc = _find("nvcc", ["/usr/local/cuda/bin/nvcc"])
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build the sm_100a kernel library")
    # Every rank of a job may find the library stale at the same moment: one builds, the others wait on the lock and
    # then see a fresh library.  The output is written under a private name and renamed into place.
    with _build_lock(KERNEL_LIB):
        if not force and not _stale(KERNEL_LIB, deps):
            return KERNEL_LIB
        OBJ_DIR.mkdir(exist_ok=True)
        procs, objs, log = [], [], []
        for src in sources:
            obj = OBJ_DIR / (src.stem + ".o")
            objs.append(obj)
            if force or _stale(obj, [src] + headers):
                cmd = [nvcc, *_flags_for(src), "-c", str(src), "-o", str(obj)]
                if verbose:
                    cmd.insert(1, "-Xptxas=-v")
                procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        failed = []
        for src, obj, proc in procs:                      # the objects compile side by side
            out, _ = proc.communicate()
            log.append(out)
            if proc.returncode != 0:
                obj.unlink(missing_ok=True)
                failed.append(f"{src.name}:\n{out}")
        if failed:
            raise RuntimeError("nvcc failed:\n" + "\n".join(failed))
        tmp = KERNEL_LIB.with_suffix(f".so.tmp{os.getpid()}")
        res = subprocess.run([nvcc, "-shared", "-o", str(tmp), *map(str, objs)], capture_output=True, text=True)
        if res.returncode != 0:
            tmp.unlink(missing_ok=True)
            raise RuntimeError("nvcc link failed:\n" + res.stdout + res.stderr)
        os.replace(tmp, KERNEL_LIB)
    if verbose:
        print("\n".join(log))
    return KERNEL_LIB


def accounting_ext_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return PKG / "accounting" / ("_native" + suffix)


def build_accounting(force: bool = False) -> Path:
    """Compile the C++17 PLD accountant into a pybind11 extension module."""
    import pybind11
    target = accounting_ext_path()
    sources = sorted(p for p in ACC_SRC.glob("*.cpp") if p.name != "selftest.cpp")     # selftest.cpp has its own main()
    deps = sources + sorted(ACC_SRC.glob("*.hpp"))
    if not sources:
        raise RuntimeError("accounting sources missing")
    if not force and not _stale(target, deps):
        return target
    gxx = _find("g++", ["/usr/bin/g++"])
    if gxx is None:
        raise RuntimeError("g++ not found: cannot build the accountant")
    with _build_lock(target):
        if not force and not _stale(target, deps):
            return target
        tmp = target.with_suffix(f".tmp{os.getpid()}")
        cmd = [gxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-pthread", "-fopenmp",
               f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}",
               "-o", str(tmp), *map(str, sources)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            tmp.unlink(missing_ok=True)
            raise RuntimeError("g++ failed:\n" + res.stdout + res.stderr)
        os.replace(tmp, target)
    return target


def build_all(force: bool = False) -> None:
    build_kernels(force)
    build_accounting(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built:", KERNEL_LIB, accounting_ext_path())
