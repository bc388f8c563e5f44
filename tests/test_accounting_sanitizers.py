"""The C++ PLD core under AddressSanitizer + UndefinedBehaviorSanitizer (host code only; no GPU involved)."""
import os
import shutil
import subprocess

import pytest

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "opaque_b200", "accounting", "csrc")


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_pld_core_is_clean_under_asan_and_ubsan(tmp_path):
    exe = tmp_path / "pld_selftest"
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined",
                            "-fno-omit-frame-pointer", "-fopenmp", os.path.join(CSRC, "pld.cpp"),
                            os.path.join(CSRC, "selftest.cpp"), "-o", str(exe)], capture_output=True, text=True, timeout=900)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=900,
                         env=dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", OMP_NUM_THREADS="4"))
    assert run.returncode == 0, run.stdout[-3000:] + run.stderr[-3000:]
    assert "all checks passed" in run.stdout and "runtime error" not in run.stderr
