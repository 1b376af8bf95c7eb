"""The host C++ library under AddressSanitizer + UndefinedBehaviorSanitizer: a driver links the
sources directly (no Python in the process), works on exactly-sized heap buffers and feeds the
bincode reader every truncation of a valid stream."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "axonml_b200", "csrc", "host")


@pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")
def test_host_library_is_clean_under_asan_and_ubsan(tmp_path):
    exe = str(tmp_path / "sanitize_driver")
    srcs = [os.path.join(HOST, f) for f in ("bincode.cpp", "quant.cpp", "cpu_kernels.cpp")]
    srcs.append(os.path.join(HOST, "tests", "sanitize_driver.cpp"))
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
           "-fno-sanitize-recover=all", "-fopenmp", *srcs, "-o", exe]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip("the sanitizer runtimes are not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1",
               OMP_NUM_THREADS="2")
    run = subprocess.run([exe], capture_output=True, text=True, timeout=600, env=env)
    assert run.returncode == 0, (run.stdout[-2000:] + run.stderr[-4000:])
    assert "sanitize_driver: ok" in run.stdout
