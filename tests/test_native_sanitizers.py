"""Host-side native code (thread pool + AVX Adam, shared-memory collectives) under AddressSanitizer + UBSan and under
ThreadSanitizer.  The device code cannot be run under compute-sanitizer here; the C++ runtime around it can be
checked on the CPU, which is what this does: ``tests/native/sanitize_driver.cpp`` is compiled together with the library
sources and has to finish without a sanitizer report."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "bmtrain_b200", "csrc")


@pytest.mark.parametrize("sanitizer", ["address,undefined", "thread"])
def test_native_host_code_under_sanitizer(sanitizer, tmp_path):
    # the toolchain named by $CXX may come without sanitizer runtimes: fall back to the system compiler
    candidates = [c for c in dict.fromkeys([os.environ.get("CXX"), "g++", "/usr/bin/g++"]) if c and shutil.which(c)]
    if not candidates:
        pytest.skip("no C++ compiler")
    exe = str(tmp_path / "driver")
    built = None
    for cxx in candidates:
        cmd = [cxx, "-O1", "-g", "-std=c++17", "-pthread", "-mavx2", "-mfma", "-mf16c", f"-fsanitize={sanitizer}",
               "-fno-omit-frame-pointer", "-o", exe, os.path.join(ROOT, "tests", "native", "sanitize_driver.cpp"),
               os.path.join(CSRC, "cpu_adam.cpp"), os.path.join(CSRC, "cpu_comm.cpp"), "-I", CSRC, "-lrt"]
        built = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
        if built.returncode == 0:
            break
    if built.returncode != 0:
        pytest.skip("sanitizer runtime not available: " + built.stderr[-300:])
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1",
               TSAN_OPTIONS="halt_on_error=1")
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300, env=env)
    report = run.stdout[-3000:] + run.stderr[-3000:]
    assert run.returncode == 0, report
    assert "all checks passed" in run.stdout and "Sanitizer" not in report and "runtime error" not in report, report
