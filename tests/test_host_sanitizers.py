"""The host C++ (AVX-512 Adam, streaming copy, locked allocations, NVMe engine)
under AddressSanitizer + UBSan and under ThreadSanitizer: the stand-alone driver
``csrc/host/selftest/host_selftest.cpp`` is compiled together with the library
sources and must exit 0 with no sanitizer report.  The ThreadSanitizer build
leaves OpenMP out (libgomp is not instrumented); what it checks is the explicit
threading: the NVMe engine's workers, the registries and concurrent callers."""
import glob
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "csrc", "host")
CXX = os.environ.get("FLEXTRAIN_CXX", "/usr/bin/g++")


def _build_and_run(tmp_path, name, flags, env_extra):
    if not shutil.which(CXX):
        pytest.skip("no host compiler")
    exe = str(tmp_path / name)
    srcs = sorted(glob.glob(os.path.join(HOST, "*.cpp"))) + [os.path.join(HOST, "selftest", "host_selftest.cpp")]
    cmd = [CXX, "-O1", "-g", "-std=c++17", "-Wno-unknown-pragmas", "-mavx2", "-mfma", "-mf16c",
           "-fno-omit-frame-pointer", *flags, f"-I{os.path.join(ROOT, 'csrc')}", *srcs, "-o", exe, "-lpthread"]
    built = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if built.returncode != 0 and ("cannot find -l" in built.stderr or "unrecognized" in built.stderr):
        pytest.skip("sanitizer runtime not installed: " + built.stderr[-300:])
    assert built.returncode == 0, built.stderr[-3000:]
    scratch = tmp_path / "scratch"
    scratch.mkdir()
    run = subprocess.run([exe, str(scratch)], capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, **env_extra))
    out = run.stdout + run.stderr
    assert run.returncode == 0, out[-4000:]
    assert "host_selftest: ok" in out
    for marker in ("ERROR: AddressSanitizer", "runtime error:", "WARNING: ThreadSanitizer", "LeakSanitizer"):
        assert marker not in out, out[-4000:]


def test_host_code_under_asan_ubsan(tmp_path):
    _build_and_run(tmp_path, "selftest_asan", ["-fopenmp", "-fsanitize=address,undefined"],
                   {"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0", "UBSAN_OPTIONS": "print_stacktrace=1"})


def test_host_code_under_tsan(tmp_path):
    _build_and_run(tmp_path, "selftest_tsan", ["-fsanitize=thread"], {"TSAN_OPTIONS": "halt_on_error=0"})
