"""Runs the C++ unit-test executable that the in-tree build produces (host code, no GPU)."""
import subprocess

from mnnvl_sharp_b200 import _build


def test_native_cpp_suite():
    paths = _build.build_native()
    proc = subprocess.run([str(paths["tests"])], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "all native tests passed" in proc.stdout


def test_native_cpp_suite_under_address_and_ub_sanitizers():
    exe = _build.build_sanitized_tests()
    env = {"ASAN_OPTIONS": "detect_leaks=1:protect_shadow_gap=0", "UBSAN_OPTIONS": "print_stacktrace=1"}
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "all native tests passed" in proc.stdout
