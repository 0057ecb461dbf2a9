"""Builds and runs the C++ contract test of the header-only host mirror
(``include/rwkv7_b200.hpp``) against the C-ABI library.  No GPU is needed: every
case fails the input checks before any CUDA call."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_host_api_contract(pkg, tmp_path):
    lib_dir = os.path.dirname(pkg.LIB_PATH)
    exe = str(tmp_path / "host_api_contract")
    cmd = ["/usr/bin/g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "host_api_contract.cpp"), "-o", exe,
           "-L", lib_dir, "-lrwkv7_b200", f"-Wl,-rpath,{lib_dir}"]
    subprocess.check_call(cmd)
    res = subprocess.run([exe], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 failure(s)" in res.stdout
