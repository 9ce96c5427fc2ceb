"""The C++ host mirror (include/candle_b200.hpp): compiles with g++ against the C-ABI library and
decides every argument error on the host with candle's messages.  No GPU."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_mirror_compiles_and_rejects_bad_arguments_like_candle(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    import candle_b200  # noqa: F401  (makes sure the library is built)

    lib_dir = os.path.join(ROOT, "candle_b200", "_lib")
    exe = str(tmp_path / "host_mirror_checks")
    subprocess.run([gxx, "-std=c++17", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"), "-o", exe,
                    os.path.join(ROOT, "tests", "cpp", "host_mirror_checks.cpp"), "-L", lib_dir,
                    "-l:libcandle_b200.so", f"-Wl,-rpath,{lib_dir}"], check=True)
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    lines = out.stdout.strip().splitlines()
    assert len(lines) >= 19 and all(l.startswith("ok ") for l in lines), out.stdout
