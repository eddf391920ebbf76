"""A C program (not C++, not Python) against the public header and the shared library."""
import os
import shutil
import subprocess

import pytest

from nfai_b200 import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cabi", "smoke.c")


def _compile(tmp_path):
    gcc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else shutil.which("gcc")
    if not gcc:
        pytest.skip("no C compiler")
    lib = build.build()
    exe = str(tmp_path / "cabi_smoke")
    subprocess.run([gcc, "-std=c11", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), SRC, "-o", exe,
                    "-L", os.path.dirname(lib), "-lnfai_cuda", "-Wl,-rpath," + os.path.dirname(lib)], check=True)
    return exe


def test_header_is_c_and_host_entry_points_run(tmp_path):
    exe = _compile(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    assert r.stdout.startswith("ok ")


@pytest.mark.gpu
def test_context_from_c(tmp_path):
    exe = _compile(tmp_path)
    r = subprocess.run([exe, "gpu"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
