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


@pytest.mark.gpu
def test_hot_path_from_plain_c(tmp_path):
    """GGUF file -> native loader -> prompt -> greedy decode, all from a C program; the tokens must be the committed
    golden ones of the tiny float32 configuration (prompt of 64, 64 greedy tokens)."""
    import numpy as np

    from nfai_b200 import gguf_io, synth
    exe = _compile(tmp_path)
    cfg = synth.get_config("c0")
    gguf = str(tmp_path / "c0.gguf")
    gguf_io.write_synthetic_gguf(cfg, gguf, seed=0)
    gold = np.load(os.path.join(ROOT, "tests", "golden", "c0.npz"))
    toks = str(tmp_path / "tokens.txt")
    with open(toks, "w") as fh:
        fh.write(" ".join(str(int(t)) for t in gold["prompt"]) + "\n")
        fh.write(" ".join(str(int(t)) for t in gold["greedy"]) + "\n")
    r = subprocess.run([exe, "gpu", gguf, toks], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    assert "hot path ok" in r.stdout


def _compile_xchg_model(tmp_path):
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    if not gxx:
        pytest.skip("no C++ compiler")
    exe = str(tmp_path / "xchg_model")
    subprocess.run([gxx, "-O2", "-std=c++17", "-pthread", "-Wall", "-Werror", "-I", os.path.join(ROOT, "nfai_b200", "csrc"),
                    os.path.join(ROOT, "tests", "cabi", "xchg_model.cpp"), "-o", exe], check=True)
    return exe


@pytest.mark.parametrize("world,rounds,H", [(2, 400, 32), (4, 300, 64), (8, 150, 128)])
def test_exchange_protocol_with_cpu_threads_as_ranks(tmp_path, world, rounds, H):
    """The epoch / parity protocol of the tensor-parallel exchange (the header the kernels compile) run by CPU threads:
    bit-identical sums on every rank, lowest-index arg-max, epochs across the 32-bit wrap."""
    exe = _compile_xchg_model(tmp_path)
    r = subprocess.run([exe, str(world), str(rounds), str(H)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, (r.stdout, r.stderr)


def test_exchange_protocol_gives_up_when_a_rank_is_gone(tmp_path):
    """A rank that stops publishing: the others leave their bounded wait with a time-out, nothing hangs."""
    exe = _compile_xchg_model(tmp_path)
    r = subprocess.run([exe, "4", "100", "64", "2", "37"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, (r.stdout, r.stderr)
