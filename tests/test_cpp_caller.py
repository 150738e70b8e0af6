"""The C++ boundary: a caller written against the reference's headers (tsnecuda::Options, GpuOptions,
RunTsne; src/include/fit_tsne.h:33-35, src/include/options.h:59-230) compiles against include/tsnecuda/ and
links with -ltsnecuda.  The compile-and-link half runs without a GPU; the run half is a GPU test."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "run_tsne_caller.cpp")


def build_caller(tmp_path):
    from tsne_cuda_b200 import _lib
    libdir = os.path.dirname(_lib.LIB_PATH)
    exe = str(tmp_path / "run_tsne_caller")
    cxx = shutil.which("g++") or shutil.which("c++")
    assert cxx, "no C++ compiler"
    subprocess.check_call([cxx, "-std=c++17", "-O1", SRC, "-I", os.path.join(ROOT, "include"), "-L", libdir, "-ltsnecuda",
                           "-Wl,-rpath," + libdir, "-o", exe])
    return exe


def test_cpp_caller_compiles_and_links_against_the_reference_interface(tmp_path):
    exe = build_caller(tmp_path)
    out = subprocess.check_output(["nm", "-C", "--undefined-only", exe], text=True)
    assert "tsnecuda::RunTsne(tsnecuda::Options&, tsnecuda::GpuOptions&)" in out
    assert "tsnecuda::GpuOptions::GpuOptions(int)" in out


@pytest.mark.gpu
def test_cpp_caller_runs(tmp_path):
    exe = build_caller(tmp_path)
    r = subprocess.run([exe, "300"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "trained=1" in r.stdout and "finite=1" in r.stdout
