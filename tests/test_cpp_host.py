"""Builds and runs the C++ host mirror's test program (tests/cpp): the same
kernels, inputs and acceptance rules as the reference's tests/gpu.rs, written
against cute_rs_b200/host/cute_host.hpp."""
import os
import subprocess

import pytest

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "test_host_mirror.cpp")
HDR = os.path.join(ROOT, "cute_rs_b200", "host", "cute_host.hpp")


@pytest.fixture(scope="module")
def program(lib, tmp_path_factory):
    oracle.build()
    odir = os.path.join(ROOT, "oracle")
    exe = os.path.join(ROOT, "build", "test_host_mirror")
    os.makedirs(os.path.dirname(exe), exist_ok=True)
    newest = max(os.path.getmtime(p) for p in (SRC, HDR, os.path.join(ROOT, "include", "cute_b200.h")))
    if not os.path.exists(exe) or os.path.getmtime(exe) < newest:
        subprocess.run(["/usr/bin/g++", "-std=c++17", "-O1", "-Wall", "-o", exe, SRC, "-L" + odir, "-loracle",
                        "-Wl,-rpath," + odir, "-ldl", "-fopenmp"], check=True)
    env = dict(os.environ, CUTE_B200_LIB=lib.LIB_PATH)
    return exe, env


def test_cpp_host_mirror_without_a_device(program):
    exe, env = program
    r = subprocess.run([exe, "cpu"], env=env, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


@pytest.mark.gpu
def test_cpp_host_mirror_on_the_gpu(program):
    exe, env = program
    r = subprocess.run([exe, "gpu"], env=env, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
