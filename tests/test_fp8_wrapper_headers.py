"""The CUDA twins of the reference's fp8_*_wrapper headers compile as C++ and a small consumer (all-ones known
answer, as fly/main_rdna_fp8_gemm.cpp) passes on the GPU."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "abi", "fp8_consumer")


def build():
    from gigaslop_b200 import build as b
    b.build()
    cuda = "/usr/local/cuda"
    cmd = ["g++", os.path.join(ROOT, "tests", "abi", "fp8_consumer.cpp"), "-o", EXE, "-std=c++17", "-O2",
           "-I" + os.path.join(ROOT, "include", "gigaslop_b200"), "-I" + os.path.join(cuda, "include"),
           "-L" + os.path.join(cuda, "lib64"), "-lcudart_static", "-ldl", "-lrt", "-lpthread",
           "-L" + os.path.join(ROOT, "gigaslop_b200"), "-lgigaslop_b200", "-Wl,-rpath,$ORIGIN/../../gigaslop_b200"]
    subprocess.run(cmd, check=True)


def test_fp8_wrapper_header_compiles_and_links():
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    build()
    assert os.path.exists(EXE)


@pytest.mark.gpu
def test_fp8_wrapper_consumer_all_ones():
    if not os.path.exists(EXE):
        build()
    r = subprocess.run([EXE], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
