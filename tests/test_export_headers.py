"""gigaslop_b200.export_headers writes per-shape headers with the reference's names; a consumer written like
cute/main_rotary.cpp compiles and links against them (and, on a GPU, gets the known answer)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GEN = os.path.join(ROOT, "tests", "abi", "generated")
EXE = os.path.join(ROOT, "tests", "abi", "exported_consumer")


def build():
    from gigaslop_b200 import build as b
    from gigaslop_b200 import export_headers
    b.build()
    toml = os.path.join(GEN, "sweep.toml")
    os.makedirs(GEN, exist_ok=True)
    with open(toml, "w") as f:
        f.write("[[configs]]\nK = 256\nnhead = 4\nhead_dim = 64\nseqlen = 512\n")
    paths = export_headers.main(["rotary", "--config", toml, "--out", GEN])
    paths += export_headers.main(["dual_silu", "--N", "256", "--K", "128", "--out", GEN])
    assert [os.path.basename(p) for p in paths] == ["gemm_i8_rotary_N768_K256_H4D64R64S512.h", "gemm_i8_dual_silu_N256_K128.h"]
    cuda = "/usr/local/cuda"
    cmd = ["g++", os.path.join(ROOT, "tests", "abi", "exported_consumer.cpp"), "-o", EXE, "-std=c++17", "-O2",
           "-I" + GEN, "-I" + os.path.join(ROOT, "include", "gigaslop_b200"), "-I" + os.path.join(cuda, "include"),
           "-L" + os.path.join(cuda, "lib64"), "-lcudart_static", "-ldl", "-lrt", "-lpthread",
           "-L" + os.path.join(ROOT, "gigaslop_b200"), "-lgigaslop_b200", "-Wl,-rpath,$ORIGIN/../../gigaslop_b200"]
    subprocess.run(cmd, check=True)


def test_generated_headers_compile_and_link():
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    build()
    r = subprocess.run([EXE], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "linked" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_generated_headers_known_answer():
    if not os.path.exists(EXE):
        build()
    r = subprocess.run([EXE, "run"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
