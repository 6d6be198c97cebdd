"""The reference's own C++ AOT tests, compiled UNMODIFIED against the drop-in headers
(oracle/build_ref.py), must link on CPU and pass on the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_BIN = os.path.join(ROOT, "oracle", "_ref")


def test_reference_consumers_compile_and_link_unchanged():
    from oracle import build_ref
    if not os.path.isdir(build_ref.REF):
        pytest.skip("reference checkout not present on this machine")
    from gigaslop_b200 import build
    build.build()
    built = build_ref.build(force=True)
    assert {os.path.basename(b) for b in built} == {"main", "main_rotary"}
    out = subprocess.run(["nm", "-u", os.path.join(REF_BIN, "main_rotary")], capture_output=True, text=True).stdout
    assert "gsb200_gemm_i8_rotary_f16" in out and "_mlir_gemm_i8_rotary_N1536_K512_H8D64R64S1024_cuda_init" in out


def _run(name, env=None):
    exe = os.path.join(REF_BIN, name)
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref not built (needs the reference checkout at build time)")
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([exe], capture_output=True, text=True, env=e, timeout=120)


@pytest.mark.gpu
def test_reference_main_cpp_passes():
    r = _run("main")
    assert r.returncode == 0, r.stdout + r.stderr
    assert "mismatches: 0" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("env", [{}, {"ROTARY_SEQLEN": "333"}, {"ROTARY_IDENTITY": "1"}, {"ROTARY_SEQLEN": "1"}])
def test_reference_main_rotary_cpp_passes(env):
    r = _run("main_rotary", env)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "PASS" in r.stdout
