"""Recipe: compile the reference's own C++ consumer programs, from the sources where they lie in the
reference checkout and UNMODIFIED, against this repository's drop-in headers and library.

    cute/main.cpp         plain W8A8 dequant GEMM 128^3, host fp32 check, abs err <= 0.5
    cute/main_rotary.cpp  QKV GEMM + rotary M=256 N=1536 K=512, per-region abs/rel gate; env
                          ROTARY_SEQLEN / ROTARY_IDENTITY select the runtime seqlen / an identity table

They are test infrastructure (parity checkers run on the GPU by the test-suite): outputs go to
oracle/_ref/ only, no reference source is copied.  Nothing is built when the checkout is absent.
"""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref")
REF = os.environ.get("GIGASLOP_REFERENCE", "/root/reference")
PROGRAMS = {"main": "cute/main.cpp", "main_rotary": "cute/main_rotary.cpp"}


def cuda_home():
    for c in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if c and os.path.isdir(c):
            return c
    nvcc = shutil.which("nvcc")
    return os.path.dirname(os.path.dirname(nvcc)) if nvcc else None


def build(force=False):
    if not os.path.isdir(REF):
        return []
    cuda = cuda_home()
    if cuda is None or shutil.which("g++") is None:
        return []
    os.makedirs(OUT, exist_ok=True)
    lib_dir = os.path.join(ROOT, "gigaslop_b200")
    built = []
    for name, rel in PROGRAMS.items():
        src = os.path.join(REF, rel)
        dst = os.path.join(OUT, name)
        lib = os.path.join(lib_dir, "libgigaslop_b200.so")
        if not force and os.path.exists(dst) and os.path.getmtime(dst) >= max(os.path.getmtime(src), os.path.getmtime(lib)):
            built.append(dst)
            continue
        # cf. the reference's own link line (cute/build_rotary_test.sh:25-33): the exported object and the DSL
        # runtime are replaced by -lgigaslop_b200; the headers come from include/gigaslop_b200/artifacts/
        cmd = ["g++", src, "-o", dst, "-std=c++17", "-O2", "-I" + os.path.join(ROOT, "include", "gigaslop_b200"),
               "-I" + os.path.join(cuda, "include"), "-L" + os.path.join(cuda, "lib64"), "-lcudart_static", "-ldl",
               "-lrt", "-lpthread", "-L" + lib_dir, "-lgigaslop_b200", "-Wl,-rpath,$ORIGIN/../../gigaslop_b200"]
        subprocess.run(cmd, check=True)
        built.append(dst)
    return built


if __name__ == "__main__":
    print("\n".join(build(force=True)) or "reference checkout not found; nothing built")
