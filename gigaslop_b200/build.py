"""Build recipe for libgigaslop_b200.so (nvcc, sm_100a only, in-tree output)."""
import os
import shutil
import subprocess

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libgigaslop_b200.so")
SRC = os.path.join(PKG, "csrc", "lib.cu")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
              "-shared", "-Xcompiler", "-fPIC"]


def _nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libgigaslop_b200.so cannot be built")


def sources():
    d = os.path.join(PKG, "csrc")
    inc = os.path.join(ROOT, "include", "gigaslop_b200")
    out = [os.path.join(d, f) for f in sorted(os.listdir(d))]
    for base, _, files in os.walk(inc):
        out += [os.path.join(base, f) for f in files]
    return out


def is_stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(s) > t for s in sources())


def build(force=False, verbose=False):
    """Compile the CUDA library if missing or older than its sources."""
    if not force and not is_stale():
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS, "-I" + os.path.join(ROOT, "include"), "-o", LIB, SRC]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    import sys
    print(build(force=True, verbose="-v" in sys.argv))
