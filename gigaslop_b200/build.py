"""Build recipe for libgigaslop_b200.so (nvcc, sm_100a only, in-tree output)."""
import os
import shutil
import subprocess

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libgigaslop_b200.so")
PTXAS_LOG = os.path.join(PKG, "libgigaslop_b200.ptxas.txt")    # ptxas -v of the last build: registers and spills per kernel
SRC = os.path.join(PKG, "csrc", "lib.cu")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
              "-shared", "-Xcompiler", "-fPIC", "-Xptxas=-v"]


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
    if not os.path.exists(LIB) or not os.path.exists(PTXAS_LOG):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(s) > t for s in sources())


def build(force=False, verbose=False, defines=(), out=None):
    """Compile the CUDA library if missing or older than its sources.  The resource report of ptxas (registers,
    spill bytes per kernel) is kept beside the library; ``kernel_resources()`` parses it.  ``defines`` / ``out``
    build a variant (``-DGSB200_DIAG`` for the tuning diagnostics) somewhere else."""
    target = out or LIB
    if out is None and not force and not is_stale():
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS, *["-D" + d for d in defines], "-I" + os.path.join(ROOT, "include"), "-o", target, SRC]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + r.stdout[-4000:])
    with open(PTXAS_LOG if out is None else target + ".ptxas.txt", "w") as f:
        f.write(r.stdout)
    if verbose:
        print(r.stdout)
    return target


def kernel_resources(log=None):
    """{mangled kernel name: dict(registers, stack, spill_stores, spill_loads)} from the ptxas report of the build."""
    import re
    text = open(log or PTXAS_LOG).read()
    out = {}
    for block in re.split(r"ptxas info\s+: Compiling entry function '", text)[1:]:
        name = block.split("'")[0]
        sp = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", block)
        rg = re.search(r"Used (\d+) registers", block)
        if sp and rg:
            out[name] = dict(registers=int(rg.group(1)), stack=int(sp.group(1)), spill_stores=int(sp.group(2)),
                             spill_loads=int(sp.group(3)))
    return out


if __name__ == "__main__":
    import sys
    print(build(force=True, verbose="-v" in sys.argv))
