"""The compiled kernels' resource report (ptxas -v, kept beside the library by the build): no kernel may spill.

A spilled register is more than a slowdown for the tcgen05 kernels: tcgen05.ld only starts a transfer into its
destination registers, and a spill placed between the load and tcgen05.wait::ld would save the registers before the
data has arrived.  Zero spill bytes everywhere is the one state in which that cannot happen."""
import subprocess


def test_no_kernel_spills_registers():
    from gigaslop_b200 import build
    build.build()
    res = build.kernel_resources()
    assert len(res) >= 40, f"only {len(res)} kernels found in the ptxas report"
    bad = {k: v for k, v in res.items() if v["stack"] or v["spill_stores"] or v["spill_loads"]}
    if bad:
        names = subprocess.run(["c++filt", *bad], capture_output=True, text=True).stdout.split("\n")
        raise AssertionError("kernels with spills: " + "; ".join(f"{n} {v}" for n, v in zip(names, bad.values())))
    # every tcgen05 kernel keeps one CTA per SM: its register allocation fits the register file
    for name, v in res.items():
        assert v["registers"] <= 255, name


def test_twelve_warp_gemm_register_pool_covers_its_resplit():
    """The twelve-epilogue-warp GEMM raises its epilogue warps to 152 registers with setmaxnreg, which waits for the
    CTA's pool: 512 threads x the compiled register count must cover 128 x 56 + 384 x 152 (the host checks the same
    through cudaFuncGetAttributes before it ever launches that form)."""
    from gigaslop_b200 import build
    build.build()
    res = {k: v for k, v in build.kernel_resources().items() if "gemm_tcgen05_kernel" in k and k.endswith("Li12EEEv14CUtensorMap_stS1_S1_S1_NS_10GemmParamsE")}
    assert len(res) >= 12, sorted(res)
    for name, v in res.items():
        assert 512 * v["registers"] >= 128 * 56 + 384 * 152, (name, v)
        assert 512 * v["registers"] <= 65536, (name, v)
