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
