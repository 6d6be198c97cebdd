"""Write per-shape C headers with the reference's names for the exported-kernel interface.

The reference exports one object + header per kernel shape (cute/export_gemm_i8_rotary.py,
cute/export_dual_gemm_i8_silu.py, cute/export_gemm_i8.py; TOML sweeps with ``[[configs]]`` tables).  With this
library a "shape" is only a header: the kernels take every dimension at run time, so the header just fixes the
names (and, for rotary, nhead / head_dim / rotary_dim and the table extent) and forwards to the C ABI.

    python -m gigaslop_b200.export_headers rotary --K 512 --nhead 8 --head-dim 64 --seqlen 2048 --out DIR
    python -m gigaslop_b200.export_headers dual_silu --N 2048 --K 512 --out DIR
    python -m gigaslop_b200.export_headers std --prefix gemm_i8_std --name gemm_i8_standard --out DIR
    python -m gigaslop_b200.export_headers rotary --config sweep.toml --out DIR

File and prefix names follow the reference: ``gemm_i8_rotary_N{N}_K{K}_H{nhead}D{head_dim}R{rotary_dim}S{seqlen}``
(N = 3 * nhead * head_dim, cute/export_gemm_i8_rotary.py:65-67) and ``gemm_i8_dual_silu_N{N}_K{K}``
(cute/export_dual_gemm_i8_silu.py:53-63).  A consumer adds ``-I<repo>/include/gigaslop_b200 -I DIR`` and links
``-lgigaslop_b200``; the module hooks of a generated header resolve to the library's generic pair.
"""
import argparse
import os

try:
    import tomllib
except ModuleNotFoundError:          # Python < 3.11
    tomllib = None


def _parse_simple_toml(path):
    """``[[configs]]`` tables of ``key = int`` lines (the format of the reference's sweeps)."""
    configs = []
    with open(path) as f:
        for raw in f:
            line = raw.split("#", 1)[0].strip()
            if not line:
                continue
            if line == "[[configs]]":
                configs.append({})
            elif "=" in line and configs:
                key, val = (t.strip() for t in line.split("=", 1))
                configs[-1][key] = int(val)
    return {"configs": configs}


def load_configs(path):
    if tomllib is not None:
        with open(path, "rb") as f:
            return tomllib.load(f)["configs"]
    return _parse_simple_toml(path)["configs"]


def _hooks(prefix):
    return (f"#define _mlir_{prefix}_cuda_init gsb200_module_cuda_init\n"
            f"#define _mlir_{prefix}_cuda_load_to_device gsb200_module_cuda_load_to_device\n")


def rotary_header(K, nhead, head_dim, rotary_dim, seqlen):
    if head_dim not in (64, 128) or rotary_dim not in (32, 64, 96, 128) or rotary_dim > head_dim:
        raise ValueError("the rotary epilogues take head_dim 64 or 128 and rotary_dim 32 / 64 / 96 / 128 (<= head_dim)")
    N = 3 * nhead * head_dim
    name = f"gemm_i8_rotary_N{N}_K{K}_H{nhead}D{head_dim}R{rotary_dim}S{seqlen}"
    text = (f"/* {name}: W8A8 QKV GEMM + rotary, N = {N}, K = {K}, {nhead} heads x {head_dim}, sin/cos tables of\n"
            f" * {seqlen} rows (name pattern of cute/export_gemm_i8_rotary.py:65-67).  Written by\n"
            f" * gigaslop_b200.export_headers. */\n#pragma once\n" + _hooks(name) +
            f"#define GSB200_ROT_PREFIX {name}\n#define GSB200_ROT_NHEAD {nhead}\n#define GSB200_ROT_HEAD_DIM {head_dim}\n"
            f"#define GSB200_ROT_ROTARY_DIM {rotary_dim}\n#define GSB200_ROT_SEQ_TABLE {seqlen}\n"
            f'#include "artifacts/gemm_i8_rotary_template.h"\n')
    return name, text


def dual_silu_header(N, K):
    name = f"gemm_i8_dual_silu_N{N}_K{K}"
    text = (f"/* {name}: W8A8 SwiGLU dual GEMM (name pattern of cute/export_dual_gemm_i8_silu.py:53-63).  Written by\n"
            f" * gigaslop_b200.export_headers. */\n#pragma once\n" + _hooks(name) +
            f'#define GSB200_DUAL_PREFIX {name}\n#include "artifacts/gemm_i8_dual_silu_template.h"\n')
    return name, text


def std_header(prefix, name):
    text = (f"/* {name}: W8A8 GEMM with per-token x per-channel dequant, prefix {prefix} (cute/export_gemm_i8.py:16-28).\n"
            f" * Written by gigaslop_b200.export_headers. */\n#pragma once\n" + _hooks(prefix) +
            f'#define GSB200_STD_PREFIX {prefix}\n#include "artifacts/gemm_i8_std_template.h"\n')
    return name, text


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kind", choices=["rotary", "dual_silu", "std"])
    ap.add_argument("--out", required=True, help="directory the headers are written to")
    ap.add_argument("--config", help="TOML file with [[configs]] tables (keys as the options below)")
    ap.add_argument("--K", type=int, default=512)
    ap.add_argument("--N", type=int, default=2048, help="dual_silu: columns of each of gate / up")
    ap.add_argument("--nhead", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--rotary-dim", type=int, default=None)
    ap.add_argument("--seqlen", type=int, default=2048)
    ap.add_argument("--prefix", default="gemm_i8_std")
    ap.add_argument("--name", default="gemm_i8_standard")
    a = ap.parse_args(argv)
    base = dict(K=a.K, N=a.N, nhead=a.nhead, head_dim=a.head_dim, rotary_dim=a.rotary_dim, seqlen=a.seqlen)
    cfgs = [dict(base, **c) for c in load_configs(a.config)] if a.config else [base]
    os.makedirs(a.out, exist_ok=True)
    written = []
    for c in cfgs:
        if a.kind == "rotary":
            rd = c["rotary_dim"] if c.get("rotary_dim") else c["head_dim"]
            name, text = rotary_header(c["K"], c["nhead"], c["head_dim"], rd, c["seqlen"])
        elif a.kind == "dual_silu":
            name, text = dual_silu_header(c["N"], c["K"])
        else:
            name, text = std_header(a.prefix, a.name)
        path = os.path.join(a.out, name + ".h")
        with open(path, "w") as f:
            f.write(text)
        written.append(path)
        print(path)
    return written


if __name__ == "__main__":
    main()
