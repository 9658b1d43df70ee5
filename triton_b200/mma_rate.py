"""Prints the tensor pipe's per-instruction ceiling on this GPU for the MMA shapes the kernels use.

    python -m triton_b200.mma_rate

One row per shape: SM clocks per tcgen05.mma (M 128, K 16, bf16, fp32 accumulation) issued back to back by
one thread per SM, the multiply-accumulates per clock and SM that this amounts to, and the same with eight
warps streaming tensor-memory loads / stores beside it (what softmax warps do to the P v and q k^T MMAs).
"""
from __future__ import annotations

import ctypes as C
import json
import sys

from . import _lib as L

SHAPES = (("SS N64", 0, 64), ("SS N128", 1, 128), ("SS N256", 2, 256), ("TS N128", 3, 128), ("TS N64", 4, 64))


def measure(n_mma: int = 4096):
    lib = L.load()
    rows = []
    for name, code, n in SHAPES:
        row = {"shape": name}
        for key, traffic in (("clk_per_mma", 0), ("clk_per_mma_with_tmem_traffic", 1)):
            v = C.c_double()
            L.check(lib.trinity_probe_mma_rate(code, traffic, n_mma, C.byref(v)))
            row[key] = round(v.value, 1)
        row["mac_per_clk_per_sm"] = round(128 * n * 16 / row["clk_per_mma"])
        rows.append(row)
    return rows


def main(argv=None) -> int:
    rows = measure()
    if argv and "--json" in argv:
        print(json.dumps(rows))
        return 0
    print(f"{'shape':10s} {'clk / MMA':>10s} {'MAC / clk / SM':>15s} {'clk / MMA beside TMEM ld/st':>30s}")
    for r in rows:
        print(f"{r['shape']:10s} {r['clk_per_mma']:10.1f} {r['mac_per_clk_per_sm']:15d} "
              f"{r['clk_per_mma_with_tmem_traffic']:30.1f}")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
