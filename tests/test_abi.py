"""The C-ABI library on a machine without a GPU: it loads, exports every symbol the header declares,
its structs have the layout the ctypes binding assumes, and argument validation answers before any
CUDA work."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest

from triton_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "trinity_b200.h")


@pytest.fixture(scope="module")
def lib():
    if not L.LIB_PATH.exists():
        from triton_b200.build import build
        build()
    return L.load()


def test_exports_every_declared_symbol(lib):
    text = open(HEADER).read()
    declared = set(re.findall(r"\b(trinity_\w+)\s*\(", text))
    assert declared == set(L.EXPORTS), declared ^ set(L.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.trinity_abi_version() == L.ABI_VERSION


def test_struct_layout_matches_header(tmp_path):
    structs = {"TrnRmsArgs": L.TrnRmsArgs, "TrnHeadTensor": L.TrnHeadTensor, "TrnProjArgs": L.TrnProjArgs,
               "TrnAttnArgs": L.TrnAttnArgs, "TrnColStatsArgs": L.TrnColStatsArgs, "TrnTopkArgs": L.TrnTopkArgs,
               "TrnBlockArgs": L.TrnBlockArgs, "TrnBlockHostArgs": L.TrnBlockHostArgs, "TrnLoraArgs": L.TrnLoraArgs,
               "TrnGmlpArgs": L.TrnGmlpArgs}
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void) {"]
    for sname, st in structs.items():
        lines.append(f'  printf("{sname} %zu\\n", sizeof({sname}));')
        for fname, _ in st._fields_:
            lines.append(f'  printf("{sname}.{fname} %zu\\n", offsetof({sname}, {fname}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c11", "-o", str(exe), str(src)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    for line in out.splitlines():
        key, val = line.split()
        if "." in key:
            s, f = key.split(".")
            assert getattr(structs[s], f).offset == int(val), key
        else:
            assert C.sizeof(structs[key]) == int(val), key


def test_error_codes_and_messages(lib):
    for code in range(0, -10, -1):
        assert lib.trinity_strerror(code).decode() not in ("", "unknown error code")
    assert lib.trinity_strerror(-99).decode() == "unknown error code"
    # NULL argument blocks are refused before any CUDA call
    for fn in (lib.trinity_rmsnorm, lib.trinity_qkv_project, lib.trinity_lora, lib.trinity_gmlp, lib.trinity_attention, lib.trinity_attn_colstats,
               lib.trinity_topk, lib.trinity_attn_block, lib.trinity_attn_block_host):
        assert fn(None, None) == -1
    assert lib.trinity_attn_block_workspace(None) == 0
    a = L.TrnBlockArgs()
    a.B, a.M, a.Hq = 2, 100, 8
    # row scales [B*M] + two lse arrays [B,Hq,M], each padded to 256 bytes
    assert lib.trinity_attn_block_workspace(C.byref(a)) == 1024 + 2 * 6400
    with pytest.raises(L.TrinityError, match="NULL"):
        L.check(-1)


def test_no_cpu_fallback():
    import torch
    from triton_b200 import ops
    with pytest.raises(ValueError, match="no CPU path"):
        ops.rmsnorm(torch.randn(4, 64, dtype=torch.bfloat16))
    with pytest.raises(TypeError):
        ops._dtype_code(torch.randn(2, 2))


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", tmp_path / "libtrinity_b200.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        L.load()


def test_workspace_sizing_policies(lib):
    """Host-side sizing (no GPU needed): which shapes ask for split-KV partials and which keep their scores."""
    def attn_ws(B, M, P, Hq, Hkv, D):
        a = L.TrnAttnArgs()
        a.B, a.M, a.P, a.Hq, a.Hkv, a.D = B, M, P, Hq, Hkv, D
        return lib.trinity_attention_workspace(C.byref(a))

    def align(v):
        return (v + 255) // 256 * 256

    # the reference's Llama shape: 32 CTAs -> 4 key splits; two lse arrays and one o array of fp32 partials
    rows = 1 * 32 * 16
    assert attn_ws(1, 16, 1024, 32, 32, 128) == 2 * align(4 * rows * 4) + align(4 * rows * 128 * 4)
    assert attn_ws(8, 2048, 0, 32, 8, 128) == 0            # fills the GPU many times over
    assert attn_ws(1, 16, 128, 4, 4, 128) == 0             # two key blocks: nothing to split
    assert attn_ws(1, 16, 1024, 32, 32, 96) == 0           # unsupported head_dim: no claim

    def block_ws(variant, B, M, P, Hq, Hkv, D, N=4096):
        a = L.TrnBlockArgs()
        a.variant, a.B, a.M, a.P, a.N, a.Hq, a.Hkv, a.D = L.VARIANTS[variant], B, M, P, N, Hq, Hkv, D
        return lib.trinity_attn_block_workspace(C.byref(a))

    base = align(16 * 4) + 2 * align(rows * 4)
    split = attn_ws(1, 16, 1024, 32, 32, 128)
    scores = align(rows * 1056 * 4)                        # [B, Hq, M, pitch] fp32, pitch = 1040 rounded up to 32
    assert block_ws("vanilla", 1, 16, 1024, 32, 32, 128) == base + split
    assert block_ws("keyformer", 1, 16, 1024, 32, 32, 128) == base + split + scores
    assert block_ws("roco", 1, 16, 1024, 32, 32, 128) == base + split + scores
    # large statistics problems recompute q k^T instead of keeping 4 GiB of scores
    big = block_ws("keyformer", 4, 4096, 0, 32, 8, 128)
    assert big == align(4 * 4096 * 4) + 2 * align(4 * 32 * 4096 * 4)

    # keep_scores: the caller (the IR candidate's structure) can ask for either schedule
    def block_ws_keep(keep, B, M, P):
        a = L.TrnBlockArgs()
        a.variant, a.B, a.M, a.P, a.N, a.Hq, a.Hkv, a.D = L.VARIANTS["roco"], B, M, P, 4096, 32, 32, 128
        a.keep_scores = keep
        return lib.trinity_attn_block_workspace(C.byref(a))
    assert block_ws_keep(-1, 1, 16, 1024) == base + split                      # never kept: two-pass statistics
    assert block_ws_keep(1, 1, 16, 1024) == base + split + scores
    mid = 1 * 32 * 512 * 1024 * 4                                              # 64 MiB of scores: kept only on request
    assert block_ws_keep(0, 1, 512, 512) < mid <= block_ws_keep(1, 1, 512, 512)
    assert block_ws_keep(1, 4, 4096, 0) < (1 << 30)                            # 8 GiB of scores: never
