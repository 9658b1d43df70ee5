"""This library against the reference's OWN kernels on the same GPU: the Triton modules that the reference's
generator (IrParser.py -> TritonGen.py:348) emits for the packaged IR programs, produced beforehand by
oracle/make_reference_kernels.py into oracle/_ref/ (git-ignored).  Skipped when that folder is absent.

Both sides get the tensors of the reference's harness (seed 42, `randn.clamp(-1, 1) * 0.01`, fp16, M = 16 new
tokens, P = 1024 cached; vanilla_llama_benchmark.py:131-139, convert_eval_rms.py:174-183) through the same
`forward(*tensors)` surface.  The generated kernels accumulate in fp16 and have no max-subtraction
(TritonGen.py:3057-3172), so the yardstick is the fp32 oracle: this library must be at least as close to it as
the reference's kernels are, and the two must agree to within the reference's own error.
"""
import importlib.util
import os
import sys

import pytest
import torch

from oracle import attn_block_ref as O
from triton_b200 import _lib as L
from triton_b200.convert_module import convert_ir_to_triton
from triton_b200.harness import AttnBlockBenchmark, tables_for

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")
IR_DIR = os.path.join(ROOT, "triton_b200", "ir_programs")

CASES = [(p, "llama") for p in ("vanilla", "prenorm", "prenorm_fused", "qknorm", "keyformer", "roco", "rmsnorm")] + \
        [("vanilla", "falcon"), ("keyformer", "falcon"), ("lora", "base"), ("lora", "large"),
         ("gmlp", "base"), ("gmlp", "large"), ("gmlp_glu", "base")]


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _outputs(program):
    if program == "rmsnorm":
        return ["X_norm"]
    if program == "lora":
        return ["O", "D"]
    if program.startswith("gmlp"):
        return ["O"]
    outs = ["O2"]
    if program == "keyformer":
        outs.append("C_out")
    if program == "roco":
        outs += ["C_out1", "C_out2"]
    return outs


@pytest.mark.parametrize("program,model", CASES)
def test_against_the_references_generated_kernels(program, model, tmp_path):
    path = os.path.join(REF_DIR, f"{program}_{model}.py")
    if not os.path.isfile(path):
        pytest.skip("oracle/_ref not generated (needs the reference checkout: python oracle/make_reference_kernels.py)")
    pytest.importorskip("triton")
    shapes, consts = tables_for(program, model)
    M, N, P = consts["M"], consts["N"], consts.get("P", 0)
    D, H = consts.get("D"), consts.get("H")
    ref_mod = _load(path, f"refgen_{program}_{model}")
    src = convert_ir_to_triton(open(os.path.join(IR_DIR, f"{program}.txt")).read(), shapes, consts)
    our_path = tmp_path / f"ours_{program}_{model}.py"
    our_path.write_text(src)
    our_mod = _load(str(our_path), f"ours_{program}_{model}")
    assert our_mod.TENSOR_PARAMS == ref_mod.TENSOR_PARAMS        # same operator surface, same argument order

    bench = AttnBlockBenchmark(consts, seed=42, shape_dict=shapes)
    bench.create_test_tensors(ref_mod.TENSOR_PARAMS)
    T = bench.tensors
    host = {k: v.detach().cpu().clone() for k, v in T.items()}
    names = _outputs(program)

    def run(mod):
        for k, v in host.items():
            T[k].copy_(v)
        mod.forward(*[T[p] for p in mod.TENSOR_PARAMS])
        torch.cuda.synchronize()
        res = {n: T[n].float().cpu() for n in names}
        if program not in ("rmsnorm", "lora") and not program.startswith("gmlp"):
            res["K_new"] = T["K_cache"][:, P:].float().cpu()
        return res

    ref_out = run(ref_mod)
    our_out = run(our_mod)
    assert L.kernel_status() == 0

    # fp32 oracle on the same inputs
    if program == "rmsnorm":
        want = {"X_norm": O.rmsnorm(host["X"])}
    elif program == "lora":
        r = O.lora(host["X"], host["W"], host["A"], host["B"])
        want = {"O": r["O"], "D": r["D"]}
    elif program.startswith("gmlp"):
        want = {"O": O.gmlp(host["X"], host["W1"], host["W2"], gate="sigmoid" if program == "gmlp_glu" else "silu")["O"]}
    else:
        variant = program.split("_")[0]
        r = O.attn_block(variant, X=host["X"], Wq=host["WQ"], Wk=host["WK"], Wv=host["WV"],
                         cache_K=host["K_cache"].unsqueeze(0), cache_V=host["V_cache"].unsqueeze(0), B=1, M=M, P=P,
                         Hq=H, Hkv=H, D=D, noise=host["noise"].unsqueeze(0) if "noise" in host else None)
        want = {"O2": r["out_bmhd"][0].reshape(M, H * D), "K_new": r["k_all"][0, :, P:]}
        if program == "keyformer":
            want["C_out"] = r["sum_p"][0]
        if program == "roco":
            want["C_out1"], want["C_out2"] = r["sum_p"][0], r["sum_p2"][0]

    for name, w in want.items():
        ours, ref = our_out[name].reshape(w.shape), ref_out[name].reshape(w.shape)
        assert torch.isfinite(ours).all(), f"{name}: this library produced non-finite values"
        e_ours = (ours - w).abs().max().item()
        scale = w.abs().max().item()
        if not torch.isfinite(ref).all():
            # e.g. QKNorm: unit-norm q.k reaches head_dim and exp() overflows the generated kernels' fp16 (no
            # max-subtraction); nothing to agree with, the oracle check stands alone
            assert e_ours <= 2e-2 * max(scale, 1.0)
            continue
        e_ref = (ref - w).abs().max().item()
        print(f"{program}/{model} {name}: max|ref| {scale:.3e}  |ours - oracle| {e_ours:.3e}  "
              f"|reference kernels - oracle| {e_ref:.3e}  |ours - reference kernels| {(ours - ref).abs().max().item():.3e}")
        assert e_ours <= max(e_ref, 2e-3 * scale) * 1.05, f"{name}: further from the fp32 oracle than the reference's kernels"
        assert (ours - ref).abs().max().item() <= e_ref + e_ours + 1e-7
    bench.cleanup()
