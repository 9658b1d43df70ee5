"""Generates the golden fixtures that pin the CPU oracle to the reference's own PyTorch path.

Run where the reference checkout is available:

    python tests/golden/make_golden.py [/path/to/reference]

It imports the reference's ref_rms.py UNMODIFIED (a stub `tensorrt` module and a no-op
torch.cuda.set_device let the import succeed on a CPU-only machine; `ref_rms.dtype` / `ref_rms.device`
are the module's own globals, set to float32 / cpu), runs its Vanila, PreNorm, QKNorm, KeyFormer and
RoCo classes (ref_rms.py:29-280) on seeded inputs and stores

  golden_small.npz   full inputs and outputs at a small shape (M16 N128 D64 P48)
  golden_native.npz  sampled outputs at the reference's native llama / falcon shapes
                     (convert_eval_rms.py:33-60), inputs regenerated from the seed by the test
  golden_batched.npz the two reference functions that carry a batch dim or a token-major O2:
                     SimpleBatchAttention (ref_rms.py:1420-1479, B = 2, PreNorm math, output [B, M, N] token-major)
                     and reference_kernel (convert_eval_rms.py:122-162, the per-head loop; its function text is
                     executed as it stands — the module around it imports packages that do not exist)

The fixtures are committed; the tests never need the reference checkout.
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference(ref_dir: str):
    sys.modules.setdefault("tensorrt", types.ModuleType("tensorrt"))
    real_set_device = torch.cuda.set_device
    torch.cuda.set_device = lambda *_a, **_k: None
    sys.path.insert(0, ref_dir)
    try:
        import ref_rms  # noqa: the reference's module
    finally:
        torch.cuda.set_device = real_set_device
        sys.path.remove(ref_dir)
    ref_rms.dtype = torch.float32
    ref_rms.device = torch.device("cpu")
    return ref_rms


def make_inputs(seed: int, M: int, N: int, D: int, H: int, P: int):
    """Input recipe of convert_eval_rms.py:170-215 (seed, randn.clamp(-1,1)*0.01, noise ~ randn), in fp32."""
    torch.manual_seed(seed)
    std = 0.01
    t = {}
    t["X"] = torch.randn((M, N)).clamp(-1, 1) * std
    t["WQ"] = torch.randn((N, N)).clamp(-1, 1) * std
    t["WK"] = torch.randn((N, N)).clamp(-1, 1) * std
    t["WV"] = torch.randn((N, N)).clamp(-1, 1) * std
    t["K_cache"] = torch.randn((H, P + M, D)).clamp(-1, 1) * std
    t["V_cache"] = torch.randn((H, P + M, D)).clamp(-1, 1) * std
    t["noise"] = torch.randn((H, M, P + M))
    return t


def run_reference(ref, name: str, t, M, N, D, P):
    kc, vc = t["K_cache"].clone(), t["V_cache"].clone()
    if name == "vanilla":
        return (ref.Vanila(M, N, D, P, kc, vc, t["WQ"], t["WK"], t["WV"])(t["X"]),)
    if name == "prenorm":
        return (ref.PreNorm(M, N, D, P, kc, vc, t["WQ"], t["WK"], t["WV"])(t["X"]),)
    if name == "qknorm":
        return (ref.QKNorm(M, N, D, P, kc, vc, t["WQ"], t["WK"], t["WV"])(t["X"]),)
    if name == "keyformer":
        return ref.KeyFormer(M, N, D, P, t["noise"], kc, vc, t["WQ"], t["WK"], t["WV"])(t["X"])
    if name == "roco":
        return ref.RoCo(M, N, D, P, kc, vc, t["WQ"], t["WK"], t["WV"])(t["X"])
    raise ValueError(name)


def load_reference_kernel(ref_dir: str):
    """convert_eval_rms.py cannot be imported (its first lines import a missing `convert_module` and
    `baseline.inductor`); its function `reference_kernel` is compiled from the file's own text, unmodified."""
    import ast
    path = os.path.join(ref_dir, "convert_eval_rms.py")
    tree = ast.parse(open(path).read(), path)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "reference_kernel")
    ns = {"torch": torch}
    exec(compile(ast.Module([fn], []), path, "exec"), ns)
    return ns["reference_kernel"]


def make_batched(ref, ref_dir: str) -> dict:
    """B = 2 through SimpleBatchAttention, and each batch item through reference_kernel."""
    B, M, N, D, P = 2, 16, 128, 64, 48
    H = N // D
    torch.manual_seed(7)
    std = 0.01
    t = {"X": torch.randn(B, M, N).clamp(-1, 1) * std, "WQ": torch.randn(N, N).clamp(-1, 1) * std,
         "WK": torch.randn(N, N).clamp(-1, 1) * std, "WV": torch.randn(N, N).clamp(-1, 1) * std,
         "K_cache": torch.randn(B, H, P + M, D).clamp(-1, 1) * std, "V_cache": torch.randn(B, H, P + M, D).clamp(-1, 1) * std}
    out = {"dims": np.array([B, M, N, D, H, P]), "seed": np.array([7])}
    for k, v in t.items():
        out["in_" + k] = v.numpy()
    with torch.no_grad():
        kc, vc = t["K_cache"].clone(), t["V_cache"].clone()
        o2 = ref.SimpleBatchAttention(B, M, N, D, P, kc, vc, t["WQ"], t["WK"], t["WV"])(t["X"])
        out["batch_O2"] = o2.numpy()                      # [B, M, N] token-major
        out["batch_K_cache"] = kc.numpy()                 # rows [P, P+M) appended in place (ref_rms.py:1460-1461)
        out["batch_V_cache"] = vc.numpy()
        rk = load_reference_kernel(ref_dir)
        per_item = []
        for b in range(B):
            kcb, vcb = t["K_cache"][b].clone(), t["V_cache"][b].clone()
            per_item.append(rk(t["X"][b], t["WQ"], t["WK"], t["WV"], kcb, vcb, M, N, D, H, P))
        out["loop_O2"] = torch.stack(per_item).numpy()    # [B, M, N]
    return out


OUT_NAMES = {"vanilla": ("out",), "prenorm": ("out",), "qknorm": ("out",),
             "keyformer": ("out", "perturb_out"), "roco": ("out", "sum_p", "sum_p2")}


def sample_indices(numel: int, n: int = 512) -> np.ndarray:
    rng = np.random.RandomState(1234)
    return np.sort(rng.choice(numel, size=min(n, numel), replace=False))


def main() -> None:
    ref_dir = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TRINITY_REFERENCE_DIR")
    if not ref_dir:
        sys.exit("usage: python " + sys.argv[0] + " <reference checkout>   (or set TRINITY_REFERENCE_DIR)")
    ref = import_reference(ref_dir)
    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # ---- small shape: everything stored
    M, N, D, P = 16, 128, 64, 48
    H = N // D
    small = {"dims": np.array([M, N, D, H, P]), "seed": np.array([42])}
    t = make_inputs(42, M, N, D, H, P)
    for k, v in t.items():
        small["in_" + k] = v.numpy()
    with torch.no_grad():
        for name in OUT_NAMES:
            outs = run_reference(ref, name, t, M, N, D, P)
            for oname, o in zip(OUT_NAMES[name], outs):
                small[f"{name}_{oname}"] = o.detach().float().numpy()
    np.savez_compressed(os.path.join(HERE, "golden_small.npz"), **small)

    # ---- native shapes: sampled outputs
    native = {}
    for model, (M, N, D, H, P) in {"llama": (16, 4096, 128, 32, 1024), "falcon": (16, 4544, 64, 71, 1024)}.items():
        t = make_inputs(42, M, N, D, H, P)
        native[f"{model}_dims"] = np.array([M, N, D, H, P])
        with torch.no_grad():
            for name in OUT_NAMES:
                outs = run_reference(ref, name, t, M, N, D, P)
                for oname, o in zip(OUT_NAMES[name], outs):
                    flat = o.detach().float().reshape(-1)
                    idx = sample_indices(flat.numel())
                    native[f"{model}_{name}_{oname}_idx"] = idx
                    native[f"{model}_{name}_{oname}_val"] = flat[idx].numpy()
                    native[f"{model}_{name}_{oname}_stat"] = np.array(
                        [flat.numel(), flat.double().mean().item(), flat.double().abs().mean().item(),
                         flat.abs().max().item()])
                    print(model, name, oname, tuple(o.shape), native[f"{model}_{name}_{oname}_stat"])
    np.savez_compressed(os.path.join(HERE, "golden_native.npz"), **native)
    np.savez_compressed(os.path.join(HERE, "golden_batched.npz"), **make_batched(ref, ref_dir))
    print("written", os.path.join(HERE, "golden_small.npz"), os.path.join(HERE, "golden_native.npz"))


if __name__ == "__main__":
    main()
