"""Pins the CPU oracle to the reference: with every generalisation flag at its default the oracle must
reproduce what the reference's own classes (ref_rms.py:29-280) returned for the same inputs.  The
fixtures were produced by tests/golden/make_golden.py from the unmodified reference module."""
import os

import numpy as np
import pytest
import torch

from oracle import attn_block_ref as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")
VARIANTS = ("vanilla", "prenorm", "qknorm", "keyformer", "roco")


def _run_oracle(variant, t, M, N, D, H, P):
    return O.attn_block(variant, X=t["X"], Wq=t["WQ"], Wk=t["WK"], Wv=t["WV"],
                        cache_K=t["K_cache"].unsqueeze(0), cache_V=t["V_cache"].unsqueeze(0),
                        B=1, M=M, P=P, Hq=H, Hkv=H, D=D, noise=t["noise"].unsqueeze(0) if variant == "keyformer" else None)


@pytest.mark.parametrize("variant", VARIANTS)
def test_small_shape_equals_reference(variant):
    g = np.load(os.path.join(GOLD, "golden_small.npz"))
    M, N, D, H, P = (int(v) for v in g["dims"])
    t = {k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("in_")}
    r = _run_oracle(variant, t, M, N, D, H, P)
    ref_out = torch.from_numpy(g[f"{variant}_out"])
    # the reference returns .view(M, H*D) of the head-major result (ref_rms.py:80-81)
    torch.testing.assert_close(O.reference_view(r["out"]), ref_out, rtol=1e-5, atol=1e-7)
    if variant == "keyformer":
        torch.testing.assert_close(r["perturb_out"][0], torch.from_numpy(g["keyformer_perturb_out"]), rtol=1e-5, atol=1e-8)
        torch.testing.assert_close(r["sum_p"][0], torch.from_numpy(g["keyformer_perturb_out"]).sum(dim=1), rtol=1e-5, atol=1e-7)
    if variant == "roco":
        torch.testing.assert_close(r["sum_p"][0], torch.from_numpy(g["roco_sum_p"]), rtol=1e-5, atol=1e-8)
        torch.testing.assert_close(r["sum_p2"][0], torch.from_numpy(g["roco_sum_p2"]), rtol=1e-5, atol=1e-9)


def _native_inputs(seed, M, N, D, H, P):
    # input recipe of convert_eval_rms.py:170-215, same call order as tests/golden/make_golden.py
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


@pytest.mark.parametrize("model", ("llama", "falcon"))
def test_native_shapes_equal_reference_samples(model):
    g = np.load(os.path.join(GOLD, "golden_native.npz"))
    M, N, D, H, P = (int(v) for v in g[f"{model}_dims"])
    t = _native_inputs(42, M, N, D, H, P)
    for variant in VARIANTS:
        r = _run_oracle(variant, t, M, N, D, H, P)
        outs = {"out": O.reference_view(r["out"])}
        if variant == "keyformer":
            outs["perturb_out"] = r["perturb_out"][0]
        if variant == "roco":
            outs["sum_p"], outs["sum_p2"] = r["sum_p"][0], r["sum_p2"][0]
        for name, val in outs.items():
            idx = torch.from_numpy(g[f"{model}_{variant}_{name}_idx"])
            want = torch.from_numpy(g[f"{model}_{variant}_{name}_val"])
            stat = g[f"{model}_{variant}_{name}_stat"]
            flat = val.reshape(-1)
            assert flat.numel() == int(stat[0])
            scale = float(stat[3])
            assert (flat[idx] - want).abs().max().item() <= 2e-5 * scale, (model, variant, name)
            assert abs(flat.double().abs().mean().item() - stat[2]) <= 1e-5 * max(stat[2], 1e-30)


def test_rmsnorm_matches_reference_formula():
    torch.manual_seed(0)
    x = torch.randn(7, 96)
    var = x.pow(2).mean(-1, keepdim=True)               # ref_rms.py:102
    torch.testing.assert_close(O.rmsnorm(x), x * torch.rsqrt(var))   # ref_rms.py:103
    w = torch.randn(96)
    torch.testing.assert_close(O.rmsnorm(x, w, 1e-6), w * (x * torch.rsqrt(var + 1e-6)))   # ref_attn.py:348-350


def test_batched_prenorm_and_token_major_output_equal_reference():
    """The only reference code with a batch dimension and a token-major O2: SimpleBatchAttention
    (ref_rms.py:1420-1479, B = 2) and the per-head loop reference_kernel (convert_eval_rms.py:122-162).  Pins the
    oracle's B > 1 path, its cache append and `out_bmhd` (what the generated kernels store into O2[M, N])."""
    g = np.load(os.path.join(GOLD, "golden_batched.npz"))
    B, M, N, D, H, P = (int(v) for v in g["dims"])
    t = {k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("in_")}
    r = O.attn_block("prenorm", X=t["X"].reshape(B * M, N), Wq=t["WQ"], Wk=t["WK"], Wv=t["WV"], cache_K=t["K_cache"],
                     cache_V=t["V_cache"], B=B, M=M, P=P, Hq=H, Hkv=H, D=D)
    got = r["out_bmhd"].reshape(B, M, N)
    torch.testing.assert_close(got, torch.from_numpy(g["batch_O2"]), rtol=1e-5, atol=1e-8)
    torch.testing.assert_close(got, torch.from_numpy(g["loop_O2"]), rtol=1e-5, atol=1e-8)
    # rows [P, P+M) appended, prefix kept (ref_rms.py:1460-1461)
    torch.testing.assert_close(r["k_all"], torch.from_numpy(g["batch_K_cache"]), rtol=1e-5, atol=1e-9)
    torch.testing.assert_close(r["v_all"], torch.from_numpy(g["batch_V_cache"]), rtol=1e-5, atol=1e-9)
    assert torch.equal(r["k_all"][:, :, :P], t["K_cache"][:, :, :P])
