"""Whole attention blocks through trinity_attn_block (the unit the reference's generated forward()
computes) against the CPU oracle and against outputs of the reference's own classes (golden fixture).

The operator surface stores Q, K_cache and V_cache as 16-bit tensors (convert_eval_rms.py:62-108), so a
block is judged in the three steps it consists of:
  1. projection: the stored q / k / v against the fp32 oracle's, abs <= 2e-2, rel <= 1e-2 above 1e-3 of
     max|ref| (this is 16-bit rounding of an fp32-accurate value);
  2. attention and statistics: against the oracle evaluated on exactly the q / k / v the block stored,
     same tolerance — one differing bit in q or k moves a whole row of scores, so this is the only
     comparison in which the 1e-3 floor is meaningful for the block's output;
  3. end to end against the pure fp32 oracle (which never rounds q, k, v): abs <= 2e-2, and
     rel <= 5e-2 above 1e-1 of max|ref| — rounding q and k to 16 bits perturbs every score by about
     2^-9 (bf16) of its size, i.e. every probability by ~0.5 %, which no implementation of this 16-bit
     surface avoids; the 1e-2 relative bound is therefore carried by steps 1 and 2, where both sides
     see identical inputs.
"""
import importlib.util
import os
import sys

import numpy as np
import pytest
import torch

from conftest import assert_parity
from gpu_util import block_inputs, run_block
from oracle import attn_block_ref as O
from triton_b200 import _lib as L
from triton_b200 import ops
from triton_b200.convert_module import convert_ir_to_triton
from triton_b200.harness import IR_DIR, MODEL_CONFIGS, SHAPE_DICT, AttnBlockBenchmark

pytestmark = pytest.mark.gpu
BF, HF = torch.bfloat16, torch.float16
VARIANTS = ("vanilla", "prenorm", "qknorm", "keyformer", "roco")
REL_FLOOR_FP32 = 1e-1
REL_TOL_E2E = 5e-2


def _oracle(variant, t, dims, causal, scale, eps, tau, noise, round_to=None, round_x_norm=None):
    B, M, P, N, Hq, Hkv, D = dims
    return O.attn_block(variant, X=t["X"], Wq=t["WQ"], Wk=t["WK"], Wv=t["WV"], cache_K=t["K_cache"],
                        cache_V=t["V_cache"], B=B, M=M, P=P, Hq=Hq, Hkv=Hkv, D=D, causal=causal, scale=scale,
                        pre_eps=eps, pre_gamma=t["pre_gamma"], qk_eps=eps, gamma_q=t["gamma_q"], gamma_k=t["gamma_k"],
                        tau=tau, noise=noise, round_to=round_to, round_x_norm=round_x_norm)


def _check_block(variant, dims, dt, causal, scale, eps, gamma, ref_native, noise_mode=L.TRN_NOISE_TENSOR, seed=4,
                 rel_tol_e2e=REL_TOL_E2E):
    B, M, P, N, Hq, Hkv, D = dims
    t = block_inputs(seed, B, M, P, N, Hq, Hkv, D, dt, ref_native=ref_native, variant=variant, gamma=gamma,
                     noise_mode=noise_mode)
    tau = 1.5
    noise = t["noise"]
    if variant == "keyformer" and noise_mode == L.TRN_NOISE_GUMBEL:
        noise = O.gumbel_noise(11, B, Hq, M, P + M)
    got = run_block(variant, t, B=B, M=M, P=P, Hq=Hq, Hkv=Hkv, D=D, causal=causal, scale=scale, eps=eps, tau=tau,
                    noise_mode=noise_mode, seed=11)
    pure = _oracle(variant, t, dims, causal, scale, eps, tau, noise)
    # 1. projection (+ norms, + cache append) as stored.  PreNorm with gamma materialises X_norm as a
    #    16-bit tensor (gamma scales the contraction axis): it is checked on its own, and the projection is
    #    then checked on the X_norm that was stored.
    proj = pure
    x_norm = getattr(got["plan"], "_x_norm", None)
    if x_norm is not None:
        assert_parity(x_norm, O.rmsnorm(t["X"], t["pre_gamma"], eps), "X_norm")
        t2 = dict(t, X=x_norm.float().cpu())
        proj = _oracle("vanilla", t2, dims, causal, scale, eps, tau, None)
    assert_parity(got["q"], proj["q"].transpose(1, 2), f"{variant} q")
    assert_parity(got["k_cache"], proj["k_all"], f"{variant} k_cache")
    assert_parity(got["v_cache"], proj["v_all"], f"{variant} v_cache")
    # 2. attention + statistics on the stored q / k / v
    strict = O.attend(got["q"].float().cpu().transpose(1, 2), got["k_cache"].float().cpu(), got["v_cache"].float().cpu(),
                      P=P, causal=causal, scale=scale, variant=variant, tau=tau, noise=noise)
    assert_parity(got["out"], strict["out"].transpose(1, 2), f"{variant} out (attention on stored q/k/v)")
    if variant in ("keyformer", "roco"):
        assert_parity(got["sum_p"], strict["sum_p"], "sum_p", abs_tol=1e-3 * max(1.0, M / 16), rel_tol=1e-3)
    if variant == "roco":
        assert_parity(got["sum_p2"], strict["sum_p2"], "sum_p2", abs_tol=1e-3 * max(1.0, M / 16), rel_tol=1e-3)
    # 3. end to end against the fp32 oracle
    assert_parity(got["out"], pure["out_bmhd"], f"{variant} out (fp32 oracle)", rel_floor=REL_FLOOR_FP32,
                  rel_tol=rel_tol_e2e)
    if variant in ("keyformer", "roco"):
        assert_parity(got["sum_p"], pure["sum_p"], "sum_p (fp32 oracle)", abs_tol=2e-2 * max(1.0, M / 16),
                      rel_tol=rel_tol_e2e, rel_floor=REL_FLOOR_FP32)
    return got, strict, pure


@pytest.mark.parametrize("variant", VARIANTS)
def test_block_reference_semantics_small(variant):
    # the reference's semantics: non-causal, unscaled, no eps / gamma, tau 1.5, MHA, its input recipe
    _check_block(variant, (1, 16, 48, 256, 4, 4, 64), HF, False, 1.0, 0.0, False, True)


@pytest.mark.parametrize("variant", VARIANTS)
def test_block_generalised_small(variant):
    # batch, GQA, causal, scaled, eps + gamma, ragged M
    _check_block(variant, (2, 200, 0, 512, 8, 2, 64), BF, True, 0.125, 1e-5, True, False)
    _check_block(variant, (1, 130, 24, 256, 4, 2, 128), BF, True, 128 ** -0.5, 1e-5, True, False,
                 noise_mode=L.TRN_NOISE_GUMBEL)


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("model", ("llama", "falcon"))
def test_block_reference_native_shapes(variant, model):
    c = MODEL_CONFIGS[model]
    _check_block(variant, (1, c["M"], c["P"], c["N"], c["H"], c["H"], c["D"]), HF, False, 1.0, 0.0, False, True)


@pytest.mark.parametrize("variant", VARIANTS)
def test_block_against_reference_class_outputs(variant):
    """Inputs and outputs of the reference's own classes (tests/golden/golden_small.npz, fp32) — the kernels
    see the inputs rounded to fp16, as the reference's harness feeds them (convert_eval_rms.py:24)."""
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden_small.npz"))
    M, N, D, H, P = (int(v) for v in g["dims"])
    t = {k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("in_")}
    tin = dict(X=t["X"].half(), WQ=t["WQ"].half(), WK=t["WK"].half(), WV=t["WV"].half(),
               K_cache=t["K_cache"].half().unsqueeze(0), V_cache=t["V_cache"].half().unsqueeze(0),
               pre_gamma=None, gamma_q=None, gamma_k=None,
               noise=t["noise"].half().unsqueeze(0) if variant == "keyformer" else None)
    got = run_block(variant, tin, B=1, M=M, P=P, Hq=H, Hkv=H, D=D, causal=False, scale=1.0, tau=1.5)
    # the reference returns the head-major result viewed as [M, H*D] (ref_rms.py:80-81)
    ref_out = torch.from_numpy(g[f"{variant}_out"]).view(H, M, D).permute(1, 0, 2)
    assert_parity(got["out"][0], ref_out, f"{variant} vs reference class", rel_floor=REL_FLOOR_FP32,
                  rel_tol=REL_TOL_E2E)
    if variant == "keyformer":
        assert_parity(got["sum_p"][0], torch.from_numpy(g["keyformer_perturb_out"]).sum(1), "C_out",
                      rel_floor=REL_FLOOR_FP32)
    if variant == "roco":
        assert_parity(got["sum_p"][0], torch.from_numpy(g["roco_sum_p"]), "C_out1", rel_floor=REL_FLOOR_FP32)
        assert_parity(got["sum_p2"][0], torch.from_numpy(g["roco_sum_p2"]), "C_out2", rel_floor=REL_FLOOR_FP32, rel_tol=2e-2)


def test_batched_block_against_reference_batched_outputs():
    """B = 2 against the reference's only batched code, SimpleBatchAttention (ref_rms.py:1420-1479; fixture
    tests/golden/golden_batched.npz): PreNorm math, cache append per batch item, token-major O2[B, M, N]."""
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden_batched.npz"))
    B, M, N, D, H, P = (int(v) for v in g["dims"])
    t = {k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("in_")}
    tin = dict(X=t["X"].reshape(B * M, N).half(), WQ=t["WQ"].half(), WK=t["WK"].half(), WV=t["WV"].half(),
               K_cache=t["K_cache"].half(), V_cache=t["V_cache"].half(), pre_gamma=None, gamma_q=None, gamma_k=None,
               noise=None)
    got = run_block("prenorm", tin, B=B, M=M, P=P, Hq=H, Hkv=H, D=D, causal=False, scale=1.0)
    assert_parity(got["out"].reshape(B, M, N), torch.from_numpy(g["batch_O2"]), "batched prenorm vs SimpleBatchAttention",
                  rel_floor=REL_FLOOR_FP32, rel_tol=REL_TOL_E2E)
    assert_parity(got["k_cache"][:, :, P:], torch.from_numpy(g["batch_K_cache"])[:, :, P:], "batched cache append",
                  rel_floor=REL_FLOOR_FP32, rel_tol=REL_TOL_E2E)
    assert torch.equal(got["k_cache"][:, :, :P].cpu(), tin["K_cache"][:, :, :P])


def _load_generated(src, name):
    import tempfile
    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as f:
        f.write(src)
    spec = importlib.util.spec_from_file_location(name, f.name)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    os.unlink(f.name)
    return mod


@pytest.mark.parametrize("variant", VARIANTS + ("rmsnorm",))
def test_generated_forward_in_place_and_graph_capturable(variant):
    """The drop-in path end to end: IR text -> convert_ir_to_triton -> module.forward(*tensors) with the
    reference's tensor names, layouts and dtypes, replayed from a CUDA graph as the reference's harness
    does (vanilla_llama_benchmark.py:263-285)."""
    consts = {"M": 16, "N": 256, "D": 64, "H": 4, "P": 48}
    src = convert_ir_to_triton(open(IR_DIR / f"{variant}.txt").read(), SHAPE_DICT, consts)
    mod = _load_generated(src, f"gen_{variant}")
    bench = AttnBlockBenchmark(consts, seed=42)
    bench.create_test_tensors(mod.TENSOR_PARAMS)
    T = bench.tensors
    args = [T[p] for p in mod.TENSOR_PARAMS]
    host = {k: v.detach().cpu().clone() for k, v in T.items()}
    assert mod.forward(*args) is None
    torch.cuda.synchronize()
    if variant == "rmsnorm":
        assert_parity(T["X_norm"], O.rmsnorm(host["X"]), "X_norm")
    else:
        o_variant, o_x = variant, host["X"]
        if variant == "prenorm":
            # this program stores X_norm from a kernel of its own: the caller's tensor must receive it, and the
            # rest of the block is the Vanilla block on the X_norm that was stored
            assert mod.SCHEDULE["x_norm_in_memory"] and "X_norm" in mod.TENSOR_PARAMS
            assert_parity(T["X_norm"], O.rmsnorm(host["X"]), "X_norm left in the caller's tensor")
            o_variant, o_x = "vanilla", T["X_norm"].float().cpu()
        r = O.attn_block(o_variant, X=o_x, Wq=host["WQ"], Wk=host["WK"], Wv=host["WV"],
                         cache_K=host["K_cache"].unsqueeze(0), cache_V=host["V_cache"].unsqueeze(0), B=1, M=16, P=48,
                         Hq=4, Hkv=4, D=64, noise=host["noise"].unsqueeze(0) if "noise" in host else None,
                         round_to=HF, round_x_norm=None)
        if variant == "prenorm":
            # unit-variance rows times 0.01-sized weights: a last-bit difference in a stored q or k moves a whole
            # row of scores, so the output is held to the end-to-end bound here; the strict bound is carried by
            # the attention check on the stored q / k / v
            strict = O.attend(T["Q"].float().cpu().unsqueeze(0), T["K_cache"].float().cpu().unsqueeze(0),
                              T["V_cache"].float().cpu().unsqueeze(0), P=48, causal=False, scale=1.0)
            assert_parity(T["O2"].view(16, 4, 64), strict["out"][0].transpose(0, 1), "O2 (attention on stored q/k/v)")
            assert_parity(T["O2"].view(16, 4, 64), r["out_bmhd"][0], "O2", rel_floor=REL_FLOOR_FP32, rel_tol=REL_TOL_E2E)
        else:
            assert_parity(T["O2"].view(16, 4, 64), r["out_bmhd"][0], "O2")
        assert_parity(T["K_cache"][:, 48:], r["k_all"][0, :, 48:], "cache append")
        assert torch.equal(T["K_cache"][:, :48].cpu(), host["K_cache"][:, :48])
        if variant == "keyformer":
            assert_parity(T["C_out"], r["sum_p"][0], "C_out")
        if variant == "roco":
            assert_parity(T["C_out1"], r["sum_p"][0], "C_out1")
            assert_parity(T["C_out2"], r["sum_p2"][0], "C_out2", rel_tol=2e-2)
    # positional block sizes (convert_eval_rms.py:275-291) and keyword block sizes (rms_benchmark.py:246-263)
    mod.forward(*args, *([32] * len(mod.BLOCK_PARAMS)))
    mod.forward(*args, **{b: 64 for b in mod.BLOCK_PARAMS})
    out_name = "X_norm" if variant == "rmsnorm" else "O2"
    want = T[out_name].clone()
    ms = bench.benchmark_kernel(mod, warmup_runs=2, benchmark_runs=5)      # zeroes outputs, captures, replays
    assert ms > 0 and torch.equal(T[out_name], want)
    bench.cleanup()


def test_harness_records_errors_instead_of_raising():
    bench = AttnBlockBenchmark({"M": 16, "N": 256, "D": 64, "H": 4, "P": 48})
    r = bench.run_single_benchmark(5, "(frobnicate X)")
    assert r.error is not None and r.execution_time == float("inf") and r.ir_id == 5
    good = bench.run_single_benchmark(0, open(IR_DIR / "vanilla.txt").read())
    assert good.error is None and good.execution_time > 0
    bench.cleanup()


def test_block_argument_validation():
    t = block_inputs(0, 1, 16, 0, 128, 2, 2, 64, BF)
    with pytest.raises(ValueError, match="weight shapes"):
        bad = dict(t)
        bad["WK"] = t["WK"][:, :64].contiguous()
        run_block("vanilla", bad, B=1, M=16, P=0, Hq=2, Hkv=2, D=64, causal=False, scale=1.0)
    # KeyFormer without noise and without the Gumbel generator
    with pytest.raises(L.TrinityError):
        run_block("keyformer", t, B=1, M=16, P=0, Hq=2, Hkv=2, D=64, causal=False, scale=1.0, noise_mode=L.TRN_NOISE_TENSOR)
    assert L.kernel_status() == 0


def test_fp32_vanilla_configuration():
    """The fp32 Vanilla Llama3-8B configuration (X[1,512,4096] ~ N(0,1), Wq 4096x4096, Wk/Wv 4096x1024 ~ N(0,1/4096),
    32 query / 8 kv heads of 128, causal softmax(q k^T / sqrt(128)) v, seed 0) through the drop-in path with fp32
    tensors.  The kernels compute on bf16-rounded operands with fp32 accumulation, so this is an end-to-end
    comparison (abs <= 2e-2; rel <= 5e-2 above 10 % of max|ref|) against the fp32 oracle on the fp32 inputs."""
    consts = {"M": 512, "N": 4096, "D": 128, "H": 32, "P": 0, "HKV": 8, "CAUSAL": 1, "SCALE_RSQRT_D": 1}
    shapes = dict(SHAPE_DICT)
    shapes["WK"] = ("N", 1024)
    shapes["WV"] = ("N", 1024)
    shapes["K_cache"] = (8, "P+M", "D")
    shapes["V_cache"] = (8, "P+M", "D")
    src = convert_ir_to_triton(open(IR_DIR / "vanilla.txt").read(), shapes, consts)
    mod = _load_generated(src, "gen_cfg1")
    torch.manual_seed(0)
    host = {"X": torch.randn(512, 4096), "WQ": torch.randn(4096, 4096) / 64, "WK": torch.randn(4096, 1024) / 64,
            "WV": torch.randn(4096, 1024) / 64, "K_cache": torch.zeros(8, 512, 128), "V_cache": torch.zeros(8, 512, 128),
            "Q": torch.zeros(32, 512, 128), "O2": torch.zeros(512, 4096)}
    T = {k: v.cuda() for k, v in host.items()}
    mod.forward(*[T[p] for p in mod.TENSOR_PARAMS])
    torch.cuda.synchronize()
    assert L.kernel_status() == 0 and T["O2"].dtype == torch.float32
    r = O.attn_block("vanilla", X=host["X"], Wq=host["WQ"], Wk=host["WK"], Wv=host["WV"], B=1, M=512, P=0, Hq=32, Hkv=8,
                     D=128, causal=True, scale=128 ** -0.5)
    cfg = "cfg1 Vanilla Llama fp32"
    assert_parity(T["O2"].view(512, 32, 128), r["out_bmhd"][0], "fp32 vanilla out (fp32 oracle, fp32 inputs)",
                  rel_floor=REL_FLOOR_FP32, rel_tol=REL_TOL_E2E, config=cfg)
    assert_parity(T["K_cache"], r["k_all"][0], "fp32 vanilla k", rel_floor=REL_FLOOR_FP32, rel_tol=REL_TOL_E2E, config=cfg)
    # the attention core on the q / k / v the block stored (the step in which both sides see the same inputs)
    strict = O.attend(T["Q"].cpu().unsqueeze(0), T["K_cache"].cpu().unsqueeze(0), T["V_cache"].cpu().unsqueeze(0), P=0,
                      causal=True, scale=128 ** -0.5)
    assert_parity(T["O2"].view(512, 32, 128), strict["out"][0].transpose(0, 1), "fp32 vanilla out (attention on stored q/k/v)",
                  config=cfg)


def test_fp32_caller_keeps_the_cached_prefix_bit_for_bit():
    """fp32 tensors with P > 0 cached keys: the operator appends rows [P, P+M) of K_cache / V_cache and must leave
    rows [0, P) exactly as the caller stored them (the reference's kernels store only the appended rows) — also
    when the kernels work on 16-bit shadows of the caller's fp32 tensors."""
    consts = {"M": 16, "N": 256, "D": 64, "H": 4, "P": 48}
    mod = _load_generated(convert_ir_to_triton(open(IR_DIR / "vanilla.txt").read(), SHAPE_DICT, consts), "gen_fp32_prefix")
    torch.manual_seed(3)
    host = {"X": torch.randn(16, 256) * 0.3, "WQ": torch.randn(256, 256) / 16, "WK": torch.randn(256, 256) / 16,
            "WV": torch.randn(256, 256) / 16, "K_cache": torch.randn(4, 64, 64), "V_cache": torch.randn(4, 64, 64),
            "Q": torch.zeros(4, 16, 64), "O2": torch.zeros(16, 256)}
    T = {k: v.cuda() for k, v in host.items()}
    for _ in range(2):
        mod.forward(*[T[p] for p in mod.TENSOR_PARAMS])
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    for name in ("K_cache", "V_cache"):
        assert torch.equal(T[name][:, :48].cpu(), host[name][:, :48]), f"{name} prefix was rewritten"
        assert not torch.equal(T[name][:, 48:].cpu(), host[name][:, 48:])
    r = O.attn_block("vanilla", X=host["X"], Wq=host["WQ"], Wk=host["WK"], Wv=host["WV"],
                     cache_K=host["K_cache"].unsqueeze(0), cache_V=host["V_cache"].unsqueeze(0), B=1, M=16, P=48,
                     Hq=4, Hkv=4, D=64)
    assert_parity(T["K_cache"][:, 48:], r["k_all"][0, :, 48:], "fp32 cache append", rel_floor=REL_FLOOR_FP32,
                  rel_tol=REL_TOL_E2E)
    assert_parity(T["O2"].view(16, 4, 64), r["out_bmhd"][0], "fp32 out with prefix", rel_floor=REL_FLOOR_FP32,
                  rel_tol=REL_TOL_E2E)


@pytest.mark.parametrize("variant,B,stats", (("prenorm", 4, False), ("roco", 3, True), ("keyformer", 9, True),
                                             ("keyformer_gumbel", 5, True)))
def test_host_activation_path_pipelines_batch_items_with_identical_results(variant, B, stats):
    """trinity_attn_block_host copies batch items in and out while others compute; every output element
    must equal the one-pass device result bit for bit (odd batch counts: uneven last group)."""
    gumbel = variant == "keyformer_gumbel"                # generated noise: batch groups must see the uncut problem's
    variant = variant.split("_")[0]
    M, P, N, Hq, Hkv, D = 512, 64, 1024, 8, 2, 128        # x and o: 1 MB per batch item each
    L_ = P + M
    torch.manual_seed(31)
    dt = BF
    x = torch.randn(B * M, N).to(dt)
    wq, wk, wv = ((torch.randn(N, h * D) / N ** 0.5).to(dt).cuda() for h in (Hq, Hkv, Hkv))
    kc0, vc0 = torch.randn(B, Hkv, L_, D).to(dt), torch.randn(B, Hkv, L_, D).to(dt)
    noise = torch.randn(B, Hq, M, L_).to(dt).cuda() if (variant == "keyformer" and not gumbel) else None
    gamma = (1 + 0.1 * torch.randn(N)).to(dt).cuda() if variant == "prenorm" else None

    def make():
        kc, vc = kc0.clone().cuda(), vc0.clone().cuda()
        q = torch.zeros(B, M, Hq, D, dtype=dt, device="cuda")
        o = torch.zeros(B, M, Hq, D, dtype=dt, device="cuda")
        sp = torch.zeros(B, Hq, L_, device="cuda") if stats else None
        sp2 = torch.zeros(B, Hq, L_, device="cuda") if variant == "roco" else None
        xd = torch.zeros(B * M, N, dtype=dt, device="cuda")
        plan = ops.BlockPlan(variant, B=B, M=M, P=P, Hq=Hq, Hkv=Hkv, D=D, q=q, k_cache=ops.as_bshd(kc, "bhsd"),
                             v_cache=ops.as_bshd(vc, "bhsd"), o=o, x=xd, wq=wq, wk=wk, wv=wv, causal=True,
                             scale=D ** -0.5, pre_eps=1e-5, pre_gamma=gamma,
                             noise_mode=(L.TRN_NOISE_GUMBEL if gumbel else L.TRN_NOISE_TENSOR) if variant == "keyformer"
                             else L.TRN_NOISE_NONE, tau=1.5, seed=77, noise=noise, sum_p=sp, sum_p2=sp2)
        return plan, xd, o, kc, vc, sp, sp2

    plan, xd, o_ref, kc_ref, vc_ref, sp_ref, sp2_ref = make()
    xd.copy_(x)
    plan.run()
    torch.cuda.synchronize()

    plan2, xd2, o2, kc2, vc2, sp_d, sp2_d = make()
    xh = x.clone().pin_memory()
    oh = torch.zeros(B, M, Hq, D, dtype=dt).pin_memory()
    sph = torch.zeros(B, Hq, L_).pin_memory() if stats else None
    sp2h = torch.zeros(B, Hq, L_).pin_memory() if variant == "roco" else None
    for _ in range(2):                               # the second call reuses the streams and events
        plan2.run_host(xh, oh, sph, sp2h)
    assert L.kernel_status() == 0
    assert torch.equal(oh, o_ref.cpu())
    assert torch.equal(kc2, kc_ref) and torch.equal(vc2, vc_ref)
    if stats:
        assert torch.equal(sph, sp_ref.cpu())
    if sp2h is not None:
        assert torch.equal(sp2h, sp2_ref.cpu())


def test_prenorm_candidate_that_keeps_x_norm_in_registers_selects_the_fused_schedule():
    """Two PreNorm candidates that differ only in their fusion structure: the packaged one stores X_norm in a
    kernel of its own, the second normalises inside the projection loop.  Both give the same block; the
    first leaves X_norm in the caller's tensor, the second has no X_norm tensor at all."""
    consts = {"M": 16, "N": 256, "D": 64, "H": 4, "P": 48}
    stored = open(IR_DIR / "prenorm.txt").read()
    fused = open(IR_DIR / "prenorm_fused.txt").read()
    outs = {}
    for name, ir in (("stored", stored), ("fused", fused)):
        mod = _load_generated(convert_ir_to_triton(ir, SHAPE_DICT, consts), f"gen_prenorm_{name}")
        bench = AttnBlockBenchmark(consts, seed=42)
        bench.create_test_tensors(mod.TENSOR_PARAMS)
        mod.forward(*[bench.tensors[p] for p in mod.TENSOR_PARAMS])
        torch.cuda.synchronize()
        outs[name] = (mod, bench.tensors["O2"].clone(), {k: v.detach().cpu().clone() for k, v in bench.tensors.items()})
    assert outs["stored"][0].SCHEDULE["x_norm_in_memory"] is True
    assert outs["fused"][0].SCHEDULE["x_norm_in_memory"] is False and "X_norm" not in outs["fused"][0].TENSOR_PARAMS
    host = outs["fused"][2]
    r = O.attn_block("prenorm", X=host["X"], Wq=host["WQ"], Wk=host["WK"], Wv=host["WV"],
                     cache_K=torch.zeros(1, 4, 64, 64), cache_V=torch.zeros(1, 4, 64, 64), B=1, M=16, P=48,
                     Hq=4, Hkv=4, D=64, round_to=HF, round_x_norm=None)
    del r
    # same inputs (same seed), two schedules: the outputs agree to 16-bit rounding of X_norm
    assert_parity(outs["fused"][1], outs["stored"][1].float().cpu(), "fused vs stored schedule", rel_tol=5e-2,
                  rel_floor=0.1)
    assert L.kernel_status() == 0


@pytest.mark.parametrize("M", (16, 32))
def test_candidate_structure_selects_the_statistics_schedule(M):
    """Two RoCo candidates with the same arithmetic: the packaged one keeps C_exp in memory between its two key loops
    (-> scores kept in the workspace, statistics summed from memory), the second recomputes exp(q k^T) in the
    statistics loop and holds no score tensor (-> second q k^T pass).  Both give the same operator.  With at most 16
    queries the library sums the statistics inside the attention launch whichever candidate asks (M = 16 here);
    M = 32 runs the two schedules proper."""
    consts = {"M": M, "N": 256, "D": 64, "H": 4, "P": 48}
    kept = open(IR_DIR / "roco.txt").read()
    load_cexp = "(load (tensor C_exp) (index (elem n) fulltile (tile p)))"
    again = ("(exp (* (load (input Q) (index (elem n) fulltile fulltile)) "
             "(permute3 (load (input K_cache) (index (elem n) (tile p) fulltile)) 0 2 1)))")
    head, sep, tail = kept.rpartition("(sloop 0 P+M tile_p p")
    recompute = head + sep + tail.replace(load_cexp, again)
    assert recompute != kept
    outs = {}
    for name, ir in (("kept", kept), ("recompute", recompute)):
        mod = _load_generated(convert_ir_to_triton(ir, SHAPE_DICT, consts), f"gen_roco_{name}_{M}")
        bench = AttnBlockBenchmark(consts, seed=42)
        bench.create_test_tensors(mod.TENSOR_PARAMS)
        mod.forward(*[bench.tensors[p] for p in mod.TENSOR_PARAMS])
        torch.cuda.synchronize()
        outs[name] = (mod, {k: bench.tensors[k].float().cpu() for k in ("O2", "C_out1", "C_out2")})
    assert outs["kept"][0].SCHEDULE["scores_in_memory"] == ["C_exp"] and "C_exp" in outs["kept"][0].TENSOR_PARAMS
    assert outs["recompute"][0].SCHEDULE["scores_in_memory"] == [] and "C_exp" not in outs["recompute"][0].TENSOR_PARAMS
    assert outs["kept"][0]._op.keep_scores == 1 and outs["recompute"][0]._op.keep_scores == -1
    # the two schedules may run different attention kernels: the same softmax in another summation order
    assert_parity(outs["recompute"][1]["O2"].cuda().half(), outs["kept"][1]["O2"], "O2: recompute vs kept scores", rel_tol=2e-2)
    for k in ("C_out1", "C_out2"):
        assert_parity(outs["recompute"][1][k].cuda().half(), outs["kept"][1][k], f"{k}: recompute vs kept scores", rel_tol=2e-2)
    assert L.kernel_status() == 0


@pytest.mark.parametrize("variant,B,M,P,Hq,Hkv,D,dt,causal,stats_dtype", (
    ("keyformer", 1, 16, 1024, 8, 8, 128, HF, False, torch.float32),     # the reference's shape
    ("roco", 1, 16, 1024, 6, 6, 64, HF, False, torch.float16),
    ("keyformer", 2, 9, 300, 4, 4, 64, BF, True, torch.float32),        # causal, ragged, 16-bit io with fp32 sums
    ("roco", 1, 16, 40, 4, 2, 128, BF, True, torch.bfloat16),           # GQA with 16 queries: heads are not packed
))
def test_statistics_summed_inside_the_small_attention_launch_equal_the_two_kernel_path(variant, B, M, P, Hq, Hkv, D, dt,
                                                                                      causal, stats_dtype):
    """With at most 16 queries the block sums the per-key statistics inside the attention launch.  The same numbers
    through the public pieces — attention that keeps its scores, then the statistics kernel on them — agree bit for
    bit: both add 2^(t - lse) over the queries in ascending order."""
    scale, tau = D ** -0.5, 1.5
    t = block_inputs(31, B, M, P, 64, Hq, Hkv, D, dt, variant=variant)
    torch.manual_seed(32)
    t["Q"] = torch.randn(B, M, Hq, D).to(dt)
    r = run_block(variant, t, B=B, M=M, P=P, Hq=Hq, Hkv=Hkv, D=D, causal=causal, scale=scale, tau=tau,
                  stats_dtype=stats_dtype, project=False)
    L_ = P + M
    pitch = (L_ + 31) // 32 * 32
    qv, kv, vv = ops.as_bshd(t["Q"].cuda(), "bshd"), ops.as_bshd(t["K_cache"].cuda(), "bhsd"), ops.as_bshd(t["V_cache"].cuda(), "bhsd")
    o = torch.zeros(B, M, Hq, D, device="cuda", dtype=dt)
    lse, lse2 = torch.zeros(B, Hq, M, device="cuda"), torch.zeros(B, Hq, M, device="cuda")
    sc = torch.full((B, Hq, M, pitch), float("nan"), device="cuda")
    kw = dict(P=P, causal=causal, scale=scale)
    sp, sp2 = (torch.zeros(B, Hq, L_, device="cuda", dtype=stats_dtype) for _ in range(2))
    if variant == "keyformer":
        ops.attention(qv, kv, vv, o, lse=lse, lse_pert=lse2, scores=sc, noise_mode=L.TRN_NOISE_TENSOR, tau=tau,
                      noise=t["noise"].cuda(), **kw)
        ops.attn_colstats(qv, kv, lse2, sp, None, scores=sc, **kw)
    else:
        ops.attention(qv, kv, vv, o, lse=lse, scores=sc, **kw)
        ops.attn_colstats(qv, kv, lse, sp, sp2, scores=sc, **kw)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    assert torch.equal(r["out"], o)
    assert torch.equal(r["sum_p"], sp)
    if variant == "roco":
        assert torch.equal(r["sum_p2"], sp2)


@pytest.mark.parametrize("variant,M,P,N,Hq,Hkv,D", (
    ("prenorm", 16, 1024, 1024, 8, 8, 128),        # split-K projection (weights requested before the dependency wait)
    ("keyformer", 16, 200, 512, 4, 4, 64),         # + the small attention kernel with the statistics inside
    ("qknorm", 300, 40, 512, 4, 2, 128),           # persistent projection + tensor-memory attention
))
def test_plain_stream_order_gives_the_same_block_as_dependent_launch(variant, M, P, N, Hq, Hkv, D, monkeypatch):
    """TRINITY_NO_PDL=1 launches every kernel plainly stream-ordered (the library reads the variable per launch):
    the results equal those of the default, programmatic dependent launch, bit for bit."""
    t = block_inputs(41, 1, M, P, N, Hq, Hkv, D, HF, variant=variant)
    kw = dict(B=1, M=M, P=P, Hq=Hq, Hkv=Hkv, D=D, causal=True, scale=D ** -0.5, eps=1e-5)
    a = run_block(variant, t, **kw)
    monkeypatch.setenv("TRINITY_NO_PDL", "1")
    b = run_block(variant, t, **kw)
    monkeypatch.delenv("TRINITY_NO_PDL")
    for k in ("out", "q", "k_cache", "v_cache", "sum_p"):
        if a[k] is not None:
            assert torch.equal(a[k], b[k]), k
