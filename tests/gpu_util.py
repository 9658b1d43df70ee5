"""Helpers shared by the GPU parity tests: seeded inputs, device copies and one function that runs a
whole attention block through the C-ABI (ops.BlockPlan -> trinity_attn_block)."""
import math

import torch

from triton_b200 import _lib as L
from triton_b200 import ops


def block_inputs(seed, B, M, P, N, Hq, Hkv, D, dt, ref_native=False, variant="vanilla", gamma=False,
                 noise_mode=L.TRN_NOISE_TENSOR):
    """ref_native: the reference's recipe randn.clamp(-1,1)*0.01 (convert_eval_rms.py:175-183);
    otherwise X ~ N(0,1), W ~ N(0, 1/N), caches ~ N(0,1) (the benchmark configurations)."""
    torch.manual_seed(seed)
    L_ = P + M
    if ref_native:
        mk = lambda *s: (torch.randn(*s).clamp(-1, 1) * 0.01).to(dt)
        t = dict(X=mk(B * M, N), WQ=mk(N, Hq * D), WK=mk(N, Hkv * D), WV=mk(N, Hkv * D),
                 K_cache=mk(B, Hkv, L_, D), V_cache=mk(B, Hkv, L_, D))
    else:
        t = dict(X=torch.randn(B * M, N).to(dt), WQ=(torch.randn(N, Hq * D) / N ** 0.5).to(dt),
                 WK=(torch.randn(N, Hkv * D) / N ** 0.5).to(dt), WV=(torch.randn(N, Hkv * D) / N ** 0.5).to(dt),
                 K_cache=torch.randn(B, Hkv, L_, D).to(dt), V_cache=torch.randn(B, Hkv, L_, D).to(dt))
    t["pre_gamma"] = (1 + 0.1 * torch.randn(N)).to(dt) if (gamma and variant == "prenorm") else None
    t["gamma_q"] = (1 + 0.1 * torch.randn(D)).to(dt) if (gamma and variant == "qknorm") else None
    t["gamma_k"] = (1 + 0.1 * torch.randn(D)).to(dt) if (gamma and variant == "qknorm") else None
    t["noise"] = None
    if variant == "keyformer" and noise_mode == L.TRN_NOISE_TENSOR:
        t["noise"] = torch.randn(B, Hq, M, L_).to(dt)
    return t


def run_block(variant, t, *, B, M, P, Hq, Hkv, D, causal, scale, eps=0.0, tau=1.5, noise_mode=L.TRN_NOISE_TENSOR,
              seed=0, stats_dtype=torch.float32, single_p=False, project=True, noise_heads=0, noise_bh0=0):
    """Returns dict(out [B,M,Hq,D], q, k_cache, v_cache, sum_p, sum_p2) of device tensors."""
    dev = lambda x: None if x is None else x.cuda()
    dt = t["K_cache"].dtype
    L_ = P + M
    kc, vc = t["K_cache"].clone().cuda(), t["V_cache"].clone().cuda()
    q = t["Q"].cuda() if not project else torch.zeros(B, M, Hq, D, device="cuda", dtype=dt)
    o = torch.zeros(B, M, Hq, D, device="cuda", dtype=dt)
    stats = variant in ("keyformer", "roco")
    sp = torch.zeros(B, Hq, L_, device="cuda", dtype=stats_dtype) if stats else None
    sp2 = torch.zeros(B, Hq, L_, device="cuda", dtype=stats_dtype) if variant == "roco" else None
    kw = {}
    if project:
        kw = dict(x=dev(t["X"]), wq=dev(t["WQ"]), wk=dev(t["WK"]), wv=dev(t["WV"]), pre_eps=eps, qk_eps=eps,
                  pre_gamma=dev(t["pre_gamma"]), gamma_q=dev(t["gamma_q"]), gamma_k=dev(t["gamma_k"]))
    plan = ops.BlockPlan(variant, B=B, M=M, P=P, Hq=Hq, Hkv=Hkv, D=D, q=ops.as_bshd(q, "bshd"),
                         k_cache=ops.as_bshd(kc, "bhsd"), v_cache=ops.as_bshd(vc, "bhsd"), o=ops.as_bshd(o, "bshd"),
                         causal=causal, scale=scale, noise_mode=noise_mode if variant == "keyformer" else 0, tau=tau,
                         noise=dev(t.get("noise")), seed=seed, sum_p=sp, sum_p2=sp2, single_p=single_p,
                         noise_heads=noise_heads, noise_bh0=noise_bh0, **kw)
    plan.run()
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    return dict(out=o, q=q, k_cache=kc, v_cache=vc, sum_p=sp, sum_p2=sp2, plan=plan)


def default_scale(D):
    return 1.0 / math.sqrt(D)
