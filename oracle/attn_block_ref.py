"""CPU oracle for the fused attention block — TEST INFRASTRUCTURE, not a product path.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may import this module; the
shipped package (triton_b200/) never does and has no CPU fallback.

It restates, in fp32 torch, what the reference's own PyTorch path computes, op for op:

  Vanila.forward     ref_rms.py:45-83      project -> view [M,H,D] -> transpose -> cat cache ->
                                            q k^T (unscaled) -> softmax -> @ v
  PreNorm.forward    ref_rms.py:101-127    x * rsqrt(mean x^2) first (no eps, no gamma)
  QKNorm.forward     ref_rms.py:197-231    per-head rsqrt(mean^2) on q and on the NEW k only (:217-222)
  KeyFormer.forward  ref_rms.py:147-179    + softmax((scores + noise) / 1.5)
  RoCo.forward       ref_rms.py:249-280    + weights.sum(dim=1), weights.pow(2).sum(dim=1)

and adds, each behind a flag that defaults to the reference behaviour, the generalisations the
benchmark configurations need: batch B, GQA / MQA (Hkv < Hq; K/V heads repeated), a causal mask offset
by the prefix P, a score scale, eps and gamma in both norms, tau, and Gumbel noise generated from a
seed.  With every flag at its default and B = 1, Hkv = Hq this function IS the reference class; that
identity is pinned by tests/test_oracle_golden.py against outputs of the reference's classes
(fixtures produced by tests/golden/make_golden.py from the reference's ref_rms.py).

Parity status: pinned against reference outputs for the reference-native semantics; the flagged
generalisations have no reference counterpart (the reference ships no causal / GQA / eps path), so
for them this file is the specification.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch

VARIANTS = ("vanilla", "prenorm", "qknorm", "keyformer", "roco")


# ------------------------------------------------------------------------------------------------
# RMSNorm (ref_rms.py:102-103; with eps / weight: ref_attn.py:348-350)
# ------------------------------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, gamma: Optional[torch.Tensor] = None, eps: float = 0.0) -> torch.Tensor:
    xf = x.float()
    variance = xf.pow(2).mean(-1, keepdim=True)
    y = xf * torch.rsqrt(variance + eps)
    if gamma is not None:
        y = y * gamma.float()
    return y


# ------------------------------------------------------------------------------------------------
# Counter-based Gumbel noise: host restatement of the noise functions in
# triton_b200/csrc/attn_common.cuh (same integer mixing; logs in float64, result rounded to fp32)
# ------------------------------------------------------------------------------------------------
def _mix32(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.uint32, copy=True)
    x ^= x >> np.uint32(16)
    x *= np.uint32(0x7FEB352D)
    x ^= x >> np.uint32(15)
    x *= np.uint32(0x846CA68B)
    x ^= x >> np.uint32(16)
    return x


def noise_bits(seed: int, bh: np.ndarray, i: np.ndarray, j: np.ndarray) -> np.ndarray:
    """32 hashed bits of element (b*Hq+h, query i, key j): headkey -> rowhash -> per-element mix, the integer
    steps of noise_headkey / noise_rowhash / noise_elem_bits in triton_b200/csrc/attn_common.cuh."""
    s_lo = np.uint32(seed & 0xFFFFFFFF)
    s_hi = np.uint32((seed >> 32) & 0xFFFFFFFF)
    with np.errstate(over="ignore"):
        headkey = _mix32(s_lo ^ _mix32(bh.astype(np.uint32) + s_hi * np.uint32(0x9E3779B9)))
        rowhash = _mix32(headkey + i.astype(np.uint32) * np.uint32(0x9E3779B9))
        x = rowhash ^ (j.astype(np.uint32) * np.uint32(0x85EBCA6B))
        x = x ^ (x >> np.uint32(16))
        x = x * np.uint32(0x7FEB352D)
        x = x ^ (x >> np.uint32(15))
    return x


def gumbel_noise(seed: int, B: int, Hq: int, M: int, L: int, b0: int = 0, b1: Optional[int] = None,
                 h0: int = 0, h1: Optional[int] = None) -> torch.Tensor:
    """Gumbel(0,1) field [b1-b0, h1-h0, M, L] of the [B, Hq, M, L] noise the kernels generate from `seed`."""
    b1 = B if b1 is None else b1
    h1 = Hq if h1 is None else h1
    bb = np.arange(b0, b1, dtype=np.uint32)[:, None, None, None]
    hh = np.arange(h0, h1, dtype=np.uint32)[None, :, None, None]
    ii = np.arange(M, dtype=np.uint32)[None, None, :, None]
    jj = np.arange(L, dtype=np.uint32)[None, None, None, :]
    bits = noise_bits(seed, bb * np.uint32(Hq) + hh, ii, jj)
    u = ((bits >> np.uint32(9)).astype(np.float64) + 0.5) * 2.0 ** -23
    g = -np.log(-np.log(u))
    return torch.from_numpy(g.astype(np.float32))


# ------------------------------------------------------------------------------------------------
# the block
# ------------------------------------------------------------------------------------------------
def project(variant: str, X: torch.Tensor, Wq: torch.Tensor, Wk: torch.Tensor, Wv: torch.Tensor, *,
            B: int, M: int, Hq: int, Hkv: int, D: int, pre_eps: float = 0.0,
            pre_gamma: Optional[torch.Tensor] = None, qk_eps: float = 0.0,
            gamma_q: Optional[torch.Tensor] = None, gamma_k: Optional[torch.Tensor] = None,
            round_x_norm: Optional[torch.dtype] = None):
    """q [B,Hq,M,D], k, v [B,Hkv,M,D] in fp32, following ref_rms.py:47-56 (+102-103, +217-220)."""
    Xf = X.float().reshape(B, M, -1)
    if variant == "prenorm":
        variance = Xf.pow(2).mean(-1, keepdim=True)          # ref_rms.py:102
        Xf = Xf * torch.rsqrt(variance + pre_eps)            # ref_rms.py:103
        if pre_gamma is not None:
            Xf = Xf * pre_gamma.float()
        if round_x_norm is not None:                         # X_norm stored as a 16-bit tensor
            Xf = Xf.to(round_x_norm).float()
    q = torch.matmul(Xf, Wq.float())                         # ref_rms.py:47
    k = torch.matmul(Xf, Wk.float())
    v = torch.matmul(Xf, Wv.float())
    q = q.view(B, M, Hq, D).transpose(1, 2)                  # ref_rms.py:51,75
    k = k.view(B, M, Hkv, D).transpose(1, 2)
    v = v.view(B, M, Hkv, D).transpose(1, 2)
    if variant == "qknorm":
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + qk_eps)   # ref_rms.py:217-220
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + qk_eps)
        if gamma_q is not None:
            q = q * gamma_q.float()
        if gamma_k is not None:
            k = k * gamma_k.float()
    return q, k, v


def attend(q: torch.Tensor, k_all: torch.Tensor, v_all: torch.Tensor, *, P: int, causal: bool = False,
           scale: float = 1.0, variant: str = "vanilla", tau: float = 1.5,
           noise: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
    """q [B,Hq,M,D]; k_all, v_all [B,Hkv,L,D] with L = P + M (prefix + new).  fp32 throughout.

    Returns out [B,Hq,M,D] and, per variant, perturb_out [B,Hq,M,L] / sum_p / sum_p2 [B,Hq,L]."""
    B, Hq, M, D = q.shape
    Hkv, L = k_all.shape[1], k_all.shape[2]
    g = Hq // Hkv
    if g > 1:
        k_all = k_all.repeat_interleave(g, dim=1)
        v_all = v_all.repeat_interleave(g, dim=1)
    scores = torch.matmul(q, k_all.transpose(-1, -2))        # ref_rms.py:77
    if scale != 1.0:
        scores = scores * scale
    mask = None
    if causal:
        i = torch.arange(M).view(M, 1)
        j = torch.arange(L).view(1, L)
        mask = j > (i + P)
        scores = scores.masked_fill(mask, float("-inf"))
    weights = torch.softmax(scores, dim=-1)                  # ref_rms.py:78
    res = {"out": torch.matmul(weights, v_all)}              # ref_rms.py:80
    if variant == "keyformer":
        perturb = (scores + noise.float()) / tau             # ref_rms.py:172
        perturb_out = torch.softmax(perturb, dim=-1)         # ref_rms.py:174
        res["perturb_out"] = perturb_out
        res["sum_p"] = perturb_out.sum(dim=-2)               # the IR's C_out reduction over queries
    if variant == "roco":
        res["sum_p"] = weights.sum(dim=-2)                   # ref_rms.py:274
        res["sum_p2"] = weights.pow(2).sum(dim=-2)           # ref_rms.py:275
    return res


def attn_block(variant: str, *, X: Optional[torch.Tensor] = None, Wq=None, Wk=None, Wv=None,
               Q: Optional[torch.Tensor] = None, K: Optional[torch.Tensor] = None,
               V: Optional[torch.Tensor] = None, cache_K: Optional[torch.Tensor] = None,
               cache_V: Optional[torch.Tensor] = None, B: int = 1, M: int, P: int = 0, Hq: int, Hkv: int, D: int,
               causal: bool = False, scale: float = 1.0, pre_eps: float = 0.0, pre_gamma=None,
               qk_eps: float = 0.0, gamma_q=None, gamma_k=None, tau: float = 1.5, noise=None,
               round_to: Optional[torch.dtype] = None,
               round_x_norm: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
    """Whole block.  X [B*M, N] with weights, or Q [B,Hq,M,D], K, V [B,Hkv,M,D] given directly.
    cache_K / cache_V: [B,Hkv,>=P,D] prefix (rows [0,P) are used, as ref_rms.py:72-73).

    round_to: if set, q / k / v are rounded to that dtype after projection before attention — the
    operator surface defines Q, K_cache and V_cache as 16-bit tensors (convert_eval_rms.py:71-84), and
    the reference's own fp16 path rounds them there too.  round_x_norm does the same for X_norm
    (convert_eval_rms.py:65) where an implementation materialises it.
    """
    assert variant in VARIANTS
    if X is not None:
        q, k, v = project(variant, X, Wq, Wk, Wv, B=B, M=M, Hq=Hq, Hkv=Hkv, D=D, pre_eps=pre_eps,
                          pre_gamma=pre_gamma, qk_eps=qk_eps, gamma_q=gamma_q, gamma_k=gamma_k,
                          round_x_norm=round_x_norm)
    else:
        q, k, v = Q.float(), K.float(), V.float()
    if round_to is not None:
        q, k, v = q.to(round_to).float(), k.to(round_to).float(), v.to(round_to).float()
    if P > 0:
        k_all = torch.cat([cache_K.float()[:, :, :P], k], dim=2)    # ref_rms.py:72
        v_all = torch.cat([cache_V.float()[:, :, :P], v], dim=2)    # ref_rms.py:73
    else:
        k_all, v_all = k, v
    res = attend(q, k_all, v_all, P=P, causal=causal, scale=scale, variant=variant, tau=tau, noise=noise)
    res["q"], res["k_all"], res["v_all"] = q, k_all, v_all
    # token-major [B, M, Hq, D]: what the generated kernels store into O2[M, N] (TritonGen.py:2855)
    res["out_bmhd"] = res["out"].transpose(1, 2).contiguous()
    return res


def reference_view(out_bhmd: torch.Tensor) -> torch.Tensor:
    """The reference classes return `output.view(M, H*D)` of the head-major [H, M, D] result
    (ref_rms.py:80-81) — a reinterpretation of memory, not a transpose.  B must be 1."""
    assert out_bhmd.shape[0] == 1
    H, M, D = out_bhmd.shape[1:]
    return out_bhmd[0].contiguous().view(M, H * D)


def topk_keys(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest scores per row, descending; equal scores keep the lower index first."""
    order = torch.sort(scores.float(), dim=-1, descending=True, stable=True).indices
    return order[..., :k].to(torch.int32)


def roco_mean_std(sum_p: torch.Tensor, sum_p2: torch.Tensor, n_queries: int):
    """Per-key mean and standard deviation of the attention probabilities across queries."""
    mean = sum_p / n_queries
    var = (sum_p2 / n_queries - mean * mean).clamp_min(0.0)
    return mean, var.sqrt()


def attn_block_chunked(variant: str, *, head_chunk: int = 4, **kw) -> Dict[str, torch.Tensor]:
    """Same as attn_block with Q/K/V given, evaluated `head_chunk` query heads at a time so that the
    [heads, M, L] fp32 score tensor fits host memory at the large configurations."""
    Q, K, V = kw.pop("Q"), kw.pop("K"), kw.pop("V")
    noise_fn = kw.pop("noise_fn", None)
    B, Hq, M, D = Q.shape
    Hkv = K.shape[1]
    g = Hq // Hkv
    assert head_chunk % g == 0 or g % head_chunk == 0 or g == 1 or Hkv == 1
    outs, sp, sp2 = [], [], []
    for b in range(B):
        ob, spb, sp2b = [], [], []
        for h0 in range(0, Hq, head_chunk):
            h1 = min(Hq, h0 + head_chunk)
            kv_idx = torch.arange(h0, h1) // g
            noise = noise_fn(b, h0, h1) if noise_fn is not None else None
            r = attend(Q[b:b + 1, h0:h1].float(), K[b:b + 1].float()[:, kv_idx], V[b:b + 1].float()[:, kv_idx],
                       P=kw.get("P", 0), causal=kw.get("causal", False), scale=kw.get("scale", 1.0),
                       variant=variant, tau=kw.get("tau", 1.5), noise=noise)
            ob.append(r["out"])
            if "sum_p" in r:
                spb.append(r["sum_p"])
            if "sum_p2" in r:
                sp2b.append(r["sum_p2"])
        outs.append(torch.cat(ob, dim=1))
        if spb:
            sp.append(torch.cat(spb, dim=1))
        if sp2b:
            sp2.append(torch.cat(sp2b, dim=1))
    res = {"out": torch.cat(outs, dim=0)}
    res["out_bmhd"] = res["out"].transpose(1, 2).contiguous()
    if sp:
        res["sum_p"] = torch.cat(sp, dim=0)
    if sp2:
        res["sum_p2"] = torch.cat(sp2, dim=0)
    return res


def lora(X: torch.Tensor, W: torch.Tensor, A: torch.Tensor, B: torch.Tensor,
         round_d: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
    """LoRA linear layer in fp32: D = X @ A, O = X @ W + D @ B (tensor table lora_benchmark.py:41-64; the arithmetic
    as the reference generator spells it, TritonGen.py:3092-3094).  round_d: D is kept as a 16-bit tensor between the
    two steps by the operator surface (and by the reference's kernels); rounding it here gives the like-for-like value."""
    Xf, Wf, Af, Bf = X.float(), W.float(), A.float(), B.float()
    D = Xf @ Af
    if round_d is not None:
        D = D.to(round_d).float()
    return {"D": D, "O": Xf @ Wf + D @ Bf}


def gmlp(X: torch.Tensor, W1: torch.Tensor, W2: torch.Tensor, gate: str = "silu") -> Dict[str, torch.Tensor]:
    """Gated MLP in fp32 (tensor table gmlp_benchmark.py:53-74; sigmoid as the reference generator lowers it,
    TritonGen.py:2207-2208, 3069-3071): C1 = X @ W1, C2 = X @ W2, C1_exp = sigmoid(C1),
    O = (C1 * C1_exp) * C2 (gate "silu") or C1_exp * C2 (gate "sigmoid")."""
    Xf = X.float()
    C1, C2 = Xf @ W1.float(), Xf @ W2.float()
    S = torch.sigmoid(C1)
    return {"C1": C1, "C2": C2, "C1_exp": S, "O": (C1 * S if gate == "silu" else S) * C2}
