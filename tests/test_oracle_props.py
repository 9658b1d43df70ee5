"""Properties of the CPU oracle's generalisations (the flags the reference does not have), checked
against independent formulations."""
import math

import numpy as np
import torch

from oracle import attn_block_ref as O


def test_gqa_causal_scale_against_per_head_loop():
    torch.manual_seed(1)
    B, M, P, Hq, Hkv, D = 2, 9, 5, 4, 2, 8
    L = P + M
    q = torch.randn(B, Hq, M, D)
    k = torch.randn(B, Hkv, L, D)
    v = torch.randn(B, Hkv, L, D)
    r = O.attend(q, k, v, P=P, causal=True, scale=D ** -0.5)
    for b in range(B):
        for h in range(Hq):
            kv = h // (Hq // Hkv)
            for i in range(M):
                n = P + i + 1                                     # query i sees keys [0, P+i]
                s = (k[b, kv, :n] @ q[b, h, i]) * D ** -0.5
                w = torch.softmax(s, 0)
                torch.testing.assert_close(r["out"][b, h, i], w @ v[b, kv, :n], rtol=1e-5, atol=1e-6)


def test_prenorm_eps_gamma_and_qknorm_follow_the_formulas():
    torch.manual_seed(2)
    B, M, N, Hq, Hkv, D = 1, 6, 32, 4, 2, 8
    X = torch.randn(B * M, N)
    Wq, Wk, Wv = torch.randn(N, Hq * D), torch.randn(N, Hkv * D), torch.randn(N, Hkv * D)
    gamma = 1 + 0.1 * torch.randn(N)
    q, k, v = O.project("prenorm", X, Wq, Wk, Wv, B=B, M=M, Hq=Hq, Hkv=Hkv, D=D, pre_eps=1e-5, pre_gamma=gamma)
    xn = X * torch.rsqrt(X.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma
    torch.testing.assert_close(q, (xn @ Wq).view(B, M, Hq, D).transpose(1, 2))
    gq, gk = 1 + 0.1 * torch.randn(D), 1 + 0.1 * torch.randn(D)
    q2, k2, v2 = O.project("qknorm", X, Wq, Wk, Wv, B=B, M=M, Hq=Hq, Hkv=Hkv, D=D, qk_eps=1e-5, gamma_q=gq, gamma_k=gk)
    q_raw = (X @ Wq).view(B, M, Hq, D).transpose(1, 2)
    torch.testing.assert_close(q2, q_raw * torch.rsqrt(q_raw.pow(2).mean(-1, keepdim=True) + 1e-5) * gq)
    torch.testing.assert_close(v2, (X @ Wv).view(B, M, Hkv, D).transpose(1, 2))     # v untouched (ref_rms.py:223)


def test_cached_keys_are_not_renormalised():
    # ref_rms.py:222: only the new k is normalised; cache rows are taken as stored
    torch.manual_seed(3)
    M, N, D, P = 4, 16, 8, 3
    H = N // D
    X, W = torch.randn(M, N), [torch.randn(N, N) for _ in range(3)]
    cK, cV = 5 * torch.randn(1, H, P + M, D), torch.randn(1, H, P + M, D)
    r = O.attn_block("qknorm", X=X, Wq=W[0], Wk=W[1], Wv=W[2], cache_K=cK, cache_V=cV, B=1, M=M, P=P, Hq=H, Hkv=H, D=D)
    torch.testing.assert_close(r["k_all"][:, :, :P], cK[:, :, :P])
    new_k = r["k_all"][:, :, P:]
    torch.testing.assert_close(new_k.pow(2).mean(-1), torch.ones(1, H, M), rtol=1e-5, atol=1e-5)


def test_statistics_are_column_sums_and_rows_sum_to_one():
    torch.manual_seed(4)
    B, Hq, M, L, D = 1, 2, 7, 7, 8
    q, k, v = torch.randn(B, Hq, M, D), torch.randn(B, Hq, L, D), torch.randn(B, Hq, L, D)
    r = O.attend(q, k, v, P=0, causal=True, scale=0.3, variant="roco")
    torch.testing.assert_close(r["sum_p"].sum(-1), torch.full((B, Hq), float(M)))
    mean, std = O.roco_mean_std(r["sum_p"], r["sum_p2"], M)
    w = torch.softmax((q @ k.transpose(-1, -2) * 0.3).masked_fill(torch.triu(torch.ones(M, L, dtype=torch.bool), 1), -math.inf), -1)
    torch.testing.assert_close(mean, w.mean(-2))
    torch.testing.assert_close(std, w.std(-2, unbiased=False), rtol=1e-4, atol=1e-6)
    noise = torch.randn(B, Hq, M, L)
    rk = O.attend(q, k, v, P=0, causal=False, scale=1.0, variant="keyformer", tau=1.5, noise=noise)
    torch.testing.assert_close(rk["sum_p"], torch.softmax((q @ k.transpose(-1, -2) + noise) / 1.5, -1).sum(-2))


def test_topk_rule_descending_ties_to_lower_index():
    s = torch.tensor([[0.5, 2.0, 2.0, -1.0, 0.5, 3.0]])
    assert O.topk_keys(s, 4).tolist() == [[5, 1, 2, 0]]
    assert O.topk_keys(torch.tensor([[0.0, -0.0, 0.0]]), 3).tolist() == [[0, 1, 2]]


def test_gumbel_noise_is_deterministic_sliceable_and_gumbel():
    a = O.gumbel_noise(11, 2, 3, 5, 64)
    b = O.gumbel_noise(11, 2, 3, 5, 64)
    assert torch.equal(a, b) and a.dtype == torch.float32
    assert torch.equal(O.gumbel_noise(11, 2, 3, 5, 64, b0=1, b1=2, h0=1, h1=3), a[1:2, 1:3])
    assert not torch.equal(a, O.gumbel_noise(12, 2, 3, 5, 64))
    g = O.gumbel_noise(5, 1, 8, 128, 512).double()
    assert abs(g.mean().item() - 0.5772) < 0.01 and abs(g.var().item() - math.pi ** 2 / 6) < 0.03
    # known-answer: the integer mixing behind the field (matches the device function bit for bit)
    bits = O.noise_bits(7, np.array([0, 0, 3], dtype=np.uint32), np.array([0, 1, 5], dtype=np.uint32),
                        np.array([0, 0, 9], dtype=np.uint32))
    assert bits.dtype == np.uint32 and len(set(bits.tolist())) == 3


def test_chunked_evaluation_equals_direct():
    torch.manual_seed(6)
    B, Hq, Hkv, M, D = 2, 8, 2, 40, 16
    Q, K, V = torch.randn(B, Hq, M, D), torch.randn(B, Hkv, M, D), torch.randn(B, Hkv, M, D)
    direct = O.attn_block("roco", Q=Q, K=K, V=V, B=B, M=M, P=0, Hq=Hq, Hkv=Hkv, D=D, causal=True, scale=0.25)
    chunk = O.attn_block_chunked("roco", Q=Q, K=K, V=V, head_chunk=4, P=0, causal=True, scale=0.25)
    for key in ("out", "sum_p", "sum_p2"):
        torch.testing.assert_close(chunk[key], direct[key], rtol=1e-5, atol=1e-6)
