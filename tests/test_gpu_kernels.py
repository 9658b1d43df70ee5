"""Parity of the individual sm_100a kernels (through the C ABI) against the fp32 CPU oracle on the same
seeded inputs: RMSNorm, QKV projection with its fused epilogues, the attention core, the per-key
statistics and top-k.  Tolerances: see tests/conftest.py (abs 2e-2, rel 1e-2 above 1e-3 of max|ref|)."""
import math

import pytest
import torch

from conftest import assert_parity, parity_errors
from oracle import attn_block_ref as O
from triton_b200 import _lib as L
from triton_b200 import ops

pytestmark = pytest.mark.gpu
BF, HF = torch.bfloat16, torch.float16


@pytest.mark.parametrize("dt", (BF, HF))
@pytest.mark.parametrize("rows,cols", ((1, 8), (5, 64), (16, 4096), (33, 4544), (7, 1024), (3, 8192), (2, 20000)))
@pytest.mark.parametrize("use_gamma", (False, True))
def test_rmsnorm(dt, rows, cols, use_gamma):
    torch.manual_seed(0)
    x = torch.randn(rows, cols).to(dt)
    g = (1 + 0.1 * torch.randn(cols)).to(dt) if use_gamma else None
    eps = 1e-5 if use_gamma else 0.0
    y = ops.rmsnorm(x.cuda(), None if g is None else g.cuda(), eps)
    rstd = torch.empty(rows, device="cuda")
    ops.rmsnorm(x.cuda(), None, eps, rstd_out=rstd, stats_only=True)
    ref = O.rmsnorm(x, g, eps)
    assert_parity(y, ref, f"rmsnorm {rows}x{cols}")
    ref_rstd = torch.rsqrt(x.float().pow(2).mean(-1) + eps)
    assert (rstd.cpu() - ref_rstd).abs().max().item() <= 1e-5 * ref_rstd.abs().max().item()


def test_rmsnorm_empty_strided_and_errors():
    x = torch.randn(0, 64, device="cuda", dtype=BF)
    assert ops.rmsnorm(x).shape == (0, 64)
    big = torch.randn(6, 256, device="cuda", dtype=BF)
    view = big[:, :128]                                   # row stride 256, 128 columns
    out = torch.zeros(6, 128, device="cuda", dtype=BF)
    ops.rmsnorm(view, None, 0.0, out=out)
    assert_parity(out, O.rmsnorm(view.cpu()), "strided rows")
    with pytest.raises(L.TrinityError, match="shape"):
        ops.rmsnorm(torch.randn(4, 12, device="cuda", dtype=BF))           # cols not a multiple of 8
    with pytest.raises(L.TrinityError, match="aligned"):
        ops.rmsnorm(torch.randn(4, 72, device="cuda", dtype=BF)[:, 4:68])   # misaligned base


PROJ_CASES = [
    # B, M, P, N, Hq, Hkv, D, dtype, qk_norm, row_scale
    (1, 128, 0, 64, 2, 2, 128, BF, False, False),
    (1, 16, 4, 256, 2, 1, 128, HF, False, False),
    (2, 200, 8, 512, 8, 2, 128, BF, False, True),
    (1, 100, 0, 320, 5, 1, 64, BF, False, False),
    (2, 96, 16, 512, 8, 2, 64, BF, True, False),
    (2, 96, 16, 520, 4, 2, 128, HF, True, True),      # hidden size not a multiple of the 64-wide K step
    (1, 16, 1024, 4544, 71, 71, 64, HF, False, False),
    # at most 32 rows and a long contraction: the cluster split-K kernel
    (1, 16, 1024, 4096, 32, 32, 128, HF, False, False),   # the reference's Llama shape
    (2, 16, 16, 1024, 8, 2, 128, BF, True, True),         # 32 rows over two batches, per-head norm, row scale, GQA
    (1, 9, 0, 4096, 32, 8, 128, HF, True, False),
    (1, 16, 8, 2048, 16, 4, 64, BF, True, True),          # head_dim 64: a thread's 64 columns are one head
    (3, 1, 40, 1536, 12, 12, 64, BF, False, True),        # decode rows of three sequences
    # wider than the device holds clusters of 256-column tiles for: 384-column tiles (1.5 / 3 heads of 128, 6 of 64)
    (1, 16, 8, 512, 64, 64, 128, BF, True, True),
    (2, 10, 0, 640, 128, 128, 64, HF, True, False),
    # at least a wave of 256 x 256 tiles: the CTA-pair kernel, with a ragged last row tile (the second CTA of the last
    # pair holds 68 / 1 valid rows), per-head norm + row scale, and a hidden size that is not a multiple of the k step
    (1, 2500, 12, 512, 8, 4, 128, BF, True, True),
    (5, 333, 7, 520, 16, 16, 64, HF, False, False),
]


@pytest.mark.parametrize("B,M,P,N,Hq,Hkv,D,dt,qk_norm,rowscale", PROJ_CASES)
def test_qkv_projection(B, M, P, N, Hq, Hkv, D, dt, qk_norm, rowscale):
    torch.manual_seed(1)
    x = torch.randn(B * M, N).to(dt)
    wq, wk, wv = ((torch.randn(N, h * D) / N ** 0.5).to(dt) for h in (Hq, Hkv, Hkv))
    rs = (torch.rand(B * M) + 0.5) if rowscale else None
    gq = (1 + 0.1 * torch.randn(D)).to(dt) if qk_norm else None
    gk = (1 + 0.1 * torch.randn(D)).to(dt) if qk_norm else None
    q = torch.zeros(B, M, Hq, D, device="cuda", dtype=dt)
    sentinel = 3.0
    kc = torch.full((B, Hkv, P + M, D), sentinel, device="cuda", dtype=dt)
    vc = torch.full((B, Hkv, P + M, D), sentinel, device="cuda", dtype=dt)
    dev = lambda t: None if t is None else t.cuda()
    ops.qkv_project(x.cuda(), wq.cuda(), wk.cuda(), wv.cuda(), q=ops.as_bshd(q, "bshd"),
                    k_cache=ops.as_bshd(kc, "bhsd"), v_cache=ops.as_bshd(vc, "bhsd"), B=B, M=M, P=P, Hq=Hq, Hkv=Hkv,
                    D=D, row_scale=dev(rs), qk_norm=qk_norm, qk_eps=1e-5, gamma_q=dev(gq), gamma_k=dev(gk))
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    xf = x.float() * (rs[:, None] if rs is not None else 1.0)
    qr, kr, vr = O.project("qknorm" if qk_norm else "vanilla", xf, wq, wk, wv, B=B, M=M, Hq=Hq, Hkv=Hkv, D=D,
                           qk_eps=1e-5, gamma_q=gq, gamma_k=gk)
    assert_parity(q, qr.transpose(1, 2), "q")
    assert_parity(kc[:, :, P:], kr, "k rows [P,P+M)")
    assert_parity(vc[:, :, P:], vr, "v rows [P,P+M)")
    # the cached prefix is left exactly as it was
    assert bool((kc[:, :, :P] == sentinel).all()) and bool((vc[:, :, :P] == sentinel).all())


ATTN_CASES = [
    # B, M, P, Hq, Hkv, D, dtype, causal, scale
    (1, 128, 0, 1, 1, 128, BF, False, None),
    (1, 128, 0, 1, 1, 64, BF, False, None),
    (1, 1, 0, 1, 1, 64, HF, True, None),              # a single query, a single key
    (1, 256, 0, 2, 2, 128, BF, True, None),
    (2, 300, 0, 4, 2, 128, HF, True, None),           # ragged: M not a multiple of the 128-row tile
    (1, 16, 1024, 4, 4, 128, HF, False, 0.125),       # the reference's chunked-prefill shape
    (1, 16, 1024, 3, 3, 64, HF, False, 0.125),
    (2, 200, 72, 6, 2, 64, BF, True, None),           # prefix + causal + GQA
    (1, 1000, 0, 8, 1, 64, BF, True, None),           # MQA
    (1, 640, 0, 2, 1, 128, BF, True, 1.0),            # unscaled scores: large row maxima, O rescaling
]


def _attn_inputs(B, M, P, Hq, Hkv, D, dt, seed=2):
    torch.manual_seed(seed)
    L_ = P + M
    return torch.randn(B, M, Hq, D).to(dt), torch.randn(B, Hkv, L_, D).to(dt), torch.randn(B, Hkv, L_, D).to(dt)


def _run_attention(q, kc, vc, P, causal, scale, single_p=False, want_lse=True):
    B, M, Hq, D = q.shape
    o = torch.zeros(B, M, Hq, D, device="cuda", dtype=q.dtype)
    lse = torch.zeros(B, Hq, M, device="cuda") if want_lse else None
    ops.attention(ops.as_bshd(q.cuda(), "bshd"), ops.as_bshd(kc.cuda(), "bhsd"), ops.as_bshd(vc.cuda(), "bhsd"),
                  ops.as_bshd(o, "bshd"), P=P, causal=causal, scale=scale, lse=lse, single_p=single_p)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    return o, lse


@pytest.mark.parametrize("B,M,P,Hq,Hkv,D,dt,causal,scale", ATTN_CASES)
def test_attention_core(B, M, P, Hq, Hkv, D, dt, causal, scale):
    scale = D ** -0.5 if scale is None else scale
    q, kc, vc = _attn_inputs(B, M, P, Hq, Hkv, D, dt)
    o, lse = _run_attention(q, kc, vc, P, causal, scale)
    r = O.attend(q.float().transpose(1, 2), kc.float(), vc.float(), P=P, causal=causal, scale=scale)
    assert not torch.isnan(o).any()
    assert_parity(o, r["out"].transpose(1, 2), "attention output")
    sc = torch.matmul(q.float().transpose(1, 2), kc.float().repeat_interleave(Hq // Hkv, 1).transpose(-1, -2)) * scale
    if causal:
        i = torch.arange(M).view(M, 1)
        j = torch.arange(P + M).view(1, P + M)
        sc = sc.masked_fill(j > i + P, -math.inf)
    lref = torch.logsumexp(sc, -1) / math.log(2)
    assert (lse.cpu() - lref).abs().max().item() <= 1e-4


SPLIT_CASES = [
    # B, M, P, Hq, Hkv, D, dtype, causal: launches that fill less than half of the SMs
    (1, 16, 1024, 32, 32, 128, HF, False),            # the reference's chunked-prefill shape: 4 splits
    (1, 16, 1024, 8, 2, 128, BF, True),               # GQA head pairs, 8 splits
    (1, 200, 900, 4, 4, 64, BF, True),                # MHA: two query blocks of unequal length per CTA
    (2, 1, 2047, 6, 3, 64, HF, True),                 # decode: one query, ragged last key block
    (1, 300, 1500, 3, 1, 128, BF, True),              # MQA, odd group: a CTA with a single tile
    (3, 16, 100, 5, 5, 64, HF, True),                 # <= 32 queries, too few keys to split: replicas only
    (2, 32, 0, 4, 2, 128, BF, True),                  # no prefix: causal mask inside the only key block
    (1, 7, 300, 2, 2, 128, BF, False),                # 7 queries, ragged last key block
]


@pytest.mark.parametrize("B,M,P,Hq,Hkv,D,dt,causal", SPLIT_CASES)
def test_attention_split_kv_matches_unsplit_and_oracle(B, M, P, Hq, Hkv, D, dt, causal):
    scale = D ** -0.5
    q, kc, vc = _attn_inputs(B, M, P, Hq, Hkv, D, dt, seed=11)
    nbytes = ops.attention_workspace_bytes(B, M, P, Hq, Hkv, D)
    assert nbytes > 0 or M <= 32, "case is meant to split (or, with <= 32 queries, to run as four replicas)"
    o0, l0 = _run_attention(q, kc, vc, P, causal, scale)
    qd, kd, vd = q.cuda(), kc.cuda(), vc.cuda()
    for avail in ((nbytes, nbytes // 2 + 256) if nbytes else (256,)):   # full scratch, and scratch for fewer splits
        ws = torch.empty(avail, dtype=torch.uint8, device="cuda")
        ws.fill_(0xff)                                 # contents must not matter (0xff..: NaN as fp32)
        o1 = torch.zeros(B, M, Hq, D, device="cuda", dtype=dt)
        l1 = torch.zeros(B, Hq, M, device="cuda")
        ops.attention(ops.as_bshd(qd, "bshd"), ops.as_bshd(kd, "bhsd"), ops.as_bshd(vd, "bhsd"), ops.as_bshd(o1, "bshd"),
                      P=P, causal=causal, scale=scale, lse=l1, workspace=ws)
        torch.cuda.synchronize()
        assert L.kernel_status() == 0
        assert not torch.isnan(o1).any()
        assert (l1 - l0).abs().max().item() <= 1e-4
        # same softmax, different summation order: within one 16-bit rounding of the unsplit result
        assert_parity(o1, o0.float().cpu(), "split vs unsplit")
        r = O.attend(q.float().transpose(1, 2), kc.float(), vc.float(), P=P, causal=causal, scale=scale)
        assert_parity(o1, r["out"].transpose(1, 2), "split attention output")


SMALL_CASES = [
    # B, M, P, Hq, Hkv, D, dtype, causal: at most 16 queries per head (the cluster-merged mma.sync kernel)
    (1, 16, 1024, 32, 32, 128, HF, False),            # the reference's Llama shape: clusters of 4
    (1, 16, 1024, 71, 71, 64, HF, False),             # the reference's Falcon shape: clusters of 2
    (1, 1, 4095, 2, 1, 128, BF, True),                # decode, long prefix: clusters of 8
    (2, 16, 0, 3, 3, 64, BF, True),                   # no prefix: one chunk, three of the four warps see no key
    (1, 5, 27, 2, 2, 128, HF, True),                  # exactly one chunk of 32 keys
    (4, 9, 500, 40, 8, 64, BF, True),                 # more heads than SMs: no cluster
    (1, 16, 8000, 4, 4, 128, HF, False),              # 250 chunks over 32 warps
    (1, 13, 70, 6, 2, 128, BF, True),                 # GQA, ragged last chunk
    (8, 1, 4095, 32, 8, 128, BF, True),               # GQA decode: the 4 query heads of a kv head share one CTA's rows
    (2, 1, 300, 16, 1, 64, HF, True),                 # MQA decode: 16 heads in the 16 rows
    (1, 4, 200, 8, 2, 128, BF, True),                 # 4 heads x 4 queries: the causal limit follows the query, not the row
    (1, 3, 100, 12, 2, 64, HF, True),                 # group of 6, 3 queries: packs of 3 heads (9 rows)
]


@pytest.mark.parametrize("B,M,P,Hq,Hkv,D,dt,causal", SMALL_CASES)
def test_attention_with_at_most_16_queries(B, M, P, Hq, Hkv, D, dt, causal):
    scale = D ** -0.5
    q, kc, vc = _attn_inputs(B, M, P, Hq, Hkv, D, dt, seed=21)
    o, lse = _run_attention(q, kc, vc, P, causal, scale)
    o2, lse2 = _run_attention(q, kc, vc, P, causal, scale)
    assert torch.equal(o, o2) and torch.equal(lse, lse2)          # fixed merge order
    r = O.attend(q.float().transpose(1, 2), kc.float(), vc.float(), P=P, causal=causal, scale=scale)
    assert not torch.isnan(o).any()
    assert_parity(o, r["out"].transpose(1, 2), "small-M attention output")
    sc = torch.matmul(q.float().transpose(1, 2), kc.float().repeat_interleave(Hq // Hkv, 1).transpose(-1, -2)) * scale
    if causal:
        i = torch.arange(M).view(M, 1)
        j = torch.arange(P + M).view(1, P + M)
        sc = sc.masked_fill(j > i + P, -math.inf)
    assert (lse.cpu() - torch.logsumexp(sc, -1) / math.log(2)).abs().max().item() <= 1e-4
    # token-major caches [B, L, Hkv, D] (the layout cache append writes): same numbers, other strides
    kt, vt = kc.transpose(1, 2).contiguous().cuda(), vc.transpose(1, 2).contiguous().cuda()
    o3 = torch.zeros_like(o)
    ops.attention(ops.as_bshd(q.cuda(), "bshd"), ops.as_bshd(kt, "bshd"), ops.as_bshd(vt, "bshd"), ops.as_bshd(o3, "bshd"),
                  P=P, causal=causal, scale=scale)
    torch.cuda.synchronize()
    assert torch.equal(o3, o)
    # one 16-bit part of p (single_p): looser, still inside the absolute bound
    o4, _ = _run_attention(q, kc, vc, P, causal, scale, single_p=True)
    assert parity_errors(o4, r["out"].transpose(1, 2))[0] <= 2e-2


def test_attention_workspace_is_zero_for_launches_that_fill_the_gpu():
    assert ops.attention_workspace_bytes(4, 4096, 0, 32, 8, 128) == 0
    assert ops.attention_workspace_bytes(1, 16, 128, 4, 4, 128) == 0          # two key blocks: nothing to split
    assert ops.attention_workspace_bytes(1, 16, 1024, 32, 32, 128) > 0


def test_attention_single_p_mode_is_looser_but_bounded():
    q, kc, vc = _attn_inputs(1, 256, 0, 2, 2, 128, BF)
    r = O.attend(q.float().transpose(1, 2), kc.float(), vc.float(), P=0, causal=True, scale=128 ** -0.5)
    o1, _ = _run_attention(q, kc, vc, 0, True, 128 ** -0.5, single_p=True)
    o2, _ = _run_attention(q, kc, vc, 0, True, 128 ** -0.5, single_p=False)
    a1, _ = parity_errors(o1, r["out"].transpose(1, 2))
    a2, r2 = parity_errors(o2, r["out"].transpose(1, 2))
    assert a1 <= 2e-2 and a2 <= 2e-2 and r2 <= 1e-2


def test_attention_is_bitwise_reproducible():
    q, kc, vc = _attn_inputs(2, 300, 40, 4, 2, 128, BF, seed=5)
    o1, l1 = _run_attention(q, kc, vc, 40, True, 0.1)
    o2, l2 = _run_attention(q, kc, vc, 40, True, 0.1)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)


def test_attention_layouts_head_major_and_token_major_agree():
    # the reference's tensors are head-major [H, M, D] (Q, O) or token-major [M, N] (O2): same numbers
    q, kc, vc = _attn_inputs(1, 48, 16, 4, 4, 64, HF, seed=6)
    o_tok, _ = _run_attention(q, kc, vc, 16, False, 1.0)
    qh = q[0].permute(1, 0, 2).contiguous().cuda()              # [H, M, D]
    oh = torch.zeros(4, 48, 64, device="cuda", dtype=HF)
    ops.attention(ops.as_bshd(qh, "hsd"), ops.as_bshd(kc[0].cuda(), "hsd"), ops.as_bshd(vc[0].cuda(), "hsd"),
                  ops.as_bshd(oh, "hsd"), P=16, causal=False, scale=1.0)
    torch.cuda.synchronize()
    assert torch.equal(oh.permute(1, 0, 2), o_tok[0])


def test_attention_argument_errors():
    q, kc, vc = _attn_inputs(1, 16, 0, 2, 2, 64, BF)
    o = torch.zeros(1, 16, 2, 64, device="cuda", dtype=BF)
    args = (ops.as_bshd(q.cuda(), "bshd"), ops.as_bshd(kc.cuda(), "bhsd"), ops.as_bshd(vc.cuda(), "bhsd"), ops.as_bshd(o, "bshd"))
    with pytest.raises(L.TrinityError, match="shape"):
        ops.attention(*args, P=0, causal=False, scale=0.0)                    # scale must be positive
    q3 = torch.randn(1, 16, 3, 64, device="cuda", dtype=BF)
    with pytest.raises(L.TrinityError, match="shape"):                        # 3 query heads over 2 kv heads
        ops.attention(q3, args[1], args[2], torch.zeros_like(q3), P=0, causal=False, scale=1.0)
    q96 = torch.randn(1, 16, 2, 96, device="cuda", dtype=BF)
    with pytest.raises(L.TrinityError, match="shape"):                        # head_dim 96 unsupported
        ops.attention(q96, q96.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3), q96, torch.zeros_like(q96),
                      P=0, causal=False, scale=1.0)
    assert L.kernel_status() == 0


STATS_CASES = [
    # variant, B, M, P, Hq, Hkv, D, dtype, causal, noise_mode, topk
    ("roco", 1, 128, 0, 1, 1, 64, BF, False, 0, 16),
    ("roco", 1, 256, 0, 2, 1, 64, BF, True, 0, 64),
    ("roco", 2, 300, 40, 4, 2, 128, HF, True, 0, 100),
    ("roco", 1, 16, 1024, 4, 4, 128, HF, False, 0, 128),
    ("keyformer", 1, 128, 0, 1, 1, 128, BF, False, L.TRN_NOISE_TENSOR, 16),
    ("keyformer", 1, 256, 0, 2, 1, 128, BF, True, L.TRN_NOISE_TENSOR, 64),
    ("keyformer", 1, 256, 0, 2, 1, 128, BF, True, L.TRN_NOISE_GUMBEL, 64),
    ("keyformer", 1, 16, 1024, 4, 4, 128, HF, False, L.TRN_NOISE_TENSOR, 128),
    ("keyformer", 2, 300, 40, 4, 2, 64, BF, True, L.TRN_NOISE_GUMBEL, 100),
]


@pytest.mark.parametrize("variant,B,M,P,Hq,Hkv,D,dt,causal,noise_mode,topk", STATS_CASES)
def test_key_statistics_and_topk(variant, B, M, P, Hq, Hkv, D, dt, causal, noise_mode, topk):
    from gpu_util import run_block
    torch.manual_seed(3)
    L_ = P + M
    scale = D ** -0.5
    tau = 1.5 if variant == "keyformer" else 1.0
    t = dict(Q=torch.randn(B, M, Hq, D).to(dt), K_cache=torch.randn(B, Hkv, L_, D).to(dt),
             V_cache=torch.randn(B, Hkv, L_, D).to(dt), noise=None)
    noise = None
    if variant == "keyformer":
        if noise_mode == L.TRN_NOISE_TENSOR:
            t["noise"] = noise = torch.randn(B, Hq, M, L_).to(dt)
        else:
            noise = O.gumbel_noise(7, B, Hq, M, L_)
    got = run_block(variant, t, B=B, M=M, P=P, Hq=Hq, Hkv=Hkv, D=D, causal=causal, scale=scale, tau=tau,
                    noise_mode=noise_mode, seed=7, project=False)
    r = O.attend(t["Q"].float().transpose(1, 2), t["K_cache"].float(), t["V_cache"].float(), P=P, causal=causal,
                 scale=scale, variant=variant, tau=tau, noise=noise)
    assert_parity(got["out"], r["out"].transpose(1, 2), "out")
    # statistics are fp32 sums of fp32 probabilities: far tighter than the 16-bit tolerance
    assert_parity(got["sum_p"], r["sum_p"], "sum_p", abs_tol=1e-4, rel_tol=1e-4)
    if variant == "roco":
        assert_parity(got["sum_p2"], r["sum_p2"], "sum_p2", abs_tol=1e-4, rel_tol=1e-4)
        assert (got["sum_p"].sum(-1).cpu() - M).abs().max().item() <= 1e-3 * M       # rows of p sum to 1
    # top-k: exact indices (order included) on the scores the kernel produced ...
    idx = ops.topk_keys(got["sum_p"], topk)
    torch.cuda.synchronize()
    assert torch.equal(idx.cpu(), O.topk_keys(got["sum_p"].cpu(), topk))
    # ... and the same selection as the oracle's own scores, except where two scores at the rank
    # boundary are closer than the fp32 noise of the sums
    want = O.topk_keys(r["sum_p"], topk)
    if not torch.equal(idx.cpu(), want):
        srt = torch.sort(r["sum_p"], -1, descending=True).values
        gaps = (srt[..., :-1] - srt[..., 1:])
        rows = (idx.cpu() != want).any(-1)
        pos = (idx.cpu() != want)[rows].float().argmax(-1)
        assert (gaps[rows].gather(-1, pos.clamp(max=gaps.shape[-1] - 1).unsqueeze(-1)) <= 1e-5 * srt[rows][..., :1]).all()


def test_topk_edge_cases():
    s = torch.tensor([[0.5, 2.0, 2.0, -1.0, 0.5, 3.0], [1.0, 1.0, 1.0, 1.0, 1.0, 1.0]], device="cuda")
    assert ops.topk_keys(s, 4).cpu().tolist() == [[5, 1, 2, 0], [0, 1, 2, 3]]
    assert ops.topk_keys(s, 6).cpu().tolist()[0] == [5, 1, 2, 0, 4, 3]
    torch.manual_seed(9)
    big = torch.randn(3, 8192, device="cuda")
    big[1, 100:200] = big[1, 50]                         # a run of equal scores
    assert torch.equal(ops.topk_keys(big, 2048).cpu(), O.topk_keys(big.cpu(), 2048))
    odd = torch.randn(5, 1040, device="cuda")
    assert torch.equal(ops.topk_keys(odd, 1).cpu(), O.topk_keys(odd.cpu(), 1))
    # every size class of the sort (keys per thread 1 / 2 / 4 / 8, padded and exact powers of two, one warp and less)
    for n, k in ((1, 1), (7, 3), (32, 32), (33, 5), (500, 499), (1024, 100), (1025, 1025), (2048, 2048), (3000, 17),
                 (4096, 1024), (5000, 4999), (8192, 8192)):
        t = torch.randn(4, n, device="cuda")
        t[2, : n // 2] = 0.25                              # ties over half of a row
        assert torch.equal(ops.topk_keys(t, k).cpu(), O.topk_keys(t.cpu(), k)), (n, k)
    with pytest.raises(L.TrinityError, match="shape"):
        ops.topk_keys(torch.randn(2, 9000, device="cuda"), 10)
    with pytest.raises(L.TrinityError, match="shape"):
        ops.topk_keys(odd, 2000)


@pytest.mark.parametrize("B,M,P,Hq,Hkv,D,dt,causal,noise_mode", (
    (1, 16, 1024, 8, 8, 128, HF, False, L.TRN_NOISE_TENSOR),      # the reference's shape (split-KV with a workspace)
    (2, 200, 72, 6, 2, 64, BF, True, L.TRN_NOISE_GUMBEL),
    (1, 300, 0, 4, 4, 128, BF, True, L.TRN_NOISE_TENSOR),
    # at most 16 queries: the warp-level kernel's fused / score-keeping modes
    (1, 16, 1024, 71, 71, 64, HF, False, L.TRN_NOISE_TENSOR),     # the reference's Falcon shape
    (2, 12, 100, 8, 2, 64, BF, True, L.TRN_NOISE_GUMBEL),         # generated noise, causal, grouped heads (one per CTA)
    (1, 4, 333, 8, 2, 128, BF, True, L.TRN_NOISE_TENSOR),         # four heads packed in the rows; odd noise row length
    (3, 1, 95, 4, 1, 128, HF, True, L.TRN_NOISE_TENSOR),          # decode
))
def test_fused_attention_and_perturbed_lse_equals_two_passes_and_kept_scores_give_the_same_statistics(
        B, M, P, Hq, Hkv, D, dt, causal, noise_mode):
    """One pass (o, lse, perturbed lse, scores kept) against the two separate passes, and per-key statistics summed
    from the kept scores against the recomputing kernel."""
    scale, tau, seed = D ** -0.5, 1.5, 5
    L_ = P + M
    q, kc, vc = _attn_inputs(B, M, P, Hq, Hkv, D, dt, seed=21)
    torch.manual_seed(22)
    noise = torch.randn(B, Hq, M, L_).to(dt).cuda() if noise_mode == L.TRN_NOISE_TENSOR else None
    qv, kv, vv = ops.as_bshd(q.cuda(), "bshd"), ops.as_bshd(kc.cuda(), "bhsd"), ops.as_bshd(vc.cuda(), "bhsd")
    kw = dict(P=P, causal=causal, scale=scale)
    nkw = dict(noise_mode=noise_mode, tau=tau, noise=noise, seed=seed)
    # two passes
    o_a = torch.zeros(B, M, Hq, D, device="cuda", dtype=dt)
    lse_a, lse2_a = torch.zeros(B, Hq, M, device="cuda"), torch.zeros(B, Hq, M, device="cuda")
    ops.attention(qv, kv, vv, o_a, lse=lse_a, **kw)
    ops.attention(qv, kv, vv, None, lse=lse2_a, **kw, **nkw)
    sp_a, sp_r, sp2_r = (torch.zeros(B, Hq, L_, device="cuda") for _ in range(3))
    ops.attn_colstats(qv, kv, lse2_a, sp_a, None, **kw, **nkw)
    ops.attn_colstats(qv, kv, lse_a, sp_r, sp2_r, **kw)
    for use_ws in (False, True):
        nb = ops.attention_workspace_bytes(B, M, P, Hq, Hkv, D) if use_ws else 0
        ws = torch.empty(nb, dtype=torch.uint8, device="cuda").fill_(0xff) if nb else None
        pitch = (L_ + 31) // 32 * 32
        o_b = torch.zeros_like(o_a)
        lse_b, lse2_b = torch.zeros_like(lse_a), torch.zeros_like(lse_a)
        sc = torch.full((B, Hq, M, pitch), float("nan"), device="cuda")
        ops.attention(qv, kv, vv, o_b, lse=lse_b, lse_pert=lse2_b, scores=sc, workspace=ws, **kw, **nkw)
        sp_b = torch.zeros_like(sp_a)
        ops.attn_colstats(qv, kv, lse2_b, sp_b, None, scores=sc, **kw)
        # plain scores kept by an un-noised pass, for the RoCo sums
        sc0 = torch.full((B, Hq, M, pitch), float("nan"), device="cuda")
        o_c, lse_c = torch.zeros_like(o_a), torch.zeros_like(lse_a)
        ops.attention(qv, kv, vv, o_c, lse=lse_c, scores=sc0, workspace=ws, **kw)
        sp_c, sp2_c = torch.zeros_like(sp_a), torch.zeros_like(sp_a)
        ops.attn_colstats(qv, kv, lse_c, sp_c, sp2_c, scores=sc0, **kw)
        torch.cuda.synchronize()
        assert L.kernel_status() == 0
        assert_parity(o_b, o_a.float().cpu(), "o fused vs separate")
        assert (lse_b - lse_a).abs().max().item() <= 1e-4 and (lse2_b - lse2_a).abs().max().item() <= 1e-4
        if not causal:          # under a causal mask the scores of keys a query must not see are never written
            assert not torch.isnan(sc[..., :L_]).any() and not torch.isnan(sc0[..., :L_]).any()
        assert_parity(sp_b, sp_a.cpu(), "KeyFormer sums from kept scores", abs_tol=1e-3 * max(1.0, M / 16), rel_tol=1e-3)
        assert_parity(sp_c, sp_r.cpu(), "RoCo sum p from kept scores", abs_tol=1e-3 * max(1.0, M / 16), rel_tol=1e-3)
        assert_parity(sp2_c, sp2_r.cpu(), "RoCo sum p^2 from kept scores", abs_tol=1e-3 * max(1.0, M / 16), rel_tol=1e-3)


@pytest.mark.parametrize("M,N,P,R,dt", (
    (16, 1024, 512, 64, HF),          # the reference's LoRA configuration (lora_benchmark.py:545)
    (16, 2048, 1024, 128, HF),        # its "larger model"
    (200, 520, 320, 64, BF),          # two row tiles, hidden size not a multiple of the 64-wide K step
    (1, 4096, 4096, 64, BF),          # a single token
    (9, 1024, 512, 128, BF),          # a partial row block on the path for at most 16 tokens
    (17, 1024, 512, 64, HF),          # one token too many for it: the tiled kernels
))
def test_lora_linear_layer(M, N, P, R, dt):
    """o = x @ w + (x @ a) @ b against the fp32 oracle; d = x @ a is delivered as a 16-bit tensor like the reference's D."""
    torch.manual_seed(3)
    x = torch.randn(M, N).to(dt)
    w, a = (torch.randn(N, P) / N ** 0.5).to(dt), (torch.randn(N, R) / N ** 0.5).to(dt)
    b = (torch.randn(R, P) / R ** 0.5).to(dt)            # keeps o at unit scale (the tolerance is absolute)
    o = torch.full((M, P), float("nan"), device="cuda", dtype=dt)
    d = torch.full((M, R), float("nan"), device="cuda", dtype=dt)
    ops.lora(x.cuda(), w.cuda(), a.cuda(), b.cuda(), o, d)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    pure = O.lora(x, w, a, b)
    assert_parity(d, pure["D"], "D = X @ A")
    # the second step on the D that was stored (one differing bit in D moves a whole row of O slightly)
    stored = O.lora(x, w, a, b, round_d=dt)
    like = x.float() @ w.float() + d.float().cpu() @ b.float()
    assert_parity(o, like, "O on the stored D")
    assert_parity(o, stored["O"], "O", rel_floor=1e-1, rel_tol=5e-2)
    o2 = ops.lora(x.cuda(), w.cuda(), a.cuda(), b.cuda())          # allocating form, deterministic
    torch.cuda.synchronize()
    assert torch.equal(o2, o)
    with pytest.raises(L.TrinityError, match="shape"):
        ops.lora(x.cuda(), w.cuda()[:, :P - 8].contiguous(), a.cuda(), b.cuda()[:, :P - 8].contiguous())


def test_wait_that_runs_out_is_reported_and_leaves_the_context_usable():
    """The device-side failure path all kernels share: a bounded wait on a barrier nothing arrives at gives up
    after its limit, the kernel returns normally (tensor memory freed, no trap), the status word holds the code,
    later kernels of the library return at once while it is set, and after trinity_clear_kernel_status() the
    library works as before."""
    import ctypes as C
    lib = L.load()
    assert L.kernel_status() == 0
    x = torch.randn(64, 256, device="cuda").to(BF)
    want = ops.rmsnorm(x, None, 1e-5).clone()
    L.check(lib.trinity_selftest_wait_timeout(1000, None))          # 1 ms
    st = C.c_int(0)
    assert lib.trinity_last_kernel_status(C.byref(st)) == -9           # TRN_E_KERNEL
    assert st.value == 103                                             # KST_TIMEOUT_CONSUMER
    with pytest.raises(L.TrinityError, match="bounded wait"):
        L.check(-9)
    # sticky until cleared; tensor-core kernels launched meanwhile return without touching their outputs
    assert L.kernel_status() == 103
    q = torch.randn(1, 128, 2, 64, device="cuda").to(BF)
    kv = torch.randn(1, 128, 2, 64, device="cuda").to(BF)
    o = torch.full_like(q, 7.0)
    ops.attention(q, kv, kv, o, P=0, causal=True, scale=0.125)
    torch.cuda.synchronize()
    assert torch.equal(o, torch.full_like(q, 7.0))
    L.check(lib.trinity_clear_kernel_status())
    assert L.kernel_status() == 0
    ops.attention(q, kv, kv, o, P=0, causal=True, scale=0.125)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0 and not torch.equal(o, torch.full_like(q, 7.0))
    assert torch.equal(ops.rmsnorm(x, None, 1e-5), want)
    with pytest.raises(L.TrinityError, match="shape"):
        L.check(lib.trinity_selftest_wait_timeout(0, None))


@pytest.mark.parametrize("B,M,P,Hq,Hkv,D,dt,causal,single_p", (
    (1, 256, 0, 2, 1, 128, BF, True, False),
    (2, 300, 40, 4, 2, 64, BF, True, False),
    (1, 130, 24, 4, 4, 128, HF, False, True),
    (1, 16, 1024, 8, 8, 128, HF, False, False),       # few queries per head: row-replicated tiles + split-KV
    (3, 1, 700, 8, 2, 64, BF, True, False),           # decode
))
def test_keyformer_tau_one_generated_noise(B, M, P, Hq, Hkv, D, dt, causal, single_p):
    """tau = 1 with generated Gumbel noise (the KeyFormer benchmark configuration): exp(s + g) = exp(s) / E, so the
    fused pass takes the perturbed weight as the plain weight times 1 / E.  Checked against the oracle
    (ref_rms.py:172-174 with tau = 1 on the same noise), against the separate perturbed-lse pass, and through the
    whole block."""
    from gpu_util import run_block
    scale, seed = D ** -0.5, 9
    L_ = P + M
    q, kc, vc = _attn_inputs(B, M, P, Hq, Hkv, D, dt, seed=33)
    noise = O.gumbel_noise(seed, B, Hq, M, L_)
    r = O.attend(q.float().transpose(1, 2), kc.float(), vc.float(), P=P, causal=causal, scale=scale, variant="keyformer",
                 tau=1.0, noise=noise)
    qv, kv, vv = ops.as_bshd(q.cuda(), "bshd"), ops.as_bshd(kc.cuda(), "bhsd"), ops.as_bshd(vc.cuda(), "bhsd")
    kw = dict(P=P, causal=causal, scale=scale)
    nkw = dict(noise_mode=L.TRN_NOISE_GUMBEL, tau=1.0, seed=seed)
    lse_sep = torch.zeros(B, Hq, M, device="cuda")
    ops.attention(qv, kv, vv, None, lse=lse_sep, **kw, **nkw)                      # perturbed lse only
    for use_ws in (False, True):
        nb = ops.attention_workspace_bytes(B, M, P, Hq, Hkv, D) if use_ws else 0
        ws = torch.empty(nb, dtype=torch.uint8, device="cuda").fill_(0xff) if nb else None
        o = torch.zeros(B, M, Hq, D, device="cuda", dtype=dt)
        lse, lse2 = torch.zeros(B, Hq, M, device="cuda"), torch.zeros(B, Hq, M, device="cuda")
        ops.attention(qv, kv, vv, o, lse=lse, lse_pert=lse2, workspace=ws, single_p=single_p, **kw, **nkw)
        sp = torch.zeros(B, Hq, L_, device="cuda")
        ops.attn_colstats(qv, kv, lse2, sp, None, **kw, **nkw)
        torch.cuda.synchronize()
        assert L.kernel_status() == 0
        if single_p:
            assert_parity(o, r["out"].transpose(1, 2), "tau=1 fused out (one 16-bit part of p)", rel_floor=0.1, rel_tol=5e-2)
        else:
            assert_parity(o, r["out"].transpose(1, 2), "tau=1 fused out")
        assert (lse2 - lse_sep).abs().max().item() <= 2e-4                          # base-2 log units
        want_lse2 = torch.logsumexp(_perturbed_scores(q, kc, noise, P, causal, scale), dim=-1) / math.log(2.0)
        assert (lse2.cpu() - want_lse2).abs().max().item() <= 1e-3
        assert_parity(sp, r["sum_p"], "tau=1 sum_p", abs_tol=1e-4 * max(1.0, M / 16), rel_tol=2e-4)
        assert (sp.sum(-1).cpu() - M).abs().max().item() <= 1e-3 * M
    # whole block (attention + perturbed lse in one pass, statistics, as trinity_attn_block composes them)
    t = dict(Q=q, K_cache=kc, V_cache=vc, noise=None)
    got = run_block("keyformer", t, B=B, M=M, P=P, Hq=Hq, Hkv=Hkv, D=D, causal=causal, scale=scale, tau=1.0,
                    noise_mode=L.TRN_NOISE_GUMBEL, seed=seed, project=False)
    assert_parity(got["out"], r["out"].transpose(1, 2), "tau=1 block out")
    assert_parity(got["sum_p"], r["sum_p"], "tau=1 block sum_p", abs_tol=1e-4 * max(1.0, M / 16), rel_tol=2e-4)


def _perturbed_scores(q, kc, noise, P, causal, scale):
    """(scale * q k^T + noise) with the causal mask, [B, Hq, M, L] fp32, natural-log domain."""
    B, M, Hq, D = q.shape
    grp = Hq // kc.shape[1]
    s = torch.matmul(q.float().transpose(1, 2), kc.float().repeat_interleave(grp, dim=1).transpose(-1, -2)) * scale + noise
    if causal:
        L_ = kc.shape[2]
        mask = torch.arange(L_).view(1, L_) > (torch.arange(M).view(M, 1) + P)
        s = s.masked_fill(mask, float("-inf"))
    return s


@pytest.mark.parametrize("M,K,N,dt,gate", (
    (16, 1024, 4096, HF, "silu"), (16, 512, 192, BF, "sigmoid"), (300, 1024, 1024, BF, "silu"),
    (2048, 512, 640, HF, "silu"), (1, 64, 64, BF, "silu"), (129, 136, 320, BF, "sigmoid"),
    (16, 2048, 8192, HF, "silu"), (7, 128, 96, BF, "sigmoid"), (16, 1024, 64, BF, "silu"), (13, 384, 160, HF, "silu"),
))
def test_gated_mlp(M, K, N, dt, gate):
    """o = gate(x @ w1) * (x @ w2) (gmlp_benchmark.py:53-74) against the fp32 oracle; both products share one
    accumulator tile and o is rounded once."""
    torch.manual_seed(17)
    x = torch.randn(M, K).to(dt)
    w1, w2 = (torch.randn(K, N) / K ** 0.5).to(dt), (torch.randn(K, N) / K ** 0.5).to(dt)
    o = torch.full((M, N), float("nan"), dtype=dt, device="cuda")
    ops.gmlp(x.cuda(), w1.cuda(), w2.cuda(), o, gate=gate)
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    want = O.gmlp(x, w1, w2, gate=gate)["O"]
    # |o| reaches tens here: the absolute bound scales with the output's 16-bit spacing at its largest value
    assert_parity(o, want, f"gmlp {gate} M{M} K{K} N{N}", abs_tol=max(2e-2, 2.0 ** -8 * want.abs().max().item()))
    with pytest.raises(L.TrinityError, match="shape"):
        ops.gmlp(x.cuda(), w1[:, :N - 8].contiguous().cuda(), w2[:, :N - 8].contiguous().cuda(), None, gate=gate)


def test_sliced_keyformer_problem_sees_the_whole_problems_noise():
    """A rank that runs only some (batch item, head) units of a KeyFormer problem with generated noise passes the whole
    problem's head count and its first unit's flat index: its slice of the per-key scores must equal the unsliced
    run's bit for bit (same noise, same kernels)."""
    from gpu_util import run_block
    B, M, P, Hq, Hkv, D, dt = 3, 200, 56, 8, 4, 64, BF
    q, kc, vc = _attn_inputs(B, M, P, Hq, Hkv, D, dt, seed=41)
    t = dict(Q=q, K_cache=kc, V_cache=vc, noise=None)
    kw = dict(M=M, P=P, D=D, causal=True, scale=D ** -0.5, tau=1.0, noise_mode=L.TRN_NOISE_GUMBEL, seed=5, project=False)
    full = run_block("keyformer", t, B=B, Hq=Hq, Hkv=Hkv, **kw)
    grp = Hq // Hkv
    for b0, nb, kv0, kv1 in ((1, 2, 0, 4), (2, 1, 1, 3), (0, 1, 3, 4)):
        h0, h1 = kv0 * grp, kv1 * grp
        ts = dict(Q=q[b0:b0 + nb, :, h0:h1].contiguous(), K_cache=kc[b0:b0 + nb, kv0:kv1].contiguous(),
                  V_cache=vc[b0:b0 + nb, kv0:kv1].contiguous(), noise=None)
        part = run_block("keyformer", ts, B=nb, Hq=h1 - h0, Hkv=kv1 - kv0, noise_heads=Hq, noise_bh0=b0 * Hq + h0, **kw)
        assert torch.equal(part["sum_p"], full["sum_p"][b0:b0 + nb, h0:h1])
        assert torch.equal(part["out"], full["out"][b0:b0 + nb, :, h0:h1])
