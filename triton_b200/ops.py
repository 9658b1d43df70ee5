"""Operators of the attention block on torch CUDA tensors, each a thin call into the C-ABI library.

torch is used for device memory and the current stream only; every computation is done by the
sm_100a kernels behind include/trinity_b200.h.  All operators write into caller-provided tensors
and launch on ``torch.cuda.current_stream()`` without synchronising, so a sequence of them can be
captured in a CUDA graph exactly like the reference's generated ``forward``
(vanilla_llama_benchmark.py:263-285).
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from . import _lib as L

_DTYPES = {torch.bfloat16: L.TRN_BF16, torch.float16: L.TRN_FP16}

# layout strings name the dims of a tensor in memory order; the kernels see (b, s, h, d) strides
_LAYOUT_PERM = {
    "bshd": (0, 1, 2, 3),
    "bhsd": (0, 2, 1, 3),
    "shd": None,   # handled by unsqueeze
    "hsd": None,
}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"triton_b200 kernels take bfloat16 or float16 tensors, got {t.dtype}") from None


def _need_cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("triton_b200 operators need CUDA tensors (there is no CPU path)")


def as_bshd(t: torch.Tensor, layout: str) -> torch.Tensor:
    """View of ``t`` with dims (batch, position, head, head_dim), whatever its memory layout."""
    if layout == "bshd":
        v = t
    elif layout == "bhsd":
        v = t.permute(0, 2, 1, 3)
    elif layout == "shd":
        v = t.unsqueeze(0)
    elif layout == "hsd":
        v = t.unsqueeze(0).permute(0, 2, 1, 3)
    else:
        raise ValueError(f"unknown layout {layout!r}")
    if v.dim() != 4 or v.stride(3) != 1:
        raise ValueError(f"tensor of shape {tuple(t.shape)} does not fit layout {layout!r} with contiguous head_dim")
    return v


def _head_tensor(v: Optional[torch.Tensor]) -> L.TrnHeadTensor:
    if v is None:
        return L.TrnHeadTensor(None, 0, 0, 0)
    return L.TrnHeadTensor(v.data_ptr(), v.stride(0), v.stride(1), v.stride(2))


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def rmsnorm(x: torch.Tensor, gamma: Optional[torch.Tensor] = None, eps: float = 0.0,
            out: Optional[torch.Tensor] = None, rstd_out: Optional[torch.Tensor] = None,
            stats_only: bool = False) -> Optional[torch.Tensor]:
    """y = x * rsqrt(mean(x^2, -1) + eps) * gamma over the last dim of a 2-D (or flattenable) tensor."""
    _need_cuda(x, gamma, out, rstd_out)
    x2 = x.reshape(-1, x.shape[-1]) if x.dim() != 2 else x
    if x2.stride(1) != 1:
        raise ValueError("rmsnorm needs a contiguous last dim")
    if out is None and not stats_only:
        out = torch.empty_like(x)
    y2 = None
    if out is not None:
        y2 = out.reshape(-1, out.shape[-1]) if out.dim() != 2 else out
        if y2.shape != x2.shape or y2.dtype != x2.dtype or y2.stride(1) != 1:
            raise ValueError("rmsnorm output must match the input's shape and dtype")
    if rstd_out is not None and (rstd_out.dtype != torch.float32 or rstd_out.numel() < x2.shape[0]):
        raise ValueError("rstd_out must be float32 with one entry per row")
    a = L.TrnRmsArgs(x2.data_ptr(), _ptr(y2), _ptr(gamma), _ptr(rstd_out), x2.shape[0], x2.shape[1],
                     x2.stride(0), y2.stride(0) if y2 is not None else x2.shape[1], float(eps), _dtype_code(x2))
    L.check(L.load().trinity_rmsnorm(C.byref(a), _stream()))
    return out


def qkv_project(x: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, *,
                q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                B: int, M: int, P: int, Hq: int, Hkv: int, D: int,
                row_scale: Optional[torch.Tensor] = None, qk_norm: bool = False, qk_eps: float = 0.0,
                gamma_q: Optional[torch.Tensor] = None, gamma_k: Optional[torch.Tensor] = None) -> None:
    """q, k, v = x @ wq, x @ wk, x @ wv with fused row scale / per-head norm; k, v land at rows
    [P, P+M) of the caches.  ``q``, ``k_cache``, ``v_cache`` are (b, s, h, d) views (see as_bshd)."""
    _need_cuda(x, wq, wk, wv, q, k_cache, v_cache, row_scale, gamma_q, gamma_k)
    N = x.shape[-1]
    if not (x.is_contiguous() and wq.is_contiguous() and wk.is_contiguous() and wv.is_contiguous()):
        raise ValueError("x and the weights must be contiguous")
    if wq.shape != (N, Hq * D) or wk.shape != (N, Hkv * D) or wv.shape != (N, Hkv * D):
        raise ValueError("weight shapes must be [N, heads*D] (used as x @ w)")
    if x.numel() != B * M * N:
        raise ValueError("x must hold B*M rows of N")
    a = L.TrnProjArgs(x.data_ptr(), wq.data_ptr(), wk.data_ptr(), wv.data_ptr(), _ptr(row_scale),
                      B, M, P, N, Hq, Hkv, D, _dtype_code(x), int(qk_norm), float(qk_eps),
                      _ptr(gamma_q), _ptr(gamma_k), _head_tensor(q), _head_tensor(k_cache), _head_tensor(v_cache))
    L.check(L.load().trinity_qkv_project(C.byref(a), _stream()))


def lora(x: torch.Tensor, w: torch.Tensor, a: torch.Tensor, b: torch.Tensor, o: Optional[torch.Tensor] = None,
         d: Optional[torch.Tensor] = None) -> torch.Tensor:
    """o = x @ w + (x @ a) @ b (lora_benchmark.py:41-64).  x [M, N], w [N, P], a [N, R], b [R, P]; ``d`` [M, R] receives
    x @ a (allocated when not given: pass it when the call is to be captured in a CUDA graph)."""
    _need_cuda(x, w, a, b, o, d)
    M, N = x.shape
    P, R = w.shape[1], a.shape[1]
    if w.shape != (N, P) or a.shape != (N, R) or b.shape != (R, P):
        raise ValueError("lora: expected w [N, P], a [N, R], b [R, P]")
    o = torch.empty(M, P, dtype=x.dtype, device=x.device) if o is None else o
    d = torch.empty(M, R, dtype=x.dtype, device=x.device) if d is None else d
    for t in (x, w, a, b, o, d):
        if not t.is_contiguous() or t.dtype != x.dtype:
            raise ValueError("lora: tensors must be contiguous and of one 16-bit dtype")
    args = L.TrnLoraArgs(x.data_ptr(), w.data_ptr(), a.data_ptr(), b.data_ptr(), o.data_ptr(), d.data_ptr(),
                         M, N, P, R, _dtype_code(x))
    L.check(L.load().trinity_lora(C.byref(args), _stream()))
    return o


def gmlp(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, o: Optional[torch.Tensor] = None,
         gate: str = "silu") -> torch.Tensor:
    """o = gate(x @ w1) * (x @ w2) (gmlp_benchmark.py:53-74); gate "silu" = c * sigmoid(c), "sigmoid" = sigmoid(c).
    x [M, K], w1 / w2 [K, N]; one kernel, fp32 accumulation, o rounded once."""
    _need_cuda(x, w1, w2, o)
    M, K = x.shape
    N = w1.shape[1]
    if w1.shape != (K, N) or w2.shape != (K, N):
        raise ValueError("gmlp: expected w1, w2 [K, N]")
    o = torch.empty(M, N, dtype=x.dtype, device=x.device) if o is None else o
    for t in (x, w1, w2, o):
        if not t.is_contiguous() or t.dtype != x.dtype:
            raise ValueError("gmlp: tensors must be contiguous and of one 16-bit dtype")
    if o.shape != (M, N):
        raise ValueError("gmlp: o must be [M, N]")
    code = {"silu": L.TRN_GATE_SILU, "sigmoid": L.TRN_GATE_SIGMOID}[gate]
    args = L.TrnGmlpArgs(x.data_ptr(), w1.data_ptr(), w2.data_ptr(), o.data_ptr(), M, K, N, _dtype_code(x), code)
    L.check(L.load().trinity_gmlp(C.byref(args), _stream()))
    return o


def _noise_fields(noise: Optional[torch.Tensor]):
    """noise is a (b, h, i, j) view with contiguous j."""
    if noise is None:
        return None, 0, 0, 0
    if noise.dim() != 4 or noise.stride(3) != 1:
        raise ValueError("noise must be a 4-D (b, h, query, key) view with contiguous keys")
    return noise.data_ptr(), noise.stride(0), noise.stride(1), noise.stride(2)


def attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, o: Optional[torch.Tensor], *,
              P: int, causal: bool, scale: float, lse: Optional[torch.Tensor] = None,
              noise_mode: int = L.TRN_NOISE_NONE, tau: float = 1.0, noise: Optional[torch.Tensor] = None,
              seed: int = 0, single_p: bool = False, workspace: Optional[torch.Tensor] = None,
              lse_pert: Optional[torch.Tensor] = None, scores: Optional[torch.Tensor] = None) -> None:
    """o = softmax(scale * q k^T [causal]) v over keys [0, P+M).  All tensors are (b, s, h, d) views.
    ``workspace`` (a uint8 CUDA tensor of attention_workspace_bytes(...) bytes) lets small launches
    split the key range over more CTAs.  With noise and ``lse_pert`` ([B, Hq, M] fp32) one pass gives o, lse
    and the perturbed scores' lse; ``scores`` ([B, Hq, M, pitch] fp32, pitch a multiple of 32) receives every
    score in the log2 domain for attn_colstats(scores=...)."""
    _need_cuda(q, k_cache, v_cache, o, lse, noise, workspace, lse_pert, scores)
    B, M, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    if k_cache.shape[1] < P + M or v_cache.shape[1] < P + M:
        raise ValueError("caches must hold P+M positions")
    nptr, nb, nh, ni = _noise_fields(noise)
    a = L.TrnAttnArgs(_head_tensor(q), _head_tensor(k_cache), _head_tensor(v_cache), _head_tensor(o), _ptr(lse),
                      B, M, P, Hq, Hkv, D, _dtype_code(q), int(causal), float(scale), noise_mode, float(tau),
                      nptr, nb, nh, ni, seed, int(single_p), _ptr(workspace),
                      0 if workspace is None else workspace.numel() * workspace.element_size())
    a.lse_pert = _ptr(lse_pert)
    if scores is not None:
        if scores.dtype != torch.float32 or scores.dim() != 4 or not scores.is_contiguous():
            raise ValueError("scores must be a contiguous float32 [B, Hq, M, pitch] tensor")
        a.scores, a.score_pitch = scores.data_ptr(), scores.shape[3]
    L.check(L.load().trinity_attention(C.byref(a), _stream()))


def attention_workspace_bytes(B: int, M: int, P: int, Hq: int, Hkv: int, D: int) -> int:
    """Scratch with which trinity_attention would split the key range for this shape (0: it would not)."""
    a = L.TrnAttnArgs()
    a.B, a.M, a.P, a.Hq, a.Hkv, a.D = B, M, P, Hq, Hkv, D
    return int(L.load().trinity_attention_workspace(C.byref(a)))


def attn_colstats(q: torch.Tensor, k_cache: torch.Tensor, lse: torch.Tensor, sum_p: torch.Tensor,
                  sum_p2: Optional[torch.Tensor] = None, *, P: int, causal: bool, scale: float,
                  noise_mode: int = L.TRN_NOISE_NONE, tau: float = 1.0, noise: Optional[torch.Tensor] = None,
                  seed: int = 0, scores: Optional[torch.Tensor] = None) -> None:
    """Per-key sums over queries of the attention probabilities (and of their squares).  With ``scores`` (kept by
    attention(scores=...)) they are summed from memory instead of recomputing q k^T."""
    _need_cuda(q, k_cache, lse, sum_p, sum_p2, noise, scores)
    B, M, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    nptr, nb, nh, ni = _noise_fields(noise)
    a = L.TrnColStatsArgs(_head_tensor(q), _head_tensor(k_cache), lse.data_ptr(), sum_p.data_ptr(), _ptr(sum_p2),
                          B, M, P, Hq, Hkv, D, _dtype_code(q), int(sum_p.dtype == torch.float32), int(causal),
                          float(scale), noise_mode, float(tau), nptr, nb, nh, ni, seed)
    if scores is not None:
        a.scores, a.score_pitch = scores.data_ptr(), scores.shape[3]
    L.check(L.load().trinity_attn_colstats(C.byref(a), _stream()))


def topk_keys(scores: torch.Tensor, k: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Indices of the k largest entries of each row of ``scores`` ([..., n] fp32), descending, ties
    to the lower index."""
    _need_cuda(scores, out)
    if scores.dtype != torch.float32 or scores.stride(-1) != 1:
        raise ValueError("scores must be float32 with a contiguous last dim")
    s2 = scores.reshape(-1, scores.shape[-1])
    if out is None:
        out = torch.empty(*scores.shape[:-1], k, dtype=torch.int32, device=scores.device)
    a = L.TrnTopkArgs(s2.data_ptr(), out.data_ptr(), s2.shape[0], s2.shape[1], k, s2.stride(0))
    L.check(L.load().trinity_topk(C.byref(a), _stream()))
    return out


class BlockPlan:
    """Arguments of one attention block bound once (pointers, strides, workspace), launched many times.

    Construction validates shapes and allocates the workspace through torch — do it before CUDA-graph
    capture.  ``run()`` only fills nothing and launches: it is what gets captured / replayed.
    """

    def __init__(self, variant: str, *, B: int, M: int, P: int, Hq: int, Hkv: int, D: int,
                 q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, o: torch.Tensor,
                 x: Optional[torch.Tensor] = None, wq: Optional[torch.Tensor] = None,
                 wk: Optional[torch.Tensor] = None, wv: Optional[torch.Tensor] = None,
                 causal: bool = False, scale: float = 1.0,
                 pre_eps: float = 0.0, pre_gamma: Optional[torch.Tensor] = None,
                 qk_eps: float = 0.0, gamma_q: Optional[torch.Tensor] = None,
                 gamma_k: Optional[torch.Tensor] = None,
                 noise_mode: int = L.TRN_NOISE_NONE, tau: float = 1.0, noise: Optional[torch.Tensor] = None,
                 seed: int = 0, sum_p: Optional[torch.Tensor] = None, sum_p2: Optional[torch.Tensor] = None,
                 single_p: bool = False, x_norm: Optional[torch.Tensor] = None, keep_scores: int = 0,
                 noise_heads: int = 0, noise_bh0: int = 0):
        _need_cuda(q, k_cache, v_cache, o, x, wq, wk, wv, pre_gamma, gamma_q, gamma_k, noise, sum_p, sum_p2, x_norm)
        self.variant = variant
        skip = x is None
        N = 0 if skip else x.shape[-1]
        a = L.TrnBlockArgs()
        a.variant = L.VARIANTS[variant]
        a.dtype = _dtype_code(q)
        a.B, a.M, a.P, a.N, a.Hq, a.Hkv, a.D = B, M, P, N, Hq, Hkv, D
        a.skip_projection = int(skip)
        self._keep = [q, k_cache, v_cache, o, x, wq, wk, wv, pre_gamma, gamma_q, gamma_k, noise, sum_p, sum_p2]
        if not skip:
            if not (x.is_contiguous() and wq.is_contiguous() and wk.is_contiguous() and wv.is_contiguous()):
                raise ValueError("x and the weights must be contiguous")
            if wq.shape != (N, Hq * D) or wk.shape != (N, Hkv * D) or wv.shape != (N, Hkv * D):
                raise ValueError("weight shapes must be [N, heads*D] (used as x @ w)")
            a.x, a.wq, a.wk, a.wv = x.data_ptr(), wq.data_ptr(), wk.data_ptr(), wv.data_ptr()
        a.pre_eps = float(pre_eps)
        a.pre_gamma = _ptr(pre_gamma)
        if x_norm is not None and not skip:
            # the caller's own X_norm tensor: PreNorm runs as normalise-then-project and leaves X_norm there
            if variant != "prenorm" or x_norm.shape != x.shape or x_norm.dtype != x.dtype or not x_norm.is_contiguous():
                raise ValueError("x_norm must be a contiguous tensor like x, and only PreNorm takes one")
            self._x_norm = x_norm
            a.x_norm = x_norm.data_ptr()
        elif pre_gamma is not None and not skip:
            self._x_norm = torch.empty_like(x)
            a.x_norm = self._x_norm.data_ptr()
        a.qk_eps = float(qk_eps)
        a.gamma_q, a.gamma_k = _ptr(gamma_q), _ptr(gamma_k)
        a.q, a.k_cache, a.v_cache, a.o = (_head_tensor(q), _head_tensor(k_cache), _head_tensor(v_cache),
                                          _head_tensor(o))
        a.causal, a.scale = int(causal), float(scale)
        a.noise_mode, a.tau = int(noise_mode), float(tau)
        a.noise, a.noise_stride_b, a.noise_stride_h, a.noise_stride_i = _noise_fields(noise)
        a.seed = seed
        a.sum_p, a.sum_p2 = _ptr(sum_p), _ptr(sum_p2)
        a.stats_fp32 = int(sum_p is not None and sum_p.dtype == torch.float32)
        a.single_p = int(single_p)
        # KeyFormer / RoCo statistics: 0 = by size, 1 = from scores kept in the workspace, -1 = second q k^T pass
        a.keep_scores = int(keep_scores)
        # generated noise of a slice of a larger problem: the whole problem's head count and the slice's first (b, h)
        a.noise_heads, a.noise_bh0 = int(noise_heads), int(noise_bh0)
        lib = L.load()
        nbytes = lib.trinity_attn_block_workspace(C.byref(a))
        self._ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=q.device)
        a.workspace, a.workspace_bytes = self._ws.data_ptr(), self._ws.numel()
        self.args = a
        self._lib = lib

    def run(self) -> None:
        L.check(self._lib.trinity_attn_block(C.byref(self.args), _stream()))

    def run_host(self, x_host: torch.Tensor, o_host: torch.Tensor, sum_p_host: Optional[torch.Tensor] = None,
                 sum_p2_host: Optional[torch.Tensor] = None) -> None:
        """The block with HOST activations (trinity_attn_block_host): x_host -> the plan's device x, the block,
        o (and the statistics) -> host.  Pinned buffers let the copies of different batch items overlap
        with the kernels.  Returns after the stream has drained."""
        for t in (x_host, o_host, sum_p_host, sum_p2_host):
            if t is not None and (t.is_cuda or not t.is_contiguous()):
                raise ValueError("run_host needs contiguous host tensors")
        h = L.TrnBlockHostArgs()
        C.memmove(C.byref(h.dev), C.byref(self.args), C.sizeof(L.TrnBlockArgs))
        h.x_host, h.o_host = x_host.data_ptr(), o_host.data_ptr()
        h.x_bytes = x_host.numel() * x_host.element_size()
        h.o_bytes = o_host.numel() * o_host.element_size()
        h.sum_p_host, h.sum_p2_host = _ptr(sum_p_host), _ptr(sum_p2_host)
        h.stats_bytes = 0 if sum_p_host is None else sum_p_host.numel() * sum_p_host.element_size()
        L.check(self._lib.trinity_attn_block_host(C.byref(h), _stream()))


def convert(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """fp32 -> bf16/fp16 (rounding) or bf16/fp16 -> fp32 (widening) of contiguous tensors of equal numel."""
    _need_cuda(src, dst)
    if not (src.is_contiguous() and dst.is_contiguous()) or src.numel() != dst.numel():
        raise ValueError("convert needs contiguous tensors of equal size")
    if src.dtype == torch.float32 and dst.dtype in _DTYPES:
        code, to32 = _DTYPES[dst.dtype], 0
    elif dst.dtype == torch.float32 and src.dtype in _DTYPES:
        code, to32 = _DTYPES[src.dtype], 1
    else:
        raise TypeError(f"convert: unsupported pair {src.dtype} -> {dst.dtype}")
    L.check(L.load().trinity_convert(src.data_ptr(), dst.data_ptr(), src.numel(), code, to32, _stream()))
    return dst


def default_scale(D: int) -> float:
    return 1.0 / math.sqrt(D)
