"""trinity_attn_block_static — the block for callers that cannot hand over or allocate a workspace (a plugin
that only receives the operator's inputs and outputs, a serving loop that bans cudaMalloc once warm): its
scratch is a fixed array inside the library.  The results must equal those of trinity_attn_block, which
gets its scratch from the caller, on two calls in a row that share the array (the second on other inputs
and another shape, so stale contents of the first are in it).  Collected last on purpose."""
import ctypes as C

import pytest
import torch

from triton_b200 import _lib as L
from triton_b200 import ops

pytestmark = pytest.mark.gpu


def _plan(variant, seed, B, M, P, N, Hq, Hkv, D, dt):
    torch.manual_seed(seed)
    dev = "cuda"
    x = torch.randn(B * M, N, device=dev).to(dt)
    wq, wk, wv = ((torch.randn(N, h * D, device=dev) / N ** 0.5).to(dt) for h in (Hq, Hkv, Hkv))
    kc = torch.randn(B, Hkv, P + M, D, device=dev).to(dt)
    vc = torch.randn(B, Hkv, P + M, D, device=dev).to(dt)
    q = torch.zeros(B, M, Hq, D, device=dev, dtype=dt)
    o = torch.zeros(B, M, Hq, D, device=dev, dtype=dt)
    sp = torch.zeros(B, Hq, P + M, device=dev)
    sp2 = torch.zeros(B, Hq, P + M, device=dev) if variant == "roco" else None
    plan = ops.BlockPlan(variant, B=B, M=M, P=P, Hq=Hq, Hkv=Hkv, D=D, q=ops.as_bshd(q, "bshd"),
                         k_cache=ops.as_bshd(kc, "bhsd"), v_cache=ops.as_bshd(vc, "bhsd"), o=ops.as_bshd(o, "bshd"),
                         x=x, wq=wq, wk=wk, wv=wv, causal=True, scale=D ** -0.5, pre_eps=1e-5,
                         noise_mode=L.TRN_NOISE_GUMBEL if variant == "keyformer" else 0, tau=1.5, seed=3,
                         sum_p=sp, sum_p2=sp2)
    return plan, dict(o=o, q=q, kc=kc, vc=vc, sp=sp, sp2=sp2)


def _snapshot(t):
    return {k: v.clone() for k, v in t.items() if v is not None}


@pytest.mark.parametrize("first,second", [
    (("roco", 1, 2, 200, 24, 256, 4, 2, 64, torch.bfloat16), ("keyformer", 2, 1, 130, 0, 512, 8, 8, 128, torch.float16)),
])
def test_static_scratch_block_matches_workspace_block_twice(first, second):
    lib = L.load()
    stream = torch.cuda.current_stream().cuda_stream
    for case in (first, second):          # two calls in a row on the shared array
        plan, t = _plan(*case)
        plan.run()                         # existing entry point, caller-owned workspace
        torch.cuda.synchronize()
        want = _snapshot(t)
        for v in t.values():
            if v is not None and v is not t["kc"] and v is not t["vc"]:
                v.zero_()
        L.check(lib.trinity_attn_block_static(C.byref(plan.args), stream))
        torch.cuda.synchronize()
        assert L.kernel_status() == 0
        for name, w in want.items():
            got = t[name]
            # same kernels on the same inputs: the tolerance of the parity tests is met with room to spare
            assert (got.float() - w.float()).abs().max().item() <= 2e-2, name
            assert torch.equal(got, w), f"{name}: static-scratch result differs from the workspace result"


def test_static_scratch_call_allocates_nothing_and_uses_optional_areas_as_far_as_they_fit():
    """A KeyFormer problem whose required scratch is small but whose optional areas (split-KV partials, 16 MiB of
    kept scores) exceed the 8 MiB array: the call is accepted, runs the schedule that fits, allocates no device
    memory (free bytes of the device and torch's own counter unchanged across the call), and equals bit for bit
    trinity_attn_block given a caller workspace of exactly the array's size."""
    lib = L.load()
    stream = torch.cuda.current_stream().cuda_stream
    cap = lib.trinity_static_scratch_capacity()
    plan, t = _plan("keyformer", 5, 1, 512, 512, 256, 8, 2, 64, torch.bfloat16)
    assert lib.trinity_attn_block_workspace(C.byref(plan.args)) > cap          # total does not fit ...
    ws = torch.empty(cap, dtype=torch.uint8, device="cuda")                     # ... the required part does
    plan.args.workspace, plan.args.workspace_bytes = ws.data_ptr(), cap
    plan.run()
    torch.cuda.synchronize()
    want = _snapshot(t)
    full_plan, full_t = _plan("keyformer", 5, 1, 512, 512, 256, 8, 2, 64, torch.bfloat16)
    full_plan.run()                                                             # everything lent: kept scores
    L.check(lib.trinity_attn_block_static(C.byref(plan.args), stream))          # first static call on this shape
    torch.cuda.synchronize()
    for v in (t["o"], t["q"], t["sp"]):
        v.zero_()
    torch.cuda.synchronize()
    free0, alloc0, resv0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    L.check(lib.trinity_attn_block_static(C.byref(plan.args), stream))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0, "device memory was allocated or freed during the call"
    assert torch.cuda.memory_allocated() == alloc0 and torch.cuda.memory_reserved() == resv0
    assert L.kernel_status() == 0
    for name, w in want.items():
        assert torch.equal(t[name], w), f"{name}: differs from trinity_attn_block with a workspace of the array's size"
    # the other schedule (scores kept in memory) agrees within the statistics' tolerance
    assert (t["sp"] - full_t["sp"]).abs().max().item() <= 1e-3 * 32
    assert (t["o"].float() - full_t["o"].float()).abs().max().item() <= 2e-2


def test_static_scratch_rejects_problems_beyond_its_capacity():
    lib = L.load()
    cap = lib.trinity_static_scratch_capacity()
    assert cap == 8 << 20
    a = L.TrnBlockArgs()
    a.variant, a.B, a.M, a.P, a.Hq, a.Hkv, a.D = L.TRN_ROCO, 2, 8192, 0, 71, 1, 64     # RoCo Falcon: 9.4 MB of scratch
    assert lib.trinity_attn_block_workspace(C.byref(a)) > cap
    rc = lib.trinity_attn_block_static(C.byref(a), None)
    assert rc == -10
    with pytest.raises(L.TrinityError, match="built-in"):
        L.check(rc)
