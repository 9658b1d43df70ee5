"""Two GPUs, one process each, NCCL: the (batch, kv-group) units of a RoCo block are split over the ranks
(triton_b200/shard.py), each rank runs the CUDA block on its own slices only — no kernel touches a peer's
memory, no collective on the data path — and the validation gather must reproduce the single-GPU result.
Skipped where fewer than two GPUs are visible."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_q):
    import datetime
    import traceback
    import torch.distributed as dist
    from triton_b200 import _lib as L
    from triton_b200 import ops, shard
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))
    try:
        torch.manual_seed(0)                                    # identical inputs on every rank
        B, M, Hq, Hkv, D = 3, 300, 8, 4, 64
        dt = torch.bfloat16
        Q = torch.randn(B, M, Hq, D).to(dt)
        K = torch.randn(B, Hkv, M, D).to(dt)
        V = torch.randn(B, Hkv, M, D).to(dt)
        grp = Hq // Hkv

        def compute(s):
            q = Q[s.b:s.b + 1, :, s.h0:s.h1].contiguous().cuda()
            k = K[s.b:s.b + 1, s.kv0:s.kv1].contiguous().cuda()
            v = V[s.b:s.b + 1, s.kv0:s.kv1].contiguous().cuda()
            nh = s.h1 - s.h0
            o = torch.zeros(1, M, nh, D, device="cuda", dtype=dt)
            sp = torch.zeros(1, nh, M, device="cuda")
            sp2 = torch.zeros(1, nh, M, device="cuda")
            plan = ops.BlockPlan("roco", B=1, M=M, P=0, Hq=nh, Hkv=s.kv1 - s.kv0, D=D, q=q, k_cache=ops.as_bshd(k, "bhsd"),
                                 v_cache=ops.as_bshd(v, "bhsd"), o=o, causal=True, scale=D ** -0.5, sum_p=sp, sum_p2=sp2)
            plan.run()
            torch.cuda.synchronize()
            assert L.kernel_status() == 0
            return {"out": o[0].permute(1, 0, 2).contiguous(), "sum_p": sp[0], "sum_p2": sp2[0]}

        local = shard.run_sharded(compute, B, Hq, Hkv, rank, world)
        full = shard.gather_outputs(local, B, Hq)
        ok = True
        if rank == 0:
            q, k, v = Q.cuda(), K.cuda(), V.cuda()
            o = torch.zeros(B, M, Hq, D, device="cuda", dtype=dt)
            sp = torch.zeros(B, Hq, M, device="cuda")
            sp2 = torch.zeros(B, Hq, M, device="cuda")
            ops.BlockPlan("roco", B=B, M=M, P=0, Hq=Hq, Hkv=Hkv, D=D, q=q, k_cache=ops.as_bshd(k, "bhsd"),
                          v_cache=ops.as_bshd(v, "bhsd"), o=o, causal=True, scale=D ** -0.5, sum_p=sp, sum_p2=sp2).run()
            torch.cuda.synchronize()
            # same kernels on the same numbers: bitwise equal
            ok = (torch.equal(full["out"], o.permute(0, 2, 1, 3).cpu()) and torch.equal(full["sum_p"], sp.cpu())
                  and torch.equal(full["sum_p2"], sp2.cpu()))
        out_q.put((rank, len(local), bool(ok), ""))
    except Exception:                                            # reported, never left hanging
        out_q.put((rank, 0, False, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_shard_matches_single_gpu():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        got = sorted(q.get(timeout=240) for _ in procs)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.terminate()
    assert all(g[2] for g in got), [g[3] for g in got]
