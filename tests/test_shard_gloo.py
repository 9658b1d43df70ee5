"""Multi-GPU sharding logic on CPU ranks (gloo, world size 2): the (batch, kv-group) partition covers
every unit exactly once, each rank computes only its slices, and the validation gather reassembles the
full result.  The per-slice computation here is the CPU oracle; on GPUs it is the CUDA block."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from triton_b200 import shard


def test_partition_covers_all_units_once():
    for B, Hkv, W in ((1, 8, 8), (8, 8, 8), (4, 8, 3), (2, 1, 2), (3, 5, 4)):
        parts = shard.partition_units(B, Hkv, W)
        flat = [u for p in parts for u in p]
        assert len(flat) == B * Hkv and len(set(flat)) == B * Hkv
        assert max(map(len, parts)) - min(map(len, parts)) <= 1
    # falcon MQA: 4 x 71 query heads over 8 ranks -> 98.6 % balance
    q = shard.partition_query_heads(4, 71, 8)
    assert sum(map(len, q)) == 284 and abs(shard.balance(q) - 284 / (8 * 36)) < 1e-9
    assert shard.balance(shard.partition_units(8, 8, 8)) == 1.0


def test_local_slices_merge_contiguous_groups():
    units = shard.partition_units(2, 4, 3)[1]          # units 3,4,5 of 8 -> (0,3), (1,0), (1,1)
    sl = shard.local_slices(units, group=4)
    assert [(s.b, s.h0, s.h1, s.kv0, s.kv1) for s in sl] == [(0, 12, 16, 3, 4), (1, 0, 8, 0, 2)]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import attn_block_ref as O
        torch.manual_seed(0)                               # same inputs on every rank
        B, Hq, Hkv, M, D = 3, 8, 4, 12, 16
        Q, K, V = torch.randn(B, Hq, M, D), torch.randn(B, Hkv, M, D), torch.randn(B, Hkv, M, D)

        def compute(s):
            r = O.attend(Q[s.b:s.b + 1, s.h0:s.h1], K[s.b:s.b + 1, s.kv0:s.kv1], V[s.b:s.b + 1, s.kv0:s.kv1],
                         P=0, causal=True, scale=0.25, variant="roco")
            return {"out": r["out"][0], "sum_p": r["sum_p"][0]}

        local = shard.run_sharded(compute, B, Hq, Hkv, rank, world)
        n_units = sum((s.kv1 - s.kv0) for s, _ in local)
        full = shard.gather_outputs(local, B, Hq)
        want = O.attend(Q, K, V, P=0, causal=True, scale=0.25, variant="roco")
        ok = torch.allclose(full["out"], want["out"], atol=1e-6) and torch.allclose(full["sum_p"], want["sum_p"], atol=1e-6)
        q.put((rank, n_units, bool(ok)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_shard_and_gather():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [g[1] for g in got] == [6, 6]        # 12 units split evenly
    assert all(g[2] for g in got)


def test_rank_launches_cover_the_problem_once_for_gqa_and_mqa():
    """What the sharded benchmark binds per rank: batch items x query heads x kv heads, merged over consecutive batch
    items.  GQA / MHA units are (batch, kv group); with ONE shared kv head (MQA) they are (batch, query head), so that
    more than B ranks have work and the kv head is replicated."""
    for B, Hq, Hkv, W in ((8, 32, 8, 8), (8, 32, 8, 2), (8, 32, 8, 3), (4, 71, 1, 8), (2, 71, 1, 8), (1, 32, 8, 8), (4, 32, 8, 8)):
        seen = set()
        per_rank = []
        for r in range(W):
            ls = shard.rank_launches(B, Hq, Hkv, r, W)
            per_rank.append(sum(l.nb * (l.h1 - l.h0) for l in ls))
            for l in ls:
                grp = Hq // Hkv
                assert 0 <= l.kv0 < l.kv1 <= Hkv and (l.kv0, l.kv1) == (l.h0 // grp, (l.h1 - 1) // grp + 1)
                for b in range(l.b0, l.b0 + l.nb):
                    for h in range(l.h0, l.h1):
                        assert (b, h) not in seen
                        seen.add((b, h))
        assert len(seen) == B * Hq
        assert abs(sum(shard.launch_flop_share(shard.rank_launches(B, Hq, Hkv, r, W), B, Hq) for r in range(W)) - 1.0) < 1e-12
        unit = 1 if Hkv == 1 else Hq // Hkv
        assert max(per_rank) - min(per_rank) <= unit           # balanced to one unit
    # whole batch items merge into one launch; MQA splits a batch item's heads across ranks
    assert [(l.b0, l.nb, l.h0, l.h1) for l in shard.rank_launches(8, 32, 8, 1, 2)] == [(4, 4, 0, 32)]
    assert [(l.b0, l.nb, l.h0, l.h1, l.kv0, l.kv1) for l in shard.rank_launches(4, 71, 1, 1, 8)] == [(0, 1, 36, 71, 0, 1), (1, 1, 0, 1, 0, 1)]
