"""Sharding of the attention block across the GPUs of one node: one process per GPU, no collective
on the data path.

Every (batch, kv-head group) pair is independent — a group is one KV head with the Hq/Hkv query heads
that read it — so the work units are flattened as (b, g) and dealt out in contiguous ranges.  A rank
needs only: the X rows of its batches, the WQ columns of its query heads, the WK/WV columns and the
cache heads of its KV heads.  Per-key statistics and top-k are per (batch, head) and shard the same
way.  The only communication is an optional all_gather of the outputs for validation, outside any
timed region (the reference itself is single-GPU: vanilla_llama_benchmark.py:119).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Unit:
    b: int      # batch index
    g: int      # kv head index (the group's query heads are [g*group, (g+1)*group))


def partition_units(B: int, Hkv: int, world_size: int) -> List[List[Unit]]:
    """Contiguous, balanced ranges of the B*Hkv units; the first (n % world) ranks get one more."""
    units = [Unit(b, g) for b in range(B) for g in range(Hkv)]
    n = len(units)
    base, extra = divmod(n, world_size)
    out, pos = [], 0
    for r in range(world_size):
        cnt = base + (1 if r < extra else 0)
        out.append(units[pos:pos + cnt])
        pos += cnt
    return out


def partition_query_heads(B: int, Hq: int, world_size: int) -> List[List[Tuple[int, int]]]:
    """MQA (one shared KV head): units are (b, query head); the KV head is replicated to every rank
    that owns one of its query heads."""
    units = [(b, h) for b in range(B) for h in range(Hq)]
    base, extra = divmod(len(units), world_size)
    out, pos = [], 0
    for r in range(world_size):
        cnt = base + (1 if r < extra else 0)
        out.append(units[pos:pos + cnt])
        pos += cnt
    return out


def balance(parts: Sequence[Sequence]) -> float:
    """Load balance of a partition: mean / max units per rank (1.0 = perfect)."""
    sizes = [len(p) for p in parts]
    return (sum(sizes) / len(sizes)) / max(sizes) if max(sizes) else 1.0


@dataclass
class LocalSlice:
    """What one rank holds for a contiguous run of units inside one batch."""
    b: int
    h0: int     # first query head
    h1: int     # one past the last query head
    kv0: int    # first kv head
    kv1: int


def local_slices(units: Sequence[Unit], group: int) -> List[LocalSlice]:
    """Groups a rank's units by batch into head ranges (units are contiguous, so one range per batch)."""
    out: List[LocalSlice] = []
    for u in units:
        if out and out[-1].b == u.b and out[-1].kv1 == u.g:
            last = out[-1]
            out[-1] = LocalSlice(last.b, last.h0, (u.g + 1) * group, last.kv0, u.g + 1)
        else:
            out.append(LocalSlice(u.b, u.g * group, (u.g + 1) * group, u.g, u.g + 1))
    return out


def query_head_slices(units: Sequence[Tuple[int, int]]) -> List[LocalSlice]:
    """MQA: a rank's contiguous (b, query head) units grouped by batch; every slice reads the one shared KV head."""
    out: List[LocalSlice] = []
    for b, h in units:
        if out and out[-1].b == b and out[-1].h1 == h:
            out[-1] = LocalSlice(b, out[-1].h0, h + 1, 0, 1)
        else:
            out.append(LocalSlice(b, h, h + 1, 0, 1))
    return out


def rank_slices(B: int, Hq: int, Hkv: int, rank: int, world_size: int) -> List[LocalSlice]:
    """What rank `rank` computes: (batch, kv group) units for GQA / MHA; (batch, query head) units when all query
    heads share ONE KV head (MQA), where kv groups alone could not occupy more than B ranks."""
    if Hkv == 1 and Hq > 1:
        return query_head_slices(partition_query_heads(B, Hq, world_size)[rank])
    return local_slices(partition_units(B, Hkv, world_size)[rank], Hq // Hkv)


@dataclass
class Launch:
    """One call of the block on a rank: batch items [b0, b0 + nb) with query heads [h0, h1) and kv heads [kv0, kv1).
    The rank binds only the X rows of those batch items, the WQ columns [h0*D, h1*D), the WK / WV columns
    [kv0*D, kv1*D) and the cache heads [kv0, kv1)."""
    b0: int
    nb: int
    h0: int
    h1: int
    kv0: int
    kv1: int


def rank_launches(B: int, Hq: int, Hkv: int, rank: int, world_size: int) -> List[Launch]:
    """rank_slices with consecutive batch items of the same head range merged into one launch."""
    out: List[Launch] = []
    for s in rank_slices(B, Hq, Hkv, rank, world_size):
        last = out[-1] if out else None
        if last and (last.h0, last.h1, last.kv0, last.kv1) == (s.h0, s.h1, s.kv0, s.kv1) and last.b0 + last.nb == s.b:
            out[-1] = Launch(last.b0, last.nb + 1, s.h0, s.h1, s.kv0, s.kv1)
        else:
            out.append(Launch(s.b, 1, s.h0, s.h1, s.kv0, s.kv1))
    return out


def launch_flop_share(launches: Sequence[Launch], B: int, Hq: int) -> float:
    """Fraction of the whole problem's (batch, query head) pairs in `launches`."""
    return sum(l.nb * (l.h1 - l.h0) for l in launches) / float(B * Hq)


def run_sharded(compute: Callable[[LocalSlice], Dict[str, torch.Tensor]], B: int, Hq: int, Hkv: int,
                rank: int, world_size: int) -> List[Tuple[LocalSlice, Dict[str, torch.Tensor]]]:
    """Runs `compute` on this rank's slices.  `compute` receives the slice and returns named outputs
    whose dim 0 is the slice's query heads (e.g. out [h1-h0, M, D], sum_p [h1-h0, L])."""
    return [(s, compute(s)) for s in rank_slices(B, Hq, Hkv, rank, world_size)]


def gather_outputs(local: List[Tuple[LocalSlice, Dict[str, torch.Tensor]]], B: int, Hq: int,
                   group: Optional[dist.ProcessGroup] = None) -> Dict[str, torch.Tensor]:
    """Validation only: all ranks exchange their slices (all_gather_object on small tensors, or
    all_gather on padded buffers) and assemble full [B, Hq, ...] outputs on every rank."""
    world = dist.get_world_size(group)
    payload = [(s.b, s.h0, s.h1, {k: v.detach().cpu() for k, v in outs.items()}) for s, outs in local]
    gathered: List = [None] * world
    dist.all_gather_object(gathered, payload, group=group)
    full: Dict[str, torch.Tensor] = {}
    for part in gathered:
        for b, h0, h1, outs in part:
            for name, t in outs.items():
                if name not in full:
                    full[name] = torch.zeros((B, Hq) + tuple(t.shape[1:]), dtype=t.dtype)
                full[name][b, h0:h1] = t
    return full
