"""Multi-GPU partitioning of the MSA hot path by (batch, KV-head group).

Every quantity of the path is independent across batch elements and across KV-head groups: KV head
g is touched only by main heads g*Hq/Hkv.., by proxy heads g*Hp/Hkv.. and - when Hpkv is a multiple
of the number of groups a rank boundary cuts - by its own proxy-K head(s)
(index maps in the reference: flash_msa/msa_backward_cutedsl.py:328-329).  So a rank simply calls
the single-GPU functions on head-sliced views; there is no collective on the kernel path.

The only cross-rank arithmetic is the normalisation of the KL term: the kernels divide proxy
gradients by the number of (batch, proxy head, position) rows OF THE CALL, so a rank that holds a
fraction f of those rows must scale the upstream gradient of its kl_loss by f
(`Shard.kl_weight`), and the global kl_loss is the kl_weight-weighted sum of the ranks' values.
If proxy-K heads are shared across a rank boundary (Hpkv smaller than the number of groups cut),
dk_proxy of the shared head must be summed over the ranks that hold it
(`needs_dk_proxy_allreduce`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List


@dataclass(frozen=True)
class Shard:
    """A rectangular piece of the (batch, KV head) grid: batches [b0,b1) x KV heads [kv0,kv1)."""
    b0: int
    b1: int
    kv0: int
    kv1: int

    @property
    def units(self) -> int:
        return (self.b1 - self.b0) * (self.kv1 - self.kv0)


def partition(batch: int, n_kv_heads: int, world: int) -> List[List[Shard]]:
    """Deal the batch*Hkv units, flattened batch-major, in contiguous equal ranges to `world`
    ranks.  Returns, per rank, a list of rectangular shards (one in the common cases)."""
    units = batch * n_kv_heads
    if world < 1 or units % world != 0:
        raise ValueError(f"{units} (batch, KV head) units cannot be dealt evenly to {world} ranks")
    per = units // world
    out: List[List[Shard]] = []
    for r in range(world):
        lo, hi = r * per, (r + 1) * per
        pieces: List[Shard] = []
        u = lo
        while u < hi:
            b, kv = divmod(u, n_kv_heads)
            if kv == 0 and hi - u >= n_kv_heads:            # whole batches
                nb = (hi - u) // n_kv_heads
                pieces.append(Shard(b, b + nb, 0, n_kv_heads))
                u += nb * n_kv_heads
            else:                                           # part of one batch element
                end = min(n_kv_heads, kv + (hi - u))
                pieces.append(Shard(b, b + 1, kv, end))
                u += end - kv
        out.append(pieces)
    return out


def head_ranges(shard: Shard, hq: int, hkv: int, hp: int, hpkv: int):
    """Head slices (main, kv, proxy, proxy-kv) of a shard as (start, stop) pairs."""
    g, ppk = hq // hkv, hp // hkv
    pg = hp // hpkv
    p0, p1 = shard.kv0 * ppk, shard.kv1 * ppk
    kp0, kp1 = p0 // pg, (p1 - 1) // pg + 1
    # The kernels recompute pg from the shard's own head counts and map local proxy head i to local proxy-K
    # head i // pg_local.  That equals the global map only if the shard lies inside one proxy-K group
    # (one local proxy-K head) or both of its ends fall on group boundaries.
    if (kp1 - kp0) > 1 and (p0 % pg != 0 or p1 % pg != 0):
        raise ValueError("shard boundary cuts a proxy-K head group unevenly")
    return (shard.kv0 * g, shard.kv1 * g), (shard.kv0, shard.kv1), (p0, p1), (kp0, kp1)


def needs_dk_proxy_allreduce(hkv: int, hp: int, hpkv: int, shards: List[List[Shard]]) -> bool:
    """True if some proxy-K head is read by more than one rank (its gradient must be summed)."""
    owners = {}
    ppk, pg = hp // hkv, hp // hpkv
    for r, pieces in enumerate(shards):
        for s in pieces:
            for b in range(s.b0, s.b1):
                for p in range(s.kv0 * ppk, s.kv1 * ppk):
                    owners.setdefault((b, p // pg), set()).add(r)
    return any(len(v) > 1 for v in owners.values())


def allreduce_dk_proxy(dk_proxy_local, shard: Shard, batch: int, hq: int, hkv: int, hp: int, hpkv: int, group=None):
    """Sums dk_proxy over the ranks that share a proxy-K head (needed when `needs_dk_proxy_allreduce`, e.g. the
    reference's default Hpkv = 1 cut by KV group): every rank places its local gradient [b, kp, S, D] into a
    zero tensor of the global shape [batch, Hpkv, S, D], one all-reduce(SUM) runs over `group`, and the rank
    reads its own slice back.  Returns a tensor shaped like `dk_proxy_local`.  This is the only collective the
    path can need; it is off the kernel path (after the backward) and all BASELINE configurations avoid it."""
    import torch
    import torch.distributed as dist
    _, _, _, (kp0, kp1) = head_ranges(shard, hq, hkv, hp, hpkv)
    s, d = dk_proxy_local.shape[2], dk_proxy_local.shape[3]
    full = torch.zeros(batch, hpkv, s, d, dtype=torch.float32, device=dk_proxy_local.device)
    full[shard.b0:shard.b1, kp0:kp1] = dk_proxy_local.float()
    dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group)
    return full[shard.b0:shard.b1, kp0:kp1].to(dk_proxy_local.dtype)


def slice_inputs(shard: Shard, q_proxy, k_proxy, q, k, v):
    """Views of the (B,H,S,D) inputs that belong to a shard.  When the shard's proxy heads do not
    start at a proxy-K group boundary the proxy-K slice still begins at the right head because the
    kernels index it as (local proxy head // pg)."""
    hq, hkv, hp, hpkv = q.shape[1], k.shape[1], q_proxy.shape[1], k_proxy.shape[1]
    (h0, h1), (kv0, kv1), (p0, p1), (kp0, kp1) = head_ranges(shard, hq, hkv, hp, hpkv)
    bs = slice(shard.b0, shard.b1)
    return (q_proxy[bs, p0:p1], k_proxy[bs, kp0:kp1], q[bs, h0:h1], k[bs, kv0:kv1], v[bs, kv0:kv1])


def kl_weight(shard: Shard, batch: int, hkv: int) -> float:
    """Fraction of the global (batch, proxy head, position) rows held by the shard."""
    return shard.units / float(batch * hkv)


def shard_workload(cfg: dict, rank: int, world: int) -> dict:
    """Local problem sizes of `rank` for a benchmark configuration given as a dict with keys
    b, s, hq, hkv, hp, hpkv, kb (first shard of the rank; benchmark shapes give exactly one)."""
    pieces = partition(cfg["b"], cfg["hkv"], world)[rank]
    if len(pieces) != 1:
        raise ValueError("benchmark shapes must give one rectangular shard per rank")
    s = pieces[0]
    (h0, h1), (kv0, kv1), (p0, p1), (kp0, kp1) = head_ranges(s, cfg["hq"], cfg["hkv"], cfg["hp"], cfg["hpkv"])
    out = dict(cfg)
    out.update(b=s.b1 - s.b0, hq=h1 - h0, hkv=kv1 - kv0, hp=p1 - p0, hpkv=kp1 - kp0)
    return out
