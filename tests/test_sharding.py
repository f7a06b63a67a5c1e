"""Host-side logic of the (batch, KV-head group) partition, including a world_size-2 gloo run in
which each rank evaluates only its shard (with the oracle standing in for the kernels) and the
gathered result equals the unsharded one - i.e. the path needs no data-path collective."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_msa_b200 import sharding as sh
from oracle import msa_oracle as O

SCALE = 128 ** -0.5


def test_partition_covers_every_unit_once():
    for b, hkv, world in [(1, 8, 8), (1, 8, 2), (2, 8, 4), (4, 2, 2), (8, 4, 8), (2, 8, 1), (3, 4, 6)]:
        seen = set()
        for pieces in sh.partition(b, hkv, world):
            assert sum(p.units for p in pieces) == b * hkv // world
            for p in pieces:
                for bb in range(p.b0, p.b1):
                    for kv in range(p.kv0, p.kv1):
                        assert (bb, kv) not in seen
                        seen.add((bb, kv))
        assert len(seen) == b * hkv
    with pytest.raises(ValueError):
        sh.partition(1, 8, 3)


def test_shard_workload_config5():
    cfg = dict(b=1, s=65536, hq=64, hkv=8, hp=16, hpkv=8, kb=32)
    loc = sh.shard_workload(cfg, 3, 8)
    assert (loc["b"], loc["hq"], loc["hkv"], loc["hp"], loc["hpkv"]) == (1, 8, 1, 2, 1)
    loc = sh.shard_workload(cfg, 1, 2)
    assert (loc["hq"], loc["hkv"], loc["hp"], loc["hpkv"]) == (32, 4, 8, 4)


def test_dk_proxy_allreduce_detection():
    assert not sh.needs_dk_proxy_allreduce(8, 16, 8, sh.partition(1, 8, 8))
    assert sh.needs_dk_proxy_allreduce(2, 4, 1, sh.partition(1, 2, 2))      # reference default Hpkv=1


def test_head_ranges_reject_shards_that_break_the_proxy_k_map():
    """A shard is usable only if the kernels' local map (local proxy head // local pg) equals the global one."""
    # starts on a proxy-K group boundary but ends inside one, spanning two proxy-K heads: rejected
    pieces = sh.partition(3, 8, 4)[0]
    assert (pieces[0].kv0, pieces[0].kv1) == (0, 6)
    with pytest.raises(ValueError):
        sh.head_ranges(pieces[0], 32, 8, 8, 2)
    # every accepted shard reproduces the global map
    for b, hq, hkv, hp, hpkv, world in [(1, 64, 8, 16, 8, 8), (1, 64, 8, 16, 8, 2), (2, 32, 8, 8, 2, 4), (1, 16, 2, 4, 1, 2),
                                        (2, 32, 8, 8, 8, 16), (1, 32, 8, 8, 2, 8), (3, 32, 8, 8, 2, 4), (1, 48, 4, 8, 4, 2)]:
        pg = hp // hpkv
        for pcs in sh.partition(b, hkv, world):
            for s in pcs:
                try:
                    _, _, (p0, p1), (kp0, kp1) = sh.head_ranges(s, hq, hkv, hp, hpkv)
                except ValueError:
                    continue
                assert (p1 - p0) % (kp1 - kp0) == 0
                pg_local = (p1 - p0) // (kp1 - kp0)
                for p in range(p0, p1):
                    assert (p - p0) // pg_local + kp0 == p // pg


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, cfg, result_file):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    qp, kp, q, k, v, do = O.make_inputs(cfg["b"], cfg["s"], cfg["hq"], cfg["hkv"], cfg["hp"], cfg["hpkv"], seed=11)
    (shard,) = sh.partition(cfg["b"], cfg["hkv"], world)[rank]
    lqp, lkp, lq, lk, lv = sh.slice_inputs(shard, qp, kp, q, k, v)
    (h0, h1), _, _, _ = sh.head_ranges(shard, cfg["hq"], cfg["hkv"], cfg["hp"], cfg["hpkv"])
    ldo = do.view(cfg["b"], cfg["s"], cfg["hq"], 128)[shard.b0:shard.b1, :, h0:h1].reshape(shard.b1 - shard.b0, cfg["s"], -1)
    w = sh.kl_weight(shard, cfg["b"], cfg["hkv"])
    r = O.sparse_forward_backward(lqp, lkp, lq, lk, lv, cfg["kb"] * 128, SCALE, ldo, grad_kl=w)
    # gather per-rank pieces (test-side only; the data path itself exchanges nothing)
    pieces = [None] * world
    dist.all_gather_object(pieces, {"shard": shard, "dq": r["dq"], "dv": r["dv"], "dqp": r["dq_proxy"],
                                    "dkp": r["dk_proxy"], "out": r["out"], "kl": float(r["kl"]) * w})
    if rank == 0:
        full = O.sparse_forward_backward(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, do, grad_kl=1.0)
        ok = True
        kl = 0.0
        for pc in pieces:
            s = pc["shard"]
            (h0, h1), (kv0, kv1), (p0, p1), (kp0, kp1) = sh.head_ranges(s, cfg["hq"], cfg["hkv"], cfg["hp"], cfg["hpkv"])
            bs = slice(s.b0, s.b1)
            ok &= torch.allclose(pc["dq"], full["dq"][bs, h0:h1], atol=1e-5)
            ok &= torch.allclose(pc["dv"], full["dv"][bs, kv0:kv1], atol=1e-5)
            ok &= torch.allclose(pc["dqp"], full["dq_proxy"][bs, p0:p1], atol=1e-9)
            ok &= torch.allclose(pc["dkp"], full["dk_proxy"][bs, kp0:kp1], atol=1e-9)
            ok &= torch.allclose(pc["out"].view(s.b1 - s.b0, cfg["s"], h1 - h0, 128),
                                 full["out"].view(cfg["b"], cfg["s"], cfg["hq"], 128)[bs, :, h0:h1], atol=1e-5)
            kl += pc["kl"]
        ok &= abs(kl - float(full["kl"])) < 1e-6
        with open(result_file, "w") as f:
            f.write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


def _worker_shared_kp(rank, world, port, cfg, result_file):
    """Ranks split the KV groups of a problem with ONE proxy-K head: dk_proxy needs the all-reduce."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    qp, kp, q, k, v, do = O.make_inputs(cfg["b"], cfg["s"], cfg["hq"], cfg["hkv"], cfg["hp"], cfg["hpkv"], seed=5)
    shards = sh.partition(cfg["b"], cfg["hkv"], world)
    assert sh.needs_dk_proxy_allreduce(cfg["hkv"], cfg["hp"], cfg["hpkv"], shards)
    (shard,) = shards[rank]
    lqp, lkp, lq, lk, lv = sh.slice_inputs(shard, qp, kp, q, k, v)
    (h0, h1), _, _, _ = sh.head_ranges(shard, cfg["hq"], cfg["hkv"], cfg["hp"], cfg["hpkv"])
    ldo = do.view(cfg["b"], cfg["s"], cfg["hq"], 128)[shard.b0:shard.b1, :, h0:h1].reshape(shard.b1 - shard.b0, cfg["s"], -1)
    w = sh.kl_weight(shard, cfg["b"], cfg["hkv"])
    r = O.sparse_forward_backward(lqp, lkp, lq, lk, lv, cfg["kb"] * 128, SCALE, ldo, grad_kl=w)
    dkp = sh.allreduce_dk_proxy(r["dk_proxy"], shard, cfg["b"], cfg["hq"], cfg["hkv"], cfg["hp"], cfg["hpkv"])
    full = O.sparse_forward_backward(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, do, grad_kl=1.0)
    ok = torch.allclose(dkp.double(), full["dk_proxy"].double(), atol=1e-7)
    flags = [None] * world
    dist.all_gather_object(flags, bool(ok))
    if rank == 0:
        with open(result_file, "w") as f:
            f.write("ok" if all(flags) else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


def test_dk_proxy_allreduce_two_ranks(tmp_path):
    cfg = dict(b=1, s=256, hq=8, hkv=2, hp=4, hpkv=1, kb=2)      # the reference's default: one proxy-K head
    result = tmp_path / "result.txt"
    mp.spawn(_worker_shared_kp, args=(2, _free_port(), cfg, str(result)), nprocs=2, join=True)
    assert result.read_text() == "ok"


@pytest.mark.parametrize("cfg", [dict(b=2, s=256, hq=4, hkv=2, hp=2, hpkv=2, kb=2),      # split by batch
                                 dict(b=1, s=384, hq=8, hkv=2, hp=4, hpkv=2, kb=2)])     # split by KV group
def test_two_rank_shards_reproduce_the_full_problem(tmp_path, cfg):
    result = tmp_path / "result.txt"
    mp.spawn(_worker, args=(2, _free_port(), cfg, str(result)), nprocs=2, join=True)
    assert result.read_text() == "ok"


def test_host_pipeline_chunks_cover_the_grid():
    """Chunking of the host-buffer pipeline: every (batch, KV head) unit in exactly one rectangular chunk;
    a proxy-K head is never needed by two chunks (its gradient would have to be summed across them)."""
    from flash_msa_b200.host import _chunks
    from flash_msa_b200.sharding import head_ranges
    for b, hq, hkv, hp, hpkv, want in [(2, 32, 8, 8, 8, 4), (1, 64, 8, 16, 8, 4), (2, 16, 2, 4, 1, 4), (1, 8, 2, 2, 2, 8),
                                        (3, 12, 2, 2, 1, 4), (8, 48, 4, 8, 4, 16)]:
        chunks = _chunks(b, hq, hkv, hp, hpkv, want)
        seen = set()
        owners = {}
        for ci, c in enumerate(chunks):
            (h0, h1), (kv0, kv1), (p0, p1), (kp0, kp1) = head_ranges(c, hq, hkv, hp, hpkv)
            assert h1 - h0 == (kv1 - kv0) * (hq // hkv) and p1 - p0 == (kv1 - kv0) * (hp // hkv)
            for bb in range(c.b0, c.b1):
                for kv in range(c.kv0, c.kv1):
                    assert (bb, kv) not in seen
                    seen.add((bb, kv))
                for kp in range(kp0, kp1):
                    owners.setdefault((bb, kp), set()).add(ci)
        assert len(seen) == b * hkv
        assert all(len(v) == 1 for v in owners.values())
        assert 1 <= len(chunks) <= want
