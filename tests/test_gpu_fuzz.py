"""Seeded random head configurations, lengths, selections, dtypes, layouts and document packings through the public
functions, against the oracle (selection bit-exact on the kernel's own scores; tensors within twice the 16-bit eager
yardstick).  The shapes are small enough for the eager restatement; what varies is everything the index arithmetic
depends on: heads per proxy head (also values that do not divide 128), proxy heads per KV head, proxy-K sharing,
ragged reverse-index rows, top-k larger than the number of visible blocks, documents that start inside blocks, fewer
proxy heads than KV heads, softmax sinks."""
import random

import pytest
import torch

from oracle import msa_oracle as O
from tests.gpu_util import SCALE, bf16_inputs, yardstick_check

pytestmark = pytest.mark.gpu
NAMES = ["dq_proxy", "dk_proxy", "dq", "dk", "dv"]


def _draw(seed):
    rng = random.Random(1000 + seed)
    hkv = rng.choice([1, 2, 3, 4])
    if hkv in (2, 4) and rng.random() < 0.25:      # fewer proxy heads than KV heads
        hp = hkv // 2
        hq = hkv * rng.choice([1, 2, 3])
    else:
        hp = hkv * rng.choice([1, 1, 2])
        hq = hp * rng.choice([1, 2, 3, 4, 6])
    hpkv = rng.choice([d for d in range(1, hp + 1) if hp % d == 0])
    s = 128 * rng.choice([1, 2, 3, 5, 8])
    kb = rng.randint(1, s // 128)
    cfg = dict(b=rng.choice([1, 2, 3]), s=s, hq=hq, hkv=hkv, hp=hp, hpkv=hpkv, kb=kb, seed=500 + seed)
    mode = rng.choice(["sparse", "sparse", "warmup"])
    dtype = rng.choice([torch.bfloat16, torch.bfloat16, torch.float16])
    layout = rng.choice(["bhsd", "bshd"])
    cu = None
    if rng.random() < 0.5:
        cuts = sorted(rng.sample(range(1, s), k=min(s - 1, rng.randint(1, 4))))
        cu = [0] + cuts + [s]
    grad_kl = rng.choice([1.0, 0.4, None])
    return cfg, mode, dtype, layout, cu, grad_kl, rng.random() < 0.3


@pytest.mark.parametrize("seed", range(48))
def test_random_configuration(seed):
    import flash_msa_b200 as fm
    from flash_msa_b200 import api, ops
    cfg, mode, dtype, layout, cu, grad_kl, with_sinks = _draw(seed)
    sinks = None
    if with_sinks:
        sinks = (torch.randn(cfg["hq"], generator=torch.Generator().manual_seed(seed)) * 0.7 + 0.5).cuda().requires_grad_(True)
    api.DEBUG_CHECK_STATUS = True
    try:
        qp, kp, q, k, v, do = bf16_inputs(cfg, layout=layout, dtype=dtype)
        leaves = [t.detach().requires_grad_(True) for t in (qp, kp, q, k, v)]
        top_k = cfg["kb"] * 128
        if mode == "warmup":
            out, kl = (fm.flash_msa_warmup_func(*leaves, top_k, SCALE, sinks=sinks) if cu is None
                       else fm.flash_msa_warmup_varlen_func(*leaves, cu, top_k, SCALE, sinks=sinks))
        else:
            out, kl = (fm.flash_msa_func(*leaves, top_k, SCALE, sinks=sinks) if cu is None
                       else fm.flash_msa_varlen_func(*leaves, cu, top_k, SCALE, sinks=sinks))
        loss = (out.float() * do.reshape(out.shape).float()).sum()
        if grad_kl is not None:
            loss = loss + grad_kl * kl
        loss.backward()
    finally:
        api.DEBUG_CHECK_STATUS = False
    ds = None if cu is None else ops.doc_start_from_cu_seqlens(cu, cfg["b"], cfg["s"], qp.device)
    ds_cpu = None if ds is None else ds.cpu()
    cpu16 = [t.cpu() for t in (qp, kp, q, k, v)]
    cpu32 = [t.float() for t in cpu16]
    sk32 = None if sinks is None else sinks.detach().float().cpu()
    sk16 = None if sinks is None else sinks.detach().to(dtype).cpu().requires_grad_(True)
    extra = [] if sinks is None else [sk16]
    if mode == "warmup":
        r32 = O.warmup_forward_backward(*cpu32, SCALE, do.float().cpu(), grad_kl, doc_start=ds_cpu, sinks=sk32)
        o16, _, g16 = O.eager_forward_backward(lambda *t: O.eager_warmup(*t, SCALE, doc_start=ds_cpu, sinks=sk16), cpu16, do.cpu(),
                                               grad_kl, extra=extra)
    else:
        idx, scores = ops.select_blocks(qp, kp, scale=SCALE, num_blocks=cfg["s"] // 128, top_k_blocks=cfg["kb"],
                                        return_scores=True, doc_start=ds)
        nb = cfg["s"] // 128
        vis = torch.arange(nb).view(1, 1, 1, nb) <= (torch.arange(cfg["s"]) // 128).view(1, 1, -1, 1)
        mine = torch.where(vis.expand_as(scores.cpu()), scores.cpu(), torch.full_like(scores.cpu(), float("-inf")))
        assert torch.equal(idx.cpu(), O.stable_topk(mine, cfg["kb"]))
        r32 = O.sparse_forward_backward(*cpu32, top_k, SCALE, do.float().cpu(), grad_kl, block_indices=idx.cpu(), doc_start=ds_cpu,
                                        sinks=sk32)
        o16, _, g16 = O.eager_forward_backward(
            lambda *t: O.eager_sparse(*t, top_k, SCALE, block_indices=idx.cpu(), doc_start=ds_cpu, sinks=sk16), cpu16, do.cpu(),
            grad_kl, extra=extra)
    assert out.dtype == dtype
    yardstick_check("out", out.cpu(), r32["out"], o16, 2e-3 if sinks is not None else 1e-3)
    if sinks is not None:
        # (a sum over all rows of exp(sink - lse) * delta: the log-sum-exp is held to 2e-3 absolute elsewhere, i.e. the
        # sink's probability to 0.2 %, and that error is systematic over the rows of a head)
        yardstick_check("dsinks", sinks.grad.cpu(), r32["dsinks"], g16[5].float(), 5e-3 * max(1.0, r32["dsinks"].abs().max().item()))
    for n, leaf, y in zip(NAMES, leaves, g16[:5]):
        got = leaf.grad.cpu()
        if grad_kl is None and n in ("dq_proxy", "dk_proxy"):
            assert got.abs().max().item() == 0.0
            continue
        floor = 1e-3 * max(1.0, r32[n].abs().max().item()) if n in ("dq", "dk", "dv") else 1e-3 * r32[n].abs().max().item()
        yardstick_check(f"{n} {cfg} {mode} {dtype} {layout} docs={cu}", got, r32[n], y, floor)
