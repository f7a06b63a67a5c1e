"""Document masking of packed sequences (`flash_msa_varlen_func`): an extension without a counterpart in the
reference.  The oracle's restatement of it is checked on the CPU against its own definition (a dense selection must
equal independent dense attention per document: tests/test_oracle_golden.py); here the kernels are compared with that
oracle.  Tolerances as everywhere: selection bit-exact, tensors within twice the 16-bit eager yardstick."""
import pytest
import torch

from oracle import msa_oracle as O
from tests.gpu_util import SCALE, bf16_inputs, max_err, yardstick_check

pytestmark = pytest.mark.gpu

NAMES = ["dq_proxy", "dk_proxy", "dq", "dk", "dv"]
CASES = {
    # document boundaries inside blocks, on block boundaries, one-token and sub-block documents
    "ragged": (dict(b=2, s=1024, hq=8, hkv=2, hp=2, hpkv=2, kb=4, seed=21), [0, 100, 101, 333, 512, 700, 1024]),
    "per_batch": (dict(b=2, s=1024, hq=4, hkv=2, hp=4, hpkv=1, kb=3, seed=22), [[0, 130, 1024, 1024], [0, 5, 640, 1024]]),
    "one_document": (dict(b=1, s=512, hq=6, hkv=1, hp=1, hpkv=1, kb=2, seed=23), [0, 512]),
    "longer": (dict(b=1, s=4096, hq=8, hkv=2, hp=2, hpkv=2, kb=8, seed=24), [0, 1000, 1900, 1901, 3333, 4096]),
}


@pytest.fixture(scope="module")
def fm():
    import flash_msa_b200
    from flash_msa_b200 import api
    api.DEBUG_CHECK_STATUS = True
    yield flash_msa_b200
    api.DEBUG_CHECK_STATUS = False


@pytest.mark.parametrize("name", list(CASES))
def test_selection_respects_documents(name):
    from flash_msa_b200 import ops
    cfg, cu = CASES[name]
    qp, kp, *_ = bf16_inputs(cfg)
    ds = ops.doc_start_from_cu_seqlens(cu, cfg["b"], cfg["s"], qp.device)
    assert torch.equal(ds.cpu(), O.doc_start_from_cu_seqlens(cu, cfg["s"], cfg["b"]))
    idx, scores = ops.select_blocks(qp, kp, scale=SCALE, num_blocks=cfg["s"] // 128, top_k_blocks=cfg["kb"], return_scores=True,
                                    doc_start=ds)
    nb = cfg["s"] // 128
    want = O.proxy_block_scores(qp.float().cpu(), kp.float().cpu(), SCALE, doc_start=ds.cpu())
    vis = torch.arange(nb).view(1, 1, 1, nb) <= (torch.arange(cfg["s"]) // 128).view(1, 1, -1, 1)
    got = scores.cpu()
    assert torch.equal(torch.isinf(got[vis.expand_as(got)]), torch.isinf(want[vis.expand_as(want)]))   # the same blocks are hidden
    fin = vis.expand_as(got) & torch.isfinite(want)
    assert max_err(got[fin], want[fin]) <= 1e-4
    # bit-exact against the stable top-k of the kernel's own scores
    mine = torch.where(vis.expand_as(got), got, torch.full_like(got, float("-inf")))
    assert torch.equal(idx.cpu(), O.stable_topk(mine, cfg["kb"]))
    lo_blk = (ds.cpu() // 128).view(cfg["b"], 1, cfg["s"], 1)
    assert not bool(((idx.cpu() < lo_blk) & (idx.cpu() < nb)).any())   # no block from an earlier document


@pytest.mark.parametrize("grad_kl", [1.0, None])
@pytest.mark.parametrize("name", list(CASES))
def test_varlen_forward_backward(fm, name, grad_kl):
    from flash_msa_b200 import ops
    cfg, cu = CASES[name]
    if grad_kl is None and name != "ragged":
        pytest.skip("the no-KL variant is covered on one case")
    qp, kp, q, k, v, do = bf16_inputs(cfg)
    leaves = [t.detach().clone().requires_grad_(True) for t in (qp, kp, q, k, v)]
    out, kl = fm.flash_msa_varlen_func(*leaves, cu, cfg["kb"] * 128, SCALE)
    loss = (out.float() * do.reshape(out.shape).float()).sum() + (0.0 if grad_kl is None else grad_kl * kl)
    loss.backward()
    ds = ops.doc_start_from_cu_seqlens(cu, cfg["b"], cfg["s"], qp.device)
    idx = ops.select_blocks(qp, kp, scale=SCALE, num_blocks=cfg["s"] // 128, top_k_blocks=cfg["kb"], doc_start=ds)
    cpu = [t.float().cpu() for t in (qp, kp, q, k, v)]
    r32 = O.sparse_forward_backward(*cpu, cfg["kb"] * 128, SCALE, do.float().cpu(), grad_kl, block_indices=idx.cpu(), doc_start=ds.cpu())
    o16, _, g16 = O.eager_forward_backward(
        lambda *t: O.eager_sparse(*t, cfg["kb"] * 128, SCALE, block_indices=idx.cpu(), doc_start=ds.cpu()),
        [t.cpu() for t in (qp, kp, q, k, v)], do.cpu(), grad_kl)
    yardstick_check("out", out.cpu(), r32["out"], o16, 1e-3)
    for n, leaf, y in zip(NAMES, leaves, g16):
        got = leaf.grad.cpu()
        if grad_kl is None and n in ("dq_proxy", "dk_proxy"):
            assert got.abs().max().item() == 0.0
            continue
        yardstick_check(n, got, r32[n], y, 1e-3 * max(1.0, r32[n].abs().max().item()) if n in ("dq", "dk", "dv")
                        else 1e-3 * r32[n].abs().max().item())


def test_one_document_equals_the_plain_call(fm):
    """cu_seqlens = [0, S] must reproduce flash_msa_func (bit for bit where the sums have a fixed order)."""
    cfg = CASES["one_document"][0]
    qp, kp, q, k, v, do = bf16_inputs(cfg)
    res = []
    for fn in (lambda *t: fm.flash_msa_varlen_func(*t, [0, cfg["s"]], cfg["kb"] * 128, SCALE),
               lambda *t: fm.flash_msa_func(*t, cfg["kb"] * 128, SCALE)):
        leaves = [t.detach().clone().requires_grad_(True) for t in (qp, kp, q, k, v)]
        out, kl = fn(*leaves)
        ((out.float() * do.reshape(out.shape).float()).sum() + kl).backward()
        res.append([out] + [t.grad for t in leaves])
    for n, a, b in zip(["out"] + NAMES, *res):
        if n in ("out", "dq", "dq_proxy"):
            assert torch.equal(a, b), n
        else:   # fp32 reductions whose order is free once a reverse-index row spans several sub-units
            assert max_err(a, b) <= 2 ** -7 * b.float().abs().max().item() + 1e-6, n


def test_varlen_argument_errors(fm):
    cfg = CASES["one_document"][0]
    qp, kp, q, k, v, _ = bf16_inputs(cfg)
    with pytest.raises(ValueError):
        fm.flash_msa_varlen_func(qp, kp, q, k, v, [0, 100], cfg["kb"] * 128, SCALE)         # does not end at S
    with pytest.raises(ValueError):
        fm.flash_msa_varlen_func(qp, kp, q, k, v, [0, 300, 200, 512], cfg["kb"] * 128, SCALE)   # not rising


@pytest.mark.parametrize("name", ["ragged", "per_batch"])
def test_varlen_warmup_forward_backward(fm, name):
    """Dense warmup on packed sequences: block pairs that straddle documents are masked, rows that see nothing of a
    block contribute nothing."""
    from flash_msa_b200 import ops
    cfg, cu = CASES[name]
    qp, kp, q, k, v, do = bf16_inputs(cfg)
    leaves = [t.detach().clone().requires_grad_(True) for t in (qp, kp, q, k, v)]
    out, kl = fm.flash_msa_warmup_varlen_func(*leaves, cu, 0, SCALE)
    ((out.float() * do.reshape(out.shape).float()).sum() + 0.6 * kl).backward()
    ds = ops.doc_start_from_cu_seqlens(cu, cfg["b"], cfg["s"], qp.device).cpu()
    cpu = [t.float().cpu() for t in (qp, kp, q, k, v)]
    r32 = O.warmup_forward_backward(*cpu, SCALE, do.float().cpu(), 0.6, doc_start=ds)
    o16, _, g16 = O.eager_forward_backward(lambda *t: O.eager_warmup(*t, SCALE, doc_start=ds),
                                           [t.cpu() for t in (qp, kp, q, k, v)], do.cpu(), 0.6)
    assert torch.isfinite(out.float()).all()
    yardstick_check("out", out.cpu(), r32["out"], o16, 1e-3)
    for n, leaf, y in zip(NAMES, leaves, g16):
        yardstick_check(n, leaf.grad.cpu(), r32[n], y, 1e-3 * max(1.0, r32[n].abs().max().item()) if n in ("dq", "dk", "dv")
                        else 1e-3 * r32[n].abs().max().item())
