"""Forward parity on the GPU through the C ABI: block scores, bit-exact selection, sparse and
dense (warmup) attention output, log-sum-exp of the main and proxy heads."""
import pytest
import torch

from oracle import msa_oracle as O
from tests.gpu_util import SCALE, bf16_inputs, max_err, yardstick_check

pytestmark = pytest.mark.gpu

CFGS = {
    "tiny": dict(b=1, s=512, hq=4, hkv=1, hp=2, hpkv=1, kb=2, seed=1),
    "c1": dict(b=2, s=1024, hq=8, hkv=2, hp=2, hpkv=2, kb=4, seed=0),
    "mpp6": dict(b=1, s=2048, hq=12, hkv=2, hp=2, hpkv=1, kb=5, seed=2),
    "ref_default": dict(b=1, s=2048, hq=16, hkv=2, hp=4, hpkv=1, kb=4, seed=67),
    "pg2": dict(b=1, s=1536, hq=8, hkv=2, hp=4, hpkv=4, kb=3, seed=4),
}


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from flash_msa_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("name", list(CFGS))
def test_block_scores_and_selection(ops, name):
    cfg = CFGS[name]
    qp, kp, *_ = bf16_inputs(cfg)
    nb = cfg["s"] // 128
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    scores = ops.proxy_block_scores(qp, kp, SCALE, status=status)
    ops.check_status(status, "select_scores")
    want = O.proxy_block_scores(qp, kp, SCALE)
    vis = torch.isfinite(want)
    assert max_err(scores[vis], want[vis]) <= 1e-4          # same bf16 inputs, fp32 accumulation both sides
    # bit-exact selection on the kernel's own scores
    idx = ops.select_topk(scores, cfg["kb"])
    masked = torch.where(vis, scores, torch.full_like(scores, float("-inf")))
    assert torch.equal(idx.cpu(), O.stable_topk(masked, cfg["kb"]).cpu())
    # flips against independently computed scores are only allowed at near-ties
    idx_o = O.stable_topk(want, cfg["kb"])
    flips = (idx.sort(-1).values != idx_o.sort(-1).values).any(-1).sum().item()
    near = O.near_tie_report(want, cfg["kb"], 1e-4)["near_ties"]
    assert flips <= near, (flips, near)


@pytest.mark.parametrize("layout", ["bhsd", "bshd"])
@pytest.mark.parametrize("name", list(CFGS))
def test_sparse_forward(ops, name, layout):
    cfg = CFGS[name]
    if layout == "bshd" and name not in ("tiny", "c1"):
        pytest.skip("layout variant covered on the small shapes")
    qp, kp, q, k, v, _ = bf16_inputs(cfg, layout=layout)
    nb = cfg["s"] // 128
    idx = ops.select_blocks(qp, kp, scale=SCALE, num_blocks=nb, top_k_blocks=cfg["kb"])
    rix = ops.build_reverse_index(idx)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse, lse_p = ops.attention_forward(q, k, v, qp, kp, SCALE, rix, status=status)
    ops.check_status(status, "sparse_fwd")
    r32 = O.sparse_forward(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, block_indices=idx)
    r16 = O.sparse_forward(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, block_indices=idx, dtype=torch.bfloat16)
    yardstick_check("out", out, r32["out"], r16["out"], 1e-3)
    assert max_err(lse, r32["lse"]) <= 2e-3
    assert max_err(lse_p, r32["lse_proxy"]) <= 2e-3


@pytest.mark.parametrize("name", ["tiny", "c1", "mpp6"])
def test_dense_forward(ops, name):
    cfg = CFGS[name]
    qp, kp, q, k, v, _ = bf16_inputs(cfg)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse, lse_p = ops.attention_forward(q, k, v, qp, kp, SCALE, None, dense=True, status=status)
    ops.check_status(status, "dense_fwd")
    r32 = O.warmup_forward(qp, kp, q, k, v, SCALE)
    r16 = O.warmup_forward(qp, kp, q, k, v, SCALE, dtype=torch.bfloat16)
    yardstick_check("out", out, r32["out"], r16["out"], 1e-3)
    assert max_err(lse, r32["lse"]) <= 2e-3
    assert max_err(lse_p, r32["lse_proxy"]) <= 2e-3


@pytest.mark.parametrize("name", ["tiny", "c1"])
def test_sparse_forward_fp16(ops, name):
    """fp16 activations (accepted by the reference kernels too, flash_msa/msa_backward_cutedsl.py:169-183): the same
    check as for bf16 with the fp16 restatement as the yardstick."""
    cfg = CFGS[name]
    qp, kp, q, k, v, _ = bf16_inputs(cfg, dtype=torch.float16)
    nb = cfg["s"] // 128
    idx = ops.select_blocks(qp, kp, scale=SCALE, num_blocks=nb, top_k_blocks=cfg["kb"])
    rix = ops.build_reverse_index(idx)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse, lse_p = ops.attention_forward(q, k, v, qp, kp, SCALE, rix, status=status)
    ops.check_status(status, "sparse_fwd")
    assert out.dtype == torch.float16
    r32 = O.sparse_forward(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, block_indices=idx)
    r16 = O.sparse_forward(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, block_indices=idx, dtype=torch.float16)
    yardstick_check("out", out, r32["out"], r16["out"], 1e-3)
    assert max_err(lse, r32["lse"]) <= 2e-3
    assert max_err(lse_p, r32["lse_proxy"]) <= 2e-3
    # the selection on fp16 inputs is bit-exact against the stable top-k of the kernel's own scores as well
    scores = ops.proxy_block_scores(qp, kp, SCALE)
    qblk = (torch.arange(cfg["s"], device="cuda") // 128).view(1, 1, -1, 1)
    masked = scores.masked_fill(torch.arange(nb, device="cuda").view(1, 1, 1, nb) > qblk, float("-inf"))
    assert torch.equal(idx.cpu(), O.stable_topk(masked.cpu(), cfg["kb"]))


@pytest.mark.parametrize("s,kb,hp,hpkv", [(128, 1, 1, 1), (512, 2, 2, 1), (1024, 4, 2, 2), (2048, 8, 3, 1), (2048, 9, 2, 2), (4096, 16, 2, 1),
                                          (4096, 17, 1, 1), (8192, 32, 2, 2), (8192, 5, 1, 1), (8192, 33, 1, 1),
                                          (8192, 48, 2, 1), (8192, 64, 2, 2), (16384, 64, 1, 1)])
@pytest.mark.parametrize("docs", [False, True])
def test_fused_selection_equals_scores_plus_topk(s, kb, hp, hpkv, docs):
    """The fused kernel (block scores and the per-row top-k in one pass, nothing materialised) must give, bit for bit,
    what the score kernel followed by the top-k kernel gives - also with ties (a proxy head made of repeated rows) and
    with documents."""
    from flash_msa_b200 import ops
    cfg = dict(b=2, s=s, hq=hp, hkv=1, hp=hp, hpkv=hpkv, seed=7 * s + kb)
    qp, kp, *_ = bf16_inputs(cfg)
    kp = kp.clone()
    kp[:, :, 128:256] = kp[:, :, 0:128] if s >= 256 else kp[:, :, 128:256]   # two identical key blocks: exact ties
    ds = None
    if docs:
        cu = sorted({0, s} | {int(x) for x in torch.randint(1, s, (3,), generator=torch.Generator().manual_seed(s + kb))})
        ds = ops.doc_start_from_cu_seqlens(cu, 2, s, qp.device)
    want = ops.select_blocks(qp, kp, scale=SCALE, num_blocks=s // 128, top_k_blocks=kb, doc_start=ds)
    got = ops.select_blocks_fused(qp, kp, SCALE, kb, doc_start=ds)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
