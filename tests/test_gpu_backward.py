"""Backward parity on the GPU through the public autograd API: dQ, dK, dV, dQp, dKp of the sparse
and the warmup function against the fp32 oracle, with the reference's bf16 eager arithmetic as the
error yardstick (tolerance: at most twice its error, plus a small floor)."""
import pytest
import torch

from oracle import msa_oracle as O
from tests.gpu_util import SCALE, bf16_inputs, kernel_selection, max_err, yardstick_check

pytestmark = pytest.mark.gpu
NAMES = ["dq_proxy", "dk_proxy", "dq", "dk", "dv"]

CFGS = {
    "tiny": dict(b=1, s=512, hq=4, hkv=1, hp=2, hpkv=1, kb=2, seed=1),
    "c1": dict(b=2, s=1024, hq=8, hkv=2, hp=2, hpkv=2, kb=4, seed=0),
    "mpp6": dict(b=1, s=2048, hq=12, hkv=2, hp=2, hpkv=1, kb=5, seed=2),
    "ref_default": dict(b=1, s=2048, hq=16, hkv=2, hp=4, hpkv=1, kb=4, seed=67),
    "pg2": dict(b=1, s=1536, hq=8, hkv=2, hp=4, hpkv=4, kb=3, seed=4),
}


@pytest.fixture(scope="module")
def fm():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import flash_msa_b200
    from flash_msa_b200 import api
    api.DEBUG_CHECK_STATUS = True
    return flash_msa_b200


def _run_kernel(fn, tensors, do, top_k, grad_kl):
    leaves = [t.detach().clone().requires_grad_(True) for t in tensors]
    out, kl = fn(*leaves, top_k, SCALE)
    assert kl.item() == 0.0 and kl.dtype == torch.float32
    loss = (out.float() * do.float()).sum()
    if grad_kl is not None:
        loss = loss + grad_kl * kl
    loss.backward()
    return out, [t.grad for t in leaves], out.grad_fn


def _floors(ref):
    return 1e-3 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("grad_kl", [1.0, 0.37, None])
@pytest.mark.parametrize("name", list(CFGS))
def test_sparse_backward(fm, name, grad_kl):
    cfg = CFGS[name]
    if grad_kl != 1.0 and name not in ("tiny", "c1"):
        pytest.skip("grad_kl variants covered on the small shapes")
    qp, kp, q, k, v, do = bf16_inputs(cfg, layout="bshd" if name == "c1" else "bhsd")
    out, grads, node = _run_kernel(fm.flash_msa_func, (qp, kp, q, k, v), do, cfg["kb"] * 128, grad_kl)
    idx = kernel_selection(qp, kp, cfg["kb"])
    r32 = O.sparse_forward_backward(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, do, grad_kl, block_indices=idx)
    _, _, g16 = O.eager_forward_backward(lambda *t: O.eager_sparse(*t, cfg["kb"] * 128, SCALE, block_indices=idx),
                                         (qp, kp, q, k, v), do, grad_kl)
    for n, got, y in zip(NAMES, grads, g16):
        assert got.shape == r32[n].shape and got.dtype == torch.bfloat16
        if grad_kl is None and n in ("dq_proxy", "dk_proxy"):
            assert got.abs().max().item() == 0.0
            continue
        yardstick_check(n, got, r32[n], y, _floors(r32[n]) if n in ("dq", "dk", "dv") else 1e-3 * r32[n].abs().max().item())


@pytest.mark.parametrize("grad_kl", [1.0, None])
@pytest.mark.parametrize("name", ["tiny", "c1", "mpp6"])
def test_warmup_backward(fm, name, grad_kl):
    cfg = CFGS[name]
    qp, kp, q, k, v, do = bf16_inputs(cfg)
    out, grads, _ = _run_kernel(fm.flash_msa_warmup_func, (qp, kp, q, k, v), do, cfg["kb"] * 128, grad_kl)
    r32 = O.warmup_forward_backward(qp, kp, q, k, v, SCALE, do, grad_kl)
    _, _, g16 = O.eager_forward_backward(lambda *t: O.eager_warmup(*t, SCALE), (qp, kp, q, k, v), do, grad_kl)
    o16 = O.warmup_forward(qp, kp, q, k, v, SCALE, dtype=torch.bfloat16)["out"]
    yardstick_check("out", out, r32["out"], o16, 1e-3)
    for n, got, y in zip(NAMES, grads, g16):
        if grad_kl is None and n in ("dq_proxy", "dk_proxy"):
            assert got.abs().max().item() == 0.0
            continue
        yardstick_check(n, got, r32[n], y, _floors(r32[n]) if n in ("dq", "dk", "dv") else 1e-3 * r32[n].abs().max().item())


def test_grad_out_none_and_error_behaviour(fm):
    cfg = CFGS["tiny"]
    qp, kp, q, k, v, do = bf16_inputs(cfg)
    # only kl_loss feeds the loss: main gradients are zero, proxy gradients are not
    leaves = [t.detach().clone().requires_grad_(True) for t in (qp, kp, q, k, v)]
    out, kl = fm.flash_msa_func(*leaves, 256, SCALE)
    kl.backward()
    assert leaves[2].grad.abs().max().item() == 0.0 and leaves[4].grad.abs().max().item() == 0.0
    assert leaves[0].grad.abs().max().item() > 0.0
    with pytest.raises(ValueError):
        fm.flash_msa_func(qp, kp, q, k, v, 200, SCALE)                  # top_k not a multiple of 128
    with pytest.raises(ValueError):
        fm.flash_msa_func(qp, kp, q, k, v, 128 * 64, SCALE)             # more blocks than the sequence has
    with pytest.raises(ValueError):
        fm.flash_msa_func(qp[:, :, :500], kp, q, k, v, 256, SCALE)      # shapes disagree
    with pytest.raises(NotImplementedError):
        fm.flash_msa_func(qp[..., :64], kp[..., :64], q[..., :64], k[..., :64], v[..., :64], 256, SCALE)
    with pytest.raises(TypeError):
        fm.flash_msa_func(qp.float(), kp.float(), q.float(), k.float(), v.float(), 256, SCALE)
    with pytest.raises(RuntimeError):
        fm.flash_msa_warmup_func(qp.cpu(), kp.cpu(), q.cpu(), k.cpu(), v.cpu(), 256, SCALE)


@pytest.mark.parametrize("name", ["tiny", "c1", "mpp6", "pg2"])
def test_kl_value(fm, name):
    """Optional KL loss value computed inside the backward kernel, against the oracle's value on the same
    selection (tolerance 2 % + 1e-4: teacher and probabilities come from bf16 operands and fp16 sums)."""
    from flash_msa_b200 import api
    cfg = CFGS[name]
    qp, kp, q, k, v, do = bf16_inputs(cfg)
    api.COMPUTE_KL_VALUE = True
    try:
        _, _, node = _run_kernel(fm.flash_msa_func, (qp, kp, q, k, v), do, cfg["kb"] * 128, 1.0)
        got = fm.last_kl_value()
        assert got is not None and got.shape == () and got.dtype == torch.float32
        ref = O.sparse_forward(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, block_indices=kernel_selection(qp, kp, cfg["kb"]))["kl"]
        assert abs(got.item() - ref.item()) <= 2e-2 * abs(ref.item()) + 1e-4, (got.item(), ref.item())
        _run_kernel(fm.flash_msa_warmup_func, (qp, kp, q, k, v), do, cfg["kb"] * 128, 1.0)
        got_w = fm.last_kl_value()
        ref_w = O.warmup_forward(qp, kp, q, k, v, SCALE)["kl"]
        assert abs(got_w.item() - ref_w.item()) <= 2e-2 * abs(ref_w.item()) + 1e-4, (got_w.item(), ref_w.item())
        # without a gradient for kl_loss the proxy work is skipped and nothing new is published
        before = fm.last_kl_value()
        _run_kernel(fm.flash_msa_func, (qp, kp, q, k, v), do, cfg["kb"] * 128, None)
        assert fm.last_kl_value() is before
    finally:
        api.COMPUTE_KL_VALUE = False



@pytest.mark.parametrize("warmup", [False, True])
def test_backward_fp16(fm, warmup):
    """fp16 activations through the public functions: gradients come back in fp16 and stay within twice the error of
    the fp16 eager arithmetic."""
    cfg = CFGS["c1"]
    qp, kp, q, k, v, do = bf16_inputs(cfg, dtype=torch.float16)
    fn = fm.flash_msa_warmup_func if warmup else fm.flash_msa_func
    out, grads, _ = _run_kernel(fn, (qp, kp, q, k, v), do, cfg["kb"] * 128, 1.0)
    assert out.dtype == torch.float16
    if warmup:
        r32 = O.warmup_forward_backward(qp, kp, q, k, v, SCALE, do, 1.0)
        _, _, g16 = O.eager_forward_backward(lambda *t: O.eager_warmup(*t, SCALE), (qp, kp, q, k, v), do, 1.0)
    else:
        idx = kernel_selection(qp, kp, cfg["kb"])
        r32 = O.sparse_forward_backward(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, do, 1.0, block_indices=idx)
        _, _, g16 = O.eager_forward_backward(lambda *t: O.eager_sparse(*t, cfg["kb"] * 128, SCALE, block_indices=idx),
                                             (qp, kp, q, k, v), do, 1.0)
    for n, got, y in zip(NAMES, grads, g16):
        assert got.dtype == torch.float16 and got.shape == r32[n].shape
        yardstick_check(n, got, r32[n], y, _floors(r32[n]) if n in ("dq", "dk", "dv") else 1e-3 * r32[n].abs().max().item())


@pytest.mark.parametrize("warmup", [False, True])
def test_gradients_in_caller_layout(fm, warmup):
    """Inputs that are (B,H,S,D) views of (B,S,H,D) storage (the reference's callers: flash_msa/tests/testing_model.py:173-185)
    get their gradients back in that same storage layout, written there by the kernels (no transposing copy), with
    the values of a run on (B,H,S,D)-contiguous inputs."""
    from flash_msa_b200 import ops
    cfg = CFGS["c1"]
    views = bf16_inputs(cfg, layout="bshd")
    plain = bf16_inputs(cfg, layout="bhsd")
    gk = torch.tensor(0.5, device="cuda")
    results = []
    for qp, kp, q, k, v, do in (views, plain):
        if warmup:
            rix = None
            out, lse, lse_p = ops.attention_forward(q, k, v, qp, kp, SCALE, None, dense=True)
        else:
            rix = ops.build_reverse_index(ops.select_blocks(qp, kp, scale=SCALE, num_blocks=cfg["s"] // 128, top_k_blocks=cfg["kb"]))
            out, lse, lse_p = ops.attention_forward(q, k, v, qp, kp, SCALE, rix)
        go = do if do.dim() == 3 else do.permute(0, 2, 1, 3).reshape(out.shape).contiguous()
        results.append(ops.attention_backward(q, k, v, qp, kp, out, go, lse, lse_p, SCALE, rix, gk, dense=warmup))
    for n, g_view, g_plain, x in zip(NAMES, results[0], results[1], (views[0], views[1], views[2], views[3], views[4])):
        assert g_view.stride() == x.stride() and g_view.transpose(1, 2).is_contiguous()
        assert g_plain.is_contiguous()
        if n in ("dq", "dq_proxy"):
            assert torch.equal(g_view, g_plain), n
        else:   # fp32 reductions whose order is free once a reverse-index row spans several sub-units
            assert max_err(g_view, g_plain) <= 2 ** -7 * g_plain.float().abs().max().item() + 1e-6, n


@pytest.mark.parametrize("warmup", [False, True])
def test_passes_over_groups_give_the_same_result(fm, warmup):
    """When the per-edge partial rows of a call would exceed `ops.MAX_PARTIAL_BYTES` the forward and the backward run in
    several passes over (batch, KV head) groups, reusing one partial buffer.  One group per pass must give what one
    pass over everything gives: out, lse and dQ bit for bit (they are sums in a fixed order), dK / dV / dKp up to the
    order of their fp32 reductions."""
    from flash_msa_b200 import ops
    cfg = dict(b=2, s=1024, hq=12, hkv=3, hp=6, hpkv=3, kb=3, seed=31)
    qp, kp, q, k, v, do = bf16_inputs(cfg)
    fn = fm.flash_msa_warmup_func if warmup else fm.flash_msa_func
    saved = ops.MAX_PARTIAL_BYTES
    results = []
    try:
        for cap in (saved, 1):
            ops.MAX_PARTIAL_BYTES = cap
            results.append(_run_kernel(fn, (qp, kp, q, k, v), do, cfg["kb"] * 128, 0.8))
    finally:
        ops.MAX_PARTIAL_BYTES = saved
    (out_a, grads_a, _), (out_b, grads_b, _) = results
    assert torch.equal(out_a, out_b)
    for n, ga, gb in zip(NAMES, grads_a, grads_b):
        if n in ("dq", "dq_proxy"):
            assert torch.equal(ga, gb), n
        else:
            assert max_err(ga, gb) <= 2 ** -7 * ga.float().abs().max().item() + 1e-6, n


@pytest.mark.parametrize("warmup", [False, True])
@pytest.mark.parametrize("heads", [(8, 4, 2, 1), (12, 6, 2, 2), (6, 3, 1, 1)])
def test_fewer_proxy_heads_than_kv_heads(fm, heads, warmup):
    """Hp < Hkv (refused by the reference): every proxy head steers the main heads of several KV heads and its KL teacher
    is the mean over all of them.  The public functions spread the proxy query heads over the KV heads and let autograd
    sum the copies' gradients; the result must be the oracle's for the original head counts."""
    hq, hkv, hp, hpkv = heads
    cfg = dict(b=2, s=512, hq=hq, hkv=hkv, hp=hp, hpkv=hpkv, kb=2, seed=41)
    qp, kp, q, k, v, do = bf16_inputs(cfg)
    fn = fm.flash_msa_warmup_func if warmup else fm.flash_msa_func
    out, grads, _ = _run_kernel(fn, (qp, kp, q, k, v), do, cfg["kb"] * 128, 0.7)
    assert grads[0].shape == qp.shape
    if warmup:
        r32 = O.warmup_forward_backward(qp, kp, q, k, v, SCALE, do, 0.7)
        o16, _, g16 = O.eager_forward_backward(lambda *t: O.eager_warmup(*t, SCALE), (qp, kp, q, k, v), do, 0.7)
    else:
        idx = kernel_selection(qp, kp, cfg["kb"])
        r32 = O.sparse_forward_backward(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, do, 0.7, block_indices=idx)
        o16, _, g16 = O.eager_forward_backward(lambda *t: O.eager_sparse(*t, cfg["kb"] * 128, SCALE, block_indices=idx),
                                               (qp, kp, q, k, v), do, 0.7)
    yardstick_check("out", out, r32["out"], o16, 1e-3)
    for n, got, y in zip(NAMES, grads, g16):
        yardstick_check(n, got, r32[n], y, _floors(r32[n]) if n in ("dq", "dk", "dv") else 1e-3 * r32[n].abs().max().item())


@pytest.mark.parametrize("warmup", [False, True])
@pytest.mark.parametrize("mpp", [5, 7, 8, 12, 16])
def test_main_heads_per_proxy_head(fm, mpp, warmup):
    """Hq/Hp beyond the BASELINE shapes: 5, 7 and 8 main heads per proxy head take the three- and four-sweep forms of the
    combine kernels, 12 and 16 the one-head-at-a-time forms; 5 and 7 do not divide 128 (the reference refuses them,
    flash_msa/flash_msa.py:153-158)."""
    cfg = dict(b=1, s=768, hq=2 * mpp, hkv=2, hp=2, hpkv=1, kb=3, seed=50 + mpp)
    qp, kp, q, k, v, do = bf16_inputs(cfg)
    fn = fm.flash_msa_warmup_func if warmup else fm.flash_msa_func
    out, grads, _ = _run_kernel(fn, (qp, kp, q, k, v), do, cfg["kb"] * 128, 0.7)
    if warmup:
        r32 = O.warmup_forward_backward(qp, kp, q, k, v, SCALE, do, 0.7)
        o16, _, g16 = O.eager_forward_backward(lambda *t: O.eager_warmup(*t, SCALE), (qp, kp, q, k, v), do, 0.7)
    else:
        idx = kernel_selection(qp, kp, cfg["kb"])
        r32 = O.sparse_forward_backward(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, do, 0.7, block_indices=idx)
        o16, _, g16 = O.eager_forward_backward(lambda *t: O.eager_sparse(*t, cfg["kb"] * 128, SCALE, block_indices=idx),
                                               (qp, kp, q, k, v), do, 0.7)
    yardstick_check("out", out, r32["out"], o16, 1e-3)
    for n, got, y in zip(NAMES, grads, g16):
        yardstick_check(n, got, r32[n], y, _floors(r32[n]) if n in ("dq", "dk", "dv") else 1e-3 * r32[n].abs().max().item())


@pytest.mark.parametrize("warmup", [False, True])
def test_softmax_sinks(fm, warmup):
    """One softmax-bias logit per main head (an extension: the reference lists it as missing).  Output, all five
    gradients and the gradient of the sinks against the oracle, whose closed forms with sinks equal autograd through
    the eager restatement (softmax over the logits and one extra column)."""
    cfg = dict(b=2, s=512, hq=8, hkv=2, hp=2, hpkv=1, kb=2, seed=43)
    qp, kp, q, k, v, do = bf16_inputs(cfg)
    sinks = (torch.randn(cfg["hq"], generator=torch.Generator().manual_seed(9)) * 0.7 + 1.0).cuda().requires_grad_(True)
    leaves = [t.detach().requires_grad_(True) for t in (qp, kp, q, k, v)]
    fn = fm.flash_msa_warmup_func if warmup else fm.flash_msa_func
    out, kl = fn(*leaves, cfg["kb"] * 128, SCALE, sinks=sinks)
    ((out.float() * do.reshape(out.shape).float()).sum() + 0.7 * kl).backward()
    sk = sinks.detach()
    if warmup:
        r32 = O.warmup_forward_backward(qp, kp, q, k, v, SCALE, do, 0.7, sinks=sk)
        sk16 = sk.to(torch.bfloat16).requires_grad_(True)
        o16, _, g16 = O.eager_forward_backward(lambda *t: O.eager_warmup(*t, SCALE, sinks=sk16), (qp, kp, q, k, v), do, 0.7, extra=[sk16])
    else:
        idx = kernel_selection(qp, kp, cfg["kb"])
        r32 = O.sparse_forward_backward(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, do, 0.7, block_indices=idx, sinks=sk)
        sk16 = sk.to(torch.bfloat16).requires_grad_(True)
        o16, _, g16 = O.eager_forward_backward(lambda *t: O.eager_sparse(*t, cfg["kb"] * 128, SCALE, block_indices=idx, sinks=sk16),
                                               (qp, kp, q, k, v), do, 0.7, extra=[sk16])
    yardstick_check("out", out, r32["out"], o16, 2e-3)
    for n, leaf, y in zip(NAMES, leaves, g16[:5]):
        yardstick_check(n, leaf.grad, r32[n], y, _floors(r32[n]) if n in ("dq", "dk", "dv") else 1e-3 * r32[n].abs().max().item())
    # (the log-sum-exp is held to 2e-3 absolute, i.e. the sink's probability to 0.2 %, systematically over a head's rows)
    yardstick_check("dsinks", sinks.grad, r32["dsinks"], g16[5].float(), 5e-3 * max(1.0, r32["dsinks"].abs().max().item()))
    # a sink that is far below every logit changes nothing
    out0, _ = fn(qp, kp, q, k, v, cfg["kb"] * 128, SCALE)
    out1, _ = fn(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, sinks=torch.full((cfg["hq"],), -1e4, device="cuda"))
    assert torch.equal(out0, out1)
