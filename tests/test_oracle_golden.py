"""The oracle against the vectors produced by the reference's own eager model
(tests/golden/make_golden.py), plus the documented tie / sentinel conventions."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import msa_oracle as O

NAMES = ["dq_proxy", "dk_proxy", "dq", "dk", "dv"]
SCALE = 128 ** -0.5


def _inputs(cfg):
    return O.make_inputs(cfg["b"], cfg["s"], cfg["hq"], cfg["hkv"], cfg["hp"], cfg["hpkv"],
                         seed=cfg["seed"])


def _close(a, ref, tol):
    ref = torch.as_tensor(ref)
    err = (a.double() - ref.double()).abs().max().item()
    bound = tol * max(1.0, ref.abs().max().item())
    assert err <= bound, (err, bound)


@pytest.mark.parametrize("kind", ["sparse", "warmup"])
def test_closed_forms_match_reference_vectors(golden_dir, kind):
    g = np.load(os.path.join(golden_dir, f"{kind}_small.npz"))
    cfg = json.loads(str(g["config"]))
    ins = _inputs(cfg)
    np.testing.assert_allclose([float(t.double().sum()) for t in ins], g["input_checksum"], rtol=0, atol=1e-6)
    qp, kp, q, k, v, do = ins
    if kind == "sparse":
        r = O.sparse_forward_backward(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, do, 1.0)
    else:
        r = O.warmup_forward_backward(qp, kp, q, k, v, SCALE, do, 1.0)
    _close(r["out"], g["out"], 2e-6)
    _close(r["kl"], g["kl"], 2e-6)
    for n in NAMES:
        _close(r[n], g[n], 2e-6)


@pytest.mark.parametrize("kind", ["sparse", "warmup"])
def test_eager_restatement_matches_reference_vectors(golden_dir, kind):
    g = np.load(os.path.join(golden_dir, f"{kind}_small.npz"))
    cfg = json.loads(str(g["config"]))
    qp, kp, q, k, v, do = _inputs(cfg)
    if kind == "sparse":
        fn = lambda *t: O.eager_sparse(*t, cfg["kb"] * 128, SCALE)
    else:
        fn = lambda *t: O.eager_warmup(*t, SCALE)
    out, kl, grads = O.eager_forward_backward(fn, (qp, kp, q, k, v), do, 1.0)
    _close(out, g["out"], 1e-6)
    _close(kl, g["kl"], 1e-6)
    for n, gr in zip(NAMES, grads):
        _close(gr, g[n], 1e-6)


@pytest.mark.parametrize("kind", ["sparse", "warmup"])
def test_config1_summary(golden_dir, kind):
    with open(os.path.join(golden_dir, "c1_summary.json")) as f:
        summ = json.load(f)
    cfg = summ["config"]
    qp, kp, q, k, v, do = _inputs(cfg)
    if kind == "sparse":
        r = O.sparse_forward_backward(qp, kp, q, k, v, cfg["kb"] * 128, SCALE, do, 1.0)
    else:
        r = O.warmup_forward_backward(qp, kp, q, k, v, SCALE, do, 1.0)
    for name, s in summ[kind].items():
        t = r[name].double().reshape(-1)
        scale = max(1.0, max(abs(x) for x in s["sample"]))
        got = t[torch.tensor(s["sample_idx"])] if t.numel() > 1 else t
        assert (got - torch.tensor(s["sample"], dtype=torch.float64)).abs().max().item() <= 5e-6 * scale, name
        assert abs(float(t.pow(2).sum().sqrt()) - s["l2"]) <= 1e-5 * max(1.0, s["l2"]), name


def test_grad_kl_none_gives_zero_proxy_grads():
    qp, kp, q, k, v, do = O.make_inputs(1, 256, 2, 1, 1, 1, seed=3)
    r = O.sparse_forward_backward(qp, kp, q, k, v, 128, SCALE, do, None)
    assert r["dq_proxy"].abs().max().item() == 0.0 and r["dk_proxy"].abs().max().item() == 0.0


def test_stable_topk_lower_index_wins_and_sentinel():
    nb = 6
    sc = torch.full((1, 1, nb * 128, nb), float("-inf"))
    # row in block 3: blocks 0..3 visible; scores tie between block 1 and 2
    q = 3 * 128 + 5
    sc[0, 0, q, :4] = torch.tensor([0.5, 1.0, 1.0, -2.0])
    idx = O.stable_topk(sc, 3)
    assert idx[0, 0, q].tolist() == [3, 1, 2]            # local first (+inf), then tie -> lower index
    # row in block 0 has a single visible block: remaining slots are the sentinel NB
    sc[0, 0, 7, 0] = 0.25
    idx = O.stable_topk(sc, 3)
    assert idx[0, 0, 7].tolist() == [0, nb, nb]


def test_reverse_index_is_canonical():
    qp, kp, *_ = O.make_inputs(2, 640, 4, 2, 4, 2, seed=5)
    idx, _ = O.select_blocks(qp, kp, SCALE, 3)
    nb = 5
    row_ptr, col_q, edge_pos = O.reverse_index(idx, nb)
    b, hp, s, kb = idx.shape
    assert row_ptr[0].item() == 0 and row_ptr[-1].item() == col_q.numel()
    seen = 0
    for bp in range(b * hp):
        for j in range(nb):
            lo, hi = row_ptr[bp * nb + j].item(), row_ptr[bp * nb + j + 1].item()
            qs = col_q[lo:hi]
            assert (qs[1:] > qs[:-1]).all()                        # ascending, unique
            assert (qs // 128 >= j).all()                          # causal
            want = ((idx.view(b * hp, s, kb)[bp] == j).any(-1)).nonzero().squeeze(1)
            assert torch.equal(qs.long(), want)
            seen += hi - lo
    assert seen == col_q.numel()
    valid = edge_pos >= 0
    assert valid.sum().item() == col_q.numel()
    # edge_pos inverts col_q
    qgrid = torch.arange(s).view(1, 1, s, 1).expand_as(idx)
    assert torch.equal(col_q[edge_pos[valid].long()].long(), qgrid[valid])


def test_flop_count_config2():
    assert O.pairs_selected(8192, 16) == 14290944
    assert abs(O.flops_sparse_fwd_bwd(2, 8192, 32, 16) - 1.639e12) < 1e9


def test_row_reference_matches_full_oracle():
    """The one-row restatement (used for parity at sequence lengths where the full eager model does not
    fit) agrees with the full closed-form oracle, which is pinned against the reference above."""
    b, s, hq, hkv, hp, hpkv, kb = 2, 512, 8, 2, 4, 2, 2
    qp, kp, q, k, v, do = O.make_inputs(b, s, hq, hkv, hp, hpkv, seed=3)
    r = O.sparse_forward_backward(qp, kp, q, k, v, kb * 128, 128 ** -0.5, do, 0.7)
    idx, mpp = r["block_indices"], hq // hp
    kl_rows = 0.0
    for bb, p, qpos in [(0, 0, 0), (1, 3, 200), (0, 2, 511), (1, 1, 128)]:
        rr = O.row_reference(qp, kp, q, k, v, do, 128 ** -0.5, bb, p, qpos, idx[bb, p, qpos], 0.7)
        heads = slice(p * mpp, (p + 1) * mpp)
        assert (r["out"][bb, qpos].view(hq, 128)[heads] - rr["out"]).abs().max() < 2e-6
        assert (r["lse"][bb, heads, qpos] - rr["lse"]).abs().max() < 2e-6
        assert (r["lse_proxy"][bb, p, qpos] - rr["lse_proxy"]).abs() < 2e-6
        assert (r["dq"][bb, heads, qpos] - rr["dq"]).abs().max() < 2e-6
        assert (r["dq_proxy"][bb, p, qpos] - rr["dq_proxy"]).abs().max() < 1e-6 * r["dq_proxy"].abs().max()
        sc = O.proxy_block_scores(qp, kp, 128 ** -0.5)[bb, p, qpos, : qpos // 128 + 1]
        assert (sc - rr["block_scores"]).abs().max() < 2e-6
        kl_rows += rr["kl"].item()
    assert kl_rows > 0.0


def test_key_block_reference_matches_the_full_restatement():
    """The per-key-block restatement (used at sequence lengths where the eager model does not fit) gives the
    dK, dV and dKp slices of the full closed-form oracle."""
    qp, kp, q, k, v, do = O.make_inputs(2, 768, 8, 2, 4, 2, seed=3)
    scale, kb = 128 ** -0.5, 3
    idx, _ = O.select_blocks(qp, kp, scale, kb)
    full = O.sparse_forward_backward(qp, kp, q, k, v, kb * 128, scale, do, 0.7, block_indices=idx)
    for b, kvh, j in [(0, 0, 0), (1, 1, 2), (0, 1, 5), (1, 0, 3)]:
        r = O.key_block_reference(qp, kp, q, k, v, do, scale, b, kvh, j, idx, 0.7, row_chunk=100)
        sl = slice(j * 128, (j + 1) * 128)
        assert (r["dv"] - full["dv"][b, kvh, sl]).abs().max().item() <= 1e-5
        assert (r["dk"] - full["dk"][b, kvh, sl]).abs().max().item() <= 1e-5
        for kph, t in r["dk_proxy"].items():
            assert (t - full["dk_proxy"][b, kph, sl]).abs().max().item() <= 1e-9


def test_document_masking_of_the_oracle():
    """Document masking (an extension: the reference has none) is pinned by its definition: with every block selected a
    packed sequence must give, document by document, plain dense causal attention; the closed-form gradients must equal
    autograd through the eager restatement; no row may select a block that lies entirely in an earlier document; and
    without documents nothing changes."""
    import torch
    from oracle import msa_oracle as O
    b, s, hq, hkv, hp, hpkv = 2, 512, 4, 2, 2, 1
    qp, kp, q, k, v, do = O.make_inputs(b, s, hq, hkv, hp, hpkv, seed=3)
    cu = [0, 100, 101, 333, 512]
    ds = O.doc_start_from_cu_seqlens(cu, s, b)
    assert ds[0, [0, 99, 100, 101, 332, 333, 511]].tolist() == [0, 0, 100, 101, 101, 333, 333]
    r0 = O.sparse_forward_backward(qp, kp, q, k, v, 256, 0.088, do, 1.0)
    r1 = O.sparse_forward_backward(qp, kp, q, k, v, 256, 0.088, do, 1.0, doc_start=torch.zeros(b, s, dtype=torch.int32))
    assert all(torch.equal(r0[n], r1[n]) for n in ("out", "dq", "dk", "dv", "dq_proxy", "dk_proxy"))
    r = O.sparse_forward_backward(qp, kp, q, k, v, 256, 0.088, do, 0.7, doc_start=ds, dtype=torch.float64)
    idx = r["block_indices"]
    out, kl, grads = O.eager_forward_backward(lambda *t: O.eager_sparse(*t, 256, 0.088, block_indices=idx, doc_start=ds),
                                              [t.double() for t in (qp, kp, q, k, v)], do.double(), 0.7)
    assert (out - r["out"]).abs().max().item() < 1e-12 and abs(kl.item() - r["kl"].item()) < 1e-12
    for n, g in zip(["dq_proxy", "dk_proxy", "dq", "dk", "dv"], grads):
        assert (g - r[n]).abs().max().item() < 1e-12, n
    nb = s // 128
    assert not bool(((idx < (ds // 128).view(b, 1, s, 1)) & (idx < nb)).any())
    dense = O.sparse_forward(qp, kp, q, k, v, s, 0.088, doc_start=ds, dtype=torch.float64)
    parts = []
    for a, e in zip(cu[:-1], cu[1:]):
        qq = q[:, :, a:e].double()
        kk = k[:, :, a:e].double().repeat_interleave(hq // hkv, 1)
        vv = v[:, :, a:e].double().repeat_interleave(hq // hkv, 1)
        att = (qq @ kk.transpose(-1, -2)) * 0.088
        att = att.masked_fill(torch.triu(torch.ones(e - a, e - a, dtype=torch.bool), 1), float("-inf"))
        parts.append((torch.softmax(att, -1) @ vv).transpose(1, 2).reshape(b, e - a, -1))
    assert (torch.cat(parts, 1) - dense["out"]).abs().max().item() < 1e-12


def test_doc_start_helper_matches_the_oracle_and_rejects_bad_packings():
    import pytest
    import torch
    from flash_msa_b200 import ops
    from oracle import msa_oracle as O
    for cu, b, s in (([0, 100, 101, 333, 512], 2, 512), ([[0, 130, 1024, 1024], [0, 5, 640, 1024]], 2, 1024), ([0, 256], 1, 256)):
        assert torch.equal(ops.doc_start_from_cu_seqlens(cu, b, s, "cpu"), O.doc_start_from_cu_seqlens(cu, s, b))
    for bad in ([1, 512], [0, 100], [0, 300, 200, 512], [[0, 512]] * 3):
        with pytest.raises(ValueError):
            ops.doc_start_from_cu_seqlens(bad, 2, 512, "cpu")


@pytest.mark.parametrize("warmup", [False, True])
def test_softmax_sinks_of_the_oracle(warmup):
    """Softmax sinks (an extension: the reference lists the softmax bias as missing) are pinned by their definition: the
    closed forms of the oracle - output, all five gradients, the gradient of the sinks - must equal autograd through the
    eager restatement, whose softmax simply gains one column per main head; and a sink of -inf changes nothing."""
    import torch
    from oracle import msa_oracle as O
    b, s, hq, hkv, hp, hpkv = 2, 384, 8, 2, 2, 1
    qp, kp, q, k, v, do = O.make_inputs(b, s, hq, hkv, hp, hpkv, seed=11)
    t64 = [t.double() for t in (qp, kp, q, k, v)]
    sinks = (torch.randn(hq, generator=torch.Generator().manual_seed(5), dtype=torch.float64) * 0.8 + 0.3).requires_grad_(True)
    if warmup:
        r = O.warmup_forward_backward(*t64, 0.088, do.double(), 0.6, dtype=torch.float64, sinks=sinks.detach())
        fn = lambda *t: O.eager_warmup(*t, 0.088, sinks=sinks)
        r_inf = O.warmup_forward_backward(*t64, 0.088, do.double(), 0.6, dtype=torch.float64,
                                          sinks=torch.full((hq,), float("-inf"), dtype=torch.float64))
        r_none = O.warmup_forward_backward(*t64, 0.088, do.double(), 0.6, dtype=torch.float64)
    else:
        r = O.sparse_forward_backward(*t64, 256, 0.088, do.double(), 0.6, dtype=torch.float64, sinks=sinks.detach())
        idx = r["block_indices"]
        fn = lambda *t: O.eager_sparse(*t, 256, 0.088, block_indices=idx, sinks=sinks)
        r_inf = O.sparse_forward_backward(*t64, 256, 0.088, do.double(), 0.6, dtype=torch.float64, block_indices=idx,
                                          sinks=torch.full((hq,), float("-inf"), dtype=torch.float64))
        r_none = O.sparse_forward_backward(*t64, 256, 0.088, do.double(), 0.6, dtype=torch.float64, block_indices=idx)
    out, kl, grads = O.eager_forward_backward(fn, t64, do.double(), 0.6, extra=[sinks])
    assert (out - r["out"]).abs().max().item() < 1e-11
    for n, g in zip(["dq_proxy", "dk_proxy", "dq", "dk", "dv", "dsinks"], grads):
        assert (g - r[n]).abs().max().item() < 1e-11, n
    assert r["dsinks"].abs().max().item() > 1e-3          # (the comparison above is not one of zeros)
    for n in ("out", "dq_proxy", "dk_proxy", "dq", "dk", "dv"):
        assert (r_inf[n] - r_none[n]).abs().max().item() < 1e-12, n


def test_fewer_proxy_heads_than_kv_heads_by_repetition():
    """Hp < Hkv (refused by the reference) is served by repeating every proxy query head Hkv/Hp times and summing the
    copies' gradients.  In fp64 on the oracle that must be the gradient of the model with the original head counts: the
    KL gradient is linear in the teacher, and the per-call factor 1/(B*Hp'*S) with Hp' = Hkv turns the copies'
    sub-means into the mean over all main heads of the proxy head."""
    import torch
    from oracle import msa_oracle as O
    b, s, hq, hkv, hp, hpkv = 2, 384, 8, 4, 2, 1
    qp, kp, q, k, v, do = [t.double() for t in O.make_inputs(b, s, hq, hkv, hp, hpkv, seed=13)]
    want_out, _, want = O.eager_forward_backward(lambda *t: O.eager_warmup(*t, 0.088), (qp, kp, q, k, v), do, 0.9)
    rep = hkv // hp
    r = O.warmup_forward_backward(qp.repeat_interleave(rep, dim=1), kp, q, k, v, 0.088, do, 0.9, dtype=torch.float64)
    assert (r["out"] - want_out).abs().max().item() < 1e-12
    got = [r["dq_proxy"].view(b, hp, rep, s, -1).sum(2), r["dk_proxy"], r["dq"], r["dk"], r["dv"]]
    for n, g, w in zip(["dq_proxy", "dk_proxy", "dq", "dk", "dv"], got, want):
        assert (g - w).abs().max().item() < 1e-11, n
