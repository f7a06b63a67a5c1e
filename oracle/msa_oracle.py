"""CPU oracle for the Flash-MSA training hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch (fp32 by default, fp64 on request), the
algorithm of the reference's eager MSA model.  It is the checker used by the
parity tests, by the smoke test and by the CPU-baseline leg of the benchmark.
It is never imported by the product package, which has no CPU path at all.

Parity status: PINNED.  ``tests/golden/make_golden.py`` runs the reference's own
``Model._attention_eager`` / ``WarmupModel._attention_eager`` (imported from the
reference tree) on seeded inputs and stores their outputs and autograd
gradients; ``tests/test_oracle_golden.py`` checks every function below against
those stored vectors.

Reference lines followed (paths inside the reference project):

* proxy scores, causal mask, max-pool, forced local block:
  flash_msa/tests/testing_model.py:75-94
* top-k: testing_model.py:96, with two documented differences: ties are broken
  towards the LOWER block index (the reference kernel's order,
  flash_msa/msa_select_cutedsl.py:370-392) by a stable descending sort, and
  slots that hold no causally valid block carry the sentinel ``NB`` (the
  kernel's convention, msa_select_cutedsl.py:219-225) instead of whatever
  ``torch.topk`` returns for ``-inf`` entries, which ``tril`` masks out anyway
  (testing_model.py:113).
* reverse index validity rule ``0 <= kb < NB and kb <= q // 128``:
  flash_msa/csrc/reverse_index_cuda.cu:41
* main sparse attention: testing_model.py:118-126
* KL term and its detached target: testing_model.py:128-167
* warmup (dense causal main + full-sequence proxy KL):
  flash_msa/tests/testing_model_warmup.py:63-104
* closed-form gradients: flash_msa/msa_backward_cutedsl.py:456-733 (P, dP, dS,
  dV, dK, dQ, teacher, ds_px, dQp, dKp) and flash_msa/flash_msa.py:99-125
  (delta, 1/(B*Hp*S) normalisation, grad_kl multiplier).
"""

from __future__ import annotations

import math
from typing import Optional

import torch

BLOCK = 128


# ----------------------------------------------------------------------------
# selection
# ----------------------------------------------------------------------------

def doc_start_from_cu_seqlens(cu_seqlens, s: int, b: int = 1) -> torch.Tensor:
    """``[B,S]`` int32: for every token of a packed sequence the position of the first token of its
    document.  ``cu_seqlens`` is ``[n+1]`` (the same packing for every batch element) or ``[B,n+1]``,
    starts at 0 and ends at ``s`` (the FlashAttention varlen convention)."""
    cu = torch.as_tensor(cu_seqlens, dtype=torch.int64)
    if cu.dim() == 1:
        cu = cu.unsqueeze(0).expand(b, -1)
    pos = torch.arange(s, dtype=torch.int64)
    out = torch.empty(b, s, dtype=torch.int32)
    for i in range(b):
        c = cu[i].contiguous()
        if int(c[0]) != 0 or int(c[-1]) != s or bool((c[1:] < c[:-1]).any()):
            raise ValueError("cu_seqlens must rise from 0 to the sequence length")
        which = torch.searchsorted(c, pos, right=True) - 1
        out[i] = c[which].to(torch.int32)
    return out


def _lo(doc_start, b, rows, dev):
    """[B,1,len(rows),1] first visible key of the query rows (0 without documents)."""
    if doc_start is None:
        return torch.zeros(b, 1, rows.stop - rows.start, 1, dtype=torch.int64, device=dev)
    return doc_start[:, rows].to(device=dev, dtype=torch.int64).view(b, 1, -1, 1)


def proxy_block_scores(q_proxy: torch.Tensor, k_proxy: torch.Tensor, scale: float,
                       dtype=torch.float32, doc_start=None) -> torch.Tensor:
    """``[B,Hp,S,NB]`` block scores: max over the causally visible keys of each
    128-key block of ``scale * Qp . Kp`` (testing_model.py:75-88).  Blocks that lie
    entirely in the future hold ``-inf``.  The local block is NOT forced here.
    ``doc_start`` ([B,S], see doc_start_from_cu_seqlens) additionally hides the keys before the row's
    own document (document masking of a packed sequence: an extension, the reference has none);
    blocks that lie entirely before the document hold ``-inf``."""
    b, hp, s, d = q_proxy.shape
    hpkv = k_proxy.shape[1]
    pg = hp // hpkv
    nb = s // BLOCK
    out = torch.full((b, hp, s, nb), float("-inf"), dtype=dtype, device=q_proxy.device)
    kf = k_proxy.to(dtype)
    for i in range(nb):
        rows = slice(i * BLOCK, (i + 1) * BLOCK)
        qf = q_proxy[:, :, rows].to(dtype)                      # [B,Hp,128,D]
        keys = kf[:, :, : (i + 1) * BLOCK]                      # [B,Hpkv,n,D]
        keys = keys.repeat_interleave(pg, dim=1)
        sc = torch.matmul(qf, keys.transpose(-1, -2)) * scale   # [B,Hp,128,n]
        qpos = torch.arange(i * BLOCK, (i + 1) * BLOCK, device=sc.device).view(-1, 1)
        kpos = torch.arange((i + 1) * BLOCK, device=sc.device).view(1, -1)
        sc = sc.masked_fill((kpos > qpos) | (kpos.view(1, 1, 1, -1) < _lo(doc_start, b, rows, sc.device)), float("-inf"))
        out[:, :, rows, : i + 1] = sc.view(b, hp, BLOCK, i + 1, BLOCK).amax(dim=-1)
    return out


def force_local_block(block_scores: torch.Tensor) -> torch.Tensor:
    """Set the score of each row's own block to ``+inf`` (testing_model.py:90-94)."""
    b, hp, s, nb = block_scores.shape
    local = (torch.arange(s, device=block_scores.device) // BLOCK).view(1, 1, s, 1)
    return block_scores.scatter(3, local.expand(b, hp, s, 1), float("inf"))


def stable_topk(block_scores: torch.Tensor, top_k_blocks: int) -> torch.Tensor:
    """Per-row top-k over ``[B,Hp,S,NB]`` scores with the total order
    (score descending, block index ascending).  The local block is forced first.
    Slots without a causally valid block carry the sentinel ``NB``.  int32."""
    b, hp, s, nb = block_scores.shape
    forced = force_local_block(block_scores)
    order = torch.sort(forced, dim=-1, descending=True, stable=True)
    idx = order.indices[..., :top_k_blocks]
    val = order.values[..., :top_k_blocks]
    qblk = (torch.arange(s, device=block_scores.device) // BLOCK).view(1, 1, s, 1)
    bad = (val == float("-inf")) | (idx > qblk)
    idx = idx.masked_fill(bad, nb)
    return idx.to(torch.int32)


def select_blocks(q_proxy, k_proxy, scale, top_k_blocks, dtype=torch.float32, doc_start=None):
    """Scores + stable top-k.  Returns ``(block_indices, block_scores)``."""
    sc = proxy_block_scores(q_proxy, k_proxy, scale, dtype=dtype, doc_start=doc_start)
    return stable_topk(sc, top_k_blocks), sc


def near_tie_report(block_scores: torch.Tensor, top_k_blocks: int, eps: float) -> dict:
    """How fragile is the selection: number of rows whose k-th and (k+1)-th
    best finite scores differ by less than ``eps``."""
    forced = force_local_block(block_scores)
    vals = torch.sort(forced, dim=-1, descending=True, stable=True).values
    if vals.shape[-1] <= top_k_blocks:
        return {"rows": int(vals[..., 0].numel()), "near_ties": 0, "eps": eps}
    a = vals[..., top_k_blocks - 1]
    c = vals[..., top_k_blocks]
    both = torch.isfinite(a) & torch.isfinite(c)
    near = both & ((a - c).abs() < eps)
    return {"rows": int(a.numel()), "near_ties": int(near.sum()), "eps": eps}


# ----------------------------------------------------------------------------
# reverse index (canonical deterministic CSR)
# ----------------------------------------------------------------------------

def reverse_index(block_indices: torch.Tensor, num_blocks: int):
    """Canonical CSR of the selection.

    Row ``(b*Hp + p)*NB + kb`` lists, in ascending order, the query positions
    that selected key block ``kb``.  An entry is an edge iff ``0 <= kb < NB``
    and ``kb <= q // 128`` (reverse_index_cuda.cu:41).

    Returns ``(row_ptr int32 [B*Hp*NB+1], col_q int32 [E], edge_pos int32
    [B,Hp,S,Kb])``; ``edge_pos`` maps a slot to its CSR position (-1 if the slot
    is not an edge), the analogue of ``edge_positions`` at
    reverse_index_cuda.cu:231.
    """
    b, hp, s, kb = block_indices.shape
    nb = num_blocks
    idx = block_indices.to(torch.int64)
    q = torch.arange(s, device=idx.device).view(1, 1, s, 1).expand_as(idx)
    valid = (idx >= 0) & (idx < nb) & (idx <= q // BLOCK)
    bp = torch.arange(b * hp, device=idx.device).view(b, hp, 1, 1).expand_as(idx)
    bucket = (bp * nb + idx.clamp(0, nb - 1))
    # sort key: (bucket, q); slots of one row hold distinct blocks, so (bucket,q) is unique
    key = bucket * s + q
    key_v = key[valid]
    flat_pos = torch.nonzero(valid.reshape(-1), as_tuple=False).squeeze(1)
    order = torch.argsort(key_v, stable=True)
    e = int(key_v.numel())
    col_q = (key_v[order] % s).to(torch.int32)
    counts = torch.bincount(bucket[valid], minlength=b * hp * nb)
    row_ptr = torch.zeros(b * hp * nb + 1, dtype=torch.int64, device=idx.device)
    row_ptr[1:] = torch.cumsum(counts, 0)
    edge_pos = torch.full((b * hp * s * kb,), -1, dtype=torch.int32, device=idx.device)
    edge_pos[flat_pos[order]] = torch.arange(e, dtype=torch.int32, device=idx.device)
    return row_ptr.to(torch.int32), col_q, edge_pos.view(b, hp, s, kb)


# ----------------------------------------------------------------------------
# masks
# ----------------------------------------------------------------------------

def _row_token_mask(block_indices_rows: torch.Tensor, q0: int, nkeys: int, nb: int):
    """``[...,128,nkeys]`` bool: key visible to the row (selected block, causal)."""
    rows = block_indices_rows.shape[-2]
    dev = block_indices_rows.device
    bm = torch.zeros(block_indices_rows.shape[:-1] + (nb + 1,), dtype=torch.bool, device=dev)
    bm.scatter_(-1, block_indices_rows.to(torch.int64).clamp(0, nb), True)
    bm = bm[..., : nkeys // BLOCK]
    tm = bm.unsqueeze(-1).expand(bm.shape + (BLOCK,)).reshape(bm.shape[:-1] + (nkeys,))
    qpos = torch.arange(q0, q0 + rows, device=dev).view(-1, 1)
    kpos = torch.arange(nkeys, device=dev).view(1, -1)
    return tm & (kpos <= qpos)


# ----------------------------------------------------------------------------
# forward / backward closed forms, chunked over query blocks
# ----------------------------------------------------------------------------

def _run(q_proxy, k_proxy, q, k, v, scale, block_indices, d_out, grad_kl, dtype,
         want_grads: bool, doc_start=None, sinks=None):
    """Shared worker.  ``block_indices is None`` means warmup (every causal block)."""
    b, hq, s, d = q.shape
    hkv = k.shape[1]
    hp = q_proxy.shape[1]
    hpkv = k_proxy.shape[1]
    nb = s // BLOCK
    mpp = hq // hp          # main heads per proxy head
    g = hq // hkv           # main heads per KV head
    pg = hp // hpkv         # proxy heads per proxy-K head
    dev = q.device

    qf, kf, vf = q.to(dtype), k.to(dtype), v.to(dtype)
    qpf, kpf = q_proxy.to(dtype), k_proxy.to(dtype)

    out = torch.empty(b, s, hq * d, dtype=dtype, device=dev)
    lse = torch.empty(b, hq, s, dtype=dtype, device=dev)
    lse_p = torch.empty(b, hp, s, dtype=dtype, device=dev)
    kl_sum = torch.zeros((), dtype=torch.float64, device=dev)

    if want_grads:
        dq = torch.zeros_like(qf)
        dk = torch.zeros_like(kf)
        dv = torch.zeros_like(vf)
        dqp = torch.zeros_like(qpf)
        dkp = torch.zeros_like(kpf)
        do = d_out.to(dtype).reshape(b, s, hq, d).permute(0, 2, 1, 3)   # [B,Hq,S,D]
        cnorm = 1.0 / float(b * hp * s)
        gk = None if grad_kl is None else float(grad_kl)
        dsink = torch.zeros(hq, dtype=dtype, device=dev)

    for i in range(nb):
        rows = slice(i * BLOCK, (i + 1) * BLOCK)
        n = (i + 1) * BLOCK
        if block_indices is None:
            qpos = torch.arange(i * BLOCK, (i + 1) * BLOCK, device=dev).view(-1, 1)
            kpos = torch.arange(n, device=dev).view(1, -1)
            vis_p = (kpos <= qpos).view(1, 1, BLOCK, n).expand(b, hp, BLOCK, n)
        else:
            vis_p = _row_token_mask(block_indices[:, :, rows], i * BLOCK, n, nb)   # [B,Hp,128,n]
        if doc_start is not None:
            vis_p = vis_p & (torch.arange(n, device=dev).view(1, 1, 1, -1) >= _lo(doc_start, b, rows, dev))
        vis = vis_p.repeat_interleave(mpp, dim=1)                                   # [B,Hq,128,n]

        kk = kf[:, :, :n].repeat_interleave(g, dim=1)           # [B,Hq,n,D]
        vv = vf[:, :, :n].repeat_interleave(g, dim=1)
        sc = torch.matmul(qf[:, :, rows], kk.transpose(-1, -2)) * scale
        sc = sc.masked_fill(~vis, float("-inf"))
        l = torch.logsumexp(sc, dim=-1)                         # [B,Hq,128]
        if sinks is not None:
            # softmax bias ("attention sink", an extension: the reference has none): one learnable logit per main head
            # joins the softmax denominator and takes probability mass without contributing a value
            l = torch.logaddexp(l, sinks.to(dtype).view(1, hq, 1).expand_as(l))
        p = torch.exp(sc - l.unsqueeze(-1))
        o = torch.matmul(p, vv)                                 # [B,Hq,128,D]
        out[:, rows] = o.permute(0, 2, 1, 3).reshape(b, BLOCK, hq * d)
        lse[:, :, rows] = l

        kkp = kpf[:, :, :n].repeat_interleave(pg, dim=1)        # [B,Hp,n,D]
        sp = torch.matmul(qpf[:, :, rows], kkp.transpose(-1, -2)) * scale
        sp = sp.masked_fill(~vis_p, float("-inf"))
        lp = torch.logsumexp(sp, dim=-1)
        lse_p[:, :, rows] = lp
        logp = sp - lp.unsqueeze(-1)
        teacher = p.view(b, hp, mpp, BLOCK, n).mean(dim=2)      # [B,Hp,128,n]
        # sum_k t*(log t - log p) with 0*log0 = 0 (testing_model.py:163-167)
        term = torch.where(teacher > 0, teacher * (torch.log(teacher.clamp_min(1e-300 if dtype == torch.float64 else 1e-38))
                                                   - logp.masked_fill(~vis_p, 0.0)),
                           torch.zeros_like(teacher))
        kl_sum += term.sum().to(torch.float64)

        if want_grads:
            dob = do[:, :, rows]                                # [B,Hq,128,D]
            dp = torch.matmul(dob, vv.transpose(-1, -2))        # [B,Hq,128,n]
            delta = (o * dob).sum(-1, keepdim=True)
            ds = p * (dp - delta)                               # dL/d(scaled logits)
            if sinks is not None:   # the sink's probability times (its zero value's dP - delta)
                dsink -= (torch.exp(sinks.to(dtype).view(1, hq, 1) - l) * delta.squeeze(-1)).sum(dim=(0, 2))
            dq[:, :, rows] = torch.matmul(ds, kk) * scale
            dk_h = torch.matmul(ds.transpose(-1, -2), qf[:, :, rows]) * scale   # [B,Hq,n,D]
            dv_h = torch.matmul(p.transpose(-1, -2), dob)
            dk[:, :, :n] += dk_h.view(b, hkv, g, n, d).sum(2)
            dv[:, :, :n] += dv_h.view(b, hkv, g, n, d).sum(2)
            if gk is not None:
                ppx = torch.exp(logp).masked_fill(~vis_p, 0.0)
                if sinks is None:
                    dsp = (ppx - teacher) * (cnorm * gk)
                else:   # the teacher's rows no longer sum to one: d/dz_j of -sum_k t_k log p_k = (sum_k t_k) p_j - t_j
                    dsp = (ppx * teacher.sum(-1, keepdim=True) - teacher) * (cnorm * gk)
                dqp[:, :, rows] = torch.matmul(dsp, kkp) * scale
                dkp_h = torch.matmul(dsp.transpose(-1, -2), qpf[:, :, rows]) * scale
                dkp[:, :, :n] += dkp_h.view(b, hpkv, pg, n, d).sum(2)

    kl = (kl_sum / float(b * hp * s)).to(dtype)
    res = {"out": out, "lse": lse, "lse_proxy": lse_p, "kl": kl}
    if want_grads:
        res.update({"dq": dq, "dk": dk, "dv": dv, "dq_proxy": dqp, "dk_proxy": dkp})
        if sinks is not None:
            res["dsinks"] = dsink
    return res


def sparse_forward(q_proxy, k_proxy, q, k, v, top_k, scale, block_indices=None,
                   dtype=torch.float32, doc_start=None):
    """Sparse MSA forward.  Returns dict(out [B,S,Hq*D], lse [B,Hq,S], lse_proxy
    [B,Hp,S], kl scalar, block_indices)."""
    kb = int(top_k) // BLOCK
    if block_indices is None:
        block_indices, _ = select_blocks(q_proxy, k_proxy, scale, kb, dtype=dtype, doc_start=doc_start)
    r = _run(q_proxy, k_proxy, q, k, v, scale, block_indices, None, None, dtype, False, doc_start=doc_start)
    r["block_indices"] = block_indices
    return r


def sparse_forward_backward(q_proxy, k_proxy, q, k, v, top_k, scale, d_out,
                            grad_kl: Optional[float] = 1.0, block_indices=None,
                            dtype=torch.float32, doc_start=None, sinks=None):
    """Forward plus closed-form gradients of ``sum(out*d_out) + grad_kl*kl``."""
    kb = int(top_k) // BLOCK
    if block_indices is None:
        block_indices, _ = select_blocks(q_proxy, k_proxy, scale, kb, dtype=dtype, doc_start=doc_start)
    r = _run(q_proxy, k_proxy, q, k, v, scale, block_indices, d_out, grad_kl, dtype, True, doc_start=doc_start, sinks=sinks)
    r["block_indices"] = block_indices
    return r


def warmup_forward(q_proxy, k_proxy, q, k, v, scale, dtype=torch.float32, doc_start=None):
    """Dense causal main attention + full-sequence proxy statistics."""
    return _run(q_proxy, k_proxy, q, k, v, scale, None, None, None, dtype, False, doc_start=doc_start)


def warmup_forward_backward(q_proxy, k_proxy, q, k, v, scale, d_out,
                            grad_kl: Optional[float] = 1.0, dtype=torch.float32, doc_start=None, sinks=None):
    return _run(q_proxy, k_proxy, q, k, v, scale, None, d_out, grad_kl, dtype, True, doc_start=doc_start, sinks=sinks)


# ----------------------------------------------------------------------------
# eager restatement (materialises S x S; autograd) - used to cross-check the
# closed forms above and as the timed CPU baseline, because it is what the
# reference's own tests run.
# ----------------------------------------------------------------------------

def _softmax_with_sinks(attn, sinks):
    """Row softmax whose denominator also holds exp(sink) of the row's head (attn [B,H,S,S], sinks [H])."""
    if sinks is None:
        return torch.softmax(attn, dim=-1)
    col = sinks.to(attn.dtype).view(1, -1, 1, 1).expand(attn.shape[0], -1, attn.shape[2], 1)
    return torch.softmax(torch.cat([attn, col], dim=-1), dim=-1)[..., :-1]


def eager_sparse(q_proxy, k_proxy, q, k, v, top_k, scale, block_indices=None, doc_start=None, sinks=None):
    """Line-by-line restatement of testing_model.py:61-169 with stable top-k (or a given
    selection).  Differentiable; returns ``(attn_out [B,S,Hq*D], kl_loss)``."""
    b, hp, s, d = q_proxy.shape
    hq, hkv, hpkv = q.shape[1], k.shape[1], k_proxy.shape[1]
    nb = s // BLOCK
    kb = int(top_k) // BLOCK
    mpp, g, pg = hq // hp, hq // hkv, hp // hpkv
    dev = q.device

    kp = k_proxy.repeat_interleave(pg, dim=1)
    proxy_scores = torch.matmul(q_proxy, kp.transpose(-2, -1)) * scale
    future = torch.triu(torch.ones(s, s, device=dev, dtype=torch.bool), diagonal=1)
    if doc_start is not None:   # document masking (extension): keys before the row's document are hidden as well
        other = torch.arange(s, device=dev).view(1, 1, 1, s) < doc_start.to(device=dev, dtype=torch.int64).view(b, 1, s, 1)
        future = future.view(1, 1, s, s) | other
    proxy_scores = proxy_scores.masked_fill(future, float("-inf"))
    block_scores = proxy_scores.view(b, hp, s, nb, BLOCK).amax(dim=-1)
    if block_indices is None:
        idx = stable_topk(block_scores.detach().float(), kb).to(torch.int64)        # sentinel nb
    else:
        idx = block_indices.to(torch.int64)
    block_mask = torch.zeros(b, hp, s, nb + 1, dtype=torch.bool, device=dev)
    block_mask.scatter_(3, idx, True)
    block_mask = block_mask[..., :nb]
    token_mask = block_mask.unsqueeze(-1).expand(b, hp, s, nb, BLOCK).reshape(b, hp, s, s)
    vis_p = token_mask & ~future
    vis = vis_p.repeat_interleave(mpp, dim=1)

    kk = k.repeat_interleave(g, dim=1)
    vv = v.repeat_interleave(g, dim=1)
    attn = torch.matmul(q, kk.transpose(-2, -1)) * scale
    attn = attn.masked_fill(~vis, float("-inf"))
    probs = _softmax_with_sinks(attn, sinks)
    out = torch.matmul(probs, vv).transpose(1, 2).reshape(b, s, -1)

    target = probs.view(b, hp, mpp, s, s).mean(dim=2).detach()
    logp = torch.log_softmax(proxy_scores.masked_fill(~vis_p, float("-inf")), dim=-1)
    logp = logp.masked_fill(~vis_p, 0.0)
    target = target.masked_fill(~vis_p, 0.0)
    kl = torch.nn.functional.kl_div(logp, target, reduction="none").sum(-1).mean()
    return out, kl


def eager_warmup(q_proxy, k_proxy, q, k, v, scale, doc_start=None, sinks=None):
    """Restatement of testing_model_warmup.py:63-104.  Differentiable."""
    b, hp, s, d = q_proxy.shape
    hq, hkv, hpkv = q.shape[1], k.shape[1], k_proxy.shape[1]
    mpp, g, pg = hq // hp, hq // hkv, hp // hpkv
    dev = q.device
    future = torch.triu(torch.ones(s, s, device=dev, dtype=torch.bool), diagonal=1)
    if doc_start is not None:   # document masking (extension): keys before the row's document are hidden as well
        other = torch.arange(s, device=dev).view(1, 1, 1, s) < doc_start.to(device=dev, dtype=torch.int64).view(b, 1, s, 1)
        future = future.view(1, 1, s, s) | other
    kp = k_proxy.repeat_interleave(pg, dim=1)
    proxy_scores = (torch.matmul(q_proxy, kp.transpose(-2, -1)) * scale).masked_fill(future, float("-inf"))
    kk = k.repeat_interleave(g, dim=1)
    vv = v.repeat_interleave(g, dim=1)
    attn = (torch.matmul(q, kk.transpose(-2, -1)) * scale).masked_fill(future, float("-inf"))
    probs = _softmax_with_sinks(attn, sinks)
    out = torch.matmul(probs, vv).transpose(1, 2).reshape(b, s, -1)
    target = probs.view(b, hp, mpp, s, s).mean(dim=2).detach().masked_fill(future, 0.0)
    logp = torch.log_softmax(proxy_scores, dim=-1).masked_fill(future, 0.0)
    kl = torch.nn.functional.kl_div(logp, target, reduction="none").sum(-1).mean()
    return out, kl


def eager_forward_backward(fn, tensors, d_out, grad_kl: Optional[float] = 1.0, extra=()):
    """Run a differentiable eager function and return its autograd gradients of
    ``sum(out*d_out) + grad_kl*kl`` w.r.t. (q_proxy,k_proxy,q,k,v), followed by those w.r.t. the
    tensors in ``extra`` (leaves that ``fn`` closes over, e.g. softmax sinks)."""
    leaves = [t.detach().clone().requires_grad_(True) for t in tensors]
    out, kl = fn(*leaves)
    loss = (out * d_out.to(out.dtype)).sum()
    if grad_kl is not None:
        loss = loss + float(grad_kl) * kl
    wrt = leaves + list(extra)
    grads = torch.autograd.grad(loss, wrt, allow_unused=True)
    grads = [torch.zeros_like(t) if gr is None else gr for gr, t in zip(grads, wrt)]
    return out.detach(), kl.detach(), grads


# --------------------------------------------------------------------------------------------
# one query position at a time (parity at sequence lengths where the full eager model does not fit)
# --------------------------------------------------------------------------------------------
def row_reference(q_proxy, k_proxy, q, k, v, d_out, scale, b, p, qpos, block_row, grad_kl=1.0,
                  rounded=False):
    """Forward and the row-local gradients of ONE query position (batch b, proxy head p, position
    qpos) whose selected key blocks are ``block_row`` (int tensor [Kb]; the sentinel NB marks unused
    slots).  Same formulas as ``_run`` (testing_model.py:77-167 restricted to one row), fp32.
    Everything that depends on this row only is returned: out [mpp,D], lse [mpp], lse_proxy, kl (the
    row's KL term), dq [mpp,D], dq_proxy [D] (dK, dV, dKp are sums over rows and are not row-local),
    and the row's causally visible proxy block scores [qpos//128+1].
    ``rounded=True`` rounds P, dS, dSp and the outputs to bf16 at the points where the reference kernels
    do (flash_msa/msa_backward_cutedsl.py:502-510, 675-679): the error yardstick."""
    bsz, hq, s, d = q.shape
    hkv, hp, hpkv = k.shape[1], q_proxy.shape[1], k_proxy.shape[1]
    mpp, grp, pg = hq // hp, hq // hkv, hp // hpkv
    nb = s // BLOCK
    f32 = torch.float32
    rnd = (lambda t: t.to(torch.bfloat16).to(f32)) if rounded else (lambda t: t)
    blocks = [int(x) for x in block_row.tolist() if 0 <= int(x) < nb]
    tok = torch.cat([torch.arange(j * BLOCK, min((j + 1) * BLOCK, qpos + 1), device=q.device) for j in sorted(blocks)])
    kph = p // pg
    kp_sel = k_proxy[b, kph, tok].to(f32)
    sp = (kp_sel @ q_proxy[b, p, qpos].to(f32)) * scale
    lse_p = torch.logsumexp(sp, 0)
    p_px = torch.exp(sp - lse_p)
    outs, lses, dqs, probs = [], [], [], []
    for i in range(mpp):
        h = p * mpp + i
        kvh = h // grp
        k_sel, v_sel = k[b, kvh, tok].to(f32), v[b, kvh, tok].to(f32)
        sc = (k_sel @ q[b, h, qpos].to(f32)) * scale
        lse = torch.logsumexp(sc, 0)
        pr = torch.exp(sc - lse)
        o = rnd(pr) @ v_sel
        do = d_out[b, qpos, h * d:(h + 1) * d].to(f32)
        dp = v_sel @ do
        delta = (rnd(o) * do).sum()
        ds = rnd(pr * (dp - delta))
        outs.append(rnd(o))
        lses.append(lse)
        dqs.append(rnd((ds @ k_sel) * scale))
        probs.append(pr)
    teacher = torch.stack(probs).mean(0)
    kl_row = torch.where(teacher > 0, teacher * (torch.log(teacher.clamp_min(1e-45)) - (sp - lse_p)), torch.zeros_like(teacher)).sum()
    gk = 0.0 if grad_kl is None else float(grad_kl)
    dsp = rnd(p_px - teacher) * (gk / float(bsz * hp * s))
    dqp = rnd((dsp @ kp_sel) * scale)
    allk = k_proxy[b, kph, : qpos + 1].to(f32)
    full = (allk @ q_proxy[b, p, qpos].to(f32)) * scale
    nvis = qpos // BLOCK + 1
    pad = nvis * BLOCK - full.numel()
    blk = torch.cat([full, full.new_full((pad,), float("-inf"))]).view(nvis, BLOCK).amax(-1)
    return {"out": torch.stack(outs), "lse": torch.stack(lses), "lse_proxy": lse_p, "kl": kl_row, "dq": torch.stack(dqs),
            "dq_proxy": dqp, "block_scores": blk}


def key_block_reference(q_proxy, k_proxy, q, k, v, d_out, scale, b, kvh, j, block_indices, grad_kl=1.0,
                        rounded=False, row_chunk=128):
    """The column-wise twin of ``row_reference``: the gradients that belong to ONE key block j of KV head
    kvh of batch b, summed over every query row that selected it (all proxy heads of the KV group, all their
    main heads): dv [128,D], dk [128,D] and dk_proxy {proxy-K head: [128,D]}.  Closed forms of the reference
    kernel (flash_msa/msa_backward_cutedsl.py:512-551 for dV, dK; :709-733 for dKp), with each row's softmax
    statistics recomputed from its own selected blocks (``block_indices`` [B,Hp,S,Kb]).  Rows are processed
    ``row_chunk`` at a time against the gathered keys of their own selected blocks, so this also runs at
    sequence lengths where the full eager model does not fit.  ``rounded=True`` rounds P, dS, dSp and out to
    bf16 at the points where the reference kernels do: the error yardstick."""
    bsz, hq, s, d = q.shape
    hkv, hp, hpkv = k.shape[1], q_proxy.shape[1], k_proxy.shape[1]
    mpp, ppk, pg = hq // hp, hp // hkv, hp // hpkv
    nb = s // BLOCK
    kb = block_indices.shape[-1]
    f32 = torch.float32
    dev = q.device
    rnd = (lambda t: t.to(torch.bfloat16).to(f32)) if rounded else (lambda t: t)
    gk = 0.0 if grad_kl is None else float(grad_kl)
    dv = torch.zeros(BLOCK, d, dtype=f32, device=dev)
    dk = torch.zeros(BLOCK, d, dtype=f32, device=dev)
    dkp = {}
    inblk = torch.arange(BLOCK, device=dev)
    for p in range(kvh * ppk, (kvh + 1) * ppk):
        kph = p // pg
        idx_p = block_indices[b, p].to(dev).long()                  # [S, Kb]
        qblk = torch.arange(s, device=dev) // BLOCK
        rows_all = torch.nonzero(((idx_p == j).any(-1)) & (qblk >= j)).flatten()
        acc_kp = dkp.setdefault(kph, torch.zeros(BLOCK, d, dtype=f32, device=dev))
        for r0 in range(0, rows_all.numel(), row_chunk):
            rows = rows_all[r0:r0 + row_chunk]
            nr = rows.numel()
            sel = idx_p[rows]                                        # [R, Kb]
            tok = sel[:, :, None] * BLOCK + inblk[None, None, :]     # [R, Kb, 128]
            valid = ((sel >= 0) & (sel < nb))[:, :, None] & (tok <= rows[:, None, None])
            tokc = tok.clamp(0, s - 1).view(nr, kb * BLOCK)
            valid = valid.view(nr, kb * BLOCK)
            jpos = (sel == j).float().argmax(1)                      # slot of block j in each row's list
            ar = torch.arange(nr, device=dev)
            pick = lambda t: t.view(nr, kb, BLOCK)[ar, jpos]         # [R, 128]: the part that belongs to block j
            mj = pick(valid)
            kp_sel = k_proxy[b, kph][tokc].to(f32)                   # [R, T, D]
            sp = torch.einsum("rd,rtd->rt", q_proxy[b, p, rows].to(f32), kp_sel) * scale
            del kp_sel
            sp = sp.masked_fill(~valid, float("-inf"))
            p_px = pick(torch.exp(sp - torch.logsumexp(sp, 1, keepdim=True)))
            del sp
            k_sel = k[b, kvh][tokc].to(f32)
            v_sel = v[b, kvh][tokc].to(f32)
            v_j = v[b, kvh, j * BLOCK:(j + 1) * BLOCK].to(f32)
            teacher = torch.zeros(nr, BLOCK, dtype=f32, device=dev)
            for i in range(mpp):
                h = p * mpp + i
                qh = q[b, h, rows].to(f32)
                sc = torch.einsum("rd,rtd->rt", qh, k_sel) * scale
                sc = sc.masked_fill(~valid, float("-inf"))
                pr = torch.exp(sc - torch.logsumexp(sc, 1, keepdim=True))
                del sc
                o = torch.einsum("rt,rtd->rd", rnd(pr), v_sel)
                do = d_out[b, rows, h * d:(h + 1) * d].to(f32)
                delta = (rnd(o) * do).sum(1, keepdim=True)
                pj = pick(pr)
                del pr
                dsj = rnd(pj * (do @ v_j.t() - delta))
                dv += rnd(pj).t() @ do
                dk += (dsj.t() @ qh) * scale
                teacher += pj
            del k_sel, v_sel
            dsp = rnd(torch.where(mj, p_px - teacher / mpp, torch.zeros_like(p_px))) * (gk / float(bsz * hp * s))
            acc_kp += (dsp.t() @ q_proxy[b, p, rows].to(f32)) * scale
    return {"dv": rnd(dv), "dk": rnd(dk), "dk_proxy": {kk: rnd(t) for kk, t in dkp.items()}}


# ----------------------------------------------------------------------------
# synthetic workloads (shapes and value distributions of the benchmark configs)
# ----------------------------------------------------------------------------

def make_inputs(b, s, hq, hkv, hp, hpkv, d=128, seed=0, dtype=torch.float32,
                device="cpu", skew=False):
    """Seeded N(0,1) inputs generated in fp32 on the CPU generator, then cast.
    ``skew=True`` builds the block-mean + sink-block distribution of the skewed
    selection workload: K and Kp rows = per-block mean ~N(0,1) + N(0,0.5) noise,
    Qp x4, four random sink key blocks per sequence scaled x3."""
    gen = torch.Generator(device="cpu").manual_seed(seed)

    def rn(*shape):
        return torch.randn(*shape, generator=gen, dtype=torch.float32)

    qp, kp = rn(b, hp, s, d), rn(b, hpkv, s, d)
    q, k, v = rn(b, hq, s, d), rn(b, hkv, s, d), rn(b, hkv, s, d)
    do = rn(b, s, hq * d)
    if skew:
        nb = s // BLOCK
        for t, h in ((k, hkv), (kp, hpkv)):
            mean = rn(b, h, nb, 1, d)
            t.copy_((mean + 0.5 * t.view(b, h, nb, BLOCK, d)).view(b, h, s, d))
        qp.mul_(4.0)
        for bi in range(b):
            sinks = torch.randperm(nb, generator=gen)[:4]
            for j in sinks.tolist():
                k[bi, :, j * BLOCK:(j + 1) * BLOCK] *= 3.0
                kp[bi, :, j * BLOCK:(j + 1) * BLOCK] *= 3.0
    return tuple(t.to(dtype).to(device) for t in (qp, kp, q, k, v, do))


def pairs_selected(s: int, kb: int) -> int:
    """Unmasked (q,k) pairs per (batch, head) in the selected set:
    128*128*sum_i (min(i+1,Kb)-1) + NB*128*129/2."""
    nb = s // BLOCK
    full = sum(min(i + 1, kb) - 1 for i in range(nb))
    return BLOCK * BLOCK * full + nb * BLOCK * (BLOCK + 1) // 2


def flops_sparse_fwd_bwd(b, s, hq, kb, d=128) -> float:
    """Headline numerator: 7 GEMM passes (2 fwd + 5 bwd) over the selected pairs."""
    return 7.0 * 2.0 * d * pairs_selected(s, kb) * b * hq


def flops_warmup_fwd_bwd(b, s, hq, d=128) -> float:
    return 7.0 * 2.0 * d * (s * (s + 1) // 2) * b * hq
