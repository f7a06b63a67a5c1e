"""Autograd boundary: the reference's public functions with the same arguments, layouts, return
values and error behaviour (flash_msa/flash_msa.py:19-64, 129-278;
flash_msa/warmup/flash_msa_warmup.py:6-106), on top of the sm_100a kernels."""
from __future__ import annotations

import torch

from . import ops

BLOCK_SIZE = 128
MAX_TOP_K_BLOCKS = 128

# The device status word of every call (a bounded wait that ran out, a bad index in metadata) is checked
# without synchronising: it is copied to pinned memory behind the call and looked at by the next call of the
# library, which raises RuntimeError then; `check_pending_status()` waits for everything queued so far.
# DEBUG_CHECK_STATUS = True reads the word right after every call instead (synchronises; for debugging).
DEBUG_CHECK_STATUS = False


def _validate_inputs(q_proxy, k_proxy, q, k, v, top_k, sparse: bool):
    if q_proxy.ndim != 4 or k_proxy.ndim != 4 or q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("all attention tensors must have shape (B, H, S, D)")
    b, n_proxy_heads, s, head_dim = q_proxy.shape
    bk, n_proxy_kv_heads, sk, dk = k_proxy.shape
    bq, n_heads, sq, dq = q.shape
    bm, n_kv_heads, sm, dm = k.shape
    bv, n_v_heads, sv, dv = v.shape
    if not (b == bk == bq == bm == bv and s == sk == sq == sm == sv and head_dim == dk == dq == dm == dv
            and n_kv_heads == n_v_heads):
        raise ValueError("q_proxy, k_proxy, q, k, and v must agree on batch, sequence, head dimension, "
                         "and KV head count")
    if s % BLOCK_SIZE != 0:
        raise ValueError(f"sequence length must be divisible by {BLOCK_SIZE}, got {s}")
    if n_proxy_heads % n_proxy_kv_heads != 0:
        raise ValueError("n_proxy_heads must be divisible by n_proxy_kv_heads")
    if n_heads % n_kv_heads != 0:
        raise ValueError("n_heads must be divisible by n_kv_heads")
    if n_heads % n_proxy_heads != 0:
        raise ValueError("n_heads must be divisible by n_proxy_heads")
    if head_dim != 128:
        raise NotImplementedError("Headdim must be 128")
    if n_proxy_heads < n_kv_heads or n_proxy_heads % n_kv_heads != 0:
        raise NotImplementedError("n_proxy_heads must be a multiple of n_kv_heads")
    dts = {t.dtype for t in (q_proxy, k_proxy, q, k, v)}
    if len(dts) != 1 or q.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"flash_msa_b200 supports bf16 or fp16 activations of one dtype, got {sorted(map(str, dts))}")
    num_blocks = s // BLOCK_SIZE
    if not sparse:
        return num_blocks, 0
    if int(top_k) % BLOCK_SIZE != 0:
        raise ValueError(f"top_k must be divisible by {BLOCK_SIZE}, got {top_k}")
    top_k_blocks = int(top_k) // BLOCK_SIZE
    if not 1 <= top_k_blocks <= num_blocks:
        raise ValueError(f"top_k selects {top_k_blocks} blocks, but sequence has {num_blocks} blocks")
    if top_k_blocks > MAX_TOP_K_BLOCKS:
        raise NotImplementedError(f"No more than {MAX_TOP_K_BLOCKS} blocks / topk={MAX_TOP_K_BLOCKS * BLOCK_SIZE} supported")
    return num_blocks, top_k_blocks


def _require_cuda(q):
    if q.device.type != "cuda":
        raise RuntimeError("flash_msa_b200 requires CUDA tensors (there is no CPU path)")


# The reference returns a zero placeholder as kl_loss and users cannot watch the distillation loss
# (flash_msa/msa_forward_cutedsl.py:69).  With COMPUTE_KL_VALUE = True every backward that receives a
# gradient for kl_loss also computes the loss value inside the backward kernel (the teacher and the proxy
# probabilities are in registers there anyway); ``last_kl_value()`` returns it.
COMPUTE_KL_VALUE = False
_last_kl_value = None


def last_kl_value():
    """0-dim fp32 CUDA tensor: the KL loss of the most recent backward that ran with
    ``COMPUTE_KL_VALUE = True`` (mean over batch, proxy heads and rows of KL(teacher || proxy), the
    value of the reference's eager model, flash_msa/tests/testing_model.py:158-167).  None before the
    first such backward.  Reading it does not synchronise; ``.item()`` does."""
    return _last_kl_value


def _kl_buffer(grad_kl, device):
    if COMPUTE_KL_VALUE and grad_kl is not None:
        return torch.zeros(1, dtype=torch.float32, device=device)
    return None


def _publish_kl(buf):
    global _last_kl_value
    if buf is not None:
        _last_kl_value = buf.reshape(())


def _maybe_check(status, what):
    if DEBUG_CHECK_STATUS:
        ops.check_status(status, what)
    else:
        ops.deferred_status.push(status, what)


def check_pending_status():
    """Waits for the status words of all calls issued so far and raises RuntimeError for a non-zero one."""
    ops.deferred_status.drain()


# Softmax bias ("attention sink": one learnable logit per main head that joins the softmax denominator and takes
# probability mass without contributing a value; the reference lists it as missing).  It changes nothing but the
# normaliser of a row, so it is applied around the kernels: lse' = logaddexp(lse, sink) and out' = out * exp(lse - lse')
# after the forward; the backward runs on (out', lse') unchanged, because P = exp(s - lse') and delta = rowsum(out' dO)
# are exactly what it needs.  The KL teacher (mean of the main probabilities) then has rows that sum to
# T = mean_h exp(lse_h - lse'_h) < 1, and the gradient of -sum_k t_k log p_k becomes T p - t: the proxy log-sum-exp handed
# to the backward is lowered by log T, which scales the proxy probabilities by T.  The sink's own gradient is
# -sum over rows of exp(sink - lse') * delta.
def _apply_sinks(out, lse_main, lse_proxy, sinks, hp):
    b, hq, s = lse_main.shape
    sk = sinks.detach().float().view(1, hq, 1)
    lse2 = torch.logaddexp(lse_main, sk)
    keep = torch.exp(lse_main - lse2)                                      # 1 - probability of the sink, [B,Hq,S]
    out2 = (out.view(b, s, hq, -1).float() * keep.transpose(1, 2).unsqueeze(-1)).to(out.dtype).view(out.shape)
    lse_proxy2 = None
    if lse_proxy is not None:
        lse_proxy2 = lse_proxy - torch.log(keep.view(b, hp, hq // hp, s).mean(dim=2))
    return out2, lse2, lse_proxy2


def _sink_grad(out_kernel, grad_out, lse_main, sinks):
    """`out_kernel` is the output as the kernels wrote it (before the sink rescaling), `lse_main` the log-sum-exp WITH the
    sink.  delta is formed from out_kernel * (1 - p_sink) in fp32: the rescaled output that the backward kernels read
    has been rounded a second time, and the sum over all rows of a head amplifies that (measured: twice the error)."""
    b, hq, s = lse_main.shape
    p_sink = torch.exp(sinks.detach().float().view(1, hq, 1) - lse_main)                                       # [B,Hq,S]
    delta = (out_kernel.view(b, s, hq, -1).float() * grad_out.reshape(b, s, hq, -1).float()).sum(-1).transpose(1, 2) * (1.0 - p_sink)
    return (-(p_sink * delta).sum(dim=(0, 2))).to(sinks.dtype)


def _check_sinks(sinks, q):
    if sinks is None:
        return None
    if sinks.ndim != 1 or sinks.shape[0] != q.shape[1] or sinks.device != q.device:
        raise ValueError("sinks must hold one logit per main query head, on the inputs' device")
    return sinks


class _SparseAttentionFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q_proxy, k_proxy, q, k, v, top_k, scale, doc_start=None, sinks=None):
        num_blocks, top_k_blocks = _validate_inputs(q_proxy, k_proxy, q, k, v, int(top_k), True)
        _require_cuda(q)
        sinks = _check_sinks(sinks, q)
        status = torch.zeros(1, dtype=torch.int32, device=q.device)
        if top_k_blocks <= ops.FUSED_SELECT_MAX_BLOCKS:
            block_indices = ops.select_blocks_fused(q_proxy, k_proxy, float(scale), top_k_blocks, status=status,
                                                    doc_start=doc_start)
        else:
            scores = ops.proxy_block_scores(q_proxy, k_proxy, float(scale), status=status, doc_start=doc_start)
            block_indices = ops.select_topk(scores, top_k_blocks)
            del scores
        rix = ops.build_reverse_index(block_indices)
        out, lse_main, lse_proxy = ops.attention_forward(q, k, v, q_proxy, k_proxy, float(scale), rix, status=status,
                                                         doc_start=doc_start)
        _maybe_check(status, "flash_msa_func forward")
        ctx.out_kernel = None
        if sinks is not None:
            ctx.out_kernel = out
            out, lse_main, lse_proxy = _apply_sinks(out, lse_main, lse_proxy, sinks, q_proxy.shape[1])
        ctx.sinks = sinks
        # kl_loss is a placeholder whose gradient switches the KL branch of the backward on
        # (reference: flash_msa/msa_forward_cutedsl.py:69)
        kl_loss = torch.zeros((), dtype=torch.float32, device=q.device)
        ctx.save_for_backward(q_proxy, k_proxy, q, k, v, out, lse_main, lse_proxy, rix.row_ptr, rix.col_q, rix.edge_pos)
        # an output that does not feed the loss arrives as None in backward (not as zeros): no gradient for
        # kl_loss then really skips the proxy work, as the reference intends (flash_msa/flash_msa.py:104-106)
        ctx.set_materialize_grads(False)
        ctx.scale = float(scale)
        ctx.top_k_blocks = top_k_blocks
        ctx.doc_start = doc_start
        return out, kl_loss

    @staticmethod
    def backward(ctx, grad_out, grad_kl):
        q_proxy, k_proxy, q, k, v, out, lse_main, lse_proxy, row_ptr, col_q, edge_pos = ctx.saved_tensors
        b, _, s, _ = q.shape
        if grad_out is None:
            grad_out = torch.zeros_like(out)
        rix = ops.ReverseIndex(row_ptr, col_q, edge_pos, b, q_proxy.shape[1], s, ctx.top_k_blocks)
        status = torch.zeros(1, dtype=torch.int32, device=q.device)
        klv = _kl_buffer(grad_kl, q.device)
        dqp, dkp, dq, dk, dv = ops.attention_backward(q, k, v, q_proxy, k_proxy, out, grad_out, lse_main, lse_proxy,
                                                      ctx.scale, rix, grad_kl, status=status, kl_value=klv,
                                                      doc_start=ctx.doc_start)
        _publish_kl(klv)
        _maybe_check(status, "flash_msa_func backward")
        dsinks = _sink_grad(ctx.out_kernel, grad_out, lse_main, ctx.sinks) if ctx.sinks is not None else None
        return dqp, dkp, dq, dk, dv, None, None, None, dsinks


class _WarmupSparseAttentionFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q_proxy, k_proxy, q, k, v, top_k, scale, doc_start=None, sinks=None):
        _ = int(top_k)                         # accepted and ignored, as in the reference
        _validate_inputs(q_proxy, k_proxy, q, k, v, 0, False)
        sinks = _check_sinks(sinks, q)
        if q.device.type != "cuda":
            raise RuntimeError("warmup MSA forward requires CUDA tensors")
        status = torch.zeros(1, dtype=torch.int32, device=q.device)
        out, lse_main, lse_proxy = ops.attention_forward(q, k, v, q_proxy, k_proxy, float(scale), None, dense=True,
                                                         status=status, doc_start=doc_start)
        _maybe_check(status, "flash_msa_warmup_func forward")
        ctx.out_kernel = None
        if sinks is not None:
            ctx.out_kernel = out
            out, lse_main, lse_proxy = _apply_sinks(out, lse_main, lse_proxy, sinks, q_proxy.shape[1])
        ctx.sinks = sinks
        kl_loss = torch.zeros((), dtype=torch.float32, device=q.device)
        ctx.save_for_backward(q_proxy, k_proxy, q, k, v, out, lse_main, lse_proxy)
        ctx.set_materialize_grads(False)
        ctx.scale = float(scale)
        ctx.doc_start = doc_start
        return out, kl_loss

    @staticmethod
    def backward(ctx, grad_out, grad_kl):
        q_proxy, k_proxy, q, k, v, out, lse_main, lse_proxy = ctx.saved_tensors
        if grad_out is None:
            grad_out = torch.zeros_like(out)
        status = torch.zeros(1, dtype=torch.int32, device=q.device)
        klv = _kl_buffer(grad_kl, q.device)
        dqp, dkp, dq, dk, dv = ops.attention_backward(q, k, v, q_proxy, k_proxy, out, grad_out, lse_main, lse_proxy,
                                                      ctx.scale, None, grad_kl, dense=True, status=status, kl_value=klv,
                                                      doc_start=ctx.doc_start)
        _publish_kl(klv)
        _maybe_check(status, "flash_msa_warmup_func backward")
        dsinks = _sink_grad(ctx.out_kernel, grad_out, lse_main, ctx.sinks) if ctx.sinks is not None else None
        return dqp, dkp, dq, dk, dv, None, None, None, dsinks


def _spread_proxy_heads(q_proxy, k_proxy, q, k):
    """Fewer proxy heads than KV heads (Hkv % Hp == 0; the reference refuses this, flash_msa/flash_msa.py:44-62): the
    kernels walk one KV head at a time and want that head's proxy head(s) with it, so every proxy query head is
    repeated Hkv/Hp times (a differentiable copy of the small proxy tensor).  Each copy then steers the main heads of
    one KV head with the same scores, hence the same selection, and autograd sums the copies' gradients.  That sum is
    exact: the gradient of the KL term is linear in the teacher, the copies' teachers are the means over their own
    main heads, and the per-call factor 1/(B*Hp'*S) with Hp' = Hkv makes their sum the gradient for the mean over all
    main heads of the proxy head.  (Only the optional KL VALUE differs: it becomes the mean of the copies' KL terms,
    an upper bound of the KL against the pooled teacher.)"""
    if q_proxy.ndim == 4 and k_proxy.ndim == 4 and q.ndim == 4 and k.ndim == 4:
        hp, hpkv, hq, hkv = q_proxy.shape[1], k_proxy.shape[1], q.shape[1], k.shape[1]
        if 0 < hp < hkv and hkv % hp == 0 and hpkv > 0 and hp % hpkv == 0 and hq % hkv == 0:
            return q_proxy.repeat_interleave(hkv // hp, dim=1)
    return q_proxy   # (anything else is judged by the shape checks of the call)


def sparse_attention(q_proxy, k_proxy, q, k, v, top_k: int, scale: float, sinks=None):
    """Block-sparse top-k GQA attention.  Returns ``(attn_out [B,S,Hq*D], kl_loss placeholder)``.
    ``sinks`` (optional, beyond the reference): one softmax-bias logit per main query head, see `_apply_sinks`."""
    return _SparseAttentionFunction.apply(_spread_proxy_heads(q_proxy, k_proxy, q, k), k_proxy, q, k, v, int(top_k), float(scale), None,
                                          sinks)


def sparse_attention_varlen(q_proxy, k_proxy, q, k, v, cu_seqlens, top_k: int, scale: float, sinks=None):
    """`sparse_attention` on packed sequences: the S positions of every batch element hold several documents laid end
    to end, `cu_seqlens` ([n+1], or [B,n+1] for a packing per batch element; starts at 0, ends at S: the FlashAttention
    varlen convention) gives their boundaries, and a query sees only the keys of its own document - in the block scores
    and the selection, in the attention and in every gradient.  Blocks stay 128 positions of the PACKED sequence, so S
    must still be a multiple of 128 (pad the last document).  The reference has no such path (its README lists
    variable-length batches as missing)."""
    if q.ndim != 4:
        raise ValueError("all attention tensors must have shape (B, H, S, D)")
    _require_cuda(q)
    doc_start = ops.doc_start_from_cu_seqlens(cu_seqlens, q.shape[0], q.shape[2], q.device)
    return _SparseAttentionFunction.apply(_spread_proxy_heads(q_proxy, k_proxy, q, k), k_proxy, q, k, v, int(top_k), float(scale), doc_start,
                                          sinks)


def sparse_attention_warmup(q_proxy, k_proxy, q, k, v, top_k: int, scale: float, sinks=None):
    """Dense causal warmup attention with full-sequence proxy KL gradients."""
    return _WarmupSparseAttentionFunction.apply(_spread_proxy_heads(q_proxy, k_proxy, q, k), k_proxy, q, k, v, int(top_k), float(scale), None,
                                                sinks)


def sparse_attention_warmup_varlen(q_proxy, k_proxy, q, k, v, cu_seqlens, top_k: int, scale: float, sinks=None):
    """`sparse_attention_warmup` on packed sequences (see `sparse_attention_varlen`): dense causal attention and the
    full-sequence proxy KL inside every document.  The schedule still visits every causal block pair of the packed
    sequence; pairs that straddle documents are masked."""
    if q.ndim != 4:
        raise ValueError("all attention tensors must have shape (B, H, S, D)")
    _require_cuda(q)
    doc_start = ops.doc_start_from_cu_seqlens(cu_seqlens, q.shape[0], q.shape[2], q.device)
    return _WarmupSparseAttentionFunction.apply(_spread_proxy_heads(q_proxy, k_proxy, q, k), k_proxy, q, k, v, int(top_k), float(scale), doc_start,
                                                sinks)
