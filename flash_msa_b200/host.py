"""Forward + backward of the attention op on buffers that live in pinned HOST memory.

The path has no exchange step between (batch, KV-head group) units (the property the multi-GPU
sharding uses, sharding.py), so a step on host buffers is pipelined over chunks of those units:
while chunk i runs its kernels, chunk i+1 is copied to the device and the results of chunk i-1 are
copied back, on three CUDA streams.  A step then costs about the larger of the copy time and the
kernel time instead of their sum.

The reference's API takes device tensors only (flash_msa/flash_msa.py:266-278); this module is what
a host-side caller of the C ABI would write around it.  It is the call `bench.py` times as `e2e`.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import _lib
from . import api
from .sharding import Shard, head_ranges, kl_weight, needs_dk_proxy_allreduce, partition


def _chunks(b: int, hq: int, hkv: int, hp: int, hpkv: int, want: int) -> List[Shard]:
    """Rectangular chunks of the (batch, KV head) grid: as many as `want` if the grid divides that way
    without cutting a proxy-K head that two chunks would both need; otherwise fewer."""
    units = b * hkv
    for n in range(min(want, units), 0, -1):
        if units % n:
            continue
        pieces = partition(b, hkv, n)
        if any(len(p) != 1 for p in pieces) or needs_dk_proxy_allreduce(hkv, hp, hpkv, pieces):
            continue
        try:
            for p in pieces:
                head_ranges(p[0], hq, hkv, hp, hpkv)
        except ValueError:
            continue
        return [p[0] for p in pieces]
    return [Shard(0, b, 0, hkv)]


class HostStep:
    """One fwd+bwd of `flash_msa_func` (or the warmup function) per `run()`, host buffers in and out.

    Inputs (pinned, contiguous): q_proxy [B,Hp,S,128], k_proxy [B,Hpkv,S,128], q [B,Hq,S,128],
    k, v [B,Hkv,S,128], d_out [B,S,Hq*128].  Results (pinned, allocated once): out [B,S,Hq*128] and the
    gradients dq_proxy, dk_proxy, dq, dk, dv shaped like the inputs.

    `chunks`: how many pieces the (batch, KV head) grid is cut into.  Measured on a B200 at B=2, S=8192,
    Hq=32, Hkv=8 (402 MB each way; one direction alone takes 7.3 ms): 1 chunk 15.6 ms per step, 2 chunks
    9.9, 4 chunks 9.6, 8 chunks 10.9, 16 chunks 15.1 (the host cannot enqueue the launches fast enough).
    """

    def __init__(self, b: int, s: int, hq: int, hkv: int, hp: int, hpkv: int, top_k: int, scale: float, *,
                 dense: bool = False, chunks: int = 4, device=None, dtype=torch.bfloat16):
        if not torch.cuda.is_available():
            raise RuntimeError("flash_msa_b200 needs a CUDA device (there is no CPU path)")
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.shape = (b, s, hq, hkv, hp, hpkv)
        self.top_k, self.scale, self.dense, self.dtype = int(top_k), float(scale), bool(dense), dtype
        self.fn = api.sparse_attention_warmup if dense else api.sparse_attention
        self.chunks = _chunks(b, hq, hkv, hp, hpkv, chunks)
        self.lib = _lib.load()
        self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(3))
        d = 128
        self.dev_in = []      # per chunk: device copies of the six inputs
        self.ev_in, self.ev_cmp, self.ev_out = [], [], []
        for c in self.chunks:
            (h0, h1), (kv0, kv1), (p0, p1), (kp0, kp1) = head_ranges(c, hq, hkv, hp, hpkv)
            nb = c.b1 - c.b0
            mk = lambda h: torch.empty(nb, h, s, d, dtype=dtype, device=self.dev)
            self.dev_in.append((mk(p1 - p0), mk(kp1 - kp0), mk(h1 - h0), mk(kv1 - kv0), mk(kv1 - kv0),
                                torch.empty(nb, s, (h1 - h0) * d, dtype=dtype, device=self.dev)))
            self.ev_in.append(torch.cuda.Event())
            self.ev_cmp.append(torch.cuda.Event())
            self.ev_out.append(torch.cuda.Event())
        pin = lambda *shape: torch.empty(*shape, dtype=dtype, pin_memory=True)
        self.host_out = (pin(b, s, hq * d), pin(b, hp, s, d), pin(b, hpkv, s, d), pin(b, hq, s, d), pin(b, hkv, s, d),
                         pin(b, hkv, s, d))
        # Device results of the step in flight, per chunk.  They are produced on the compute stream and read by the
        # copy-out stream; a chunk's results are released only after the compute stream has been made to wait for the
        # copy-out of that chunk, so the caching allocator hands their memory to later work of the compute stream alone
        # and the set of blocks in use is the same every step, however far the host runs ahead of the device.
        # (Marking them with record_stream instead lets the allocator defer their reuse by host timing: a step that
        # found no free block called cudaMalloc, which waits for the device - measured as steps of 26-29 ms among
        # steps of 9 ms.)
        self._keep = [None] * len(self.chunks)
        self._first = True

    # -- copies ------------------------------------------------------------------------------
    def _copy_heads(self, dst, src, b0, b1, h0, h1, stream):
        """(B,H,S,128) tensors: a head range of some batch elements is contiguous per batch element."""
        for i, bb in enumerate(range(b0, b1)):
            host_side = src if src.device.type == "cpu" else dst
            view = host_side[bb, h0:h1]
            if src.device.type == "cpu":
                dst[i].copy_(view, non_blocking=True)
            else:
                view.copy_(src[i], non_blocking=True)

    def _copy_rows(self, dst, src, b0, b1, h0, h1, hq, stream):
        """[B,S,Hq*128] tensors: a head range is S pieces of (h1-h0)*256 bytes, Hq*256 bytes apart."""
        width, pitch = (h1 - h0) * 256, hq * 256
        s = self.shape[1]
        for i, bb in enumerate(range(b0, b1)):
            if src.device.type == "cpu":
                d_ptr, d_pitch = dst[i].data_ptr(), width
                s_ptr, s_pitch = src[bb].data_ptr() + h0 * 256, pitch
            else:
                d_ptr, d_pitch = dst[bb].data_ptr() + h0 * 256, pitch
                s_ptr, s_pitch = src[i].data_ptr(), width
            _lib.check(self.lib.fmsa_copy2d_async(d_ptr, d_pitch, s_ptr, s_pitch, width, s, stream.cuda_stream),
                       "fmsa_copy2d_async")

    # -- the step ----------------------------------------------------------------------------
    def run(self, q_proxy, k_proxy, q, k, v, d_out, grad_kl: Optional[float] = 1.0):
        """Enqueues one step; returns the pinned result tensors (out, dq_proxy, dk_proxy, dq, dk, dv).
        They are complete after `synchronize()`."""
        b, s, hq, hkv, hp, hpkv = self.shape
        for t in (q_proxy, k_proxy, q, k, v, d_out):
            if t.device.type != "cpu" or not t.is_pinned() or not t.is_contiguous() or t.dtype != self.dtype:
                raise ValueError("HostStep.run takes contiguous pinned host tensors of the configured dtype")
        for ci, c in enumerate(self.chunks):
            (h0, h1), (kv0, kv1), (p0, p1), (kp0, kp1) = head_ranges(c, hq, hkv, hp, hpkv)
            dqp_d, dkp_d, dq_d, dk_d, dv_d, do_d = self.dev_in[ci]
            with torch.cuda.stream(self.s_in):
                if not self._first:
                    self.s_in.wait_event(self.ev_cmp[ci])     # last step's kernels have finished with these buffers
                self._copy_heads(dqp_d, q_proxy, c.b0, c.b1, p0, p1, self.s_in)
                self._copy_heads(dkp_d, k_proxy, c.b0, c.b1, kp0, kp1, self.s_in)
                self._copy_heads(dq_d, q, c.b0, c.b1, h0, h1, self.s_in)
                self._copy_heads(dk_d, k, c.b0, c.b1, kv0, kv1, self.s_in)
                self._copy_heads(dv_d, v, c.b0, c.b1, kv0, kv1, self.s_in)
                self._copy_rows(do_d, d_out, c.b0, c.b1, h0, h1, hq, self.s_in)
                self.ev_in[ci].record(self.s_in)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(self.ev_in[ci])
                if not self._first:
                    self.s_cmp.wait_event(self.ev_out[ci])    # last step's results of this chunk have reached the host
                self._keep[ci] = None
                leaves = [t.detach().requires_grad_(True) for t in (dqp_d, dkp_d, dq_d, dk_d, dv_d)]
                out, kl = self.fn(*leaves, self.top_k, self.scale)
                if grad_kl is None:
                    torch.autograd.backward([out], [do_d])
                else:
                    # every call normalises its KL term by its own row count: weight by the chunk's share
                    gk = torch.full((), float(grad_kl) * kl_weight(c, b, hkv), device=self.dev)
                    torch.autograd.backward([out, kl], [do_d, gk])
                res = [out] + [t.grad if t.grad is not None else torch.zeros_like(t) for t in leaves]
                self.ev_cmp[ci].record(self.s_cmp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_cmp[ci])
                ho, hdqp, hdkp, hdq, hdk, hdv = self.host_out
                self._copy_rows(ho, res[0], c.b0, c.b1, h0, h1, hq, self.s_out)
                self._copy_heads(hdqp, res[1], c.b0, c.b1, p0, p1, self.s_out)
                self._copy_heads(hdkp, res[2], c.b0, c.b1, kp0, kp1, self.s_out)
                self._copy_heads(hdq, res[3], c.b0, c.b1, h0, h1, self.s_out)
                self._copy_heads(hdk, res[4], c.b0, c.b1, kv0, kv1, self.s_out)
                self._copy_heads(hdv, res[5], c.b0, c.b1, kv0, kv1, self.s_out)
                self.ev_out[ci].record(self.s_out)
            self._keep[ci] = res
            del res, leaves, out, kl
        self._first = False
        return self.host_out

    def synchronize(self):
        self.s_out.synchronize()
        self.s_cmp.synchronize()

    def bytes_per_step(self):
        """(host-to-device, device-to-host) bytes one step moves."""
        b, s, hq, hkv, hp, hpkv = self.shape
        esz, d = torch.empty((), dtype=self.dtype).element_size(), 128
        h2d = b * s * d * esz * (hp + hpkv + hq + 2 * hkv + hq)
        d2h = b * s * d * esz * (hq + hp + hpkv + hq + 2 * hkv)
        return h2d, d2h
