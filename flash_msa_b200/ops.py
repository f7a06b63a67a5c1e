"""Thin launch wrappers: validate, allocate outputs with torch, call the C ABI on the current
stream.  Names follow the reference's host-side functions so tests read alike."""
from __future__ import annotations

from dataclasses import dataclass

import ctypes
import os

import torch

from . import _lib

ctypes_byref = ctypes.byref

BLOCK_SIZE = 128


# Instrumentation used by the benchmark: when KERNEL_EVENTS is a list, every C-ABI launch is
# bracketed by CUDA events on the launching stream and (name, start, end) is appended.
# LAUNCHES counts the kernels launched by this library since import.
KERNEL_EVENTS = None
LAUNCHES = 0


def _launch(name: str, n_kernels: int, status: int, device) -> None:
    global LAUNCHES
    _lib.check(status, name)
    LAUNCHES += n_kernels


class _Timed:
    def __init__(self, name, device):
        self.name, self.device = name, device

    def __enter__(self):
        if KERNEL_EVENTS is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.end = torch.cuda.Event(enable_timing=True)
            self.start.record(torch.cuda.current_stream(self.device))
        return self

    def __exit__(self, *exc):
        if KERNEL_EVENTS is not None:
            self.end.record(torch.cuda.current_stream(self.device))
            KERNEL_EVENTS.append((self.name, self.start, self.end))
        return False


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(*tensors):
    for t in tensors:
        if t.device.type != "cuda":
            raise ValueError("flash_msa_b200 kernels require CUDA tensors (there is no CPU path)")


def umma_selftest(a: torch.Tensor, b: torch.Tensor, a_mn: bool, b_mn: bool, use_tma: bool):
    """Test hook: D = A_eff @ B_eff^T for one 128x128x128 bf16 tile on the tensor cores."""
    _require_cuda(a, b)
    lib = _lib.load()
    a = a.contiguous()
    b = b.contiguous()
    d = torch.zeros(128, 128, dtype=torch.float32, device=a.device)
    status = torch.zeros(1, dtype=torch.int32, device=a.device)
    _lib.check(lib.fmsa_umma_selftest(a.data_ptr(), b.data_ptr(), d.data_ptr(), int(a_mn), int(b_mn), int(use_tma),
                                      status.data_ptr(), _stream(a.device)), "fmsa_umma_selftest")
    return d, status


def pipeline_selftest(src: torch.Tensor, rows: torch.Tensor, b: torch.Tensor, withhold: bool = False,
                      limit_ns: int = 2_000_000_000):
    """Test hook: TMA row gather -> product -> packed TMEM operand -> product, plus a swizzled TMA tile store.
    Returns (d1, d2, part, status); see fmsa_pipeline_selftest in the header."""
    _require_cuda(src, rows, b)
    lib = _lib.load()
    src, b = src.contiguous(), b.contiguous()
    rows = rows.to(torch.int32).contiguous()
    dev = src.device
    d1 = torch.zeros(128, 128, dtype=torch.float32, device=dev)
    d2 = torch.zeros(128, 128, dtype=torch.float32, device=dev)
    part = torch.zeros(128, 2, 128, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    _lib.check(lib.fmsa_pipeline_selftest(src.data_ptr(), src.shape[0], rows.data_ptr(), b.data_ptr(), d1.data_ptr(),
                                          d2.data_ptr(), part.data_ptr(), int(withhold), int(limit_ns),
                                          status.data_ptr(), _stream(dev)), "fmsa_pipeline_selftest")
    return d1, d2, part, status


def select_topk(block_scores: torch.Tensor, top_k_blocks: int) -> torch.Tensor:
    """Top-k over fp32 block scores [B,Hp,S,NB] -> int32 [B,Hp,S,Kb]; order (score desc, index
    asc), own block first, sentinel NB in unused slots."""
    _require_cuda(block_scores)
    if block_scores.dtype != torch.float32 or block_scores.ndim != 4:
        raise TypeError("block_scores must be fp32 [B,Hp,S,NB]")
    b, hp, s, nb = block_scores.shape
    if s % BLOCK_SIZE or nb != s // BLOCK_SIZE:
        raise ValueError("block_scores shape does not match the sequence length")
    block_scores = block_scores.contiguous()
    out = torch.empty(b, hp, s, int(top_k_blocks), dtype=torch.int32, device=block_scores.device)
    lib = _lib.load()
    with _Timed("select_topk", out.device):
        _launch("fmsa_select_topk", 1, lib.fmsa_select_topk(block_scores.data_ptr(), out.data_ptr(), b * hp, s,
                                                          int(top_k_blocks), _stream(out.device)), out.device)
    return out


@dataclass
class ReverseIndex:
    """CSR of the selection (the counterpart of the reference's SparseAttentionMetadata,
    flash_msa/reverse_index_cuda.py:119-136): row (b*Hp+p)*NB+kb lists ascending query positions."""
    row_ptr: torch.Tensor    # int32 [B*Hp*NB + 1]
    col_q: torch.Tensor      # int32 [B*Hp*S*Kb], first row_ptr[-1] entries used
    edge_pos: torch.Tensor   # int32 [B,Hp,S,Kb]
    batch: int
    n_proxy_heads: int
    seq_len: int
    top_k_blocks: int


def build_reverse_index(block_indices: torch.Tensor) -> ReverseIndex:
    _require_cuda(block_indices)
    if block_indices.dtype != torch.int32 or block_indices.ndim != 4:
        raise TypeError("block_indices must be int32 [B,Hp,S,Kb]")
    b, hp, s, kb = block_indices.shape
    if s % BLOCK_SIZE:
        raise ValueError("sequence length must be divisible by 128")
    nb = s // BLOCK_SIZE
    block_indices = block_indices.contiguous()
    dev = block_indices.device
    lib = _lib.load()
    row_ptr = torch.empty(b * hp * nb + 1, dtype=torch.int32, device=dev)
    col_q = torch.empty(b * hp * s * kb, dtype=torch.int32, device=dev)
    edge_pos = torch.empty(b, hp, s, kb, dtype=torch.int32, device=dev)
    ws_bytes = lib.fmsa_reverse_index_workspace_bytes(b * hp, s)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    with _Timed("reverse_index", dev):
        _launch("fmsa_reverse_index", 4, lib.fmsa_reverse_index(block_indices.data_ptr(), row_ptr.data_ptr(),
                                                              col_q.data_ptr(), edge_pos.data_ptr(), b * hp, s, kb,
                                                              ws.data_ptr(), ws_bytes, _stream(dev)), dev)
    return ReverseIndex(row_ptr, col_q, edge_pos, b, hp, s, kb)


STATIC_SCRATCH_BYTES = 8 << 20


def build_reverse_index_static(block_indices: torch.Tensor, row_ptr: torch.Tensor, col_q: torch.Tensor,
                               edge_pos: torch.Tensor) -> ReverseIndex:
    """Reverse index through the allocation-free entry point: the caller passes the three output
    tensors and the library uses the scratch array built into its image instead of a workspace.
    Meant for hosts that cannot allocate device memory around the call (a frozen memory plan, an
    FFI binding that owns only inputs and outputs).  Limits: the problem's scratch need must not
    exceed STATIC_SCRATCH_BYTES (ValueError otherwise); calls that may overlap on the GPU race on
    the shared array, so keep them ordered on one stream; the first call on a device should come
    before any stream capture."""
    _require_cuda(block_indices, row_ptr, col_q, edge_pos)
    if block_indices.dtype != torch.int32 or block_indices.ndim != 4 or not block_indices.is_contiguous():
        raise TypeError("block_indices must be contiguous int32 [B,Hp,S,Kb]")
    b, hp, s, kb = block_indices.shape
    nb = s // BLOCK_SIZE
    if (row_ptr.numel() < b * hp * nb + 1 or col_q.numel() < b * hp * s * kb or edge_pos.numel() < b * hp * s * kb
            or any(t.dtype != torch.int32 or not t.is_contiguous() for t in (row_ptr, col_q, edge_pos))):
        raise ValueError("output tensors are too small or not contiguous int32")
    lib = _lib.load()
    need = lib.fmsa_reverse_index_workspace_bytes(b * hp, s)
    if need > STATIC_SCRATCH_BYTES:
        raise ValueError(f"reverse index of this size needs {need} bytes of scratch, more than the {STATIC_SCRATCH_BYTES} "
                         "bytes built into the library; use build_reverse_index (caller-provided workspace)")
    dev = block_indices.device
    with _Timed("reverse_index", dev):
        _launch("fmsa_reverse_index_static", 4, lib.fmsa_reverse_index_static(
            block_indices.data_ptr(), row_ptr.data_ptr(), col_q.data_ptr(), edge_pos.data_ptr(), b * hp, s, kb,
            _stream(dev)), dev)
    return ReverseIndex(row_ptr, col_q, edge_pos.view(b, hp, s, kb), b, hp, s, kb)


# ----------------------------------------------------------------------------------------------
# tensor-core kernels
# ----------------------------------------------------------------------------------------------

def _as_kernel_input(t: torch.Tensor) -> torch.Tensor:
    """Kernels read (B,H,S,128) bf16 with a contiguous last dimension and strides that are multiples of one
    128-element row (so that a row of any (batch, head, position) is a row of one 2-D matrix the TMA row
    gather can index): contiguous (B,H,S,D) tensors, (B,S,H,D)-backed views and slices of a packed QKV
    buffer all qualify.  Anything else (for instance an odd storage offset) is copied once."""
    ok = (t.stride(3) == 1 and t.stride(0) % 128 == 0 and t.stride(1) % 128 == 0 and t.stride(2) % 128 == 0
          and t.data_ptr() % 16 == 0 and t.stride(0) > 0 and t.stride(1) > 0 and t.stride(2) > 0)
    return t if ok else t.contiguous()


def _tensor_arg(t: torch.Tensor) -> "_lib.FmsaTensor":
    return _lib.FmsaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _grad_like(t: torch.Tensor) -> torch.Tensor:
    """Uninitialised gradient buffer for the (B,H,S,D) input `t`, in `t`'s own memory layout when `t` is a view of
    (B,S,H,D) storage (what the reference's callers pass, flash_msa/tests/testing_model.py:173-185): autograd then
    hands the gradient back through the caller's transpose and reshape as views, with no copy.  Otherwise (B,H,S,D)
    contiguous."""
    b, h, s, d = t.shape
    if t.stride(3) == 1 and t.stride(2) == h * d and t.stride(1) == d and t.stride(0) == s * h * d and h > 1:
        return torch.empty(b, s, h, d, dtype=t.dtype, device=t.device).transpose(1, 2)
    return torch.empty(b, h, s, d, dtype=t.dtype, device=t.device)


def _dtype_code(dtype) -> int:
    """The library's code of an activation type (bf16 and fp16 are supported, as in the reference:
    flash_msa/msa_backward_cutedsl.py:169-183)."""
    if dtype == torch.bfloat16:
        return _lib.FMSA_DTYPE_BF16
    if dtype == torch.float16:
        return _lib.FMSA_DTYPE_FP16
    raise TypeError(f"flash_msa_b200 supports bf16 and fp16 activations, got {dtype}")


def _problem(q, k, q_proxy, k_proxy, top_k_blocks, scale, doc_start=None) -> "_lib.FmsaProblem":
    b, hq, s, _ = q.shape
    return _lib.FmsaProblem(b, s, hq, k.shape[1], q_proxy.shape[1], k_proxy.shape[1], int(top_k_blocks), float(scale),
                            _dtype_code(q.dtype), doc_start.data_ptr() if doc_start is not None else None)


def doc_start_from_cu_seqlens(cu_seqlens, batch: int, seq_len: int, device) -> torch.Tensor:
    """int32 [B,S] on `device`: for every token of a packed sequence the position of the first token of its document.
    `cu_seqlens` is [n+1] (one packing for every batch element) or [B,n+1]; it starts at 0 and ends at `seq_len`
    (the FlashAttention varlen convention).  The kernels take this array (`fmsa_problem.doc_start`)."""
    cu = torch.as_tensor(cu_seqlens).to(device=device, dtype=torch.int64)
    if cu.dim() == 1:
        cu = cu.unsqueeze(0).expand(batch, -1)
    if cu.dim() != 2 or cu.shape[0] != batch or cu.shape[1] < 2:
        raise ValueError("cu_seqlens must have shape [n+1] or [B, n+1]")
    cu = cu.contiguous()
    if bool((cu[:, 0] != 0).any()) or bool((cu[:, -1] != seq_len).any()) or bool((cu[:, 1:] < cu[:, :-1]).any()):
        raise ValueError("cu_seqlens must rise from 0 to the sequence length")
    pos = torch.arange(seq_len, device=device, dtype=torch.int64).unsqueeze(0).expand(batch, -1).contiguous()
    which = torch.searchsorted(cu, pos, right=True) - 1
    return torch.gather(cu, 1, which).to(torch.int32).contiguous()


def _check_doc_start(doc_start, b, s, dev):
    if doc_start is None:
        return None
    if doc_start.dtype != torch.int32 or tuple(doc_start.shape) != (b, s) or doc_start.device != dev or not doc_start.is_contiguous():
        raise ValueError("doc_start must be a contiguous int32 [B,S] tensor on the inputs' device")
    return doc_start


_STATUS_NAMES = {1: "a bounded device-side wait timed out", 2: "an out-of-range index was found in metadata",
                 3: "the shared-memory window of a kernel was not 1024-byte aligned"}


def check_status(status: torch.Tensor, what: str) -> None:
    """Reads the device status word (synchronises).  Used by tests and debug mode only."""
    code = int(status.item())
    if code != 0:
        raise RuntimeError(f"{what}: {_STATUS_NAMES.get(code, code)}")


class DeferredStatus:
    """Checks device status words without synchronising: `push` copies the word to a slot of a small pinned
    ring on the current stream and records an event; every later `push` (and `drain`) looks at the words
    whose events have completed and raises for a non-zero one, so a timed-out wait or a bad index surfaces
    at the next call of the library instead of passing silently.  Nothing is queued while the stream is
    being captured into a graph."""
    SLOTS = 64

    def __init__(self):
        self._host = None
        self._pending = []        # (slot, event, what, status tensor: kept alive until its copy has run)
        self._next = 0

    def _poll(self, block: bool) -> None:
        while self._pending:
            slot, event, what, _ = self._pending[0]
            if block:
                event.synchronize()
            elif not event.query():
                return
            self._pending.pop(0)
            code = int(self._host[slot])
            if code != 0:
                raise RuntimeError(f"{what} (reported late): {_STATUS_NAMES.get(code, code)}")

    def push(self, status: torch.Tensor, what: str) -> None:
        if torch.cuda.is_current_stream_capturing():
            return
        if self._host is None:
            self._host = torch.zeros(self.SLOTS, dtype=torch.int32).pin_memory()
            self._side = {}
        self._poll(block=len(self._pending) >= self.SLOTS - 1)
        slot = self._next
        self._next = (slot + 1) % self.SLOTS
        # The copy runs on a side stream behind an event of the calling stream: a device-to-host copy on the calling
        # stream itself would queue behind whatever large copies the application has on the copy engine and hold
        # the next kernels back (measured: 3.4 ms per step in the host-buffer pipeline).
        dev = status.device
        side = self._side.get(dev)
        if side is None:
            side = self._side[dev] = torch.cuda.Stream(dev)
        done = torch.cuda.Event()
        done.record(torch.cuda.current_stream(dev))
        side.wait_event(done)
        event = torch.cuda.Event()
        with torch.cuda.stream(side):
            self._host[slot:slot + 1].copy_(status, non_blocking=True)
            event.record(side)
        # (the reference held here, not record_stream: the caching allocator then never has to defer the reuse of
        # the word's block by the side stream's progress, which would make its behaviour depend on host timing)
        self._pending.append((slot, event, what, status))

    def drain(self) -> None:
        """Waits for every queued status word and raises for the first non-zero one."""
        self._poll(block=True)


deferred_status = DeferredStatus()


def proxy_block_scores(q_proxy: torch.Tensor, k_proxy: torch.Tensor, scale: float, status=None, doc_start=None) -> torch.Tensor:
    """fp32 block scores [B,Hp,S,NB]; entries of future blocks are left unwritten.  With `doc_start` (int32 [B,S]) the
    keys before a row's document are hidden and blocks that lie entirely before it score -inf."""
    _require_cuda(q_proxy, k_proxy)
    if q_proxy.dtype != k_proxy.dtype:
        raise TypeError("q_proxy and k_proxy must have one dtype")
    code = _dtype_code(q_proxy.dtype)
    b, hp, s, d = q_proxy.shape
    qp, kp = _as_kernel_input(q_proxy.detach()), _as_kernel_input(k_proxy.detach())
    dev = qp.device
    doc_start = _check_doc_start(doc_start, b, s, dev)
    scores = torch.empty(b, hp, s, s // BLOCK_SIZE, dtype=torch.float32, device=dev)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=dev)
    lib = _lib.load()
    with _Timed("select_scores", dev):
        _launch("fmsa_select_scores", 1, lib.fmsa_select_scores(_tensor_arg(qp), _tensor_arg(kp), scores.data_ptr(), b, hp,
                                                              kp.shape[1], s, float(scale), code,
                                                              doc_start.data_ptr() if doc_start is not None else None,
                                                              status.data_ptr(), _stream(dev)), dev)
    return scores


FUSED_SELECT_MAX_BLOCKS = 64


def select_blocks_fused(q_proxy: torch.Tensor, k_proxy: torch.Tensor, scale: float, top_k_blocks: int, status=None,
                        doc_start=None) -> torch.Tensor:
    """block_indices [B,Hp,S,Kb] int32 from one kernel that scores the key blocks and keeps every row's best ones in
    registers (Kb <= FUSED_SELECT_MAX_BLOCKS); the fp32 block scores are never written.  Bit for bit the result of
    `proxy_block_scores` + `select_topk`."""
    _require_cuda(q_proxy, k_proxy)
    if q_proxy.dtype != k_proxy.dtype:
        raise TypeError("q_proxy and k_proxy must have one dtype")
    kb = int(top_k_blocks)
    b, hp, s, d = q_proxy.shape
    if not 1 <= kb <= min(FUSED_SELECT_MAX_BLOCKS, s // BLOCK_SIZE):
        raise ValueError("top_k_blocks outside the range of the fused selection")
    code = _dtype_code(q_proxy.dtype)
    qp, kp = _as_kernel_input(q_proxy.detach()), _as_kernel_input(k_proxy.detach())
    dev = qp.device
    doc_start = _check_doc_start(doc_start, b, s, dev)
    idx = torch.empty(b, hp, s, kb, dtype=torch.int32, device=dev)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=dev)
    lib = _lib.load()
    with _Timed("select_scores", dev):
        _launch("fmsa_select_fused", 1, lib.fmsa_select_fused(_tensor_arg(qp), _tensor_arg(kp), idx.data_ptr(), b, hp,
                                                            kp.shape[1], s, kb, float(scale), code,
                                                            doc_start.data_ptr() if doc_start is not None else None,
                                                            status.data_ptr(), _stream(dev)), dev)
    return idx


def select_blocks(q_proxy, k_proxy, *, scale: float, num_blocks: int, top_k_blocks: int, return_scores=False, doc_start=None):
    """Counterpart of the reference's select_blocks (flash_msa/msa_select_cutedsl.py:481-538)."""
    if q_proxy.ndim != 4 or k_proxy.ndim != 4:
        raise ValueError("q_proxy and k_proxy must have shape (B, H, S, D)")
    if int(num_blocks) != q_proxy.shape[2] // BLOCK_SIZE:
        raise ValueError("num_blocks does not match q_proxy sequence length")
    scores = proxy_block_scores(q_proxy, k_proxy, scale, doc_start=doc_start)
    idx = select_topk(scores, top_k_blocks)
    return (idx, scores) if return_scores else idx


# Upper bound on the bytes of per-edge partial rows (forward O partials, backward dQ partials) held at once;
# larger problems run in several passes over (batch, KV head) groups.  4 GiB keeps the 8K training shapes in
# one pass; lower it (module attribute, or FLASH_MSA_B200_MAX_PARTIAL_BYTES in the environment) when the
# attention call has to fit beside model state.
MAX_PARTIAL_BYTES = int(os.environ.get("FLASH_MSA_B200_MAX_PARTIAL_BYTES", 4 << 30))
# Rows with more edges than this store their dQ partial rows as (value, rounding remainder) pairs.
SPLIT_PARTIALS_ABOVE = 32


def attention_forward(q, k, v, q_proxy, k_proxy, scale, rix, *, dense=False, with_proxy=True, status=None, doc_start=None):
    """Sparse (or dense warmup) forward.  Returns (out [B,S,Hq*D] bf16, lse [B,Hq,S] fp32,
    lse_proxy [B,Hp,S] fp32 or None)."""
    _require_cuda(q, k, v)
    lib = _lib.load()
    q, k, v = (_as_kernel_input(t.detach()) for t in (q, k, v))
    qp, kp = _as_kernel_input(q_proxy.detach()), _as_kernel_input(k_proxy.detach())
    b, hq, s, d = q.shape
    hkv, hp = k.shape[1], qp.shape[1]
    mpp = hq // hp
    dev = q.device
    doc_start = _check_doc_start(doc_start, q.shape[0], q.shape[2], q.device)
    pb = _problem(q, k, qp, kp, 1 if dense else rix.top_k_blocks, scale, doc_start)
    out = torch.empty(b, s, hq * d, dtype=q.dtype, device=dev)
    lse = torch.empty(b, hq, s, dtype=torch.float32, device=dev)
    lse_proxy = torch.empty(b, hp, s, dtype=torch.float32, device=dev) if with_proxy else None
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=dev)
    counter = torch.empty(1, dtype=torch.int32, device=dev)
    groups = b * hkv
    per_group = lib.fmsa_fwd_partial_slots(ctypes_byref(pb), 1, int(dense))
    bytes_per_slot = mpp * d * 2 + (mpp + 1) * 8
    gstep = max(1, min(groups, MAX_PARTIAL_BYTES // max(1, per_group * bytes_per_slot)))
    slots = per_group * gstep
    o_part = torch.empty(slots * mpp * d, dtype=q.dtype, device=dev)
    lse_part = torch.empty(slots * (mpp + 1) * 2, dtype=torch.float32, device=dev)
    row_ptr = 0 if dense else rix.row_ptr.data_ptr()
    col_q = 0 if dense else rix.col_q.data_ptr()
    edge_pos = 0 if dense else rix.edge_pos.data_ptr()
    st = _stream(dev)
    for g0 in range(0, groups, gstep):
        gc = min(gstep, groups - g0)
        with _Timed("attn_fwd", dev):
            _launch("fmsa_sparse_fwd", 1, lib.fmsa_sparse_fwd(
                ctypes_byref(pb), _tensor_arg(q), _tensor_arg(k), _tensor_arg(v), _tensor_arg(qp), _tensor_arg(kp), row_ptr,
                col_q, o_part.data_ptr(), lse_part.data_ptr(), slots, g0, gc, int(with_proxy), int(dense),
                counter.data_ptr(), status.data_ptr(), st), dev)
        with _Timed("fwd_combine", dev):
            _launch("fmsa_sparse_fwd_combine", 2 if mpp <= 8 else 1, lib.fmsa_sparse_fwd_combine(   # log-sum-exp kernel + row kernel
                ctypes_byref(pb), o_part.data_ptr(), lse_part.data_ptr(), edge_pos, row_ptr, out.data_ptr(), lse.data_ptr(),
                lse_proxy.data_ptr() if with_proxy else 0, g0, gc, int(dense), st), dev)
    return out, lse, lse_proxy


def attention_backward(q, k, v, q_proxy, k_proxy, out, grad_out, lse, lse_proxy, scale, rix, grad_kl, *, dense=False,
                       status=None, kl_value=None, doc_start=None):
    """Fused backward.  ``out`` is the [B,S,Hq*D] forward output, ``grad_out`` its upstream gradient,
    ``grad_kl`` the upstream gradient of kl_loss (0-dim tensor) or None.  Returns
    (dq_proxy, dk_proxy, dq, dk, dv) in the input dtype, shaped like the inputs.
    ``kl_value``: optional zeroed fp32 tensor of one element; the kernel adds the value of the KL loss
    (what the reference's eager model returns, flash_msa/tests/testing_model.py:158-167) to it.  Only
    with ``grad_kl`` given: without it the proxy work is skipped altogether."""
    _require_cuda(q, k, v, grad_out)
    lib = _lib.load()
    q, k, v = (_as_kernel_input(t.detach()) for t in (q, k, v))
    qp, kp = _as_kernel_input(q_proxy.detach()), _as_kernel_input(k_proxy.detach())
    b, hq, s, d = q.shape
    hkv, hp, hpkv = k.shape[1], qp.shape[1], kp.shape[1]
    mpp = hq // hp
    dev = q.device
    st = _stream(dev)
    doc_start = _check_doc_start(doc_start, q.shape[0], q.shape[2], q.device)
    pb = _problem(q, k, qp, kp, 1 if dense else rix.top_k_blocks, scale, doc_start)
    with_kl = grad_kl is not None
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=dev)
    counter = torch.empty(1, dtype=torch.int32, device=dev)

    go = grad_out.detach().reshape(b, s, hq, d)
    if go.dtype != q.dtype:
        go = go.to(q.dtype)
    go = go.permute(0, 2, 1, 3)                       # (B,Hq,S,D) view, no copy
    go = _as_kernel_input(go)
    delta = torch.empty(b, hq, s, dtype=torch.float32, device=dev)
    with _Timed("bwd_delta", dev):
        _launch("fmsa_bwd_delta", 1, lib.fmsa_bwd_delta(out.data_ptr(), _tensor_arg(go), delta.data_ptr(), b, s, hq, pb.dtype, st), dev)

    dkv_acc = torch.zeros(2, b, hkv, s, d, dtype=torch.float32, device=dev)
    if with_kl:
        gk = grad_kl.detach().to(device=dev, dtype=torch.float32).reshape(1)
        dkp_acc = torch.zeros(b, hpkv, s, d, dtype=torch.float32, device=dev)
    else:
        dqp = _grad_like(qp).zero_()
        dkp = _grad_like(kp).zero_()
    groups = b * hkv
    row_ptr = 0 if dense else rix.row_ptr.data_ptr()
    col_q = 0 if dense else rix.col_q.data_ptr()
    edge_pos = 0 if dense else rix.edge_pos.data_ptr()
    klv = kl_value.data_ptr() if (with_kl and kl_value is not None) else 0
    kl_norm = float(scale) / float(b * hp * s)

    def cast(acc, dst, scale_ptr, const_scale):
        if dst.is_contiguous():
            _launch("fmsa_cast_scaled", 1, lib.fmsa_cast_scaled(acc.data_ptr(), dst.data_ptr(), acc.numel(), scale_ptr,
                                                              float(const_scale), pb.dtype, st), dev)
        else:
            _launch("fmsa_cast_scaled_rows", 1, lib.fmsa_cast_scaled_rows(
                acc.data_ptr(), _tensor_arg(dst), acc.shape[0], acc.shape[1], acc.shape[2], scale_ptr, float(const_scale),
                pb.dtype, st), dev)

    # dQ and dQp leave the kernel as per-edge partial rows; a combine pass sums them per query row
    dq = _grad_like(q)
    if with_kl:
        dqp = _grad_like(qp)
    per_group = lib.fmsa_fwd_partial_slots(ctypes_byref(pb), 1, int(dense))
    # A query row's dQ is the sum of one bf16 partial row per selected block.  Beyond ~32 blocks the rounding of the
    # partial rows starts to show against the reference's fp32 accumulation, so each partial is then stored as a
    # (value, rounding remainder) pair in two planes.
    edges_per_row = (s // BLOCK_SIZE) if dense else rix.top_k_blocks
    split = 1 if edges_per_row > SPLIT_PARTIALS_ABOVE else 0
    planes = 2 if split else 1
    bytes_per_slot = (mpp + (1 if with_kl else 0)) * d * 2 * planes
    gstep = max(1, min(groups, MAX_PARTIAL_BYTES // max(1, per_group * bytes_per_slot)))
    slots = per_group * gstep
    dq_part = torch.empty(planes * slots * mpp * d, dtype=q.dtype, device=dev)
    dqp_part = torch.empty(planes * slots * d, dtype=q.dtype, device=dev) if with_kl else None
    for g0 in range(0, groups, gstep):
        gc = min(gstep, groups - g0)
        with _Timed("attn_bwd", dev):
            _launch("fmsa_sparse_bwd", 1, lib.fmsa_sparse_bwd(
                ctypes_byref(pb), _tensor_arg(q), _tensor_arg(k), _tensor_arg(v), _tensor_arg(qp), _tensor_arg(kp),
                _tensor_arg(go), lse.data_ptr(), lse_proxy.data_ptr() if with_kl else 0, delta.data_ptr(), row_ptr, col_q,
                dq_part.data_ptr(), dqp_part.data_ptr() if with_kl else 0, slots, split,
                dkp_acc.data_ptr() if with_kl else 0, dkv_acc[0].data_ptr(), dkv_acc[1].data_ptr(), g0, gc, int(with_kl),
                int(dense), klv, counter.data_ptr(), status.data_ptr(), st), dev)
        with _Timed("bwd_combine", dev):
            _launch("fmsa_sparse_bwd_combine", 1, lib.fmsa_sparse_bwd_combine(
                ctypes_byref(pb), dq_part.data_ptr(), dqp_part.data_ptr() if with_kl else 0, slots, split, edge_pos, row_ptr,
                _tensor_arg(dq), _tensor_arg(dqp) if with_kl else None, gk.data_ptr() if with_kl else 0, g0, gc, int(dense),
                st), dev)

    dk, dv = _grad_like(k), _grad_like(v)
    with _Timed("cast", dev):
        cast(dkv_acc[0], dk, 0, scale)
        cast(dkv_acc[1], dv, 0, 1.0)
        if with_kl:
            dkp = _grad_like(kp)
            cast(dkp_acc, dkp, gk.data_ptr(), kl_norm)
    return dqp, dkp, dq, dk, dv
