"""Thin launch wrappers: validate, allocate outputs with torch, call the C ABI on the current
stream.  Names follow the reference's host-side functions so tests read alike."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib

BLOCK_SIZE = 128


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
    _lib.check(lib.fmsa_select_topk(block_scores.data_ptr(), out.data_ptr(), b * hp, s, int(top_k_blocks),
                                    _stream(out.device)), "fmsa_select_topk")
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
    _lib.check(lib.fmsa_reverse_index(block_indices.data_ptr(), row_ptr.data_ptr(), col_q.data_ptr(),
                                      edge_pos.data_ptr(), b * hp, s, kb, ws.data_ptr(), ws_bytes, _stream(dev)),
               "fmsa_reverse_index")
    return ReverseIndex(row_ptr, col_q, edge_pos, b, hp, s, kb)
