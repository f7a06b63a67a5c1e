"""The allocation-free reverse index (scratch inside the library image) must give exactly what
the workspace-based entry point gives, call after call.  Collected last on purpose."""
import pytest
import torch

from oracle import msa_oracle as O

pytestmark = pytest.mark.gpu


def _indices(b, hp, s, kb, seed):
    nb = s // 128
    g = torch.Generator(device="cpu").manual_seed(seed)
    sc = torch.randn(b, hp, s, nb, generator=g)
    qblk = (torch.arange(s) // 128).view(1, 1, s, 1)
    sc = sc.masked_fill(torch.arange(nb).view(1, 1, 1, nb) > qblk, float("-inf"))
    return O.stable_topk(sc, kb).cuda()


def test_static_scratch_reverse_index_matches_workspace_variant():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from flash_msa_b200 import ops
    # two calls in a row on different problems: the second must not see the first one's scratch
    for b, hp, s, kb, seed in [(2, 4, 4096, 8, 1), (1, 2, 1024, 3, 2), (2, 4, 4096, 8, 3)]:
        idx = _indices(b, hp, s, kb, seed)
        want = ops.build_reverse_index(idx)
        nb = s // 128
        row_ptr = torch.full((b * hp * nb + 1,), -7, dtype=torch.int32, device="cuda")
        col_q = torch.full((b * hp * s * kb,), -7, dtype=torch.int32, device="cuda")
        edge_pos = torch.full((b, hp, s, kb), -7, dtype=torch.int32, device="cuda")
        got = ops.build_reverse_index_static(idx, row_ptr, col_q, edge_pos)
        torch.cuda.synchronize()
        e = int(want.row_ptr[-1])
        assert torch.equal(got.row_ptr, want.row_ptr)
        assert torch.equal(got.col_q[:e], want.col_q[:e])
        assert torch.equal(got.edge_pos, want.edge_pos)


def test_static_scratch_calls_allocate_nothing():
    """What the entry point is for: after the first call on the device (which looks the scratch array's address
    up) further calls on caller-owned, preallocated tensors neither allocate through torch nor change the
    amount of free device memory."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from flash_msa_b200 import ops
    b, hp, s, kb = 2, 4, 4096, 8
    nb = s // 128
    idx = _indices(b, hp, s, kb, 5)
    row_ptr = torch.empty(b * hp * nb + 1, dtype=torch.int32, device="cuda")
    col_q = torch.empty(b * hp * s * kb, dtype=torch.int32, device="cuda")
    edge_pos = torch.empty(b, hp, s, kb, dtype=torch.int32, device="cuda")
    ops.build_reverse_index_static(idx, row_ptr, col_q, edge_pos)       # warm call: symbol address looked up here
    torch.cuda.synchronize()
    want = ops.build_reverse_index(idx)
    torch.cuda.synchronize()
    free0, alloc0, reserved0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(3):
        ops.build_reverse_index_static(idx, row_ptr, col_q, edge_pos)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == alloc0 and torch.cuda.memory_reserved() == reserved0
    assert torch.cuda.mem_get_info()[0] == free0
    assert torch.equal(row_ptr, want.row_ptr) and torch.equal(edge_pos, want.edge_pos)


def test_static_scratch_rejects_oversized_problems():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from flash_msa_b200 import _lib, ops
    lib = _lib.load()
    s, rows = 65536, 16                      # 16 * 512^2 * 5 bytes > 8 MiB
    assert lib.fmsa_reverse_index_workspace_bytes(rows, s) > ops.STATIC_SCRATCH_BYTES
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    rc = lib.fmsa_reverse_index_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                       rows, s, 32, 0)
    assert rc == -3                          # FMSA_ERR_WORKSPACE, nothing launched
