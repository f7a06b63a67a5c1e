"""GPU checks of the building blocks, all through the C ABI: the tcgen05 tile product in every
operand mode, the top-k pick and the reverse index (bit-exact against the oracle)."""
import pytest
import torch

from oracle import msa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from flash_msa_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("use_tma", [0, 1])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_umma_tile_product(ops, a_mn, b_mn, use_tma):
    g = torch.Generator(device="cpu").manual_seed(7 + a_mn * 2 + b_mn)
    a = torch.randn(128, 128, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(128, 128, generator=g).to(torch.bfloat16).cuda()
    d, status = ops.umma_selftest(a, b, bool(a_mn), bool(b_mn), bool(use_tma))
    torch.cuda.synchronize()
    assert status.item() == 0
    ae = a.float().t() if a_mn else a.float()
    be = b.float().t() if b_mn else b.float()
    ref = ae @ be.t()
    err = (d - ref).abs().max().item()
    assert err <= 1e-2, err     # bf16 inputs are exact in fp32; only the summation order differs


def test_gather_tmem_operand_and_tile_store(ops):
    """TMA row gather (with out-of-range rows), a product whose A operand was written to TMEM with tcgen05.st,
    and the swizzled TMA tile store of partial rows."""
    g = torch.Generator(device="cpu").manual_seed(11)
    src = torch.randn(1000, 128, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(128, 128, generator=g).to(torch.bfloat16).cuda()
    rows = torch.randint(0, 1000, (128,), generator=g)
    rows[5] = 1000          # first row outside the matrix
    rows[77] = 2 ** 30      # far outside
    rows[100:104] = torch.tensor([999, 0, 999, 0])
    d1, d2, part, status = ops.pipeline_selftest(src, rows.cuda(), b)
    torch.cuda.synchronize()
    assert status.item() == 0
    a = src.float()[rows.clamp(max=999)]
    a[5] = 0
    a[77] = 0
    ref1 = a @ b.float().t()
    assert (d1 - ref1).abs().max().item() <= 1e-2
    a2 = (d1 * 0.0625).to(torch.bfloat16)
    ref2 = a2.float() @ b.float()
    assert (d2 - ref2).abs().max().item() <= 2e-2
    assert torch.equal(part[:, 1, :], a2)
    assert part[:, 0, :].abs().max().item() == 0


def test_bounded_wait_runs_out(ops):
    """A completion signal that never comes: the bounded wait gives up after its limit, the kernel returns
    normally and reports status 1 (nothing traps or spins on)."""
    g = torch.Generator(device="cpu").manual_seed(12)
    src = torch.randn(256, 128, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(128, 128, generator=g).to(torch.bfloat16).cuda()
    rows = torch.arange(128)
    d1, d2, part, status = ops.pipeline_selftest(src, rows.cuda(), b, withhold=True, limit_ns=3_000_000)
    torch.cuda.synchronize()
    assert status.item() == 1
    assert (d1 - src.float()[:128] @ b.float().t()).abs().max().item() <= 1e-2   # the first product still arrived
    # the context stays usable
    d1b, _, _, status_b = ops.pipeline_selftest(src, rows.cuda(), b)
    torch.cuda.synchronize()
    assert status_b.item() == 0 and torch.equal(d1, d1b)


def test_status_word_surfaces_without_synchronising(ops):
    """The status word of a call is copied to pinned memory behind it and raised by a later look: a kernel whose
    bounded wait ran out (status 1) turns into a RuntimeError at `drain`, a clean call into nothing."""
    g = torch.Generator(device="cpu").manual_seed(13)
    src = torch.randn(256, 128, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(128, 128, generator=g).to(torch.bfloat16).cuda()
    rows = torch.arange(128).cuda()
    watch = ops.DeferredStatus()
    watch.push(ops.pipeline_selftest(src, rows, b)[3], "clean call")
    watch.drain()
    watch.push(ops.pipeline_selftest(src, rows, b, withhold=True, limit_ns=2_000_000)[3], "withheld signal")
    with pytest.raises(RuntimeError, match="withheld signal.*timed out"):
        watch.drain()
    watch.drain()                                   # the queue is empty again


@pytest.mark.parametrize("s,kb", [(128, 1), (512, 2), (1024, 4), (2048, 16), (4096, 32), (8192, 33), (8192, 64), (16384, 128)])
def test_topk_bit_exact(ops, s, kb):
    nb = s // 128
    g = torch.Generator(device="cpu").manual_seed(s + kb)
    sc = torch.randn(2, 2, s, nb, generator=g)
    # heavy ties: quantise half of the rows to a few distinct values
    sc[:, 1] = torch.round(sc[:, 1] * 2) / 2
    qblk = (torch.arange(s) // 128).view(1, 1, s, 1)
    sc = sc.masked_fill(torch.arange(nb).view(1, 1, 1, nb) > qblk, float("-inf"))
    want = O.stable_topk(sc, kb)
    dev = sc.cuda()
    dev = torch.where(torch.isinf(dev) & (dev < 0), torch.full_like(dev, float("nan")), dev)   # future entries are never read
    got = ops.select_topk(dev, kb).cpu()
    assert torch.equal(got, want)


@pytest.mark.parametrize("b,hp,s,kb", [(1, 1, 128, 1), (2, 2, 640, 3), (1, 4, 2048, 16), (2, 8, 8192, 16), (1, 2, 16384, 64)])
def test_reverse_index_bit_exact(ops, b, hp, s, kb):
    nb = s // 128
    g = torch.Generator(device="cpu").manual_seed(b * 131 + s + kb)
    sc = torch.randn(b, hp, s, nb, generator=g)
    qblk = (torch.arange(s) // 128).view(1, 1, s, 1)
    sc = sc.masked_fill(torch.arange(nb).view(1, 1, 1, nb) > qblk, float("-inf"))
    idx = O.stable_topk(sc, kb)
    row_ptr, col_q, edge_pos = O.reverse_index(idx, nb)
    rix = ops.build_reverse_index(idx.cuda())
    assert torch.equal(rix.row_ptr.cpu(), row_ptr)
    e = int(row_ptr[-1])
    assert torch.equal(rix.col_q[:e].cpu(), col_q)
    assert torch.equal(rix.edge_pos.cpu(), edge_pos)


def test_reverse_index_ignores_garbage_slots(ops):
    """Out-of-range and future block ids are not edges (reference rule, reverse_index_cuda.cu:41)."""
    s, kb, nb = 512, 4, 4
    idx = torch.full((1, 1, s, kb), nb, dtype=torch.int32)
    idx[..., 0] = (torch.arange(s) // 128).to(torch.int32)
    idx[..., 1] = 3          # future for all rows outside block 3
    idx[..., 2] = -5
    idx[0, 0, 384:, 1] = 0   # rows of block 3 also pick block 0
    row_ptr, col_q, edge_pos = O.reverse_index(idx, nb)
    rix = ops.build_reverse_index(idx.cuda())
    assert torch.equal(rix.row_ptr.cpu(), row_ptr)
    assert torch.equal(rix.col_q[: int(row_ptr[-1])].cpu(), col_q)
    assert torch.equal(rix.edge_pos.cpu(), edge_pos)
