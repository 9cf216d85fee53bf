"""The peer-write exchange kernels on ONE GPU: the ranks' receive buffers are ordinary tensors of the same
device and every rank's launch is issued in turn (the kernels never wait on each other, so this is the same
index arithmetic as the multi-GPU run, minus NVLink).  Bit-exact against torch indexing."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda:0")


@pytest.mark.parametrize("world,block_elems", [(1, 1024), (2, 8 * 333), (4, 8 * 4099), (8, 8 * 1000)])
def test_peer_scatter_is_an_all_to_all(dev, world, block_elems):
    from tt_boltz_b200._lib import call, ptr, stream
    g = torch.Generator().manual_seed(world)
    send = [torch.randint(-30000, 30000, (world, block_elems), generator=g, dtype=torch.int16).to(dev) for _ in range(world)]
    recv = [torch.full((world, block_elems), -1, dtype=torch.int16, device=dev) for _ in range(world)]
    ptrs = (C.c_ulonglong * world)(*[r.data_ptr() for r in recv])
    for rank in range(world):
        call("b200pf_peer_scatter", ptr(send[rank]), ptrs, block_elems * 2, rank, world, stream())
    torch.cuda.synchronize()
    for t in range(world):
        for s in range(world):
            assert torch.equal(recv[t][s], send[s][t]), (t, s)          # rank t receives block t of every sender s


@pytest.mark.parametrize("world,block_elems", [(1, 64), (2, 8 * 777), (8, 8 * 2048)])
def test_peer_broadcast_is_an_all_gather(dev, world, block_elems):
    from tt_boltz_b200._lib import call, ptr, stream
    g = torch.Generator().manual_seed(100 + world)
    send = [torch.randint(-30000, 30000, (block_elems,), generator=g, dtype=torch.int16).to(dev) for _ in range(world)]
    recv = [torch.full((world, block_elems), -1, dtype=torch.int16, device=dev) for _ in range(world)]
    ptrs = (C.c_ulonglong * world)(*[r.data_ptr() for r in recv])
    for rank in range(world):
        call("b200pf_peer_broadcast", ptr(send[rank]), ptrs, block_elems * 2, rank, world, stream())
    torch.cuda.synchronize()
    for t in range(world):
        for s in range(world):
            assert torch.equal(recv[t][s], send[s]), (t, s)


def test_peer_scatter_rejects_bad_arguments(dev):
    from tt_boltz_b200._lib import call, ptr, stream
    send = torch.zeros(2, 24, dtype=torch.int16, device=dev)
    recv = torch.zeros(2, 24, dtype=torch.int16, device=dev)
    ptrs = (C.c_ulonglong * 2)(recv.data_ptr(), recv.data_ptr())
    with pytest.raises(RuntimeError):
        call("b200pf_peer_scatter", ptr(send), ptrs, 24, 0, 2, stream())          # 24 bytes: not a multiple of 16
    with pytest.raises(RuntimeError):
        call("b200pf_peer_scatter", ptr(send), ptrs, 48, 2, 2, stream())          # rank out of range
    bad = (C.c_ulonglong * 2)(recv.data_ptr(), 0)
    with pytest.raises(RuntimeError):
        call("b200pf_peer_scatter", ptr(send), bad, 48, 0, 2, stream())           # a null receive buffer


def test_peer_barrier_passes_when_every_peer_has_signalled(dev):
    """World of 3 on one device, seen from rank 1: the other ranks' signals are already in its pad (written here
    with torch, generation 7 and the later 8 of a peer that is one barrier ahead), so the wait ends at once, and
    rank 1's own signal lands in slot 1 of every pad."""
    from tt_boltz_b200 import _lib
    from tt_boltz_b200._lib import call, stream
    world, rank, gen = 3, 1, 7
    pads = [torch.zeros(16, dtype=torch.int32, device=dev) for _ in range(world)]
    pads[rank][0], pads[rank][2] = gen, gen + 1
    ptrs = (C.c_ulonglong * world)(*[p.data_ptr() for p in pads])
    call("b200pf_peer_barrier", ptrs, gen, rank, world, 50_000_000, stream())
    assert _lib.device_status() == 0
    for t in range(world):
        assert int(pads[t][rank]) == gen
    assert int(pads[0][0]) == 0 and int(pads[2][2]) == 0


def test_peer_barrier_gives_up_on_a_missing_rank_without_losing_the_context(dev):
    """The second rank's launch is never issued, so its signal never comes: after the 1 ms limit the kernel
    returns, the status word says why, and the device keeps working (no trap, no hang)."""
    import time
    from tt_boltz_b200 import _lib
    from tt_boltz_b200._lib import call, stream
    pads = [torch.zeros(16, dtype=torch.int32, device=dev) for _ in range(2)]
    ptrs = (C.c_ulonglong * 2)(*[p.data_ptr() for p in pads])
    assert _lib.device_status() == 0
    t0 = time.perf_counter()
    call("b200pf_peer_barrier", ptrs, 1, 0, 2, 1_000_000, stream())
    status = _lib.device_status()               # synchronises
    assert time.perf_counter() - t0 < 5.0
    assert status == 4, status
    assert "cross-rank barrier" in _lib.last_error()
    assert int(pads[1][0]) == 1                 # its own signal was sent before it started to wait
    assert _lib.device_status() == 0            # the word is cleared by the read
    x = torch.arange(1024, device=dev, dtype=torch.float32)
    assert float((x * 2).sum()) == 1023 * 1024  # the context is intact
    with pytest.raises(RuntimeError):
        call("b200pf_peer_barrier", ptrs, 2, 0, 2, 0, stream())          # a wait without a limit is refused


@pytest.mark.parametrize("world,nr,c", [(2, 8, 8), (4, 16, 12), (8, 24, 4)])
def test_strided_scatter_is_the_row_column_transposition(dev, world, nr, c):
    """Row shards -> column shards -> row shards of a [N][N][c] tensor with the strided exchange, bit-exact against
    torch indexing (strides exactly as tt_boltz_b200.sharded.rows_to_cols / cols_to_rows pass them)."""
    from tt_boltz_b200._lib import call, ptr, stream
    n = world * nr
    g = torch.Generator().manual_seed(7 * world)
    z = torch.randn(n, n, c, generator=g).to(dev)
    rows = [z[r * nr:(r + 1) * nr].contiguous() for r in range(world)]
    cols = [torch.full((n, nr, c), float("nan"), device=dev) for _ in range(world)]
    ptrs = (C.c_ulonglong * world)(*[t.data_ptr() for t in cols])
    for rank in range(world):
        call("b200pf_peer_scatter_strided", ptr(rows[rank]), ptrs, nr * c * 4, nr, nr * c * 4, n * c * 4, nr * nr * c * 4, nr * c * 4,
             rank, world, stream())
    torch.cuda.synchronize()
    for t in range(world):
        assert torch.equal(cols[t], z[:, t * nr:(t + 1) * nr]), t
    back = [torch.full((nr, n, c), float("nan"), device=dev) for _ in range(world)]
    ptrs = (C.c_ulonglong * world)(*[t.data_ptr() for t in back])
    for rank in range(world):
        call("b200pf_peer_scatter_strided", ptr(cols[rank]), ptrs, nr * c * 4, nr, nr * nr * c * 4, nr * c * 4, nr * c * 4, n * c * 4,
             rank, world, stream())
    torch.cuda.synchronize()
    for t in range(world):
        assert torch.equal(back[t], rows[t]), t


def test_exchanges_with_built_in_barrier(dev):
    """The `_sync` forms on one device: every rank's launch is issued in turn, with the peers' signals already in
    its pad (a kernel that waited for a later launch of the same stream would only run into its limit), so each
    kernel's tail finds them at once.  Checked: the data (bit-exact), the signals each launch leaves in the peers'
    pads, a clean status word, and that the CTA counter is ready for the next launch (two rounds)."""
    from tt_boltz_b200 import _lib
    from tt_boltz_b200._lib import PeerSync, call, ptr, stream
    world, block_elems = 4, 8 * 1500
    g = torch.Generator().manual_seed(3)
    pads = [torch.zeros(16, dtype=torch.int32, device=dev) for _ in range(world)]
    pad_ptrs = (C.c_ulonglong * world)(*[p.data_ptr() for p in pads])
    for gen in (1, 2):
        send = [torch.randint(-30000, 30000, (world, block_elems), generator=g, dtype=torch.int16).to(dev) for _ in range(world)]
        recv = [torch.full((world, block_elems), -1, dtype=torch.int16, device=dev) for _ in range(world)]
        ptrs = (C.c_ulonglong * world)(*[r.data_ptr() for r in recv])
        for rank in range(world):
            pads[rank].fill_(gen)                      # "every peer has arrived"
            sync = PeerSync(pad_ptrs, gen, 50_000_000, 2)
            if rank % 2 == 0:
                call("b200pf_peer_scatter_sync", ptr(send[rank]), ptrs, block_elems * 2, rank, world, C.byref(sync), stream())
            else:       # the strided form with contiguous blocks is the same exchange
                call("b200pf_peer_scatter_strided_sync", ptr(send[rank]), ptrs, block_elems * 2, 1, block_elems * 2, block_elems * 2,
                     block_elems * 2, block_elems * 2, rank, world, C.byref(sync), stream())
        assert _lib.device_status() == 0
        for t in range(world):
            for src in range(world):
                assert torch.equal(recv[t][src], send[src][t]), (gen, t, src)
            assert all(int(pads[t][r]) == gen for r in range(world))
    # all-gather form, and a missing peer: the tail gives up after its limit, status bit 4, context intact
    x = torch.arange(8 * 64, dtype=torch.int16, device=dev)
    out = [torch.zeros(2, 8 * 64, dtype=torch.int16, device=dev) for _ in range(2)]
    ptrs = (C.c_ulonglong * 2)(*[o.data_ptr() for o in out])
    pads2 = [torch.zeros(16, dtype=torch.int32, device=dev) for _ in range(2)]
    pad_ptrs2 = (C.c_ulonglong * 2)(*[p.data_ptr() for p in pads2])
    call("b200pf_peer_broadcast_sync", ptr(x), ptrs, 8 * 64 * 2, 0, 2, C.byref(PeerSync(pad_ptrs2, 1, 1_000_000, 3)), stream())
    assert _lib.device_status() == 4
    assert torch.equal(out[0][0], x) and torch.equal(out[1][0], x)
    assert float(torch.ones(4, device=dev).sum()) == 4.0
    with pytest.raises(RuntimeError):
        call("b200pf_peer_scatter_sync", ptr(x), ptrs, 64, 0, 2, C.byref(PeerSync(pad_ptrs2, 2, 1_000_000, 9)), stream())   # channel out of range


def test_narrowing_exchange_and_bf16_add(dev):
    """fp32 row shards -> bf16 column shards with the narrowing exchange (every rank's launch issued in turn, the
    peers' barrier signals preset), bit-exact against torch's round-to-nearest-even; and z += bf16 update."""
    from tt_boltz_b200 import _lib
    from tt_boltz_b200._lib import PeerSync, call, ptr, stream
    world, nr, c = 4, 8, 16
    n = world * nr
    g = torch.Generator().manual_seed(77)
    z = (torch.randn(n, n, c, generator=g) * 3).to(dev)
    rows = [z[r * nr:(r + 1) * nr].contiguous() for r in range(world)]
    cols = [torch.zeros(n, nr, c, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    ptrs = (C.c_ulonglong * world)(*[t.data_ptr() for t in cols])
    pads = [torch.ones(16, dtype=torch.int32, device=dev) for _ in range(world)]
    pad_ptrs = (C.c_ulonglong * world)(*[p.data_ptr() for p in pads])
    for rank in range(world):
        call("b200pf_peer_scatter_strided_f32_bf16_sync", ptr(rows[rank]), ptrs, nr * c, nr, nr * c, n * c, nr * nr * c, nr * c,
             rank, world, C.byref(PeerSync(pad_ptrs, 1, 50_000_000, 4)), stream())
    assert _lib.device_status() == 0
    for t in range(world):
        assert torch.equal(cols[t], z[:, t * nr:(t + 1) * nr].to(torch.bfloat16)), t
    upd = torch.randn(n * n * c, generator=g).to(torch.bfloat16).to(dev)
    acc = z.clone().view(-1)
    call("b200pf_add_bf16", ptr(acc), ptr(upd), n * n * c, stream())
    assert torch.equal(acc, z.view(-1) + upd.float())
