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
