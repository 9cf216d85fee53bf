"""Multi-rank logic on CPU (gloo, world_size 2 and 4): the exchanges of the row-sharded trunk
reproduce the unsharded oracle, and the layout helpers are exact inverses."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import pairformer_oracle as orc
from tt_boltz_b200 import synthetic
from tt_boltz_b200.sharded import all_gather_cat, cols_to_rows, rows_to_cols, shard_rows


def _free_port():
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def _worker(rank, world, port, n, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    try:
        from tests.sharded_oracle import sharded_block_cpu
        sd = synthetic.make_weights(1, seed=5, std=0.05, affine_jitter=0.3)
        s, z = synthetic.make_inputs(n, seed=4)
        g = torch.Generator().manual_seed(9)
        tm = torch.ones(n)
        tm[n - 3:] = 0
        pm = (torch.rand(n, n, generator=g) > 0.2).float() * tm[:, None] * tm[None, :]
        r0, nr = shard_rows(n, rank, world)
        z_loc = z[0, r0:r0 + nr].clone()
        # layout helpers: exact round trip and the right content
        zc = rows_to_cols(z_loc)
        assert torch.equal(zc, z[0][:, r0:r0 + nr])
        assert torch.equal(cols_to_rows(zc), z_loc)
        with torch.no_grad():
            s_sh, z_sh = sharded_block_cpu(sd, "layers.0.", s[0], z_loc, tm, pm, rank, world)
            z_full = all_gather_cat(z_sh).view(n, n, -1)
            s_ref, z_ref = orc.pairformer_layer(s[0], z[0], tm, pm, sd, "layers.0.")
        rz = float((z_full - z_ref).norm() / z_ref.norm())
        rs = float((s_sh - s_ref).norm() / s_ref.norm())
        out_q.put((rank, rz, rs, None))
    except Exception as e:  # noqa: BLE001
        out_q.put((rank, None, None, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n", [(2, 16), (4, 24)])
def test_sharded_block_matches_unsharded_oracle(world, n):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, rz, rs, err in res:
        assert err is None, f"rank {rank}: {err}"
        assert rz < 2e-6 and rs < 2e-6, (rank, rz, rs)


def _leaving_worker(rank, world, port, n, out_q):
    """Two blocks; the last rank leaves after the first (between steps, nothing of its own in flight)."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    torch.set_num_threads(1)
    from tests.sharded_oracle import sharded_block_cpu
    sd = synthetic.make_weights(1, seed=5, std=0.05)
    s, z = synthetic.make_inputs(n, seed=4)
    tm, pm = torch.ones(n), torch.ones(n, n)
    r0, nr = shard_rows(n, rank, world)
    z_loc = z[0, r0:r0 + nr].clone()
    with torch.no_grad():
        s1, z_loc = sharded_block_cpu(sd, "layers.0.", s[0], z_loc, tm, pm, rank, world)
        if rank == world - 1:
            out_q.put((rank, "left", 0.0))
            out_q.close()
            out_q.join_thread()                          # the report is out before the process dies
            os._exit(0)                                  # gone without a goodbye, like a crashed worker
        t0 = time.perf_counter()
        try:
            sharded_block_cpu(sd, "layers.0.", s1, z_loc, tm, pm, rank, world)
            out_q.put((rank, "completed", time.perf_counter() - t0))
        except Exception as e:  # noqa: BLE001
            out_q.put((rank, "raised " + type(e).__name__, time.perf_counter() - t0))
    out_q.close()
    out_q.join_thread()
    os._exit(0)                                          # the group cannot be torn down cleanly any more


def test_a_rank_that_leaves_between_blocks_ends_the_others_with_an_error():
    """Failure detection on the host side of the sharded trunk: the survivors' next exchange raises within the
    process-group timeout instead of waiting forever (the reference's counterpart is the job lease that expires
    when a worker stops reporting, tt_bio/distributed.py:22, 214)."""
    world, n = 2, 16
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_leaving_worker, args=(r, world, _free_port_shared(), n, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = dict((r, (what, dt)) for r, what, dt in (q.get(timeout=120) for _ in procs))
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    assert res[world - 1][0] == "left"
    what, dt = res[0]
    assert what.startswith("raised"), what
    assert dt < 60.0, dt


_SHARED_PORT = []


def _free_port_shared():
    if not _SHARED_PORT:
        _SHARED_PORT.append(_free_port())
    return _SHARED_PORT[0]


def test_shard_rows_rejects_ragged():
    assert shard_rows(1024, 3, 8) == (384, 128)
    with pytest.raises(RuntimeError):
        shard_rows(100, 0, 8)
