"""The column-sharded product's host logic on two CPU ranks (gloo): the partition is the
reference's (crates/tt-kernels/src/shard.rs:398-405), and slices gathered and laid side by side
equal the whole product bit for bit, as the reference's gate claims for its chips
(crates/tt-tests/tests/step14_shard.rs:56-121).  The slice products here are NumPy stand-ins for
the engine call; the collective and the layout code are the ones the GPU path runs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from metalium_rs_b200 import sharded


def test_partition_is_whole_tiles_in_order():
    assert sharded.partition(16384, 8) == [(i * 2048, (i + 1) * 2048) for i in range(8)]
    assert sharded.partition(100, 2) == [(0, 64), (64, 100)]
    assert sharded.partition(57344, 4)[3] == (43008, 57344)
    assert sharded.partition(64, 4) == [(0, 32), (32, 64), (64, 64), (64, 64)]  # trailing ranks idle
    for n, g in ((8192, 2), (28672, 8), (1000, 3)):
        parts = sharded.partition(n, g)
        assert parts[0][0] == 0 and parts[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        assert all(lo % 32 == 0 for lo, _ in parts)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(7)  # the same A and B on every rank
        m, k, n = 48, 40, 128
        a = rng.integers(-7, 8, (m, k)).astype(np.float32)
        b = rng.integers(-7, 8, (k, n)).astype(np.float32)
        lo, hi = sharded.partition(n, world)[rank]
        local = torch.from_numpy(a @ b[:, lo:hi])          # K whole: the same sums as one device
        staged = sharded.gather_columns(local, world)
        full = sharded.interleave(staged, n)
        mesh = sharded.MeshExecution(rank, world)           # shard.rs:139-145: completion evidence, gathered over the ranks
        for _ in range(rank + 2):
            mesh.count(1, local.numel() * 4 * (world - 1))
        q.put((rank, bool(np.array_equal(full.numpy(), a @ b)), tuple(staged.shape), mesh.report()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.timeout(120)
def test_two_ranks_gather_the_whole_product_bit_for_bit():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=90) for _ in procs]
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    assert sorted(r[0] for r in res) == [0, 1]
    assert all(r[1] for r in res)
    assert all(r[2] == (2, 48, 64) for r in res)
    for r in res:
        assert r[3] == {"completed_matmuls": [2, 3], "acknowledged_transfers": r[0] + 2,
                        "acknowledged_bytes": (r[0] + 2) * 48 * 64 * 4}


def _failing_worker(rank, world, port, q):
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=15))
    dist.barrier()
    if rank == 1:
        q.put((1, "raised", 0.0))
        q.close(); q.join_thread()     # the message is out before the process goes
        os._exit(3)                    # the rank dies between steps: no collective of its own in flight, no clean-up
    t0 = time.monotonic()
    try:
        sharded.gather_columns(torch.zeros((4, 8)), world)
        q.put((0, "completed", time.monotonic() - t0))
    except Exception as ex:            # the survivor's gather ends in an error (a closed connection or the group's timeout)
        q.put((0, "error: " + type(ex).__name__, time.monotonic() - t0))
    q.close(); q.join_thread()
    os._exit(0)


@pytest.mark.timeout(120)
def test_a_rank_that_dies_before_the_gather_is_an_error_on_the_other_not_a_hang():
    # Failure is made on the host only: rank 1 exits before the all-gather; rank 0's collective must return with an
    # error inside the process group's timeout (crates/tt-device/src/transport.rs:208-217: every wait is bounded).
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict()
    for _ in procs:
        r = q.get(timeout=60)
        res[r[0]] = r
    for p in procs:
        p.join(30)
    assert res[1][1] == "raised" and procs[1].exitcode == 3
    assert res[0][1].startswith("error"), res[0]
    assert res[0][2] < 30.0 and procs[0].exitcode == 0
