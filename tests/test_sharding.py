"""Host logic of the multi-GPU path on CPU: world_size 2 over gloo."""
import os
import socket

import numpy as np
import torch.multiprocessing as mp

from rustygradients_b200.sharding import gather_ids, max_over_ranks, shard_range


def test_shard_range_partitions():
    for n in (0, 1, 7, 8, 64, 65):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, n, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = shard_range(n, rank, world)
    local = (np.arange(lo, hi, dtype=np.uint32)[:, None] * 10 + np.arange(4, dtype=np.uint32)[None, :])
    ids = gather_ids(local, n, rank, world)
    slow = max_over_ranks(1.0 + rank, world)
    q.put((rank, ids.tolist(), slow))
    dist.barrier()
    dist.destroy_process_group()


def test_gather_over_gloo_world_2():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    n, world = 5, 2   # ragged: 3 + 2
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, q)) for r in range(world)]
    [p.start() for p in procs]
    res = [q.get(timeout=120) for _ in range(world)]
    [p.join(60) for p in procs]
    want = (np.arange(n)[:, None] * 10 + np.arange(4)[None, :]).tolist()
    for rank, ids, slow in res:
        assert ids == want and slow == 2.0


def _worker_with_a_missing_rank(rank, world, port, q):
    """Rank 1 leaves between steps (host-side failure); rank 0 must get an error from its next gather, not hang."""
    import datetime
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=10))
    local = np.full((1, 4), rank, np.uint32)
    first = gather_ids(local, world, rank, world)          # step 1: both ranks present
    if rank == 1:
        q.put((rank, "left"))
        q.close()
        q.join_thread()                                     # the item is on the pipe before the process goes
        os._exit(0)                                         # no collective in flight
    try:
        gather_ids(local, world, rank, world)               # step 2: the peer is gone
        q.put((rank, "no error"))
    except Exception as e:  # noqa: BLE001  (gloo raises RuntimeError / DistBackendError depending on the version)
        q.put((rank, "error:" + type(e).__name__, first.tolist()))


def test_gather_reports_a_rank_that_left():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_with_a_missing_rank, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in procs]
    res = dict((r[0], r[1:]) for r in (q.get(timeout=120) for _ in range(2)))
    [p.join(60) for p in procs]
    assert res[1] == ("left",)
    assert res[0][0].startswith("error:") and res[0][1] == [[0, 0, 0, 0], [1, 1, 1, 1]]
