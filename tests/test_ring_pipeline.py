"""The layer-sharded ring pipeline on CPU: world_size 2 and 3 gloo ranks must
produce exactly what one rank applying all stages in order produces."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _stage_math(rank, m, s, x):
    return x * (1.0 + 0.25 * rank) + (m + 1) + 0.5 * s


def _expected(world, steps):
    out = {}
    for m in range(world):
        x = torch.full((4, 3), float(m))
        for s in range(steps):
            for r in range(world):
                x = _stage_math(r, m, s, x)
            out[(m, s)] = x.clone()
    return out


def _worker(rank, world, port, steps, split, q):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    from deserve_b200.engine import RingPipeline

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    seen = []

    def stage_fn(u, m, s, x):
        seen.append((m, s))
        return _stage_math(rank, m, s, x)

    pipe = RingPipeline(rank, world, stage_fn, lambda m: torch.full((4, 3), float(m)), steps, dist=dist)
    finals = {}
    total_slots = steps * world + world - 1
    done = 0
    for n in split + [total_slots - sum(split)]:  # resume after a pause, like warm-up then timed steps
        before = len(pipe.completed)
        for _ in range(n):
            pipe.advance(1)
            if rank == world - 1 and len(pipe.completed) > before:
                finals[pipe.completed[-1]] = pipe.last_output.clone()
                before = len(pipe.completed)
        done += n
        dist.barrier()
    q.put((rank, seen, {k: v.tolist() for k, v in finals.items()}))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,steps,split", [(2, 3, [2]), (3, 2, [3, 1]), (2, 1, [])])
def test_ring_pipeline_matches_sequential(world, steps, split):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, steps, split, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want = _expected(world, steps)
    by_rank = {r: (seen, finals) for r, seen, finals in results}
    for r in range(world):
        # every rank runs every (microbatch, step) unit once, in ring order
        assert by_rank[r][0] == [(u % world, u // world) for u in range(steps * world)]
    finals = by_rank[world - 1][1]
    assert set(finals) == set(want)
    for key, val in want.items():
        assert torch.tensor(finals[key]).equal(val), key


def test_single_rank_ring_is_a_plain_loop():
    sys.path.insert(0, str(ROOT))
    from deserve_b200.engine import RingPipeline

    pipe = RingPipeline(0, 1, lambda u, m, s, x: x + 1, lambda m: torch.zeros(2), 5)
    pipe.advance(5)
    assert pipe.last_output.tolist() == [5.0, 5.0] and pipe.completed == [(0, s) for s in range(5)]


def _dying_worker(rank, world, port, q):
    """Rank 1 leaves between two slots (host-side failure, nothing in flight); rank 0 must get an
    error from its next exchange within the process-group timeout instead of waiting forever."""
    sys.path.insert(0, str(ROOT))
    import datetime
    import time

    import torch.distributed as dist

    from deserve_b200.engine import RingPipeline

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    pipe = RingPipeline(rank, world, lambda u, m, s, x: x + 1, lambda m: torch.zeros(3), 50, dist=dist)
    pipe.advance(4)
    if rank == 1:
        dist.destroy_process_group()
        q.put((rank, "left"))
        return
    t0 = time.time()
    try:
        pipe.advance(20)
        q.put((rank, "no error"))
    except Exception as exc:  # gloo reports the closed / timed-out peer
        q.put((rank, f"error after {time.time() - t0:.1f}s: {type(exc).__name__}"))


def test_a_rank_that_leaves_surfaces_as_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_dying_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=90) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert got[1] == "left"
    assert got[0].startswith("error after"), got[0]
    assert float(got[0].split()[2][:-2]) < 30.0
