"""The layer-sharded ring pipeline on CPU: world_size 2, 3 and 4 gloo ranks (with as
many microbatches as stages, or more) must produce exactly what one rank applying
all stages in order produces."""
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


def _expected(world, steps, mbs=None):
    out = {}
    for m in range(mbs or world):
        x = torch.full((4, 3), float(m))
        for s in range(steps):
            for r in range(world):
                x = _stage_math(r, m, s, x)
            out[(m, s)] = x.clone()
    return out


class _GlooHop:
    """Stands in for deserve_b200.peer.PeerHop on CPU: same three calls, gloo underneath. It checks
    the protocol the ring must follow: every message sent is received once, in order, and released."""

    def __init__(self, dist, rank, world):
        self.dist, self.nxt, self.prv = dist, (rank + 1) % world, (rank - 1) % world
        self.sent = self.received = self.released = 0
        self._pending = []
        self.depth = 16  # inbox buffers: the ring asks for microbatches - stages + 2

    def send(self, y):
        self._pending.append(self.dist.isend(torch.cat([torch.tensor([float(self.sent)]), y.flatten()]), self.nxt))
        self.sent += 1

    def recv(self):
        assert self.received == self.released, "recv() before the previous message was released"
        buf = torch.empty(1 + 12)
        self.dist.recv(buf, self.prv)
        assert int(buf[0]) == self.received, "messages out of order"
        self.received += 1
        return buf[1:].reshape(4, 3).clone()

    def release(self):
        self.released += 1

    def close(self):
        for w in self._pending:
            w.wait()


def _worker(rank, world, port, steps, split, q, mbs=None):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    from deserve_b200.engine import RingPipeline

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    seen = []

    def stage_fn(u, m, s, x):
        seen.append((m, s))
        return _stage_math(rank, m, s, x)

    hop = _GlooHop(dist, rank, world) if split == "hop" else None
    split = [] if split == "hop" else split
    M = mbs or world
    pipe = RingPipeline(rank, world, stage_fn, lambda m: torch.full((4, 3), float(m)), steps, dist=dist, peer_hop=hop,
                        microbatches=M)
    finals = {}
    total_slots = steps * M + world - 1
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
    pipe.flush()
    if hop is not None:
        hop.close()
        # rank 0 takes its first `world` inputs from first_input, everything else arrives over the hop
        assert hop.received == hop.released == steps * M - (M if rank == 0 else 0)
        assert hop.sent == steps * M - (M if rank == world - 1 else 0)
    q.put((rank, seen, {k: v.tolist() for k, v in finals.items()}))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,steps,split,mbs", [(2, 3, [2], None), (3, 2, [3, 1], None), (2, 1, [], None),
                                                   (3, 3, "hop", None), (4, 2, "hop", None),
                                                   (2, 3, [5], 4), (3, 2, [4, 3], 5), (2, 2, [], 8),
                                                   (2, 3, "hop", 4), (3, 2, "hop", 5)])
def test_ring_pipeline_matches_sequential(world, steps, split, mbs):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, steps, split, q, mbs)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    M = mbs or world
    want = _expected(world, steps, M)
    by_rank = {r: (seen, finals) for r, seen, finals in results}
    for r in range(world):
        # every rank runs every (microbatch, step) unit once, in ring order
        assert by_rank[r][0] == [(u % M, u // M) for u in range(steps * M)]
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
    # three microbatches on one stage: each one's output is its own next input
    outs = {}
    pipe = RingPipeline(0, 1, lambda u, m, s, x: outs.setdefault((m, s), x * 2 + m), lambda m: torch.ones(1), 3,
                        microbatches=3)
    pipe.advance(9)
    for m in range(3):
        x = 1.0
        for s in range(3):
            x = 2 * x + m
            assert outs[(m, s)].item() == x
    assert [t.item() for t in pipe.take_finals()] == [outs[(m, 2)].item() for m in range(3)]


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


class _FakeWork:
    def __init__(self, fn=None):
        self._fn, self._done = fn, fn is None

    def wait(self):
        if not self._done:
            self._fn()
            self._done = True

    def is_completed(self):
        return True


class _RendezvousLinks:
    """All ranks of a ring in ONE process, advanced slot by slot in rank order, over links that
    behave like NCCL point-to-point: a send completes only when its receive has been posted. The
    fake keeps, per directed link, the messages sent and the receives posted, so a test can ask
    after any slot whether a send is still waiting for its receive (a device synchronisation at
    that point would then never return)."""

    def __init__(self, world):
        self.sent = {(r, (r + 1) % world): [] for r in range(world)}
        self.posted = {k: 0 for k in self.sent}
        self.taken = {k: 0 for k in self.sent}

    def for_rank(self, rank):
        links = self

        class _Dist:
            def isend(self, t, dst, group=None):
                links.sent[(rank, dst)].append(t.clone())
                return _FakeWork()

            def irecv(self, buf, src, group=None):
                key = (src, rank)
                links.posted[key] += 1
                index = links.posted[key] - 1

                def deliver():
                    assert index < len(links.sent[key]), "the receiver would block: nothing was sent yet"
                    assert index == links.taken[key], "receives completed out of order"
                    buf.copy_(links.sent[key][index])
                    links.taken[key] += 1

                return _FakeWork(deliver)

        return _Dist()

    def unmatched_sends(self):
        return {k: len(v) - self.posted[k] for k, v in self.sent.items() if len(v) > self.posted[k]}


@pytest.mark.parametrize("send_final", [False, True])
@pytest.mark.parametrize("world,mbs,steps", [(2, 2, 3), (2, 4, 3), (2, 8, 2), (4, 8, 2), (3, 5, 3), (8, 8, 2)])
def test_no_send_is_left_without_a_posted_receive_at_any_slot_boundary(world, mbs, steps, send_final):
    """With more microbatches than stages the first stage consumes the last stage's output several
    slots after it was sent; every such send must already have its receive posted when all ranks
    have run the same number of slots, because the benchmark synchronises the device there."""
    sys.path.insert(0, str(ROOT))
    from deserve_b200.engine import RingPipeline

    links = _RendezvousLinks(world)
    finals = {}

    def make(rank):
        def stage_fn(u, m, s, x):
            y = _stage_math(rank, m, s, x)
            if rank == world - 1:
                finals[(m, s)] = y.clone()
            return y
        return RingPipeline(rank, world, stage_fn, lambda m: torch.full((4, 3), float(m)), steps, dist=links.for_rank(rank),
                            microbatches=mbs, links=("send", "recv"), send_final=send_final)

    pipes = [make(r) for r in range(world)]
    for slot in range(steps * mbs + world - 1):
        for p in pipes:
            p.advance(1)
        assert not links.unmatched_sends(), (slot, links.unmatched_sends())
    want = _expected(world, steps, mbs)
    assert set(finals) == set(want)
    for key, val in want.items():
        assert finals[key].equal(val), key
    if send_final:  # the first stage also gets the last stage's outputs of the final token step
        got = pipes[0].take_finals()
        assert len(got) == mbs and all(got[m].equal(want[(m, steps - 1)]) for m in range(mbs))
        assert all(len(v) == links.taken[k] for k, v in links.sent.items())  # every message was consumed
