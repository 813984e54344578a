"""The stage-to-stage hop over peer memory: the push / signal / wait kernels on one
GPU (local buffers stand in for the peer's), the bounded wait, and on two GPUs the
ring pipeline over PeerHop against a sequential evaluation."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

from deserve_b200 import _lib

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_push_signal_wait_on_one_gpu():
    dev = torch.device("cuda:0")
    st = _lib.current_stream_ptr(dev)
    src = torch.arange(1 << 18, dtype=torch.int32, device=dev)
    dst = torch.zeros_like(src)
    flags = torch.zeros(4, dtype=torch.int32, device=dev)
    arrivals = torch.zeros(1, dtype=torch.int32, device=dev)
    for k in range(3):  # the arrival counter returns to zero after every push
        src += 1
        _lib.check(_lib.lib.dsv_peer_push(dst.data_ptr(), src.data_ptr(), src.numel() * 4, flags.data_ptr(), k + 1,
                                          arrivals.data_ptr(), 0, st))
        _lib.check(_lib.lib.dsv_peer_wait(flags.data_ptr(), k + 1, 10**9, st))
        torch.cuda.synchronize()
        assert torch.equal(dst, src) and int(flags[0]) == k + 1 and int(arrivals[0]) == 0
    _lib.check(_lib.lib.dsv_peer_signal(flags.data_ptr() + 4, 7, st))
    torch.cuda.synchronize()
    assert int(flags[1]) == 7
    assert _lib.read_device_status() == 0
    # a flag nobody raises: the wait gives up after 2 ms of GPU time, the status word says so, the
    # context lives on. While the status is unread the link counts as broken: a credit and a push
    # queued behind the failed wait are dropped, a second wait returns at once.
    _lib.check(_lib.lib.dsv_peer_wait(flags.data_ptr() + 8, 1, 2_000_000, st))
    _lib.check(_lib.lib.dsv_peer_signal(flags.data_ptr() + 12, 9, st))
    _lib.check(_lib.lib.dsv_peer_push(dst.data_ptr(), (src + 5).data_ptr(), src.numel() * 4, flags.data_ptr(), 99,
                                      arrivals.data_ptr(), 0, st))
    _lib.check(_lib.lib.dsv_peer_wait(flags.data_ptr() + 8, 1, 500 * 10**9, st))
    torch.cuda.synchronize()
    assert int(flags[3]) == 0 and int(flags[0]) == 3 and torch.equal(dst, src)
    assert _lib.read_device_status() == 4
    assert _lib.read_device_status() == 0
    _lib.check(_lib.lib.dsv_peer_signal(flags.data_ptr() + 12, 9, st))  # status read: the link works again
    torch.cuda.synchronize()
    assert int(flags[3]) == 9
    with pytest.raises(ValueError):
        _lib.check(_lib.lib.dsv_peer_push(dst.data_ptr(), src.data_ptr(), 10, flags.data_ptr(), 1, arrivals.data_ptr(), 0, st))
    with pytest.raises(ValueError):
        _lib.check(_lib.lib.dsv_peer_wait(flags.data_ptr(), 1, 0, st))
    with pytest.raises(ValueError):
        _lib.check(_lib.lib.dsv_peer_wait(flags.data_ptr(), 1, 601 * 10**9, st))


def _stage_math(rank, m, s, x):
    return x * (1.0 + 0.25 * rank) + (m + 1) + 0.5 * s


def _worker(rank, world, port, steps, q):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    from deserve_b200.engine import RingPipeline
    from deserve_b200.peer import PeerHop

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    hop = PeerHop(rank, world, (64, 8), torch.float32, dev, dist.group.WORLD)
    finals = {}

    def stage_fn(u, m, s, x):
        return _stage_math(rank, m, s, x)

    pipe = RingPipeline(rank, world, stage_fn, lambda m: torch.full((64, 8), float(m), device=dev), steps,
                        dist=dist, peer_hop=hop)
    for _ in range(steps * world + world - 1):
        before = len(pipe.completed)
        pipe.advance(1)
        if rank == world - 1 and len(pipe.completed) > before:
            finals[pipe.completed[-1]] = pipe.last_output.clone()
    status = 0
    try:
        hop.close()  # raises if a wait of this rank gave up
    except _lib.DeserveKVError:
        status = 4
    q.put((rank, status, {k: v.cpu().tolist() for k, v in finals.items()}))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ring_over_peer_memory_matches_sequential():
    world, steps = min(torch.cuda.device_count(), 4), 5  # every GPU of the box, up to four
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, steps, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        results = [q.get(timeout=240) for _ in procs]
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:
        for p in procs:  # a worker that is still here hangs: do not leave it behind
            if p.is_alive():
                p.kill()
    assert all(status == 0 for _, status, _ in results), results
    finals = {r: f for r, _, f in results}[world - 1]
    for m in range(world):
        x = torch.full((64, 8), float(m))
        for s in range(steps):
            for r in range(world):
                x = _stage_math(r, m, s, x)
            assert torch.tensor(finals[(m, s)]).equal(x), (m, s)
