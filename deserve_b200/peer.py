"""The stage-to-stage hop over peer memory.

Every rank owns an inbox of two message buffers plus four flags in memory that
its neighbours can address (torch symmetric memory: one allocation per rank,
mapped into every process of the node). A message is pushed by the sender's own
kernel with plain stores over NVLink; the same kernel raises the receiver's
data flag once all stores are visible (csrc/peer_hop.cu). The receiver's stream
waits for that flag with a bounded one-thread kernel, and tells the sender with
a credit flag when a buffer may be overwritten. Flags carry message number + 1
and only grow.

    message k of a link travels in buffer k % 2
    receiver: wait data[k % 2] >= k + 1, consume, then credit[k % 2] := k + 1 at the sender
    sender:   wait credit[k % 2] >= k - 1 (message k - 2 consumed), push, data[k % 2] := k + 1

Replaces the HTTP POST per hop of the reference
(deserve_worker/engine/pipeline/processor.py:218-224) and the NCCL send/recv
pair `engine.RingPipeline` uses otherwise.
"""
from __future__ import annotations

import torch

from . import _lib

_FLAG_INTS = 16          # data[2], credit[2], padding: one 64-byte line
WAIT_TIMEOUT_NS = 20 * 10**9  # a wait gives up after this much GPU time (ranks may be seconds apart on the host)


class PeerHopTimeout(_lib.DeserveKVError):
    """A bounded wait on a neighbour's flag ran out: a message or a credit never arrived."""


class PeerHop:
    """One rank's end of the ring: receives from (rank - 1), sends to (rank + 1)."""

    def __init__(self, rank: int, world: int, message_shape, dtype: torch.dtype, device: torch.device, group,
                 timeout_ns: int = WAIT_TIMEOUT_NS):
        import torch.distributed._symmetric_memory as symm_mem

        self.timeout_ns = int(timeout_ns)
        _lib.require_cuda(torch.empty(0, device=device))
        self.rank, self.world = rank, world
        self.shape, self.dtype = tuple(message_shape), dtype
        n = 1
        for d in self.shape:
            n *= d
        self.msg_bytes = n * torch.empty(0, dtype=dtype).element_size()
        if self.msg_bytes % 16:
            raise ValueError("peer hop: message size must be a multiple of 16 bytes")
        total = 2 * self.msg_bytes + _FLAG_INTS * 4
        self._mem = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self._mem.zero_()
        torch.cuda.synchronize(device)
        self._handle = symm_mem.rendezvous(self._mem, group)
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        view = lambda r: self._handle.get_buffer(r, (total,), torch.uint8, 0)
        self._next_mem, self._prev_mem = view(nxt), view(prv)
        self._arrivals = torch.zeros(1, dtype=torch.int32, device=device)
        self._sm_count = _lib.device_info()[0]
        self.sent = 0       # messages pushed to the next rank
        self.received = 0   # messages taken from the previous rank
        self.launches = 0   # kernels launched for the hop so far
        self._handle.barrier()  # every inbox is zeroed before anyone writes a flag

    # addresses inside a rank's allocation
    def _buf(self, mem: torch.Tensor, k: int) -> int:
        return mem.data_ptr() + (k % 2) * self.msg_bytes

    def _flag(self, mem: torch.Tensor, which: int, k: int) -> int:
        return mem.data_ptr() + 2 * self.msg_bytes + 4 * (2 * which + k % 2)

    def send(self, y: torch.Tensor) -> None:
        """Push y into the next rank's inbox (stream-ordered; returns at once)."""
        if tuple(y.shape) != self.shape or y.dtype != self.dtype or not y.is_contiguous():
            raise ValueError("peer hop: message differs from the shape / dtype the ring was set up for")
        k, st = self.sent, _lib.current_stream_ptr(y.device)
        if k >= 2:  # the buffer still holds message k - 2 until the receiver says otherwise
            _lib.check(_lib.lib.dsv_peer_wait(self._flag(self._mem, 1, k), k - 1, self.timeout_ns, st))
            self.launches += 1
        _lib.check(_lib.lib.dsv_peer_push(self._buf(self._next_mem, k), y.data_ptr(), self.msg_bytes,
                                          self._flag(self._next_mem, 0, k), k + 1, self._arrivals.data_ptr(),
                                          self._sm_count, st))
        self.sent += 1
        self.launches += 1

    def recv(self) -> torch.Tensor:
        """The next message of the previous rank: a view of this rank's inbox that is
        valid for kernels launched after this call on the current stream, until
        release() of this message."""
        k, st = self.received, _lib.current_stream_ptr(self._mem.device)
        _lib.check(_lib.lib.dsv_peer_wait(self._flag(self._mem, 0, k), k + 1, self.timeout_ns, st))
        self.launches += 1
        off = (k % 2) * self.msg_bytes
        return self._mem[off : off + self.msg_bytes].view(self.dtype).view(self.shape)

    def release(self) -> None:
        """The kernels launched so far have consumed the last received message: hand
        its buffer back to the sender."""
        k, st = self.received, _lib.current_stream_ptr(self._mem.device)
        _lib.check(_lib.lib.dsv_peer_signal(self._flag(self._prev_mem, 1, k), k + 1, st))
        self.received += 1
        self.launches += 1

    def check(self) -> None:
        """Synchronise the device and raise PeerHopTimeout if a wait of this process gave up
        (the status word is cleared by the read). After a timeout the device side of the hop
        has stopped pushing and crediting, so the data received since is not to be used."""
        status = _lib.read_device_status()
        if status == 4:
            raise PeerHopTimeout(f"rank {self.rank}: a peer-memory wait timed out after {self.timeout_ns / 1e9:.1f} s "
                                 f"(sent {self.sent}, received {self.received} messages)")
        if status != 0:
            raise _lib.DeserveKVError(f"device self-check fired: status {status}")

    def close(self) -> None:
        """Drain, verify that no wait gave up, and leave together with the neighbours."""
        try:
            self.check()
        finally:
            self._handle.barrier()
