"""The stage-to-stage hop over peer memory.

Every rank owns an inbox of `depth` message buffers (two by default) plus two
flags per buffer in memory that its neighbours can address (torch symmetric memory: one allocation per rank,
mapped into every process of the node). A message is pushed by the sender's own
kernel with plain stores over NVLink; the same kernel raises the receiver's
data flag once all stores are visible (csrc/peer_hop.cu). The receiver's stream
waits for that flag with a bounded one-thread kernel, and tells the sender with
a credit flag when a buffer may be overwritten. Flags carry message number + 1
and only grow.

    message k of a link travels in buffer k % depth
    receiver: wait data[k % depth] >= k + 1, consume, then credit[k % depth] := k + 1 at the sender
    sender:   wait credit[k % depth] >= k - depth + 1 (message k - depth consumed), push,
              data[k % depth] := k + 1

The push can also be done by the kernel that computes the message: send_buffer()
hands out the destination inside the next rank's inbox (after the credit wait), the
producing kernel stores its result there with ordinary stores, and commit() raises
the flag behind it.

Replaces the HTTP POST per hop of the reference
(deserve_worker/engine/pipeline/processor.py:218-224) and the NCCL send/recv
pair `engine.RingPipeline` uses otherwise.
"""
from __future__ import annotations

import torch

from . import _lib

WAIT_TIMEOUT_NS = 20 * 10**9  # a wait gives up after this much GPU time (ranks may be seconds apart on the host)


class PeerHopTimeout(_lib.DeserveKVError):
    """A bounded wait on a neighbour's flag ran out: a message or a credit never arrived."""


class PeerHop:
    """One rank's end of the ring: receives from (rank - 1), sends to (rank + 1)."""

    def __init__(self, rank: int, world: int, message_shape, dtype: torch.dtype, device: torch.device, group,
                 timeout_ns: int = WAIT_TIMEOUT_NS, depth: int = 2):
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
        if depth < 2:
            raise ValueError("peer hop: at least two buffers per inbox")
        self.depth = depth
        self._flag_bytes = (2 * depth * 4 + 63) // 64 * 64  # data[depth], credit[depth], padded to 64-byte lines
        total = depth * self.msg_bytes + self._flag_bytes
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
        return mem.data_ptr() + (k % self.depth) * self.msg_bytes

    def _flag(self, mem: torch.Tensor, which: int, k: int) -> int:
        return mem.data_ptr() + self.depth * self.msg_bytes + 4 * (self.depth * which + k % self.depth)

    def _wait_credit(self, k: int, st: int) -> None:
        if k >= self.depth:  # the buffer still holds message k - depth until the receiver says otherwise
            _lib.check(_lib.lib.dsv_peer_wait(self._flag(self._mem, 1, k), k - self.depth + 1, self.timeout_ns, st))
            self.launches += 1

    def send(self, y: torch.Tensor) -> None:
        """Push y into the next rank's inbox (stream-ordered; returns at once)."""
        if tuple(y.shape) != self.shape or y.dtype != self.dtype or not y.is_contiguous():
            raise ValueError("peer hop: message differs from the shape / dtype the ring was set up for")
        k, st = self.sent, _lib.current_stream_ptr(y.device)
        self._wait_credit(k, st)
        _lib.check(_lib.lib.dsv_peer_push(self._buf(self._next_mem, k), y.data_ptr(), self.msg_bytes,
                                          self._flag(self._next_mem, 0, k), k + 1, self._arrivals.data_ptr(),
                                          self._sm_count, st))
        self.sent += 1
        self.launches += 1

    def send_buffer(self) -> torch.Tensor:
        """Where the next message lives in the next rank's inbox, as a tensor of the message
        shape in PEER memory, usable by kernels launched after this call on the current
        stream (the wait for the buffer's credit is queued first). Write the message there
        with ordinary stores from a kernel of this package (or an elementwise torch kernel),
        then call commit()."""
        k, st = self.sent, _lib.current_stream_ptr(self._mem.device)
        self._wait_credit(k, st)
        off = (k % self.depth) * self.msg_bytes
        return self._next_mem[off : off + self.msg_bytes].view(self.dtype).view(self.shape)

    def commit(self, y: torch.Tensor | None = None) -> None:
        """The kernels launched so far have written the message into send_buffer(): raise the
        receiver's flag behind them. If y is given and does not already live there, it is
        pushed the ordinary way instead."""
        k, st = self.sent, _lib.current_stream_ptr(self._mem.device)
        if y is not None and y.data_ptr() != self._buf(self._next_mem, k):
            self.send(y)
            return
        _lib.check(_lib.lib.dsv_peer_signal(self._flag(self._next_mem, 0, k), k + 1, st))
        self.sent += 1
        self.launches += 1

    def recv(self) -> torch.Tensor:
        """The next message of the previous rank: a view of this rank's inbox that is
        valid for kernels launched after this call on the current stream, until
        release() of this message."""
        k, st = self.received, _lib.current_stream_ptr(self._mem.device)
        _lib.check(_lib.lib.dsv_peer_wait(self._flag(self._mem, 0, k), k + 1, self.timeout_ns, st))
        self.launches += 1
        off = (k % self.depth) * self.msg_bytes
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
