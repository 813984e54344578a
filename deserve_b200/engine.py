"""Execution of the KV hot path over a stage's layers, and the layer-sharded
ring pipeline that spreads the layers over the GPUs of one node.

`KVStage` is what one pipeline stage does with one microbatch on the KV path:
for each of its layers, append the step's new K/V rows into the pages and run
paged decode attention (the inner part of the reference's
Attention.paged_forward, deserve_worker/model/layer/attention.py:174-185,
looped by LayerStorage.forward, deserve_worker/layer_storage.py:182-197).

`RingPipeline` is the microbatch rotation of the reference
(deserve_worker/engine/pipeline/processor.py:231-243: `num_rounds` microbatches
circulate through the stages, the last stage feeding the first) with the HTTP
hop replaced by NCCL send/recv: one grouped send+recv per slot moves every
stage's activations to its successor.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import numpy as np
import torch

from . import ops
from .context import FlashDecodeCtx
from .kvcache import PagedKVCache
from .task import TaskData
from .request import StepRequest  # noqa: F401  (re-exported: the stage loop's input type)
from .trace import phase


@dataclass
class StepDescriptors:
    """Device-resident descriptors + decode plan of one microbatch step."""

    indptr: torch.Tensor
    kv_page_indices: torch.Tensor
    kv_page_indptr: torch.Tensor
    kv_last_page_lens: torch.Tensor
    plan_host: np.ndarray
    plan_dev: torch.Tensor
    workspace_bytes: int
    kv_tokens: int


def prepare_decode_step(task_datas: Sequence[TaskData], kvcaches: Sequence[PagedKVCache], n_q_heads: int,
                        sm_count: int) -> StepDescriptors:
    """Host half of a decode step: grow the caches, build the ragged descriptors
    (one H2D copy) and the split-KV plan (one more)."""
    ctx = FlashDecodeCtx.init_paged_decode_ctx(list(task_datas), list(kvcaches), None)
    pool = ctx.page_pool
    plan = torch.empty(ops.plan_capacity(ctx.bsz, sm_count), dtype=torch.int32, pin_memory=True)  # kept by the caller
    used, ws = ops.make_decode_plan(ctx.host["kv_page_indptr"], n_q_heads, pool.n_kv_heads, pool.head_dim,
                                    pool.page_size, pool.main_dtype, sm_count, plan.numpy())
    plan_dev = plan[:used].to(pool.main_device, non_blocking=True)
    kv_tokens = int(((np.diff(ctx.host["kv_page_indptr"]) - 1) * pool.page_size + ctx.host["kv_last_page_lens"]).sum())
    sd = StepDescriptors(ctx.indptr, ctx.kv_page_indices, ctx.kv_page_indptr, ctx.kv_last_page_lens, plan.numpy(),
                         plan_dev, ws, kv_tokens)
    sd._pinned = plan  # keeps the pinned plan alive as long as plan_host is used
    return sd


class KVStage:
    """The KV path of the layers [layer_begin, layer_end) of one pool."""

    def __init__(self, pool, n_q_heads: int, layer_begin: int = 0, layer_end: Optional[int] = None,
                 workspace_bytes: int = 64 << 20):
        self.pool = pool
        self.n_q_heads = n_q_heads
        self.layer_begin = layer_begin
        self.layer_end = pool.num_layers if layer_end is None else layer_end
        self.workspace = torch.empty(workspace_bytes, dtype=torch.uint8, device=pool.main_device)

    def forward(self, x: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, sd: StepDescriptors,
                on_attention: Callable[[int], None] | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """x: [B, Hq, D] query of the first layer; layer l's attention output is
        layer l+1's query. k_new, v_new: [layers, B, Hkv, D] rows to append.
        on_attention(i), if given, is called before and after every attention
        launch (i = 2*layer, 2*layer+1) so a caller can bracket it with events.
        out, if given, receives the last layer's output: the attention kernel then
        stores its result straight into that buffer, which may be the next stage's
        inbox in peer memory (the compute kernel itself does the hop)."""
        if sd.workspace_bytes > self.workspace.numel():
            raise RuntimeError(f"stage workspace too small: need {sd.workspace_bytes} bytes")
        n = self.layer_end - self.layer_begin
        for i, layer in enumerate(range(self.layer_begin, self.layer_end)):
            pages = self.pool.pages[layer]
            ops.append_paged_kv_cache(k_new[i], v_new[i], sd.indptr, pages, sd.kv_page_indices, sd.kv_page_indptr,
                                      sd.kv_last_page_lens)
            if on_attention is not None:
                on_attention(2 * i)
            x = ops.paged_decode(x, pages, sd.kv_page_indices, sd.kv_page_indptr, sd.kv_last_page_lens, sd.plan_host,
                                 sd.plan_dev, self.workspace, out=out if i == n - 1 else None)
            if on_attention is not None:
                on_attention(2 * i + 1)
        return x


def make_ring_links(dist, rank: int, world: int, device=None):
    """One two-rank process group per directed link r -> (r+1) % world, created in
    the same order on every rank. Returns (group this rank sends on, group it
    receives on). A link carries traffic in one direction only, so a receive
    posted early never sits in front of a send on the same communicator (one
    communicator for the whole ring would need grouped send+recv calls, which tie
    a stage's send to its neighbour's progress).

    With `device` given, one element travels over every link before the function
    returns. The first point-to-point call on a communicator sets up the connection
    and blocks the host until the peer makes its first call on the same
    communicator; the links are therefore opened in the order of their index (a
    rank opens the lower-numbered of its two links first), which pairs the calls
    up along the ring instead of leaving two neighbours each waiting in a different
    link's set-up. Later calls find the connections open and never block the host."""
    if world < 2:
        return None, None
    groups = [dist.new_group([r, (r + 1) % world]) for r in range(world)]
    out_link, in_link = rank, (rank - 1) % world
    if device is not None:
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        one, got = torch.ones(1, device=device), torch.zeros(1, device=device)
        works = []
        for link in sorted({out_link, in_link}):
            if link == out_link:
                works.append(dist.isend(one, nxt, group=groups[link]))
            if link == in_link:
                works.append(dist.irecv(got, prv, group=groups[link]))
        for w in works:
            w.wait()
        if torch.device(device).type == "cuda":
            torch.cuda.synchronize(device)
        if float(got.item()) != 1.0:
            raise RuntimeError("ring link warm-up: the message from the previous stage did not arrive")
    return groups[out_link], groups[in_link]


class RingPipeline:
    """W stages (ranks) and M >= W microbatches in a ring. In slot t, rank r works on
    unit u = t - r, i.e. microbatch u % M at token step u // M, and hands its output
    to rank (r+1) % W; the last stage feeds the first. After the first W-1 slots
    every rank is busy in every slot. The object keeps its position, so a caller
    can run some slots, synchronise, and continue with a full ring.

    The hop never blocks the host, and blocks the compute stream only where the data
    is needed: the send of slot t's output is queued behind the slot's kernels and is
    not waited for, the receive for slot t+1 is posted right after it, and the
    compute stream waits for a message right before the kernels that read it. Three
    transports:
      * links=(send_group, recv_group) from make_ring_links: NCCL (or gloo)
        isend / irecv, one communicator per directed link;
      * peer_hop (deserve_b200.peer.PeerHop): the sender stores into the next GPU's
        inbox; with direct=True the stage's last kernel writes its output there
        itself (stage_fn gets out=<inbox buffer>) and only a flag follows;
      * neither (W == 1): the output is the next input.

    stage_fn(unit, microbatch, token_step, x[, out=...]) -> y runs the rank's layers.
    first_input(microbatch) gives rank 0 its input for token step 0.
    recv_spec(unit) -> (shape, dtype, device) of the tensor this rank consumes as
    input of `unit`; None: same as what first_input / the previous message had.
    """

    def __init__(self, rank: int, world: int, stage_fn, first_input, total_steps: int, group=None, dist=None,
                 recv_spec=None, peer_hop=None, microbatches: int | None = None, links=None, direct: bool = False,
                 send_final: bool = False):
        # send_final: the last stage also hands on its output of every microbatch's LAST token step; the first
        # stage does not compute on it but fetches it with take_finals() once all slots have run (a pipeline
        # whose first stage finishes the last stage's work, e.g. the second half of a split output head)
        self.send_final = send_final
        if send_final and peer_hop is not None:
            raise ValueError("send_final is implemented for the NCCL / gloo links")
        self.recv_spec = recv_spec
        self.peer_hop = peer_hop
        self.direct = direct and peer_hop is not None
        self.rank, self.world = rank, world
        self.M = world if microbatches is None else microbatches
        if self.M < world:
            raise ValueError(f"{self.M} microbatches cannot keep {world} stages busy")
        if peer_hop is not None and getattr(peer_hop, "depth", 2) < self.M - world + 2:
            raise ValueError("peer hop: the inbox needs microbatches - stages + 2 buffers")
        self.stage_fn, self.first_input = stage_fn, first_input
        self.units = total_steps * self.M
        self.dist = dist
        if world > 1 and peer_hop is None and links is None:
            like = first_input(0)
            links = make_ring_links(dist, rank, world, like.device if like.is_cuda else None)
        self.send_group, self.recv_group = links if links is not None else (None, None)
        self.slot = 0
        self.last_output: torch.Tensor | None = None
        self.completed: list[tuple[int, int]] = []  # (microbatch, token_step) finished on the last rank
        self._carry: dict = {}                       # W == 1: microbatch -> the output that is its next input
        self._posted: dict = {}                      # slot -> (work, buffer) of receives in flight
        self._sends: list = []                       # (work, tensor) of sends in flight (keeps the tensor alive)
        self._like = None

    # ---- schedule ---------------------------------------------------------------------------
    def _unit(self, rank: int, slot: int) -> int | None:
        u = slot - rank
        return u if 0 <= u < self.units else None

    def _computes(self, rank: int, slot: int) -> bool:
        return self._unit(rank, slot) is not None

    def _from_hop(self, slot: int) -> bool:
        """Does a message for this rank's `slot` arrive over the hop? (With send_final the first stage
        also receives, in the M slots after its last unit, the last stage's final outputs.)"""
        if self.world == 1:
            return False
        u = self._unit(self.rank, slot)
        if u is None:
            return self.send_final and self.rank == 0 and self.units <= slot < self.units + self.M
        return not (self.rank == 0 and u < self.M)

    def _sends_after(self, slot: int) -> bool:
        """Is this rank's output of `slot` somebody's input? (The last stage's output of a
        microbatch's final token step is not, unless send_final.)"""
        u = self._unit(self.rank, slot)
        return u is not None and self.world > 1 and (self.rank < self.world - 1 or self.send_final
                                                      or u + self.M < self.units)

    def take_finals(self) -> list:
        """First stage, after every slot has run: the last stage's outputs of the final token step, one per
        microbatch in microbatch order (send_final=True). On one stage: that stage's own last outputs."""
        if self.world == 1:
            return [self._carry[m] for m in range(self.M)]
        if self.rank != 0:
            return []
        return [self._take_recv(self.units + m) for m in range(self.M)]

    # ---- NCCL / gloo links ---------------------------------------------------------------------
    def _post_recv(self, slot: int) -> None:
        if slot in self._posted or not self._from_hop(slot):
            return
        if self.recv_spec is not None:
            shape, dtype, device = self.recv_spec(slot - self.rank)  # the unit; >= units for a final output
            buf = torch.empty(shape, dtype=dtype, device=device)
        else:
            buf = torch.empty_like(self._like if self._like is not None else self.first_input(0))
        prv = (self.rank - 1) % self.world
        self._posted[slot] = (self.dist.irecv(buf, prv, group=self.recv_group), buf)

    def _take_recv(self, slot: int) -> torch.Tensor:
        self._post_recv(slot)
        work, buf = self._posted.pop(slot)
        with phase("recv"):
            work.wait()  # NCCL: the compute stream waits for the message; gloo: the host does
        return buf

    def _send(self, y: torch.Tensor) -> None:
        nxt = (self.rank + 1) % self.world
        self._sends = [(w, t) for w, t in self._sends if not w.is_completed()]
        with phase("send"):
            self._sends.append((self.dist.isend(y, nxt, group=self.send_group), y))

    def flush(self) -> None:
        """Wait for the sends still in flight (end of a run)."""
        for w, _ in self._sends:
            w.wait()
        self._sends = []

    # ---- slots ----------------------------------------------------------------------------------
    def advance(self, n_slots: int) -> None:
        W, r, M = self.world, self.rank, self.M
        hop = self.peer_hop
        for _ in range(n_slots):
            t = self.slot
            u = self._unit(r, t)
            y = None
            if u is not None:
                m, s = u % M, u // M
                from_hop = self._from_hop(t)
                if not from_hop:
                    x = self.first_input(m) if s == 0 else self._carry.pop(m)
                elif hop is not None:
                    x = hop.recv()
                else:
                    x = self._take_recv(t)
                sends = self._sends_after(t)
                if W == 1 and s + 1 == self.units // M:
                    sends = False  # one stage: the final outputs stay in _carry for take_finals()
                if self.direct and sends:
                    y = self.stage_fn(u, m, s, x, out=hop.send_buffer())
                else:
                    y = self.stage_fn(u, m, s, x)
                if from_hop and hop is not None:
                    hop.release()
                if r == W - 1:
                    self.completed.append((m, s))
                    self.last_output = y
                if self._like is None:
                    self._like = x
                if sends:
                    if hop is None:
                        self._send(y)
                    elif self.direct:
                        hop.commit(y)
                    else:
                        hop.send(y)
                elif W == 1:
                    self._carry[m] = y
            if hop is None and W > 1:
                # Receives are posted right AFTER this slot's work and send have been queued, never before:
                # a posted receive is a kernel that spins until the peer's send arrives, and any call on the
                # host that implicitly waits for the device (a pinned allocation, a lazily loaded kernel
                # module, a cudaFree) then waits for it. Posted here, a receive only ever depends on work
                # its peers queued for EARLIER slots, so such a wait always ends; posted before this slot's
                # own work, two neighbours could wait for each other's current slot forever.
                # The first stage consumes the last stage's output M - W + 1 slots after it was sent and
                # posts that far ahead, so that every send has its receive whenever all ranks have run the
                # same number of slots (a send completes only once its receive is posted, and callers
                # synchronise the device at such points).
                for ahead in range(1, (M - W + 1 if r == 0 else 1) + 1):
                    self._post_recv(t + ahead)
            self.slot += 1


# =================================================================================================
# Engine-facing classes with the reference's names and call order
# =================================================================================================
from dataclasses import field as _field  # noqa: E402

from .context import FlashPrefillCtx  # noqa: E402
from .kvcache import ChunkHandle, KVCacheManager, PageTableAllocator, VirtualPagedKVCache, CopiedPinnedMemory  # noqa: E402
from .task import SamplingParams, TaskManager  # noqa: E402


@dataclass
class BatchResult:
    """deserve_worker/execution/result.py:6-13."""

    ongoing_xs: torch.Tensor
    ongoing_task_ids: list
    all_xs: torch.Tensor
    all_task_ids: list
    done_task_ids: list
    needed_probs: dict


_WRAPPERS: dict = {}


def stage_wrappers(device) -> tuple:
    """One 128 MiB workspace and one decode + one prefill wrapper per device (the
    reference creates them at import time, deserve_worker/execution/exec.py:20-22)."""
    key = torch.device(device).index or 0
    if key not in _WRAPPERS:
        ws = torch.empty(128 << 20, dtype=torch.uint8, device=device)
        ws2 = torch.empty(64 << 20, dtype=torch.uint8, device=device)
        _WRAPPERS[key] = (ops.BatchDecodeWithPagedKVCacheWrapper(ws), ops.BatchPrefillWithPagedKVCacheWrapper(ws2))
    return _WRAPPERS[key]


@dataclass
class BatchExec:
    """deserve_worker/execution/exec.py:58-147 (the parts the microbatch path uses)."""

    xs: torch.Tensor
    layer_storage: object
    task_datas: list
    kvcaches: list

    def bsz(self) -> int:
        return len(self.task_datas)

    def seqlens(self) -> list:
        return [t.seqlen for t in self.task_datas]

    def total_seqlen(self) -> int:
        return sum(self.seqlens())

    # Regrouping of ragged batches (exec.py:74-106): rows are stored request after request,
    # request i owning seqlen_i of them.
    @classmethod
    def merge(cls, execs: Sequence["BatchExec"]) -> "BatchExec":
        return cls(torch.cat([e.xs for e in execs]), execs[0].layer_storage,
                   [t for e in execs for t in e.task_datas], [c for e in execs for c in e.kvcaches])

    def split(self) -> list:
        parts = self.xs.split(self.seqlens()) if self.task_datas else []
        return [type(self)(x, self.layer_storage, [t], [c]) for x, t, c in zip(parts, self.task_datas, self.kvcaches)]

    def pop(self) -> "BatchExec":
        """Take the last request out of the batch (with its rows)."""
        task, cache = self.task_datas.pop(), self.kvcaches.pop()
        tail = type(self)(self.xs[-task.seqlen:], self.layer_storage, [task], [cache])
        self.xs = self.xs[: -task.seqlen]
        return tail

    def post_process(self, result: torch.Tensor, ignore_eos: bool) -> BatchResult:
        ids = [t.task_id for t in self.task_datas]
        if not self.layer_storage.need_sample:
            return BatchResult(result, ids, result, ids, [], {})
        tokens, produced, done = self.layer_storage.sample(result, self.task_datas, ignore_eos)
        if not done and all(produced):  # plain decode step: every request got a token and goes on
            return BatchResult(tokens, ids, tokens, list(ids), [], {})
        all_idx = [i for i, p in enumerate(produced) if p]
        on_idx = [i for i in all_idx if ids[i] not in done]
        pick = lambda idx: tokens[torch.as_tensor(idx, dtype=torch.long, device=tokens.device)] if idx else tokens[:0]
        return BatchResult(pick(on_idx), [ids[i] for i in on_idx], pick(all_idx), [ids[i] for i in all_idx], list(done), {})


@dataclass
class BatchDecode(BatchExec):
    """All rows have seqlen 1 (exec.py:150-199)."""

    decode_ctx: Optional[FlashDecodeCtx] = None

    def prepare(self) -> None:
        wrapper, _ = stage_wrappers(self.kvcaches[0].pool.main_device)
        self.decode_ctx = FlashDecodeCtx.init_paged_decode_ctx(self.task_datas, self.kvcaches, wrapper)
        a, c = self.layer_storage.model_args, self.decode_ctx
        wrapper.begin_forward(indptr=c.kv_page_indptr, indices=c.kv_page_indices, last_page_len=c.kv_last_page_lens,
                              num_qo_heads=a.n_heads, num_kv_heads=a.n_kv_heads, head_dim=a.dim // a.n_heads,
                              page_size=c.page_pool.page_size, data_type=c.page_pool.main_dtype,
                              indptr_host=c.host["kv_page_indptr"])

    def step(self, ignore_eos: bool) -> BatchResult:
        with torch.inference_mode():
            result = self.layer_storage.forward(self.xs, self.decode_ctx)
            self.decode_ctx.decode_wrapper.end_forward()
            return self.post_process(result, ignore_eos)


@dataclass
class BatchPrefill(BatchExec):
    """Prompt chunks, possibly mixed with decode rows (exec.py:202-243)."""

    prefill_ctx: Optional[FlashPrefillCtx] = None

    def prepare(self) -> None:
        _, wrapper = stage_wrappers(self.kvcaches[0].pool.main_device)
        self.prefill_ctx = FlashPrefillCtx.init_paged_prefill_ctx(self.task_datas, self.kvcaches, wrapper)
        a, c = self.layer_storage.model_args, self.prefill_ctx
        wrapper.begin_forward(qo_indptr=c.indptr, paged_kv_indptr=c.kv_page_indptr, paged_kv_indices=c.kv_page_indices,
                              paged_kv_last_page_len=c.kv_last_page_lens, num_qo_heads=a.n_heads,
                              num_kv_heads=a.n_kv_heads, head_dim=a.dim // a.n_heads, page_size=c.page_pool.page_size,
                              data_type=c.page_pool.main_dtype, causal=True, qo_indptr_host=c.host["indptr"],
                              kv_indptr_host=c.host["kv_page_indptr"], last_page_len_host=c.host["kv_last_page_lens"],
                              kv_indices_host=c.host["kv_page_indices"])

    def step(self, ignore_eos: bool) -> BatchResult:
        with torch.inference_mode():
            result = self.layer_storage.forward(self.xs, self.prefill_ctx)
            self.prefill_ctx.prefill_wrapper.end_forward()
            return self.post_process(result, ignore_eos)


class MicroBatchProcessor:
    """One microbatch: its tasks' KV caches and the pinned image of its swap
    region (deserve_worker/engine/microbatch/processor.py:24-149)."""

    def __init__(self, kvcache_manager: KVCacheManager, task_data_manager: TaskManager, layer_storage,
                 page_table_allocator: PageTableAllocator, ignore_eos: bool) -> None:
        self.kvcache_manager = kvcache_manager
        pool = kvcache_manager.virtual_page_pool
        self.pinned_memory = CopiedPinnedMemory(size=pool.calc_swap_size(), num_pages_swap=pool.num_pages_swap,
                                                device=pool.main_device, dtype=pool.main_dtype)
        self.task_data_manager = task_data_manager
        self.layer_storage = layer_storage
        self.ongoing_paged_kvcaches: dict = {}
        self.ignore_eos = ignore_eos
        self.page_table_allocator = page_table_allocator

    def join(self, task_ids: list) -> None:
        for task_id in task_ids:
            self.ongoing_paged_kvcaches[task_id] = VirtualPagedKVCache.empty(
                self.page_table_allocator, self.kvcache_manager.virtual_page_pool)

    def adjust(self) -> None:
        vpp = self.kvcache_manager.virtual_page_pool
        offset = vpp.num_pages_swap if vpp.on == 1 else -vpp.num_pages_swap
        for kv in self.ongoing_paged_kvcaches.values():
            kv.adjust(offset)

    def offload(self, task_ids: list) -> list:
        """Tasks leave the device: one pipelined transfer for all of them, then
        their pages and table rows are freed."""
        kvs = [self.ongoing_paged_kvcaches.pop(t) for t in task_ids]
        handles = self.kvcache_manager.offload_many(kvs) if kvs else []
        for kv in kvs:
            kv.free()
        return handles

    def reload(self, task_ids: list, cpu_chunk_handles: list) -> None:
        kvs = self.kvcache_manager.reload_many(cpu_chunk_handles) if cpu_chunk_handles else []
        for task_id, kv in zip(task_ids, kvs):
            self.ongoing_paged_kvcaches[task_id] = kv
        for h in cpu_chunk_handles:
            h.free()

    def cancel(self, task_ids: list) -> None:
        for task_id in task_ids:
            kv = self.ongoing_paged_kvcaches.pop(task_id, None)
            if kv is not None:
                kv.free()

    def _batch(self, task_ids: list, xs: torch.Tensor):
        task_datas = [self.task_data_manager.get(t) for t in task_ids]
        kvcaches = [self.ongoing_paged_kvcaches[t] for t in task_ids]
        cls = BatchDecode if all(t.seqlen == 1 for t in task_datas) else BatchPrefill
        return cls(xs, self.layer_storage, task_datas, kvcaches)

    def exec(self, xs: torch.Tensor, task_ids: list) -> BatchResult:
        batch = self._batch(task_ids, xs)
        batch.prepare()
        return batch.step(self.ignore_eos)

    def step(self, task_ids: list, xs: torch.Tensor, prev_group: "MicroBatchProcessor",
             next_group: "MicroBatchProcessor") -> BatchResult:
        """prepare (grow caches, descriptors, plan) -> start the region swap for the
        neighbours on the side streams -> run the layers (processor.py:107-146)."""
        batch = self._batch(task_ids, xs)
        with phase("alloc+descriptors+plan"):
            batch.prepare()
        pool = self.kvcache_manager.virtual_page_pool
        if pool.num_pages_swap > 0:
            with phase("swap2"):
                pool.swap2(next_group.pinned_memory, prev_group.pinned_memory)
        with phase("layers"):
            return batch.step(self.ignore_eos)

    def synchronize(self) -> None:
        self.kvcache_manager.synchronize()


class StageProcessor:
    """The per-stage ordering contract of the reference's PipelineProcessor
    (deserve_worker/engine/pipeline/processor.py:226-301) without its HTTP shell:
    synchronize() = wait for the region DMA + switch(); process_step() = (adjust)
    -> init seqlens -> cancel -> offload -> reload -> synchronize the manager ->
    join -> step (prepare, swap2, layers) -> TaskData.step."""

    def __init__(self, kvcache_manager: KVCacheManager, task_manager: TaskManager, layer_storage,
                 page_table_allocator: PageTableAllocator, num_rounds: int, ignore_eos: bool = True):
        self.kvcache_manager, self.task_manager, self.layer_storage = kvcache_manager, task_manager, layer_storage
        self.num_rounds = num_rounds
        self.microbatches = [MicroBatchProcessor(kvcache_manager, task_manager, layer_storage, page_table_allocator,
                                                 ignore_eos) for _ in range(num_rounds)]
        self.offloaded_kvcaches: dict = {}
        self.current_microbatch_id = 0
        # debug mode (DESERVE_CHECK_PAGES=1 or set the attribute): after every step's allocation the page tables
        # of the stepping microbatch are checked against the allocator's invariants (kvcache.check_page_ownership)
        self.check_pages = os.environ.get("DESERVE_CHECK_PAGES", "0") == "1"

    def _check_pages(self, mb: "MicroBatchProcessor") -> None:
        from .kvcache import check_page_ownership

        pool = self.kvcache_manager.virtual_page_pool
        away = pool.slices[1 - pool.on] if pool.num_pages_swap > 0 else None
        check_page_ownership(pool, list(mb.ongoing_paged_kvcaches.values()), in_flight=away)
        # pages of the main area belong to one cache only, whichever microbatch it is in
        main_only = []
        for other in self.microbatches:
            for kv in other.ongoing_paged_kvcaches.values():
                ids = kv.page_table.retrieve_np()
                main_only.extend(ids[ids < pool.num_pages_main].tolist())
        if len(main_only) != len(set(main_only)):
            raise AssertionError("a page of the main area is owned by two caches")

    def synchronize(self, host_wait: bool = False) -> None:
        """The region DMA queued by the previous slot must be over before this slot's
        kernels touch the region that comes `on`. The reference blocks the host on both
        DMA streams here (processor.py:226-228); a device-side edge from the DMA streams
        to the compute stream orders the same things and lets the host run ahead
        (host_wait=True gives the reference's blocking form). Then flip the regions."""
        pool = self.kvcache_manager.virtual_page_pool
        if pool.stream is not None:
            with phase("swap_wait"):
                if host_wait:
                    pool.stream.synchronize()
                    pool.stream2.synchronize()
                else:
                    pool.wait_swap()
        pool.switch()

    def metrics(self) -> dict:
        """Page accounting of this stage right now (the counterpart of the reference's
        periodic "avg available pages" log line, processor.py:113-140)."""
        pool = self.kvcache_manager.virtual_page_pool
        out_pages, in_pages = pool.last_swap_pages
        return {"pages_total": pool.num_pages, "pages_main": pool.num_pages_main, "pages_per_region": pool.num_pages_swap,
                "pages_free": pool.num_avails, "region_on": pool.on, "region_pages_in_flight_out": out_pages,
                "region_pages_in_flight_in": in_pages,
                "tasks_resident": sum(len(m.ongoing_paged_kvcaches) for m in self.microbatches),
                "tasks_offloaded": len(self.offloaded_kvcaches)}

    def process_step(self, request: StepRequest) -> tuple:
        mb = self.microbatches[request.microbatch_id]
        assert request.microbatch_id == self.current_microbatch_id
        self.current_microbatch_id = (self.current_microbatch_id + 1) % self.num_rounds
        if self.num_rounds % 2 == 1:
            mb.adjust()
        prev_mb = self.microbatches[(request.microbatch_id - 1) % self.num_rounds]
        next_mb = self.microbatches[(request.microbatch_id + 1) % self.num_rounds]
        for task_id, (prompt_len, sp) in request.init_tasks.items():
            if task_id not in self.task_manager.task_datas:
                self.task_manager.add(TaskData.empty(task_id, prompt_len, sp))
        for task_id, seqlen in zip(request.exec_task_ids, request.exec_seqlens):
            self.task_manager.get(task_id).init(seqlen)
        mb.cancel(request.cancel_task_ids)
        if request.offload_task_ids or request.reload_task_ids:
            with phase("offload+reload"):
                for task_id, h in zip(request.offload_task_ids, mb.offload(request.offload_task_ids)):
                    self.offloaded_kvcaches[task_id] = h
                mb.reload(request.reload_task_ids, [self.offloaded_kvcaches.pop(t) for t in request.reload_task_ids])
        mb.kvcache_manager.synchronize()
        result = None
        if request.exec_task_ids:
            mb.join([t for t in request.init_tasks if t not in mb.ongoing_paged_kvcaches])
            result = mb.step(request.exec_task_ids, request.xs, prev_mb, next_mb)
            if self.check_pages:
                self._check_pages(mb)
            for task_id in request.exec_task_ids:
                self.task_manager.get(task_id).step()
            if self.layer_storage.need_sample:
                request.cancel_task_ids = result.done_task_ids
            request.xs = result.ongoing_xs
            request.exec_task_ids = result.ongoing_task_ids
        else:
            pool = self.kvcache_manager.virtual_page_pool
            if pool.num_pages_swap > 0:  # an idle slot keeps the region rotation going
                pool.swap2(next_mb.pinned_memory, prev_mb.pinned_memory)
            if self.layer_storage.need_sample:
                request.cancel_task_ids = []
        return request, result
