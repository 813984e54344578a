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

from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import numpy as np
import torch

from . import ops
from .context import FlashDecodeCtx
from .kvcache import PagedKVCache
from .task import TaskData


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
    plan = torch.empty(ops.plan_capacity(ctx.bsz, sm_count), dtype=torch.int32, pin_memory=True)
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
                on_attention: Callable[[int], None] | None = None) -> torch.Tensor:
        """x: [B, Hq, D] query of the first layer; layer l's attention output is
        layer l+1's query. k_new, v_new: [layers, B, Hkv, D] rows to append.
        on_attention(i), if given, is called before and after every attention
        launch (i = 2*layer, 2*layer+1) so a caller can bracket it with events."""
        if sd.workspace_bytes > self.workspace.numel():
            raise RuntimeError(f"stage workspace too small: need {sd.workspace_bytes} bytes")
        for i, layer in enumerate(range(self.layer_begin, self.layer_end)):
            pages = self.pool.pages[layer]
            ops.append_paged_kv_cache(k_new[i], v_new[i], sd.indptr, pages, sd.kv_page_indices, sd.kv_page_indptr,
                                      sd.kv_last_page_lens)
            if on_attention is not None:
                on_attention(2 * i)
            x = ops.paged_decode(x, pages, sd.kv_page_indices, sd.kv_page_indptr, sd.kv_last_page_lens, sd.plan_host,
                                 sd.plan_dev, self.workspace)
            if on_attention is not None:
                on_attention(2 * i + 1)
        return x


class RingPipeline:
    """W stages (ranks) and W microbatches in a ring. In slot t, rank r works on
    unit u = t - r, i.e. microbatch u % W at token step u // W, then every rank
    hands its output to rank (r+1) % W in one grouped send+recv. After the first
    W-1 slots every rank is busy in every slot. The object keeps its position,
    so a caller can run some slots, synchronise, and continue with a full ring.

    stage_fn(unit, microbatch, token_step, x) -> y runs the rank's layers.
    first_input(microbatch) gives rank 0 its input for token step 0.
    """

    def __init__(self, rank: int, world: int, stage_fn, first_input, total_steps: int, group=None, dist=None):
        self.rank, self.world = rank, world
        self.stage_fn, self.first_input = stage_fn, first_input
        self.units = total_steps * world
        self.group = group
        self.dist = dist
        self.slot = 0
        self.inbox: torch.Tensor | None = None
        self.last_output: torch.Tensor | None = None
        self.completed: list[tuple[int, int]] = []  # (microbatch, token_step) finished on the last rank

    def _computes(self, rank: int, slot: int) -> bool:
        return 0 <= slot - rank < self.units

    def advance(self, n_slots: int) -> None:
        W, r = self.world, self.rank
        for _ in range(n_slots):
            t = self.slot
            y = None
            if self._computes(r, t):
                u = t - r
                m, s = u % W, u // W
                x = self.first_input(m) if (r == 0 and s == 0) else self.inbox
                y = self.stage_fn(u, m, s, x)
                if r == W - 1:
                    self.completed.append((m, s))
                    self.last_output = y
            if W > 1:
                nxt, prv = (r + 1) % W, (r - 1) % W
                # what rank r+1 computes in slot t+1 is the unit rank r computed in slot t;
                # rank 0 needs the last rank's output only while token steps remain
                send = y is not None and (r < W - 1 or t + 1 < self.units)
                recv = self._computes(prv, t) and (r > 0 or t + 1 < self.units) and self._computes(r, t + 1)
                p2p = []
                buf = None
                if send:
                    p2p.append(self.dist.P2POp(self.dist.isend, y, nxt, self.group))
                if recv:
                    like = y if y is not None else (self.inbox if self.inbox is not None else self.first_input(0))
                    buf = torch.empty_like(like)
                    p2p.append(self.dist.P2POp(self.dist.irecv, buf, prv, self.group))
                if p2p:
                    for req in self.dist.batch_isend_irecv(p2p):
                        req.wait()
                self.inbox = buf
            else:
                self.inbox = y
            self.slot += 1
