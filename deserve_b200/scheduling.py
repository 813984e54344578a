"""Per-step admission and swap policies of the first pipeline stage.

Before a microbatch's request enters the stage loop, the reference rewrites it
(PipelineScheduler.convert_step_request, deserve_worker/engine/pipeline/
scheduler.py:158-169): a JOIN policy admits waiting prompts (whole or in chunks)
and parked decode rows while pages and batch rows last, then the SWAP policy
either offloads tasks until the page budget is non-negative or brings offloaded
tasks back while pages are left. The budget `rest_pages` is the pool's free pages
plus the pages of the tasks the step cancels.

Policies (deserve_worker/engine/pipeline/stage/join.py, stage/swap.py):
  VanillaJoin          one whole prompt per step, alone (the running decodes are
                       parked); otherwise every parked decode that fits
  PrefillFirstJoin     prompts first, chunked to `max_batch_size` rows; if any
                       prompt rows were admitted the running decodes are parked,
                       and parked decodes fill what is left
  DecodeFirstJoin      the running decodes stay; prompt chunks and parked decodes
                       fill the rows that are left
  SwapPolicy           offload order: parked prompts (longest first), parked
                       decodes (last parked first), then the tail of the running
                       decodes; reload order: prompts, then decodes, longest first

The dicts (pending prompts, parked/offloaded rows) belong to the caller and are
mutated in place, as in the reference. Orders, tie-breaks and the error cases
(AssertionError of an empty chunk, RuntimeError when nothing more can be
offloaded) are the reference's.
"""
from __future__ import annotations

from typing import Callable

import torch

from .request import StepRequest
from .task import TaskManager


def _shortest_first(items):
    """Stable ascending order by row count (ties keep dict order)."""
    return sorted(items, key=lambda kv: kv[1].shape[0])


class _Rows:
    """Row budget of the request under construction."""

    def __init__(self, request: StepRequest, used: int, cap: int):
        self.request, self.used, self.cap = request, used, cap

    @property
    def full(self) -> bool:
        return self.used == self.cap

    def add_prompt(self, task_id: str, x: torch.Tensor, init_info, parked: dict) -> bool:
        """Whole prompt if it fits, else the chunk that fills the batch (the rest
        is parked under the same id). True when the scan must stop."""
        n = x.shape[0]
        if self.used + n <= self.cap:
            self.used += n
            parked.pop(task_id, None)
            self.request.append_exec(task_id, x, init_info)
            return self.full
        room = self.cap - self.used
        self.used += room
        self.request.append_exec(task_id, x[:room], init_info)
        parked[task_id] = x[room:]
        return True


class JoinPolicy:
    def __init__(self, manager: TaskManager) -> None:
        self.manager = manager

    def process(self, rest_pages: int, request: StepRequest) -> tuple[int, StepRequest]:
        raise NotImplementedError

    # -- shared scans -----------------------------------------------------------------
    def _parked_prompts(self, rows: _Rows, parked: dict) -> None:
        for task_id, x in _shortest_first(list(parked.items())):
            if rows.add_prompt(task_id, x, None, parked):
                return

    def _new_prompts(self, rows: _Rows, pending: dict, parked: dict, rest_pages: int) -> int:
        """Pending prompts, shortest first; one is admitted only if the pages of
        its WHOLE prompt are there (they are reserved at once)."""
        for task_id, (x, sp) in sorted(pending.items(), key=lambda kv: kv[1][0].shape[0]):
            need = self.manager.calc_initial_space([task_id])
            if rest_pages < need:
                continue
            rest_pages -= need
            pending.pop(task_id)
            if rows.add_prompt(task_id, x, (x.shape[0], sp), parked):
                break
        return rest_pages

    def _parked_decodes(self, rows: _Rows | None, request: StepRequest, parked: dict, rest_pages: int) -> int:
        for task_id, x in list(parked.items()):
            need = self.manager.calc_extended_space([task_id])
            if rest_pages < need:
                continue
            rest_pages -= need
            assert x.shape[0] == 1
            parked.pop(task_id)
            request.append_exec(task_id, x, None)
            if rows is not None:
                rows.used += 1
                if rows.full:
                    break
        return rest_pages

    @staticmethod
    def _park_running(request: StepRequest, parked_decodes: dict) -> None:
        for i, task_id in enumerate(request.exec_task_ids):
            parked_decodes[task_id] = request.xs[i : i + 1]


class VanillaJoin(JoinPolicy):
    """join.py:186-227."""

    def __init__(self, manager, pending_prompts: dict, parked_decodes: dict) -> None:
        super().__init__(manager)
        self.pending_prompts, self.parked_decodes = pending_prompts, parked_decodes

    def process(self, rest_pages, request):
        if self.pending_prompts:
            for task_id, (x, sp) in sorted(self.pending_prompts.items(), key=lambda kv: kv[1][0].shape[0]):
                need = self.manager.calc_initial_space([task_id])
                if rest_pages >= need:
                    fresh = StepRequest.empty(request.microbatch_id, request.xs.dtype, request.xs.device)
                    self.pending_prompts.pop(task_id)
                    fresh.append_exec(task_id, x, (x.shape[0], sp))
                    self._park_running(request, self.parked_decodes)
                    fresh.cancel_task_ids.extend(request.cancel_task_ids)
                    return rest_pages - need, fresh
        rest_pages -= self.manager.calc_extended_space(request.exec_task_ids)
        return self._parked_decodes(None, request, self.parked_decodes, rest_pages), request


class PrefillFirstJoin(JoinPolicy):
    """join.py:94-183."""

    def __init__(self, manager, pending_prompts: dict, parked_prompts: dict, parked_decodes: dict,
                 max_batch_size: int) -> None:
        super().__init__(manager)
        self.pending_prompts, self.parked_prompts, self.parked_decodes = pending_prompts, parked_prompts, parked_decodes
        self.max_batch_size = max_batch_size

    def process(self, rest_pages, request):
        rows = _Rows(request, 0, self.max_batch_size)
        admitted = False
        if self.pending_prompts or self.parked_prompts:
            fresh = StepRequest.empty(request.microbatch_id, request.xs.dtype, request.xs.device)
            rows.request = fresh
            self._parked_prompts(rows, self.parked_prompts)
            if rows.used < rows.cap:
                rest_pages = self._new_prompts(rows, self.pending_prompts, self.parked_prompts, rest_pages)
            admitted = len(fresh.exec_task_ids) > 0
            if admitted:
                self._park_running(request, self.parked_decodes)
                fresh.cancel_task_ids.extend(request.cancel_task_ids)
                request = fresh
        if not admitted:
            rest_pages -= self.manager.calc_extended_space(request.exec_task_ids)
        if rows.used < rows.cap:
            rest_pages = self._parked_decodes(rows, request, self.parked_decodes, rest_pages)
        return rest_pages, request


class DecodeFirstJoin(JoinPolicy):
    """join.py:12-91."""

    def __init__(self, manager, pending_prompts: dict, parked_prompts: dict, parked_decodes: dict,
                 max_batch_size: int) -> None:
        super().__init__(manager)
        self.pending_prompts, self.parked_prompts, self.parked_decodes = pending_prompts, parked_prompts, parked_decodes
        self.max_batch_size = max_batch_size

    def process(self, rest_pages, request):
        rest_pages -= self.manager.calc_extended_space(request.exec_task_ids)
        rows = _Rows(request, request.get_bsz(), self.max_batch_size)
        if (self.pending_prompts or self.parked_prompts) and rest_pages > 0:
            self._parked_prompts(rows, self.parked_prompts)
            if rows.used < rows.cap:
                rest_pages = self._new_prompts(rows, self.pending_prompts, self.parked_prompts, rest_pages)
        if rows.used < rows.cap:
            rest_pages = self._parked_decodes(rows, request, self.parked_decodes, rest_pages)
        return rest_pages, request


class SwapPolicy:
    """stage/swap.py:9-102."""

    def __init__(self, manager: TaskManager, parked_prompts: dict, parked_decodes: dict, offloaded_prompts: dict,
                 offloaded_decodes: dict) -> None:
        self.manager = manager
        self.parked_prompts, self.parked_decodes = parked_prompts, parked_decodes
        self.offloaded_prompts, self.offloaded_decodes = offloaded_prompts, offloaded_decodes

    def _move(self, src: dict, dst: dict, ids: list, pages_of: Callable[[list], int], rest_pages: int, out: bool) -> int:
        """Longest first (last of the stable ascending order). Going out: until the
        budget is non-negative. Coming back: while pages are left and the next one
        fits; the first that does not fit ends the scan."""
        queue = _shortest_first(list(src.items()))
        while queue and (rest_pages < 0 if out else rest_pages > 0):
            task_id, x = queue.pop()
            pages = pages_of([task_id])
            if out:
                rest_pages += pages
            elif rest_pages >= pages:
                rest_pages -= pages
            else:
                break
            src.pop(task_id)
            dst[task_id] = x
            ids.append(task_id)
        return rest_pages

    def process(self, rest_pages: int, request: StepRequest) -> tuple[int, StepRequest]:
        m = self.manager
        if rest_pages >= 0:
            rest_pages = self._move(self.offloaded_prompts, self.parked_prompts, request.reload_task_ids,
                                    m.calc_initial_space, rest_pages, out=False)
            rest_pages = self._move(self.offloaded_decodes, self.parked_decodes, request.reload_task_ids,
                                    m.calc_occupied_space, rest_pages, out=False)
            return rest_pages, request
        rest_pages = self._move(self.parked_prompts, self.offloaded_prompts, request.offload_task_ids,
                                m.calc_initial_space, rest_pages, out=True)
        rest_pages = self._move(self.parked_decodes, self.offloaded_decodes, request.offload_task_ids,
                                m.calc_occupied_space, rest_pages, out=True)
        if rest_pages >= 0:
            return rest_pages, request
        # still short: cut running decodes off the tail of the batch, fewest first
        assert all(n == 1 for n in request.exec_seqlens)
        for keep in range(len(request.exec_task_ids) + 1, 0, -1):
            victims = request.exec_task_ids[keep:]
            gain = m.calc_occupied_space(victims) + m.calc_extended_space(victims)
            if rest_pages + gain >= 0:
                cut = request.xs[keep:]
                request.offload_task_ids.extend(victims)
                request.exec_task_ids = request.exec_task_ids[:keep]
                request.xs = request.xs[:keep]
                for i, task_id in enumerate(victims):
                    self.offloaded_decodes[task_id] = cut[i : i + 1]
                    assert self.offloaded_decodes[task_id].numel() > 0
                return rest_pages + gain, request
        raise RuntimeError("Unable to fetch enough pages")


class StepPlanner:
    """convert_step_request (scheduler.py:158-169) for every microbatch of a stage:
    one join policy and one swap policy per microbatch over shared pending /
    offloaded dicts (scheduler.py:55-104)."""

    def __init__(self, manager: TaskManager, num_rounds: int, policy: str = "vanilla", max_batch_size: int = 512) -> None:
        self.manager = manager
        self.pending_prompts: dict = {}
        self.offloaded_prompts: dict = {}
        self.offloaded_decodes: dict = {}
        self.parked_prompts = [dict() for _ in range(num_rounds)]
        self.parked_decodes = [dict() for _ in range(num_rounds)]
        if policy == "vanilla":
            self.join = [VanillaJoin(manager, self.pending_prompts, d) for d in self.parked_decodes]
        elif policy in ("prefill_first", "decode_first"):
            cls = PrefillFirstJoin if policy == "prefill_first" else DecodeFirstJoin
            self.join = [cls(manager, self.pending_prompts, p, d, max_batch_size)
                         for p, d in zip(self.parked_prompts, self.parked_decodes)]
        else:
            raise ValueError(f"unknown join policy {policy!r}")
        self.swap = [SwapPolicy(manager, p, d, self.offloaded_prompts, self.offloaded_decodes)
                     for p, d in zip(self.parked_prompts, self.parked_decodes)]

    def add_prompt(self, task_id: str, x: torch.Tensor, sampling_params) -> None:
        """process_init (scheduler.py:146-155) without the buffered-request flush."""
        from .task import TaskData

        self.manager.add(TaskData.empty(task_id, x.shape[0], sampling_params))
        self.pending_prompts[task_id] = (x, sampling_params)

    def convert(self, request: StepRequest, free_pages: int) -> StepRequest:
        rest = free_pages + self.manager.calc_occupied_space(request.cancel_task_ids)
        request.refresh()
        rest, request = self.join[request.microbatch_id].process(rest, request)
        rest, request = self.swap[request.microbatch_id].process(rest, request)
        return request
