"""Requests that travel between pipeline stages (deserve_worker/request.py)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from .task import SamplingParams


@dataclass
class InitRequest:
    """A new prompt handed to the first stage (request.py:19-36)."""

    x: torch.Tensor
    task_id: str
    sampling_params: SamplingParams

    def into_safetensors(self) -> tuple[dict[str, torch.Tensor], dict[str, Any]]:
        sp = self.sampling_params
        return {"x": self.x}, {"task_id": self.task_id,
                               "sampling_params": sp.model_dump() if hasattr(sp, "model_dump") else dict(vars(sp))}

    def get_tensors_size(self) -> int:
        return self.x.numel() * self.x.element_size()


@dataclass
class StepRequest:
    """One microbatch's step (request.py:137-213): the ragged rows `xs` of the
    executing tasks in `exec_task_ids` order (`exec_seqlens[i]` rows each), the
    tasks to cancel, offload and reload before it runs, and the prompts that start
    in this step (task id -> (prompt length, sampling parameters))."""

    microbatch_id: int
    xs: torch.Tensor
    exec_task_ids: list = field(default_factory=list)
    exec_seqlens: list = field(default_factory=list)
    cancel_task_ids: list = field(default_factory=list)
    offload_task_ids: list = field(default_factory=list)
    reload_task_ids: list = field(default_factory=list)
    init_tasks: dict = field(default_factory=dict)

    @staticmethod
    def empty(group_id: int, dtype: torch.dtype, device: torch.device | str | None = None) -> "StepRequest":
        return StepRequest(group_id, torch.empty((0,), dtype=dtype, device=device))

    def is_empty(self) -> bool:
        return (self.xs.numel() == 0 and not self.exec_task_ids and not self.exec_seqlens and not self.cancel_task_ids
                and not self.offload_task_ids and not self.reload_task_ids and not self.init_tasks)

    def append_exec(self, task_id: str, x: torch.Tensor, init_info: Optional[tuple]) -> None:
        assert x.numel() > 0, "a task joins a step with at least one row"
        self.exec_task_ids.append(task_id)
        self.exec_seqlens.append(x.shape[0])
        self.xs = x if self.xs.numel() == 0 else torch.cat([self.xs, x], dim=0)
        if init_info is not None:
            self.init_tasks[task_id] = init_info

    def get_bsz(self) -> int:
        return len(self.exec_task_ids)

    def refresh(self) -> None:
        """What a request that comes back around the ring carries into its next
        step: the same tasks, one row each, nothing to move or start."""
        self.offload_task_ids = []
        self.reload_task_ids = []
        self.exec_seqlens = [1] * len(self.exec_task_ids)
        self.init_tasks = {}

    def into_safetensors(self) -> tuple[dict[str, torch.Tensor], dict[str, Any]]:
        return {"xs": self.xs}, {
            "group_id": self.microbatch_id,
            "exec_task_ids": self.exec_task_ids,
            "exec_seqlens": self.exec_seqlens,
            "cancel_task_ids": self.cancel_task_ids,
            "offload_task_ids": self.offload_task_ids,
            "reload_task_ids": self.reload_task_ids,
            "init_tasks": self.init_tasks,
        }

    @staticmethod
    def from_safetensors(tensors: dict[str, torch.Tensor], metadata: dict[str, Any],
                         device: torch.device | str | None = None) -> "StepRequest":
        """The receiving side (deserve_worker/worker_api.py:90-111)."""
        xs = tensors["xs"]
        return StepRequest(metadata["group_id"], xs.to(device) if device is not None else xs,
                           metadata["exec_task_ids"], metadata["exec_seqlens"], metadata["cancel_task_ids"],
                           metadata["offload_task_ids"], metadata["reload_task_ids"], metadata["init_tasks"])

    def get_tensors_size(self) -> int:
        return self.xs.numel() * self.xs.element_size()
