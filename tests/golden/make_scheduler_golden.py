"""Record what the REFERENCE's step scheduler policies and wire framing do
(CoLearn-Dev/deserve, CPU only):

    python tests/golden/make_scheduler_golden.py /path/to/reference

  * deserve_worker/engine/pipeline/stage/join.py (VanillaJoinStage,
    PrefillFirstAgggregatedJoinStage, DecodeFirstAgggregatedJoinStage) followed by
    stage/swap.py (SwapStage), the pair PipelineScheduler.convert_step_request runs
    (engine/pipeline/scheduler.py:158-169), on seeded random situations;
  * StepRequest.append_exec / refresh / is_empty / into_safetensors
    (deserve_worker/request.py:137-213);
  * dumps() of deserve_worker/model/utils.py:12-30 (u32be length, pickled metadata,
    safetensors with the '#name' stand-in for empty tensors).

The reference modules are imported unmodified; only request.main_device is pointed at
the CPU. Writes tests/golden/scheduler_traces.json."""
from __future__ import annotations

import json
import os
import random
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent


def rows(task_index: int, first: int, n: int) -> torch.Tensor:
    """n activation rows that name themselves: column 0 = 1000 * task + row."""
    r = torch.arange(first, first + n, dtype=torch.int32) + 1000 * task_index
    return torch.stack([r, -r], dim=1)


def ids_of(x: torch.Tensor) -> list[list[int]]:
    """Row names as runs [first, count] (rows of one task are consecutive)."""
    runs: list[list[int]] = []
    for v in (x[:, 0].tolist() if x.numel() else []):
        if runs and runs[-1][0] + runs[-1][1] == v:
            runs[-1][1] += 1
        else:
            runs.append([v, 1])
    return runs


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    os.chdir(ref_root)
    import deserve_worker.task as task_mod

    torch.set_default_dtype(torch.float32)
    import deserve_worker.request as request_mod

    request_mod.main_device = torch.device("cpu")
    from deserve_worker.engine.pipeline.stage.join import (DecodeFirstAgggregatedJoinStage,
                                                           PrefillFirstAgggregatedJoinStage, VanillaJoinStage)
    from deserve_worker.engine.pipeline.stage.swap import SwapStage
    from deserve_worker.model.utils import dumps
    from deserve_worker.request import StepRequest
    from deserve_worker.task import SamplingParams, TaskData, TaskManager

    sp = SamplingParams()
    out: dict = {"policy_cases": [], "wire": []}

    def snapshot(d: dict) -> list:
        return [[k, ids_of(v[0] if isinstance(v, tuple) else v)] for k, v in d.items()]

    def policy_case(seed: int, kind: str) -> dict:
        rng = random.Random(seed)
        ps = rng.choice([8, 16])
        cap = rng.choice([6, 16, 40, 512])
        manager = TaskManager(1000, ps)
        tasks = []  # [id, start_pos, seqlen, initial_seqlen]
        pend, sus_p, sus_d, off_p, off_d = {}, {}, {}, {}, {}
        exec_ids, cancel_ids = [], []
        xs = []
        n_tasks = rng.randint(4, 14)
        for t in range(n_tasks):
            tid = f"t{t}"
            role = rng.choice(["exec", "exec", "pending", "pending", "sus_prefill", "sus_decode", "off_prefill",
                               "off_decode", "cancel"])
            initial = rng.choice([1, 5, 8, 16, 17, 40, 100, 300])
            if role in ("exec", "sus_decode", "off_decode", "cancel"):
                start, seqlen = initial + rng.randint(0, 50), 1
            elif role == "pending":
                start, seqlen = 0, 0
            else:  # a prompt that has been fed in part
                start, seqlen = rng.randint(0, max(0, initial - 1)), 0
            td = TaskData(task_id=tid, start_pos=start, round=0, seqlen=seqlen, initial_seqlen=initial,
                          sampling_params=sp)
            manager.add(td)
            tasks.append([tid, start, seqlen, initial, role])
            if role == "exec":
                exec_ids.append(tid)
                xs.append(rows(t, 0, 1))
            elif role == "cancel":
                cancel_ids.append(tid)
            elif role == "pending":
                pend[tid] = (rows(t, 0, initial), sp)
            elif role == "sus_prefill":
                sus_p[tid] = rows(t, start, initial - start)
            elif role == "sus_decode":
                sus_d[tid] = rows(t, 0, 1)
            elif role == "off_prefill":
                off_p[tid] = rows(t, start, initial - start)
            else:
                off_d[tid] = rows(t, 0, 1)
        request = StepRequest.empty(rng.randint(0, 3), torch.int32)
        for tid, x in zip(exec_ids, xs):
            request.append_exec(tid, x, None)
        request.cancel_task_ids = list(cancel_ids)
        request.refresh()
        rest = rng.choice([-40, -10, -3, 0, 2, 5, 12, 30, 80, 400])
        rec = {"seed": seed, "kind": kind, "page_size": ps, "max_batch_size": cap, "tasks": tasks,
               "microbatch_id": request.microbatch_id, "rest_pages": rest,
               "before": {"pending": snapshot(pend), "suspended_prefills": snapshot(sus_p),
                          "suspended_decodes": snapshot(sus_d), "offloaded_prefills": snapshot(off_p),
                          "offloaded_decodes": snapshot(off_d), "exec": exec_ids, "cancel": cancel_ids}}
        if kind == "vanilla":
            join = VanillaJoinStage(manager, pend, sus_d)
        elif kind == "prefill_first":
            join = PrefillFirstAgggregatedJoinStage(manager, pend, sus_p, sus_d, cap)
        else:
            join = DecodeFirstAgggregatedJoinStage(manager, pend, sus_p, sus_d, cap)
        swap = SwapStage(manager, sus_p, sus_d, off_p, off_d)
        try:
            rest1, request = join.process(rest, request)
            rec["rest_after_join"] = rest1
            rec["exec_after_join"] = list(request.exec_task_ids)
            rest2, request = swap.process(rest1, request)
            rec["rest_after_swap"] = rest2
        except RuntimeError as e:
            rec["error"] = ["RuntimeError", str(e)]
        except AssertionError:
            rec["error"] = ["AssertionError", ""]
        rec["after"] = {"pending": snapshot(pend), "suspended_prefills": snapshot(sus_p),
                        "suspended_decodes": snapshot(sus_d), "offloaded_prefills": snapshot(off_p),
                        "offloaded_decodes": snapshot(off_d), "exec": list(request.exec_task_ids),
                        "exec_seqlens": list(request.exec_seqlens), "xs": ids_of(request.xs),
                        "cancel": list(request.cancel_task_ids), "offload": list(request.offload_task_ids),
                        "reload": list(request.reload_task_ids),
                        "init_tasks": [[k, v[0]] for k, v in request.init_tasks.items()]}
        return rec

    seed = 0
    for kind in ("vanilla", "prefill_first", "decode_first"):
        for _ in range(60):
            out["policy_cases"].append(policy_case(seed, kind))
            seed += 1

    # ---- wire frames ---------------------------------------------------------------
    def frame(req: StepRequest, note: str) -> None:
        tensors, metadata = req.into_safetensors()
        out["wire"].append({"note": note, "microbatch_id": req.microbatch_id, "dtype": str(req.xs.dtype).split(".")[-1],
                            "xs_shape": list(req.xs.shape), "xs": req.xs.flatten().tolist(),
                            "exec_task_ids": req.exec_task_ids, "exec_seqlens": req.exec_seqlens,
                            "cancel_task_ids": req.cancel_task_ids, "offload_task_ids": req.offload_task_ids,
                            "reload_task_ids": req.reload_task_ids, "is_empty": req.is_empty(),
                            "tensors_size": req.get_tensors_size(), "frame_hex": dumps(tensors, metadata).hex()})

    r = StepRequest.empty(2, torch.int32)
    frame(r, "empty request of the first stage (token ids)")
    r = StepRequest.empty(1, torch.float16)
    r.append_exec("a", torch.arange(8, dtype=torch.float16).reshape(1, 8), None)
    r.append_exec("b", (torch.arange(24, dtype=torch.float16) / 8).reshape(3, 8), None)
    r.cancel_task_ids.append("z")
    frame(r, "one decode row and a three-row prompt chunk, fp16 activations")
    r.refresh()
    frame(r, "the same after refresh()")
    r = StepRequest.empty(0, torch.int32)
    r.append_exec("t0", torch.tensor([5, 6, 7], dtype=torch.int32), None)
    r.offload_task_ids.append("t9")
    r.reload_task_ids.extend(["t3", "t4"])
    frame(r, "token ids with offload and reload lists")
    r = StepRequest.empty(3, torch.bfloat16)
    r.append_exec("q", (torch.arange(16, dtype=torch.float32) - 8).to(torch.bfloat16).reshape(2, 8), None)
    frame(r, "bf16 activations")

    (HERE / "scheduler_traces.json").write_text(json.dumps(out))
    print("wrote", HERE / "scheduler_traces.json", len(out["policy_cases"]), "policy cases,", len(out["wire"]), "frames")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_scheduler_golden.py /path/to/reference")
    main(sys.argv[1])
