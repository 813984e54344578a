"""Step-scheduler policies and wire framing against traces recorded from the
reference's own classes (tests/golden/make_scheduler_golden.py): 180 seeded
join + swap situations (orders, chunking, page budgets, the error cases) and five
frames compared byte for byte."""
import json
from functools import lru_cache

import pytest
import torch

from helpers import GOLDEN
from deserve_b200 import wire
from deserve_b200.request import StepRequest
from deserve_b200.scheduling import DecodeFirstJoin, PrefillFirstJoin, StepPlanner, SwapPolicy, VanillaJoin
from deserve_b200.task import SamplingParams, TaskData, TaskManager


@lru_cache(maxsize=None)
def traces() -> dict:
    return json.loads((GOLDEN / "scheduler_traces.json").read_text())


def _rows(runs) -> torch.Tensor:
    ids = [v for first, n in runs for v in range(first, first + n)]
    r = torch.tensor(ids, dtype=torch.int32)
    return torch.stack([r, -r], dim=1)


def _runs(x: torch.Tensor):
    out = []
    for v in (x[:, 0].tolist() if x.numel() else []):
        if out and out[-1][0] + out[-1][1] == v:
            out[-1][1] += 1
        else:
            out.append([v, 1])
    return out


def _snapshot(d):
    return [[k, _runs(v[0] if isinstance(v, tuple) else v)] for k, v in d.items()]


@pytest.mark.parametrize("idx", range(180))
def test_policy_case(idx):
    c = traces()["policy_cases"][idx]
    sp = SamplingParams()
    manager = TaskManager(1000, c["page_size"])
    for tid, start, seqlen, initial, _role in c["tasks"]:
        manager.add(TaskData(tid, start, 0, seqlen, initial, sp))
    b = c["before"]
    pend = {k: (_rows(r), sp) for k, r in b["pending"]}
    sus_p = {k: _rows(r) for k, r in b["suspended_prefills"]}
    sus_d = {k: _rows(r) for k, r in b["suspended_decodes"]}
    off_p = {k: _rows(r) for k, r in b["offloaded_prefills"]}
    off_d = {k: _rows(r) for k, r in b["offloaded_decodes"]}
    index = {t[0]: i for i, t in enumerate(c["tasks"])}
    request = StepRequest.empty(c["microbatch_id"], torch.int32)
    for tid in b["exec"]:
        request.append_exec(tid, _rows([[1000 * index[tid], 1]]), None)
    request.cancel_task_ids = list(b["cancel"])
    request.refresh()
    cap = c["max_batch_size"]
    join = {"vanilla": lambda: VanillaJoin(manager, pend, sus_d),
            "prefill_first": lambda: PrefillFirstJoin(manager, pend, sus_p, sus_d, cap),
            "decode_first": lambda: DecodeFirstJoin(manager, pend, sus_p, sus_d, cap)}[c["kind"]]()
    swap = SwapPolicy(manager, sus_p, sus_d, off_p, off_d)
    error = None
    try:
        rest, request = join.process(c["rest_pages"], request)
        assert rest == c["rest_after_join"]
        assert request.exec_task_ids == c["exec_after_join"]
        rest, request = swap.process(rest, request)
        assert rest == c["rest_after_swap"]
    except (RuntimeError, AssertionError) as e:
        if "error" not in c:
            raise
        error = type(e).__name__
    if "error" in c:
        assert error == c["error"][0]
    a = c["after"]
    assert _snapshot(pend) == a["pending"]
    assert _snapshot(sus_p) == a["suspended_prefills"]
    assert _snapshot(sus_d) == a["suspended_decodes"]
    assert _snapshot(off_p) == a["offloaded_prefills"]
    assert _snapshot(off_d) == a["offloaded_decodes"]
    assert request.exec_task_ids == a["exec"]
    assert request.exec_seqlens == a["exec_seqlens"]
    assert _runs(request.xs) == a["xs"]
    assert request.cancel_task_ids == a["cancel"]
    assert request.offload_task_ids == a["offload"]
    assert request.reload_task_ids == a["reload"]
    assert [[k, v[0]] for k, v in request.init_tasks.items()] == a["init_tasks"]


@pytest.mark.parametrize("idx", range(5))
def test_wire_frame(idx):
    w = traces()["wire"][idx]
    dtype = getattr(torch, w["dtype"])
    xs = torch.tensor(w["xs"], dtype=torch.float32).to(dtype).reshape(w["xs_shape"]) if w["xs"] else \
        torch.empty((0,), dtype=dtype)
    req = StepRequest(w["microbatch_id"], xs, w["exec_task_ids"], w["exec_seqlens"], w["cancel_task_ids"],
                      w["offload_task_ids"], w["reload_task_ids"], {})
    assert req.is_empty() == w["is_empty"]
    assert req.get_tensors_size() == w["tensors_size"]
    frame = wire.dumps(*req.into_safetensors())
    assert frame.hex() == w["frame_hex"]
    tensors, meta = wire.loads(bytes.fromhex(w["frame_hex"]))
    back = StepRequest.from_safetensors(tensors, meta)
    assert back.microbatch_id == req.microbatch_id and back.exec_task_ids == req.exec_task_ids
    assert back.exec_seqlens == req.exec_seqlens and back.offload_task_ids == req.offload_task_ids
    assert back.xs.dtype == dtype and back.xs.shape == xs.shape and torch.equal(back.xs, xs)
    # the transport's framing carries the same two parts in the other order
    t2, m2 = wire.loads_network(wire.dumps_network(*req.into_safetensors()))
    assert m2 == meta and torch.equal(t2["xs"], xs)


def test_frames_carry_sampling_params_and_nothing_else():
    import pickle

    from deserve_b200.task import SamplingParams

    req = StepRequest.empty(0, torch.int32)
    req.append_exec("p", torch.arange(4, dtype=torch.int32), (4, SamplingParams(max_new_tokens=7)))
    tensors, meta = wire.loads(wire.dumps(*req.into_safetensors()))
    assert meta["init_tasks"]["p"][1].max_new_tokens == 7 and torch.equal(tensors["xs"], req.xs)
    evil = pickle.dumps({"group_id": __import__("os").getcwd})  # a frame that names a callable of another module
    frame = len(evil).to_bytes(4, "big") + evil + wire.st_save({"xs": torch.zeros(1)})
    with pytest.raises(pickle.UnpicklingError):
        wire.loads(frame)
    for bad in (b"\x00\x00", b"\x00\x00\x10\x00abc"):
        with pytest.raises(ValueError):
            wire.loads(bad)


def test_safetensors_container_matches_the_library():
    st = pytest.importorskip("safetensors.torch")
    g = torch.Generator().manual_seed(0)
    tensors = {"b": torch.randn(2, 2, generator=g), "a": torch.arange(3, dtype=torch.int32),
               "xs": torch.randn(2, 3, generator=g).to(torch.bfloat16), "flag": torch.tensor([True, False]),
               "wide": torch.arange(5, dtype=torch.int64), "h": torch.randn(7, generator=g).to(torch.float16)}
    assert wire.st_save(tensors) == st.save(tensors)
    back = wire.st_load(st.save(tensors))
    assert all(torch.equal(back[k], v) and back[k].dtype == v.dtype for k, v in tensors.items())


def test_step_planner_budget_and_chunking():
    manager = TaskManager(1000, 16)
    planner = StepPlanner(manager, num_rounds=2, policy="prefill_first", max_batch_size=64)
    sp = SamplingParams()
    planner.add_prompt("p0", torch.arange(100, dtype=torch.int32), sp)
    planner.add_prompt("p1", torch.arange(40, dtype=torch.int32), sp)
    req = planner.convert(StepRequest.empty(0, torch.int32), free_pages=20)
    # shortest prompt first (3 pages), then a 24-row chunk of the long one (its 7 pages reserved at once)
    assert req.exec_task_ids == ["p1", "p0"] and req.exec_seqlens == [40, 24]
    assert list(planner.parked_prompts[0]) == ["p0"] and planner.parked_prompts[0]["p0"].shape[0] == 76
    assert req.init_tasks["p0"][0] == 100 and not planner.pending_prompts
    with pytest.raises(ValueError):
        StepPlanner(manager, 1, policy="nope")


def test_batch_exec_regrouping():
    from deserve_b200.engine import BatchDecode, BatchExec, BatchPrefill

    sp = SamplingParams()
    tasks = [TaskData(f"t{i}", 0, 0, n, n, sp) for i, n in enumerate([3, 1, 4])]
    xs = torch.arange(8 * 2).reshape(8, 2)
    batch = BatchPrefill(xs, "storage", list(tasks), ["c0", "c1", "c2"])
    assert batch.bsz() == 3 and batch.seqlens() == [3, 1, 4] and batch.total_seqlen() == 8
    parts = batch.split()
    assert [p.xs.shape[0] for p in parts] == [3, 1, 4] and all(isinstance(p, BatchPrefill) for p in parts)
    assert torch.equal(parts[2].xs, xs[4:]) and parts[1].kvcaches == ["c1"]
    again = BatchPrefill.merge(parts)
    assert isinstance(again, BatchPrefill) and torch.equal(again.xs, xs) and again.task_datas == tasks
    last = batch.pop()
    assert last.task_datas == [tasks[2]] and torch.equal(last.xs, xs[4:]) and batch.xs.shape[0] == 4 and batch.bsz() == 2
    assert isinstance(BatchDecode.merge([BatchExec(xs[:1], "s", tasks[1:2], ["c1"])]), BatchDecode)
