"""Pipeline schedules as explicit task lists.

Reference: infini_train/src/nn/parallel/pp/pipeline_schedule.cc — GPipe :86-127, interleaved 1F1B
:129-192 (implemented there but never executed: ``StepMicroBatches`` walks the GPipe list, :202).
Here both generators exist and the executor runs whichever is selected; 1F1B is the default.

A task is one forward or one backward of (micro-batch, global chunk).  Global chunk ``g`` lives on
stage ``g % num_stages`` as that stage's local chunk ``g // num_stages``; with virtual pipeline
parallelism (``vpp_size`` chunks per stage) the activation path is
stage0/chunk0 -> stage1/chunk0 -> ... -> last stage/chunk0 -> stage0/chunk1 -> ...

Every rank walks the same global list in the same order and executes the tasks of its own stage;
every task's producers sit at strictly earlier steps, so blocking receives paired with
asynchronous sends cannot deadlock.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List


@dataclass(frozen=True)
class Task:
    step: int
    microbatch_id: int
    global_chunk_id: int
    local_chunk_idx: int
    is_forward: bool
    stage_id: int
    is_last_chunk: bool
    is_first_chunk: bool


def CreateTask(step: int, mb: int, global_chunk: int, num_stages: int, total_chunks: int, is_forward: bool) -> Task:
    return Task(step, mb, global_chunk, global_chunk // num_stages, is_forward, global_chunk % num_stages,
                global_chunk == total_chunks - 1, global_chunk == 0)


def GenerateGPipeSchedule(n: int, num_stages: int, vpp_size: int = 1) -> List[Task]:
    """All forwards, then all backwards.  Forward of (mb, g) at step ``mb + g``; backward at step
    ``S + (S - 1 - g - mb)`` with ``S = n + chunks - 1``; ties ordered by local chunk."""
    chunks = num_stages * vpp_size
    total_steps = n + chunks - 1
    out: List[Task] = []
    for step in range(total_steps):
        for mb in range(n):
            g = step - mb
            if 0 <= g < chunks:
                out.append(CreateTask(step, mb, g, num_stages, chunks, True))
    for step in range(total_steps):
        for mb in range(n):
            g = (total_steps - 1 - step) - mb
            if 0 <= g < chunks:
                out.append(CreateTask(step + total_steps, mb, g, num_stages, chunks, False))
    out.sort(key=lambda t: (t.step, t.local_chunk_idx))
    return out


def GenerateInterleaved1F1BSchedule(n: int, num_stages: int, vpp_size: int = 1) -> List[Task]:
    """Warm-up of ``chunks - 1`` forward-only steps, ``n`` steady steps that issue one forward and
    one backward per micro-batch slot, then the cool-down of the remaining backwards.  A micro-batch
    starts its backward as soon as its forward reaches the last chunk, so at most ``chunks``
    micro-batches hold activations per stage instead of all ``n``."""
    out: List[Task] = []
    if n <= 0 or num_stages <= 0 or vpp_size <= 0:
        return out
    chunks = num_stages * vpp_size
    warmup = chunks - 1
    total_steps = 2 * warmup + n
    for step in range(warmup):
        for mb in range(n):
            g = step - mb
            if 0 <= g < chunks:
                out.append(CreateTask(step, mb, g, num_stages, chunks, True))
    for step in range(warmup, warmup + n):
        stable = step - warmup
        for mb in range(n):
            g = step - mb
            if 0 <= g < chunks:
                out.append(CreateTask(step, mb, g, num_stages, chunks, True))
            gb = (chunks - 1) - (stable - mb)
            if 0 <= gb < chunks:
                out.append(CreateTask(step, mb, gb, num_stages, chunks, False))
    for step in range(warmup + n, total_steps):
        for mb in range(n):
            gb = (chunks - 1) - ((step - warmup) - mb)
            if 0 <= gb < chunks:
                out.append(CreateTask(step, mb, gb, num_stages, chunks, False))
    return out


def ValidateSchedule(schedule: List[Task], n: int, num_stages: int, vpp_size: int) -> None:
    """Checks the invariants the executor relies on (raises AssertionError otherwise)."""
    chunks = num_stages * vpp_size
    pos = {(t.microbatch_id, t.global_chunk_id, t.is_forward): i for i, t in enumerate(schedule)}
    assert len(pos) == len(schedule) == 2 * n * chunks, "every (micro-batch, chunk) needs one forward and one backward"
    for mb in range(n):
        for g in range(chunks):
            f, b = pos[(mb, g, True)], pos[(mb, g, False)]
            assert f < b, "forward precedes backward"
            if g > 0:
                assert pos[(mb, g - 1, True)] < f and schedule[pos[(mb, g - 1, True)]].step < schedule[f].step
            if g < chunks - 1:
                assert pos[(mb, g + 1, False)] < b and schedule[pos[(mb, g + 1, False)]].step < schedule[b].step


def PrintScheduleTable(schedule: List[Task], n: int, num_stages: int, vpp_size: int) -> str:
    steps = max(t.step for t in schedule) + 1 if schedule else 0
    rows = []
    for s in range(num_stages):
        cells = []
        for step in range(steps):
            ts = [t for t in schedule if t.stage_id == s and t.step == step]
            cells.append(",".join(f"{'F' if t.is_forward else 'B'}{t.microbatch_id}.{t.local_chunk_idx}" for t in ts) or "-")
        rows.append(f"stage {s}: " + " | ".join(f"{c:>9}" for c in cells))
    return "\n".join(rows)
