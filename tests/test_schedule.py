"""Instruction-stream identity with the reference's schedule generators.

The golden streams in tests/golden/schedules.json.gz were produced by running the
reference's own ``deepspeed/runtime/pipe/schedule.py`` (see tests/golden/gen_golden.py).
"""
import re

import pytest

from bamboo_b200 import schedule as S

KEY = re.compile(r"S(\d+)M(\d+)/(train|lazy|eager)/(?:stage(\d+)|victim(\d+)/f(\d+)c(\d+)/"
                 r"(next|prev|allreduce)_on_stage(\d+))$")


def build(key):
    m = KEY.match(key)
    assert m, key
    stages, mb, base = int(m.group(1)), int(m.group(2)), m.group(3)

    def train(s):
        return S.TrainSchedule(micro_batches=mb, stages=stages, stage_id=s)

    def own(s):
        if base == "train":
            return train(s)
        cls = S.LazyRecoverySchedule if base == "lazy" else S.EagerRecoverySchedule
        return cls(train(s), train((s + 1) % stages))

    if m.group(4) is not None:
        return own(int(m.group(4)))
    victim, fs, cs, kind, on = int(m.group(5)), int(m.group(6)), int(m.group(7)), m.group(8), int(m.group(9))
    if kind == "next":
        return S.NextStageFailoverSchedule(own(on), train(victim), failed_step=fs, curr_step=cs)
    if kind == "prev":
        return S.PrevStageFailoverSchedule(train(victim), own(on), failed_step=fs, curr_step=cs)
    return S.AllReduceFailoverSchedule(own(on), [[] for _ in own(on)], failed_step=fs)


def test_every_golden_stream(golden_schedules):
    assert len(golden_schedules) > 600
    raised = 0
    for key, want in golden_schedules.items():
        sched = build(key)
        if isinstance(want, dict):
            with pytest.raises(Exception) as ei:
                S.materialize(sched)
            assert type(ei.value).__name__ == want["raises"], key
            raised += 1
            continue
        got = [[repr(c) for c in step] for step in sched]
        assert got == want, key
    assert raised > 0


def test_known_answers_two_stage_four_micro_batches(golden_schedules):
    # hand-checkable: stage 0 of a 2-stage pipeline, 4 micro-batches
    got = [[repr(c) for c in s] for s in S.TrainSchedule(4, 2, 0)]
    assert got[0] == ["LoadMicroBatch(buffer_id=0)", "ForwardPass(buffer_id=0, stage_id=0)"]
    assert got[1] == ["SendActivation(buffer_id=0, stage_id=0)"]
    assert got[8] == []
    assert got[9] == ["RecvGrad(buffer_id=3, stage_id=0)", "BackwardPass(buffer_id=3, stage_id=0)",
                      "ReduceGrads(stage_id=0)", "OptimizerStep()"]
    merged = S.materialize(S.NextStageFailoverSchedule(
        S.LazyRecoverySchedule(S.TrainSchedule(4, 2, 0), S.TrainSchedule(4, 2, 1)), S.TrainSchedule(4, 2, 1)))
    assert [repr(c) for c in merged[9]] == [
        "RecvGrad(buffer_id=3, stage_id=0)", "BackwardPass(buffer_id=3, stage_id=0)",
        "ReduceGrads(stage_id=0)", "OptimizerStep()", "ReduceGrads(stage_id=1)"]
    assert sum(len(s) for s in merged) == 40


def test_single_stage_degenerates_to_accumulation():
    steps = S.materialize(S.TrainSchedule(micro_batches=3, stages=1, stage_id=0))
    assert len(steps) == 6
    flat = [type(c).__name__ for s in steps for c in s]
    assert flat == ["LoadMicroBatch", "ForwardPass", "BackwardPass"] * 3 + ["ReduceGrads", "OptimizerStep"]


def test_schedule_queries():
    first, last = S.TrainSchedule(8, 3, 0), S.TrainSchedule(8, 3, 2)
    assert first.is_first_stage and not first.is_last_stage
    assert last.is_last_stage and last.require_data_loader
    assert not S.TrainSchedule(8, 3, 1).require_data_loader
    assert first.num_pipe_buffers() == 8 and first.num_stages == 3 and first.num_micro_batches == 8
    assert first.step_to_micro_batch(0) == (0, True)


def test_every_micro_batch_runs_once_per_direction():
    for stages, mb in ((2, 4), (4, 16), (8, 32), (3, 5)):
        for s in range(stages):
            flat = [c for st in S.TrainSchedule(mb, stages, s) for c in st]
            fwd = sorted(c.buffer_id for c in flat if type(c) is S.ForwardPass)
            bwd = sorted(c.buffer_id for c in flat if type(c) is S.BackwardPass)
            assert fwd == list(range(mb)) and bwd == list(range(mb))


def test_instruction_repr_and_kwargs():
    c = S.ForwardPass(3, 1)
    assert repr(c) == "ForwardPass(buffer_id=3, stage_id=1)"
    assert c.kwargs == {"buffer_id": 3, "stage_id": 1} and c.buffer_id == 3 and c.stage_id == 1
    assert repr(S.OptimizerStep()) == "OptimizerStep()"
    assert isinstance(S.SendGrad(0, 0), S.CommunicationInstruction)
    assert not isinstance(S.ForwardPass(0, 0), S.CommunicationInstruction)
