"""Pipeline instruction streams: 1F1B training, redundant computation, failover.

Behavioural contract (what must match, instruction for instruction, the schedule
generators of Bamboo's patched DeepSpeed, ``deepspeed/runtime/pipe/schedule.py``):

* ``TrainSchedule``            - reference ``schedule.py:225-310``
* ``LazyRecoverySchedule``     - reference ``schedule.py:469-501``
* ``EagerRecoverySchedule``    - reference ``schedule.py:504-524``
* ``NextStageFailoverSchedule``- reference ``schedule.py:343-430``
* ``PrevStageFailoverSchedule``- reference ``schedule.py:433-454``
* ``AllReduceFailoverSchedule``- reference ``schedule.py:457-466``
* instruction classes and their ``repr`` - reference ``schedule.py:552-732`` and
  ``deepspeed/runtime/utils.py:733-752``

The implementation here is organised differently: the step -> micro-batch map is a
closed form, a training stream is produced by one function over (step, stage), and the
wrappers are stream transformers driven by small rule tables.  Class names, constructor
signatures and the iteration protocol are kept so code written against the reference
(``schedule.TrainSchedule(micro_batches=..., stages=..., stage_id=...)``) keeps working.
"""
from typing import Iterable, Iterator, List, Optional, Sequence, Tuple


# --------------------------------------------------------------------------- instructions
class PipeInstruction:
    """One engine command.  Keyword arguments become attributes and are passed to the
    executor as ``**cmd.kwargs``; ``repr`` is ``Name(k=v, ...)`` in insertion order."""

    def __init__(self, **kwargs):
        self.name = type(self).__name__
        self.kwargs = kwargs
        self.__dict__.update(kwargs)

    def __repr__(self):
        return "%s(%s)" % (self.name, ", ".join("%s=%r" % kv for kv in self.kwargs.items()))

    def __eq__(self, other):
        return type(self) is type(other) and self.kwargs == other.kwargs

    def __hash__(self):
        return hash((type(self).__name__, tuple(self.kwargs.items())))


class BufferOpInstruction(PipeInstruction):
    def __init__(self, buffer_id, **kwargs):
        super().__init__(buffer_id=buffer_id, **kwargs)


class MultiStageOpInstruction(PipeInstruction):
    def __init__(self, stage_id, **kwargs):
        super().__init__(stage_id=stage_id, **kwargs)


class MultiStageBufferOpInstruction(BufferOpInstruction):
    def __init__(self, buffer_id, stage_id, **kwargs):
        super().__init__(buffer_id=buffer_id, stage_id=stage_id, **kwargs)


class CommunicationInstruction:
    """Marker mixin: the instruction talks to a neighbouring stage."""


class LoadMicroBatch(BufferOpInstruction):
    """``buffers['data'/'label'][buffer_id] = next(data_iter)``"""


class ForwardPass(MultiStageBufferOpInstruction):
    """Run stage ``stage_id`` forward on buffer ``buffer_id``."""


class BackwardPass(MultiStageBufferOpInstruction):
    """Back-propagate stage ``stage_id`` for buffer ``buffer_id``; grads accumulate."""


class SendActivation(MultiStageBufferOpInstruction, CommunicationInstruction):
    """Ship the stage output to the next stage (``buffer_id == -1``: liveness ping)."""


class RecvActivation(MultiStageBufferOpInstruction, CommunicationInstruction):
    """Take the stage input from the previous stage (``buffer_id == -1``: ping)."""


class SendGrad(MultiStageBufferOpInstruction, CommunicationInstruction):
    """Ship d(loss)/d(stage input) to the previous stage."""


class RecvGrad(MultiStageBufferOpInstruction, CommunicationInstruction):
    """Take d(loss)/d(stage output) from the next stage."""


class SendWeights(MultiStageOpInstruction):
    pass


class RecvWeights(MultiStageOpInstruction):
    pass


class ReduceGrads(MultiStageOpInstruction):
    """All-reduce the gradients of stage ``stage_id`` over its data-parallel column."""


class ReduceTiedGrads(PipeInstruction):
    pass


class OptimizerStep(PipeInstruction):
    """One optimizer step over every stage this rank owns, then zero the grads."""


# --------------------------------------------------------------------------- 1F1B map
def _is_even(x):
    return x % 2 == 0


def _is_odd(x):
    return x % 2 != 0


def _step_to_micro_batch(stages: int, stage_id: int, step_id: int) -> Tuple[int, bool]:
    """(micro_batch_id, is_forward) of pipeline step ``step_id`` on stage ``stage_id``.

    A stage runs forward when step and stage have the same parity.  Forward micro-batch
    ids trail the step by half the stage index; backward ids additionally trail by the
    pipeline depth.  Ids outside ``[0, micro_batches)`` mean "bubble".
    """
    half = step_id // 2
    if (step_id - stage_id) % 2 == 0:
        return half - stage_id // 2, True
    return half - stages + 1 + stage_id // 2, False


class PipeSchedule:
    """Base: iterating yields one list of instructions per pipeline step."""

    def __init__(self, micro_batches, stages, stage_id):
        self.micro_batches = micro_batches
        self.stages = stages
        self.stage_id = stage_id
        self.prev_stage = stage_id - 1
        self.next_stage = stage_id + 1

    def steps(self) -> Iterator[List[PipeInstruction]]:
        raise NotImplementedError

    def num_pipe_buffers(self):
        return self.micro_batches

    def _valid_micro_batch(self, mb):
        return 0 <= mb < self.micro_batches

    def _valid_stage(self, s):
        return 0 <= s < self.stages

    def _buffer_idx(self, mb):
        assert self._valid_micro_batch(mb)
        return mb % self.num_pipe_buffers()

    @property
    def stage(self):
        return self.stage_id

    @property
    def num_stages(self):
        return self.stages

    @property
    def num_micro_batches(self):
        return self.micro_batches

    @property
    def is_first_stage(self):
        return self.stage_id == 0

    @property
    def is_last_stage(self):
        return self.stage_id == self.stages - 1

    def __iter__(self):
        self.it = None
        return self

    def __next__(self):
        if self.it is None:
            self.it = self.steps()
        return next(self.it)


class TrainSchedule(PipeSchedule):
    """Interleaved one-forward-one-backward schedule, ``2*(M+S-1)`` steps.

    Buffer id equals micro-batch id (the stage keeps ``M`` buffers) so that a failover
    schedule can address the dead neighbour's buffers by micro-batch.
    """

    def __init__(self, micro_batches, stages, stage_id, **kwargs):
        super().__init__(micro_batches, stages, stage_id)

    @property
    def require_data_loader(self):
        return self.is_first_stage or self.is_last_stage

    def step_to_micro_batch(self, step_id):
        return _step_to_micro_batch(self.stages, self.stage_id, step_id)

    _step_to_micro_batch = step_to_micro_batch

    def valid_micro_batch(self, mb):
        return self._valid_micro_batch(mb)

    def steps(self):
        sid, last_step = self.stage_id, 2 * (self.micro_batches + self.stages - 1) - 1
        has_prev, has_next = self._valid_stage(self.prev_stage), self._valid_stage(self.next_stage)
        before = -1  # micro-batch handled by the preceding step
        for step in range(last_step + 1):
            mb, fwd = self.step_to_micro_batch(step)
            live, before_live = self._valid_micro_batch(mb), self._valid_micro_batch(before)
            cmds: List[PipeInstruction] = []
            if fwd:
                if live and self.require_data_loader:
                    cmds.append(LoadMicroBatch(mb))
                if live and has_prev:
                    cmds.append(RecvActivation(mb, sid))
                if before_live and has_prev:
                    cmds.append(SendGrad(before, sid))
                if live:
                    cmds.append(ForwardPass(mb, sid))
            else:
                if before_live and has_next:
                    cmds.append(SendActivation(before, sid))
                if live and has_next:
                    cmds.append(RecvGrad(mb, sid))
                if live:
                    cmds.append(BackwardPass(mb, sid))
            if step == last_step:
                cmds += [ReduceGrads(sid), OptimizerStep()]
            before = mb
            yield cmds


class DataParallelSchedule(PipeSchedule):
    """Gradient accumulation without pipelining (one buffer)."""

    def steps(self):
        for i in range(self.micro_batches):
            cmds = [LoadMicroBatch(buffer_id=0), ForwardPass(buffer_id=0, stage_id=self.stage_id),
                    BackwardPass(buffer_id=0, stage_id=self.stage_id)]
            if i == self.micro_batches - 1:
                cmds += [ReduceGrads(self.stage_id), OptimizerStep()]
            yield cmds

    def num_pipe_buffers(self):
        return 1


# --------------------------------------------------------------------------- wrappers
class ResilientPipeSchedule:
    """A stream computed from two step-aligned streams: this rank's (``sched``) and a
    neighbour's (``next_sched``).  ``failed_step``/``curr_step`` delimit the redo
    window when a failure was detected in the middle of a batch."""

    def __init__(self, sched, next_sched, failed_step=0, curr_step=0):
        self.sched = sched
        self.next_sched = next_sched
        self.failed_step = failed_step
        self.curr_step = curr_step
        self.cmd_buffer: List[List[PipeInstruction]] = []

    def steps(self):
        for i, (mine, other) in enumerate(zip(self.sched, self.next_sched)):
            yield self._merge_cmds(mine, other, i)

    def num_pipe_buffers(self):
        return self.sched.num_pipe_buffers()

    def _merge_cmds(self, cmds, next_cmds, i):
        raise NotImplementedError

    def __iter__(self):
        self.it = None
        return self

    def __next__(self):
        if self.it is None:
            self.it = self.steps()
        return next(self.it)


def _kind(seq: Sequence[PipeInstruction], pos: int):
    return type(seq[pos]) if pos < len(seq) else None


class NextStageFailoverSchedule(ResilientPipeSchedule):
    """This rank also runs the stage after it (whose owner died).

    Before ``curr_step`` the dead stage's steps are replayed alone (its sends dropped
    before ``failed_step``, since their receivers already hold the data).  From
    ``curr_step`` on, the two step lists are interleaved by a two-cursor merge: the
    pair (own SendActivation, dead RecvActivation) collapses to the latter as a local
    hand-off, the pair (dead SendGrad, own RecvGrad) collapses to the latter, the dead
    stage's OptimizerStep disappears (one step covers both stages) and its ReduceGrads
    stays.
    """

    _DROP_IN_REPLAY = (SendActivation, SendGrad)

    def _merge_cmds(self, cmds, next_cmds, i):
        if i < self.curr_step:
            if i < self.failed_step:
                return [c for c in next_cmds if type(c) not in self._DROP_IN_REPLAY]
            return list(next_cmds)

        out: List[PipeInstruction] = []
        a = b = 0  # cursors into own / dead stage's instructions
        while a < len(cmds) or b < len(next_cmds):
            mine, dead = _kind(cmds, a), _kind(next_cmds, b)
            if mine is LoadMicroBatch:
                out.append(cmds[a]); a += 1
            elif mine is RecvWeights:
                a += 1
            elif dead is SendWeights:
                b += 1
            elif dead in (LoadMicroBatch, SendActivation, RecvGrad):
                out.append(next_cmds[b]); b += 1
            elif dead is SendGrad:
                assert mine is RecvGrad, f"Unable to merge cmds ({cmds}) and ({next_cmds})"
                out.append(cmds[a]); a += 1; b += 1
            elif dead is RecvActivation:
                assert mine is SendActivation, f"Unable to merge cmds ({cmds}) and ({next_cmds})"
                out.append(next_cmds[b]); a += 1; b += 1
            elif mine is BackwardPass:
                out.append(cmds[a]); a += 1
            elif dead is BackwardPass:
                out.append(next_cmds[b]); b += 1
            elif mine is not None:
                out.append(cmds[a]); a += 1
            elif dead in (ForwardPass, RecvWeights, ReduceGrads):
                out.append(next_cmds[b]); b += 1
            elif dead is OptimizerStep:
                b += 1
            elif dead is not None:
                raise Exception(f"Unsupported cmd found in cmds ({next_cmds})")
            else:  # pragma: no cover - loop guard makes this unreachable
                raise Exception(f"Unable to merge cmds ({cmds}) and ({next_cmds})")
        return out


class PrevStageFailoverSchedule(ResilientPipeSchedule):
    """The stage before this rank died and its predecessor took it over.

    ``sched`` is the dead stage's stream (only used for alignment), ``next_sched`` is
    this rank's own.  In the replay window only gradient sends are repeated; afterwards
    the own stream runs minus liveness pings (nobody answers them any more).
    """

    def _merge_cmds(self, cmds, next_cmds, i):
        if i < self.curr_step:
            if i < self.failed_step:
                return [c for c in next_cmds if type(c) is SendGrad]
            return []
        return [c for c in next_cmds
                if type(c) is not SendWeights
                and not (type(c) is RecvActivation and c.buffer_id == -1)]


class AllReduceFailoverSchedule(ResilientPipeSchedule):
    """A data-parallel peer died: skip what completed before ``failed_step``."""

    def _merge_cmds(self, cmds, next_cmds, i):
        return [] if i < self.failed_step else cmds


class LazyRecoverySchedule(ResilientPipeSchedule):
    """Lazy redundancy: no shadow compute, only one-float pings (``buffer_id=-1``)
    that let neighbours notice a dead stage while the pipeline is filling."""

    def __init__(self, sched, next_sched, failed_step=0, curr_step=0):
        super().__init__(sched, next_sched, failed_step, curr_step)
        self.stage_id = sched.stage_id
        self.is_first_stage = sched.is_first_stage
        self.is_last_stage = sched.is_last_stage

    def _fwd(self, stage, step):
        return _step_to_micro_batch(self.sched.stages, stage, step)[1]

    def _merge_cmds(self, cmds, next_cmds, i):
        sid = self.stage_id
        filling = i < self.sched.micro_batches + self.sched.stages - 1
        quiet = not any(isinstance(c, CommunicationInstruction) for c in cmds)
        head: List[PipeInstruction] = []
        if self.is_first_stage:
            if self._fwd(sid, i):
                head = [RecvActivation(-1, sid)]
        elif self.is_last_stage:
            if quiet and filling and self._fwd(sid, i):
                head = [RecvActivation(-1, sid)]
            if self._fwd(0, i):
                head = [SendActivation(-1, sid)] + head
        elif quiet and filling:
            head = [RecvActivation(-1, sid)] if self._fwd(sid, i) else [SendActivation(-1, sid)]
        return head + cmds


class EagerRecoverySchedule(ResilientPipeSchedule):
    """Eager redundancy: the successor's input-side work (load, receive, forward) is
    queued step by step and one queued step is released in front of every own step
    that receives a gradient, i.e. where this stage would otherwise wait."""

    _SHADOWED = (RecvActivation, LoadMicroBatch, ForwardPass)

    def _merge_cmds(self, cmds, next_cmds, i):
        out: List[PipeInstruction] = []
        if self.cmd_buffer and any(type(c) is RecvGrad for c in cmds):
            out += [c for c in self.cmd_buffer.pop(0) if type(c) in self._SHADOWED]
        if any(type(c) in self._SHADOWED for c in next_cmds):
            self.cmd_buffer.append(next_cmds)
        return out + list(cmds)


def materialize(sched: Iterable[List[PipeInstruction]]) -> List[List[PipeInstruction]]:
    """Run a schedule generator to completion (raises what the generator raises)."""
    return [list(step) for step in sched]
