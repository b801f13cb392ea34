"""PipelineEngine: executes the per-step instruction stream of a pipeline stage.

Mirrors the behaviour of Bamboo's patched DeepSpeed engine on the ``train_batch`` path
(``deepspeed/runtime/pipe/engine.py``): constructor arguments and redundancy checks
(``:104-183``), pipe buffers (``:352-387``), schedule construction (``:272-293``),
``train_batch`` with failure bookkeeping (``:1068-1423``), ``check_preemptions``
(``:731-880``), the instruction executors (``:1626-2082``, ``:2139-2183``), the interpreter
``_exec_schedule`` (``:2339-2394``) and loss aggregation (``:1550-1584``); base-engine pieces
it relies on: loss scaling by gradient-accumulation steps and ``loss.backward()``
(``deepspeed/runtime/engine.py:1317-1335,1416-1478``), the data-parallel gradient average
(``:1728-1802``) and the model step (``:1526-1573``).

What is different underneath:

* stage compute is whatever the layers do - the layers in ``bamboo_b200.layers`` run on
  hand-written sm_100a kernels; parameters live in flat arenas, the optimizer is one fused
  kernel per stage and the data-parallel all-reduce sees one contiguous fp32 buffer;
* inter-stage tensors go through a ``Transport`` (IPC mailboxes + store kernels on CUDA);
* eager redundant computation runs on a separate low-priority CUDA stream;
* the shadow copy of the successor stage (weights and Adam moments) is refreshed after
  every optimizer step - the reference never implemented that transfer (its
  ``_exec_recv_weights`` returns immediately, ``engine.py:2110-2112``), so a promoted stage
  there would continue from zeros; here failover continues the same optimisation trajectory.
"""
import collections
import contextlib
import json
import os
import signal
import sys
import threading
import time
from types import MethodType
from typing import Dict, List, Optional, Tuple

import torch

from . import rendezvous as _rdzv
from . import schedule
from .arena import ParamArena
from .config import PipeConfig
from .module import PipelineModule
from .p2p import ACT, GRAD, DistTransport, NullTransport, PeerTimeout
from .partition import get_redundant_stage_ids, get_redundant_user_stage_ids

should_stop = False
_live_stores = []


def sig_handler(signum, frame):
    """SIGTERM = preemption notice: announce the failure at the next batch boundary."""
    global should_stop
    should_stop = True


class PipelineError(Exception):
    """Errors related to the use of deepspeed.PipelineEngine."""


class PrevStageException(Exception):
    ...


class NextStageException(Exception):
    ...


class AllReduceException(Exception):
    def __init__(self, src, *args):
        super().__init__(*args)
        self.src = src  # pipeline (data-parallel id) of the failed rank


class LocalStore:
    """In-process key/value store with the subset of the c10d ``Store`` API the engine uses."""

    def __init__(self):
        self._d = {}
        self._add_lock = threading.Lock()

    def set(self, key, value):
        self._d[key] = value if isinstance(value, bytes) else str(value).encode()

    def get(self, key):
        return self._d[key]

    def check(self, keys):
        return all(k in self._d for k in keys)

    def add(self, key, num):
        with self._add_lock:
            value = int(self._d.get(key, b"0")) + int(num)
            self._d[key] = str(value).encode()
            return value


@contextlib.contextmanager
def store_mutex(store, name, timeout_s=5.0):
    """Mutual exclusion between the members of a job through their key/value store: a ticket lock on the
    store's atomic ``add`` (c10d TCP / file stores, the etcd-backed store and the in-process one all have it).
    A member that waited ``timeout_s`` for a holder that never released (it died in between) goes ahead anyway
    and moves the counter past its own ticket, so that the members behind it are served again."""
    add = getattr(store, "add", None)
    if add is None:
        yield
        return
    ticket = int(add(f"{name}-ticket", 1))
    deadline = time.time() + timeout_s
    while int(add(f"{name}-serving", 0)) < ticket - 1 and time.time() < deadline:
        time.sleep(0.002)
    try:
        yield
    finally:
        behind = ticket - int(add(f"{name}-serving", 0))
        if behind > 0:
            add(f"{name}-serving", behind)


class LocalRendezvous:
    """Stand-in for the etcd rendezvous handler when a job is launched without the elastic
    agent: a fixed grid, never reconfigures."""

    def __init__(self, topology, world_size):
        from .topology import GlobalInfo
        self._decision = []
        for r in range(world_size):
            c = topology.get_coord(r)
            self._decision.append(GlobalInfo(r, [], [[c.data, c.pipe]]))
        self._kv = {}

    def get_global_decision(self):
        return self._decision

    def get_current_step(self):
        return 0

    def write(self, key, value):
        self._kv[key] = value

    def should_reconfigure(self, step, failures):
        return False

    def update_coordinates(self, rank, coordinates):
        self._kv[f"coords-{rank}"] = coordinates

    def create_lock(self, name):
        return _NullLock()


class _NullLock:
    def acquire(self, blocking=True, lock_ttl=10):
        return True

    def release(self):
        return True


def _decode(v):
    return v.decode() if isinstance(v, (bytes, bytearray)) else v


class PipelineEngine:
    def __init__(self, model: PipelineModule, config=None, redundancy_level=0, sync_save=False, eager_recovery=False,
                 training_data=None, collate_fn=None, rdzv_handler=None, store=None, transport=None, dist=None,
                 lr_scheduler=None, prev_state=None):
        assert isinstance(model, PipelineModule), "model must base PipelineModule"
        self._init_args = dict(config=config, redundancy_level=redundancy_level, sync_save=sync_save,
                               eager_recovery=eager_recovery, collate_fn=collate_fn, lr_scheduler=lr_scheduler)
        self.module = model
        self.grid = model._grid
        self.device = model.device
        if dist is None:
            import torch.distributed as _d
            dist = _d if (_d.is_available() and _d.is_initialized()) else None
        self.dist = dist
        self.global_rank = self.grid.get_global_rank()
        self.world_size = self.grid.world_size
        self.dp_world_size = self.grid.data_parallel_size
        self._config = config if isinstance(config, PipeConfig) else PipeConfig(config, self.dp_world_size)
        assert self._config.zero_stage < 2, "ZeRO-2 and ZeRO-3 are incompatible with pipeline parallelism"
        self.micro_batch_size = self._config.train_micro_batch_size_per_gpu
        self.micro_batches = self._config.gradient_accumulation_steps
        assert self._config.train_batch_size == self.micro_batch_size * self.micro_batches * self.dp_world_size

        try:
            signal.signal(signal.SIGTERM, sig_handler)
        except ValueError:
            pass  # not the main thread

        self.num_stages = self.grid.pipe_parallel_size
        self.stage_id = self.grid.get_stage_id()
        self.prev_stage = self._dec(self.stage_id)
        self.next_stage = self._inc(self.stage_id)
        self.stage_ids = [self.stage_id]

        # A job started by the launcher describes its rendezvous in the environment
        # (PROJECT_PACTUM_ENABLED / ENDPOINT / RUN_ID / MIN_NODES / MAX_NODES / RDZV_CONFIGS /
        # MAX_PIPE_PARALLEL_SIZE): the handler is built from it and its etcd-backed store carries the
        # bookkeeping keys, as in deepspeed/runtime/engine.py:152-184.
        launched = _rdzv.ENV_ENABLED in os.environ
        if launched:
            self.max_pipe_parallel_size = os.environ["PROJECT_PACTUM_MAX_PIPE_PARALLEL_SIZE"]
            if rdzv_handler is None:
                rdzv_handler = _rdzv.handler_from_env()
            if store is None:
                store = rdzv_handler.setup_kv_store()
                _live_stores.append(store)
                for rank in range(self.world_size):
                    store.set(str(rank), "0")
                store.set("failures", "{}")
        self.rdzv_handler = rdzv_handler or LocalRendezvous(self.grid.topology(), self.world_size)
        self.coordinates = [[self.grid.get_data_parallel_id(), self.stage_id]]
        for info in self.rdzv_handler.get_global_decision():
            if info.rank == self.global_rank:
                self.coordinates = [list(c) for c in info.active_coordinates]
        if store is None and self.dist is not None and self.world_size > 1:
            try:  # the job's own c10d store (env:// or rendezvous-provided) carries the bookkeeping keys
                from torch.distributed.distributed_c10d import _get_default_store
                store = self.dist.PrefixStore("bamboo_b200", _get_default_store())
            except Exception:
                store = None
        self.global_store = store or LocalStore()
        self.global_store.set(str(self.global_rank), "0")
        if isinstance(self.global_store, LocalStore) or self.global_rank == 0:
            self.global_store.set("failures", "{}")
        self.fail_lock = self.rdzv_handler.create_lock("fail-lock")
        self.global_steps = self.rdzv_handler.get_current_step()
        self.global_samples = 0
        self.join = "PROJECT_PACTUM_JOIN" in os.environ    # a worker that joins a job which is already running

        if redundancy_level > 1:
            raise NotImplementedError(f"R level {redundancy_level} > 1 is not supported now.")
        if eager_recovery and redundancy_level == 0:
            raise Exception("Must set redundancy level to enable eager recovery")
        self.redundancy_level = redundancy_level
        self.eager_recovery = eager_recovery
        self.sync_save = sync_save

        # ---- parameters and optimizer state, one flat arena per stage on this rank
        self.native = self.device.type == "cuda"
        lp_dtype = torch.bfloat16 if (self.native and self._config.bf16_enabled) else torch.float32
        self.lp_dtype = lp_dtype
        self.arenas: Dict[int, ParamArena] = {}
        self.arenas[self.stage_id] = ParamArena(self.module.stage_parameters(self.stage_id), self.device, lp_dtype)
        self._adam = self._config.adam_args()
        self.lr_scheduler = lr_scheduler
        self.optimizer = self  # exposes param_groups-like access through get_lr()

        # ---- transport
        if transport is not None:
            self.transport = transport
        elif self.num_stages == 1:
            self.transport = NullTransport()
        elif self.native:
            from .mailbox import MailboxTransport
            self.transport = MailboxTransport(self)
        else:
            self.transport = DistTransport(self.dist, timeout_s=self._config.p2p_timeout_s)

        self.init_redundancy()
        self.init_pipe_buffers()
        self.data_iterator = None
        self.training_dataloader = None
        self.batch_fn = None
        if training_data is not None:
            self._build_data_iter(training_data, collate_fn)

        self.is_pipe_parallel = self.num_stages > 1
        self.is_data_parallel = self.dp_world_size > 1
        self.loss = None
        self.total_loss = None
        self.agg_train_loss = None
        self.loss_model = self.module.loss_fn
        self._compute_loss = True
        self._losses: Dict[Tuple[int, int], torch.Tensor] = {}
        self.timers = collections.defaultdict(float)
        self.instr_counts = collections.Counter()

        # low-priority stream for redundant computation
        self.rc_stream = None
        self._rc_event = None
        self._lp_refreshed = None
        self._main_stream = None
        if self.native:
            # Priorities: the stage's own work runs on a stream of the highest priority, weight
            # gradients one level below (layers.py), redundant computation at the lowest: whenever
            # thread blocks of several streams are pending, the GPU places the own stage's first.
            # (The default stream has the LOWEST priority, so the own work must leave it for the
            # order to mean anything.)
            lo, hi = torch.cuda.Stream.priority_range() if hasattr(torch.cuda.Stream, "priority_range") else (0, -1)
            if self._config.main_stream_high_priority:
                self._main_stream = torch.cuda.Stream(device=self.device, priority=hi)
            if self.eager_recovery:
                self.rc_stream = torch.cuda.Stream(device=self.device,
                                                   priority=lo if self._config.rc_stream_priority_low else hi)

        # ---- schedule constructors (composed like the reference: base, RC wrapper, failover wrappers)
        self._sched_layers: List = []  # list of (kind, kwargs) applied on top of TrainSchedule(own stage)
        if self.r_stage_ids:
            self._sched_layers.append(("eager" if self.eager_recovery else "lazy", dict(stage_id=self.next_stage)))
        self._seq = collections.Counter()
        self._fwd_done: Dict[Tuple[int, int], object] = {}   # (stage, buffer) -> event behind that forward
        self._shadow_ctx = False        # True while an instruction of a redundant-work group executes
        self._rc_queue = collections.deque()                  # redundant forwards not yet (fully) issued
        self._rc_inflight = collections.deque()               # events behind the chunks issued in idle time
        if self.rc_stream is not None and hasattr(self.transport, "idle_hook") and self._config.rc_deferred:
            self.transport.idle_hook = self._rc_pump

        # not the first rendezvous of the run: some member already trained; fetch the layers of this
        # rank's new seat from whoever held them (reference: pipe/engine.py:149-165)
        decision = self.rdzv_handler.get_global_decision()
        if self.dist is not None and self.world_size > 1 and any(len(i.previous_coordinates) for i in decision):
            self._join_from_previous(decision, prev_state or {})

    # ------------------------------------------------------------------ helpers
    def _inc(self, s):
        return (s + 1) % self.num_stages

    def _dec(self, s):
        return (s - 1 + self.num_stages) % self.num_stages

    def is_first_stage(self):
        return self.stage_id == 0

    def is_last_stage(self):
        return self.num_stages - 1 in self.stage_ids

    def train_batch_size(self):
        return self._config.train_batch_size

    def train_micro_batch_size_per_gpu(self):
        return self.micro_batch_size

    def gradient_accumulation_steps(self):
        return self.micro_batches

    def steps_per_print(self):
        return self._config.steps_per_print

    def wall_clock_breakdown(self):
        return self._config.wall_clock_breakdown

    def get_lr(self):
        return [self._adam["lr"]]

    def log(self, msg, color=None):
        if os.environ.get("BAMBOO_QUIET"):
            return
        print(f"[ {self.global_rank:02d}|{self.global_steps:02d} ] {msg}", flush=True)

    def _stage_rank(self, stage):
        return self.grid._topo.get_rank(data=self.grid.get_data_parallel_id(), pipe=stage)

    # ------------------------------------------------------------------ redundancy
    def init_redundancy(self):
        self.r_stage_ids = get_redundant_stage_ids(self.redundancy_level, self.stage_id, self.num_stages)
        self.r_user_stage_ids = get_redundant_user_stage_ids(self.redundancy_level, self.stage_id, self.num_stages)
        if self.num_stages == 1:
            self.r_stage_ids, self.r_user_stage_ids = [], []
        self.param_buffers: Dict[int, ParamArena] = {}
        self.state_buffers: Dict[int, ParamArena] = {}
        # who holds the shadow copy of this rank's stage / who owns the stages shadowed here
        self._shadow_holder_rank = self._stage_rank(self.r_user_stage_ids[0]) if self.r_user_stage_ids else None
        # False once a state transfer into a shadow copy failed: its weights and moments may then
        # belong to different steps, and a promotion from it would leave the optimisation trajectory
        self._shadow_valid: Dict[int, bool] = {}
        self._shadow_source_rank = {sid: self._stage_rank(sid) for sid in self.r_stage_ids}
        if self.redundancy_level > 0:
            for sid in self.r_stage_ids:
                # The shadow stage is built with the same constructors (and seeds) as on its
                # owner, so it starts as an exact copy; afterwards it follows the owner through
                # the state transfer that ends every optimizer step.
                self.module.build_layers(sid)
                arena = ParamArena(self.module.stage_parameters(sid), self.device, self.lp_dtype)
                self.arenas[sid] = arena
                self.param_buffers[sid] = arena
                self.state_buffers[sid] = arena
            self.grid.init_fallback_group(self.redundancy_level)

    def init_pipe_buffers(self):
        self.num_pipe_buffers = 0
        self.pipe_buffers: Dict[str, List] = {
            "data": [], "label": [],
            f"input_{self.stage_id}": [], f"output_{self.stage_id}": [],
        }
        if self.stage_id != 0:
            self.pipe_buffers[f"input_grad_{self.stage_id}"] = []
        for sid in self.r_stage_ids:
            self.pipe_buffers[f"input_{sid}"] = []
            self.pipe_buffers[f"output_{sid}"] = []
        self.grad_layer = None

    def _clean_pipe_buffers(self):
        for k in self.pipe_buffers:
            self.pipe_buffers[k] = []
        self.num_pipe_buffers = 0
        self._losses = {}
        self._fwd_done.clear()

    def _reserve_pipe_buffers(self, n):
        for k, v in self.pipe_buffers.items():
            if len(v) < n:
                v.extend([None] * (n - len(v)))
        self.num_pipe_buffers = max(self.num_pipe_buffers, n)

    # ------------------------------------------------------------------ schedules
    def _train_sched(self, stage_id):
        return schedule.TrainSchedule(micro_batches=self.micro_batches, stages=self.num_stages, stage_id=stage_id)

    def _generate_sched(self):
        """Compose the wrappers recorded in ``_sched_layers`` around this rank's base stream."""
        sched = self._train_sched(self.stage_id)
        for kind, kw in self._sched_layers:
            fs, cs = kw.get("failed_step", 0), kw.get("curr_step", 0)
            if kind == "lazy":
                sched = schedule.LazyRecoverySchedule(sched, self._train_sched(kw["stage_id"]))
            elif kind == "eager":
                sched = schedule.EagerRecoverySchedule(sched, self._train_sched(kw["stage_id"]))
            elif kind == "next":
                sched = schedule.NextStageFailoverSchedule(sched, self._train_sched(kw["stage_id"]),
                                                           failed_step=fs, curr_step=cs)
            elif kind == "prev":
                sched = schedule.PrevStageFailoverSchedule(self._train_sched(kw["stage_id"]), sched,
                                                           failed_step=fs, curr_step=cs)
            elif kind == "allreduce":
                steps = schedule.materialize(sched)
                sched = schedule.AllReduceFailoverSchedule(iter(steps), [[] for _ in steps], failed_step=fs)
        return sched

    def _materialize_sched(self):
        """Instruction list for the coming batch.  An eager-RC stream cannot be merged with a
        dead successor's stream in the reference when the victim is not stage 0 (its merge
        asserts); in that case the pending redundant instructions are dropped and the plain
        stream is merged instead."""
        try:
            return schedule.materialize(self._generate_sched())
        except AssertionError:
            kinds = [k for k, _ in self._sched_layers]
            if "eager" in kinds and "next" in kinds:
                saved = list(self._sched_layers)
                self._sched_layers = [(k, v) for k, v in saved if k != "eager"]
                try:
                    return schedule.materialize(self._generate_sched())
                finally:
                    self._sched_layers = saved
            raise

    # ------------------------------------------------------------------ data
    def _build_data_iter(self, dataset, collate_fn=None):
        from .dataloader import RepeatingLoader, build_loader
        loader = build_loader(dataset, self.micro_batch_size, self.dp_world_size, self.grid.get_data_parallel_id(),
                              collate_fn)
        self.set_dataloader(RepeatingLoader(loader))

    def set_dataloader(self, loader):
        self.training_dataloader = loader
        self.data_iterator = iter(loader)

    def set_dataiterator(self, iterator):
        self.training_dataloader = None
        self.data_iterator = iterator

    def set_batch_fn(self, fn):
        self.batch_fn = fn

    def _next_batch(self):
        batch = next(self.data_iterator) if self.data_iterator is not None else None
        if self.batch_fn:
            batch = self.batch_fn(batch)
        return batch

    # ------------------------------------------------------------------ failure bookkeeping
    def trigger_kill(self, dp_id, stage_id, step, fatal=False):
        if self.global_steps == step and self.grid.get_data_parallel_id() == dp_id and self.stage_id == stage_id:
            if fatal:
                self.log("FAILING")
                sys.exit(13)
            self.log("PREEMPTION SOON")
            os.kill(os.getpid(), signal.SIGTERM)

    def should_kill(self, dp_id, stage_id):
        return self.grid.get_data_parallel_id() == dp_id and self.stage_id == stage_id

    def announce_preemption(self):
        """What the SIGTERM handler's flag leads to: publish 'this rank dies before step+1'.

        The record is one shared key that every announcer reads, extends and writes back (reference
        ``pipe/engine.py:1099-1109``).  Spot instances are often reclaimed several at a time, and two members
        doing this at the same moment would lose one of the two entries - that member's departure would then
        only be found by its neighbours' timeouts.  So the update runs under a mutex kept in the store itself."""
        me, when = str(self.global_rank), self.global_steps + 1
        with store_mutex(self.global_store, "failures"):
            failures = json.loads(_decode(self.global_store.get("failures")))
            failures = {r: s for r, s in failures.items() if s >= self.global_steps}
            failures[me] = when
            self.global_store.set("failures", json.dumps(failures))

    def _promote_next_stage(self):
        """Take over the successor stage from the shadow copy: its arena becomes a live stage
        of this rank (weights and Adam moments were refreshed at the last optimizer step)."""
        nxt = self.next_stage
        if nxt not in self.param_buffers or nxt not in self.state_buffers:
            raise RuntimeError("Doesn't have param or state to recover")
        if not self._shadow_valid.get(nxt, True):
            raise RuntimeError(f"the shadow copy of stage {nxt} missed a state transfer (its owner stopped answering "
                               "in the middle of one) and cannot be promoted; restart from a checkpoint")
        t0 = time.time()
        self._rc_pump(everything=True)
        if self.rc_stream is not None:
            # redundant forwards and the shadow's working-copy refresh are ordered on the RC stream
            torch.cuda.current_stream().wait_stream(self.rc_stream)
            self._rc_event = None
        next_rank = self.grid.stage_to_global(nxt)
        next_coord = self.grid.topology().get_coord(next_rank)
        self.grid.topology().modify_mapping(rank=self.global_rank, **next_coord._asdict())
        arena = self.param_buffers.pop(nxt)
        self.state_buffers.pop(nxt)
        arena.allocate_optimizer_state()
        arena.step_count = self.arenas[self.stage_id].step_count
        self.stage_ids.append(nxt)
        self.r_stage_ids = []
        self.pipe_buffers.setdefault(f"input_{nxt}", [])
        self.pipe_buffers.setdefault(f"output_{nxt}", [])
        self.next_stage = self._inc(nxt)
        self._forget_rank(next_rank)
        self.timers["promote_s"] = time.time() - t0
        return next_rank

    def _forget_rank(self, rank):
        """A rank is gone: stop exchanging shadow state with it and drop transport state."""
        if self._shadow_holder_rank == rank:
            self._shadow_holder_rank = None
        for sid, r in list(self._shadow_source_rank.items()):
            if r == rank:
                self._shadow_source_rank[sid] = None
        if hasattr(self.transport, "forget_peer"):
            self.transport.forget_peer(rank)

    def check_preemptions(self, failures):
        """Failures announced for this step by ranks this one talks to: successor, predecessor
        or a data-parallel peer."""
        dp_id = self.grid.get_data_parallel_id()
        prev_rank = self._stage_rank(self.prev_stage) if self.num_stages > 1 else -1
        next_rank = self._stage_rank(self.next_stage) if self.num_stages > 1 else -1
        seen = set()
        for rank in list(self.grid.current_dp_group) + [prev_rank, next_rank]:
            if rank in seen:
                continue  # in a two-stage ring the successor is also the predecessor
            seen.add(rank)
            key = str(rank)
            if key not in failures or self.global_steps != failures[key]:
                continue
            if rank == self.global_rank:
                self.global_store.set(str(self.global_rank), "1")
                self.transport.close()
                sys.exit(13)
            if rank == next_rank and self.num_stages > 1 and self.next_stage not in self.stage_ids:
                self.log("Next node is going to fail. Using fallback schedule")
                victim = self.next_stage
                self._sched_layers.append(("next", dict(stage_id=victim, failed_step=0, curr_step=0)))
                self._promote_next_stage()
                self.coordinates.append([dp_id, victim])
                self.rdzv_handler.update_coordinates(self.global_rank, self.coordinates)
            elif rank == prev_rank and self.num_stages > 1:
                self.log("Previous node is going to fail. Using fallback schedule")
                victim = self.prev_stage
                prev_coord = self.grid.topology().get_coord(prev_rank)
                fallback_rank = self.grid.stage_to_global(self._dec(victim))
                self.grid.topology().modify_mapping(rank=fallback_rank, **prev_coord._asdict())
                self._sched_layers.append(("prev", dict(stage_id=victim, failed_step=0, curr_step=0)))
                self._forget_rank(prev_rank)
            elif rank in self.grid.current_dp_group:
                self.log("Node in my AllReduce group is going to fail. Using fallback group")
                src = self.grid._topo.get_coord(rank=rank).data
                coord = self.grid.topology().get_coord(self.global_rank)
                except_coord = coord._replace(data=src)
                failed_rank = self.grid.topology().get_rank(**except_coord._asdict())
                self.grid.current_dp_group = self.grid.dp_fallback_groups[failed_rank]
                self._sched_layers.append(("allreduce", dict(failed_step=0, curr_step=0)))
                prev_coord = except_coord._replace(pipe=self._dec(except_coord.pipe))
                self.grid.topology().modify_mapping(self.grid.topology().get_rank(**prev_coord._asdict()),
                                                    **except_coord._asdict())
                self.grid.set_fallback_group(src)

    # ------------------------------------------------------------------ train_batch
    def train_batch(self, data_iter=None, debug=False, mem_status=False, mem_log=False):
        """Run one optimizer step over ``gradient_accumulation_steps`` micro-batches.  Returns
        the mean micro-batch loss on the rank that owns the last stage, 0 elsewhere."""
        if self._main_stream is None:
            return self._train_batch(data_iter, debug, mem_status, mem_log)
        # the step runs on the engine's high-priority stream, fenced on both sides against the
        # caller's stream (inputs produced there before the call, the returned loss used there after)
        caller = torch.cuda.current_stream(self.device)
        self._main_stream.wait_stream(caller)
        with torch.cuda.stream(self._main_stream):
            out = self._train_batch(data_iter, debug, mem_status, mem_log)
        caller.wait_stream(self._main_stream)
        if torch.is_tensor(out):
            out.record_stream(caller)
        return out

    def _train_batch(self, data_iter=None, debug=False, mem_status=False, mem_log=False):
        global should_stop
        self.rdzv_handler.write("/rdzv/cluster_status", "train")
        if should_stop:
            self.log("------- EXITING")
            self.announce_preemption()
            should_stop = False
        failures = json.loads(_decode(self.global_store.get("failures")))
        if not torch.is_grad_enabled():
            raise RuntimeError("train_batch() requires gradients enabled. Use eval_batch() instead.")
        if data_iter is not None:
            self.set_dataiterator(data_iter)
        self.module.train()
        self.total_loss = None
        self._compute_loss = True
        if not self.join and self.rdzv_handler.should_reconfigure(self.global_steps, failures):
            self._reconfigure(failures)
            failures = {}
        self.check_preemptions(failures)
        self.join = False

        t_start = time.time()
        steps = self._materialize_sched()
        status = self._exec_schedule(steps, debug=debug)
        if status is not None:
            self._handle_detected_failure(status)
            steps = self._materialize_sched()
            status = self._exec_schedule(steps, debug=debug)
            if status is not None:
                raise Exception(status[1])
            # the redo window only applies to the batch in which the failure was seen
            kind, kw = self._sched_layers[-1]
            kw["failed_step"], kw["curr_step"] = 0, 0

        self._rc_pump(everything=True)
        self.agg_train_loss = self._aggregate_total_loss()
        self.transport.end_step()
        elapsed = time.time() - t_start
        self.timers["train_batch_s"] = elapsed
        if self.global_steps % self.steps_per_print() == 0 and self.global_rank == 0 and not os.environ.get("BAMBOO_QUIET"):
            loss = float(self.agg_train_loss) if torch.is_tensor(self.agg_train_loss) else self.agg_train_loss
            print(f"steps: {self.global_steps} loss: {loss:0.4f} iter time (s): {elapsed:0.3f} "
                  f"samples/sec: {self.train_batch_size() / max(elapsed, 1e-9):0.3f}", flush=True)
        self._clean_pipe_buffers()
        return self.agg_train_loss

    # ------------------------------------------------------------------ re-partitioning
    def get_model_state(self):
        """``{layer index: [params {name: fp32 tensor}, [{"exp_avg": t, "exp_avg_sq": t}, ...]]}`` of
        every stage this rank owns: views into the arenas (reference ``get_model_state``,
        ``pipe/engine.py:565-572``, which hands out per-layer ``state_dict`` and optimizer state)."""
        from .checkpoint import _named_slices
        state = {}
        for sid in self.stage_ids:
            arena = self.arenas[sid]
            if self.native:
                self._join_wgrad_stream()
            for name, off, n, shape in _named_slices(self, arena, sid):
                layer_key, pname = name.split(".", 1)
                if not layer_key.isdigit():
                    continue                               # tied modules keep their own copy on every stage
                entry = state.setdefault(int(layer_key), [collections.OrderedDict(), []])
                entry[0][pname] = arena.master[off:off + n].view(shape)
                entry[1].append({"exp_avg": arena.exp_avg[off:off + n].view(shape),
                                 "exp_avg_sq": arena.exp_avg_sq[off:off + n].view(shape)})
        return state

    def _load_model_state(self, state, stage_ids=None):
        """Fill the arenas of the given stages (default: the owned ones) from per-layer state."""
        from .checkpoint import _named_slices
        loaded = set()
        with torch.no_grad():
            for sid in (self.stage_ids if stage_ids is None else stage_ids):
                arena = self.arenas[sid]
                seen = collections.Counter()
                for name, off, n, shape in _named_slices(self, arena, sid):
                    layer_key, pname = name.split(".", 1)
                    if not layer_key.isdigit() or int(layer_key) not in state:
                        continue
                    params, moments = state[int(layer_key)]
                    k = seen[layer_key]
                    seen[layer_key] += 1
                    arena.master[off:off + n].copy_(params[pname].reshape(-1))
                    if arena.exp_avg is not None and k < len(moments):
                        arena.exp_avg[off:off + n].copy_(moments[k]["exp_avg"].reshape(-1))
                        arena.exp_avg_sq[off:off + n].copy_(moments[k]["exp_avg_sq"].reshape(-1))
                    loaded.add(int(layer_key))
                arena.refresh_lp()
                arena.step_count = self.global_steps
        return loaded

    def _join_from_previous(self, decision, prev_state):
        from . import reconfigure as R
        from .checkpoint import _named_slices
        self.join = True
        self.global_steps = self.rdzv_handler.get_current_step()
        prev_stages = max(s for info in decision for _, s in info.previous_coordinates) + 1
        if prev_stages == self.num_stages:
            old_parts = list(self.module.parts)
        else:
            old_parts = self.module.get_new_partition(prev_stages)
        recv = R.get_recv_decisions(old_parts, self.module.parts, decision)
        send = R.get_send_decisions(recv)
        shapes = {}
        for name, off, n, shape in _named_slices(self, self.arenas[self.stage_id], self.stage_id):
            layer_key, pname = name.split(".", 1)
            if layer_key.isdigit():
                shapes.setdefault(int(layer_key), collections.OrderedDict())[pname] = tuple(shape)
        t0 = time.time()
        received = R.transfer_layers(self.dist, self.global_rank, self.world_size, recv, send, prev_state, shapes,
                                     device=self.device)
        state = dict(received)
        state.update(prev_state)                      # what this rank already held wins, like the reference
        need = set(range(self.module.parts[self.stage_id], self.module.parts[self.stage_id + 1])) & set(shapes)
        loaded = self._load_model_state(state, [self.stage_id])
        missing = need - loaded
        if missing:
            raise PipelineError(f"re-partition left layers {sorted(missing)} of stage {self.stage_id} without state")
        self.timers["layer_transfer_s"] = time.time() - t0
        self.log(f"joined at step {self.global_steps}: received layers {sorted(received)} "
                 f"in {self.timers['layer_transfer_s']:.3f} s")
        # shadow copies restart from their owners' state
        self._sync_shadow_state()

    def _layer_shapes(self, layers):
        """``{layer index: {parameter name: shape}}`` of arbitrary pipeline layers, from the layer specs."""
        from .module import LayerSpec
        shapes = {}
        for idx in sorted(layers):
            spec = self.module._layer_specs[idx]
            mod = spec.build() if isinstance(spec, LayerSpec) else spec
            if isinstance(mod, torch.nn.Module):
                named = collections.OrderedDict((n, tuple(p.shape)) for n, p in mod.named_parameters() if p.requires_grad)
                if named:
                    shapes[idx] = named
        return shapes

    def _save_shadow_node_state(self, failures):
        """A member that holds two stages (it absorbed a failed neighbour) and is itself announced to leave at
        this step carries state nobody else has: the stage it took over is no longer shadowed.  Before it goes,
        its layers and Adam moments move to the first member that stays, and that member's seats of the round
        that is ending are extended, so that the re-partition plan of the next round finds the layers there
        (reference ``save_shadow_node_state``, ``pipe/engine.py:660-727``).  Every member calls this with the
        same ``failures`` and derives the same plan; returns what this member received."""
        from . import reconfigure as R
        recv_decisions, send_decisions, seat_updates = {}, {}, []
        for fail_rank, at_step in failures.items():
            if at_step != self.global_steps:
                continue
            prev = self.rdzv_handler.get_previous_state()
            coords = self.rdzv_handler.get_rank_coordinates_for_version(prev, prev["version"])
            leaving = coords.get(str(fail_rank), [])
            if len(leaving) != 2:
                continue
            staying = [int(r) for r in coords
                       if str(r) not in failures and _decode(self.global_store.get(str(r))) == "0"]
            if not staying:
                continue
            send_node, recv_node = int(fail_rank), staying[0]
            held = [s for _, s in coords.get(str(recv_node), [])]
            stages = [s for _, s in leaving if s not in held]
            if not stages:
                continue
            layers = set(range(self.module.parts[min(stages)], self.module.parts[max(stages) + 1]))
            recv_decisions.setdefault(recv_node, {})[send_node] = layers
            send_decisions.setdefault(send_node, {})[recv_node] = layers
            if self.global_rank == recv_node:            # one writer: the update compares on the key's index
                extended = [list(c) for c in coords[str(recv_node)]] + [[leaving[0][0], s] for s in stages]
                seat_updates.append((prev["version"], recv_node, extended))
        if not recv_decisions:
            return {}
        incoming = set().union(*recv_decisions.get(self.global_rank, {}).values()) if self.global_rank in recv_decisions else set()
        t0 = time.time()
        received = R.transfer_layers(self.dist, self.global_rank, self.world_size, recv_decisions, send_decisions,
                                     self.get_model_state(), self._layer_shapes(incoming), device=self.device)
        # The seats are extended only now: the plan above is derived from the seats as they were, by every member
        # on its own, and a sender that read them after the receiver's update would find nothing left to hand over
        # and leave without sending.  The layers having arrived, the sender has made its plan; and this member joins
        # the next rendezvous after the update, so the re-partition plan of the next round sees it.
        for version, node, extended in seat_updates:
            self.rdzv_handler.update_coordinates_for_version(version, node, extended)
        if received:
            self.log(f"took over layers {sorted(received)} of a leaving member in {time.time() - t0:.3f} s")
        return received

    def _reconfigure(self, failures):
        """The rendezvous decided to re-form the cluster at this step (a member holding two stages
        is about to leave, or waiting members make another pipeline): re-join, rebuild the
        process group and the pipeline module for the new grid, move layers to their new owners
        and continue from the same optimisation state (reference: ``pipe/engine.py:1129-1164``,
        ``reconfigure_cluster`` ``:630-658``)."""
        import torch.distributed as tdist
        from .topology import PipeDataParallelTopology
        received = self._save_shadow_node_state(failures)
        if failures.get(str(self.global_rank), -1) == self.global_steps:
            self.log("We are reconfiguring and I will die soon anyway. I'm leaving")
            self.global_store.set(str(self.global_rank), "1")
            self.transport.close()
            sys.exit(13)
        state = self.get_model_state()
        state = {k: [collections.OrderedDict((n, t.clone()) for n, t in v[0].items()),
                     [{kk: tt.clone() for kk, tt in m.items()} for m in v[1]]] for k, v in state.items()}
        state.update(received)
        self.log(f"Triggered a reconfiguration on global step {self.global_steps}")
        store, rank, world, num_pipelines, num_stages, decision = self.rdzv_handler.next_rendezvous(self.global_rank)
        for info in decision:
            if info.rank == rank and len(info.active_coordinates) == 0:
                self.log("-------- I'M LEAVING!!")
                sys.exit(125)
        self.rdzv_handler.write("/rdzv/cluster_status", "init")
        self.rdzv_handler.write("/rdzv/last_reconfig", self.global_steps)
        self.transport.close()
        backend = tdist.get_backend()
        tdist.destroy_process_group()
        tdist.init_process_group(backend, store=store, rank=rank, world_size=world)
        # the process group holds the store through its C++ base only; the Python object (whose
        # methods it calls back) has to be kept alive on this side
        _live_stores.append(store)
        old = self.module
        topo = PipeDataParallelTopology(num_pp=num_stages, num_dp=num_pipelines, custom_mapping=decision)
        model = PipelineModule(layers=old._layer_specs, loss_fn=old.loss_fn, topology=topo,
                               partition_method=old.partition_method,
                               activation_checkpoint_interval=old.activation_checkpoint_interval, device=self.device)
        keep = (self.data_iterator, self.training_dataloader, self.batch_fn, self.rdzv_handler)
        args = dict(self._init_args)
        cfg = args.pop("config")
        raw = cfg._raw if isinstance(cfg, PipeConfig) else cfg
        self.__init__(model, PipeConfig(raw, num_pipelines), rdzv_handler=keep[3], prev_state=state, **args)
        self.data_iterator, self.training_dataloader, self.batch_fn = keep[:3]

    def _handle_detected_failure(self, status):
        """A neighbour stopped answering in the middle of a batch (``status`` = (step index,
        exception)).  Agree on the earliest failed step through the store, switch to the
        failover schedule with a redo window and run the batch again."""
        step_idx, exc = status
        self.rdzv_handler.write("/rdzv/last_reconfig", self.global_steps)
        if (isinstance(exc, PrevStageException) and self.num_stages == 2 and self.next_stage not in self.stage_ids
                and self.next_stage in self.param_buffers):
            # two-stage ring: the silent predecessor is also the successor whose shadow lives here
            exc = NextStageException(str(exc))
        if isinstance(exc, NextStageException):
            victim = self.next_stage
            # the other rank that talks to the victim: the owner of the stage after it
            other = self._stage_rank(self._inc(victim)) if victim != self.num_stages - 1 else None
            victim_rank = self._promote_next_stage()
            failed_step = self._agree_failed_step(victim_rank, step_idx, other)
            self._sched_layers.append(("next", dict(stage_id=victim, failed_step=failed_step, curr_step=step_idx)))
        elif isinstance(exc, PrevStageException):
            victim = self.prev_stage
            prev_rank = self.grid.stage_to_global(victim)
            prev_coord = self.grid.topology().get_coord(prev_rank)
            fallback_rank = self.grid.stage_to_global(self._dec(victim))
            self.grid.topology().modify_mapping(rank=fallback_rank, **prev_coord._asdict())
            # the other rank that talks to the victim: the owner of the stage before it
            failed_step = self._agree_failed_step(prev_rank, step_idx, fallback_rank if victim != 0 else None)
            self._sched_layers.append(("prev", dict(stage_id=victim, failed_step=failed_step, curr_step=step_idx)))
            self._forget_rank(prev_rank)
        elif isinstance(exc, AllReduceException):
            src = exc.src
            coord = self.grid.topology().get_coord(self.global_rank)
            except_coord = coord._replace(data=src)
            failed_rank = self.grid.topology().get_rank(**except_coord._asdict())
            self.grid.current_dp_group = self.grid.dp_fallback_groups[failed_rank]
            if except_coord.pipe == 0:
                raise NotImplementedError("First stage exception can not be handled now")
            self._sched_layers.append(("allreduce", dict(failed_step=step_idx, curr_step=0)))
            prev_coord = except_coord._replace(pipe=except_coord.pipe - 1)
            self.grid.topology().modify_mapping(self.grid.topology().get_rank(**prev_coord._asdict()),
                                                **except_coord._asdict())
            self.grid.set_fallback_group(src)
        else:
            raise Exception(exc)

    def _agree_failed_step(self, victim_rank, my_step, other_rank):
        """Both neighbours of a dead middle stage notice it, possibly at different schedule steps;
        the redo window starts at the earlier one.  Every detector publishes its own step under a
        key of its own (no shared read-modify-write, so concurrent detections cannot lose an
        entry) and waits - bounded - for the other detector's key.  The result always includes
        this rank's own step."""
        self.global_store.set(f"fail-step-{victim_rank}-{self.global_rank}", str(int(my_step)))
        if other_rank is None or other_rank == self.global_rank:
            return my_step
        key = f"fail-step-{victim_rank}-{other_rank}"
        deadline = time.time() + self._config.p2p_timeout_s
        while time.time() < deadline:
            if self.global_store.check([key]):
                return min(my_step, int(_decode(self.global_store.get(key))))
            time.sleep(0.01)
        return my_step

    def _aggregate_total_loss(self):
        if self.is_last_stage() and self.total_loss is not None:
            return (self.total_loss / self.micro_batches).clone().detach()
        return 0

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, save_dir, tag=None, client_state={}, save_latest=True):
        """Per-layer model files plus one state file per stage (every rank calls it); same
        signature and on-disk layout as ``DeepSpeedEngine.save_checkpoint``
        (``deepspeed/runtime/engine.py:2197-2253``)."""
        from . import checkpoint
        return checkpoint.save_checkpoint(self, save_dir, tag, client_state, save_latest)

    def load_checkpoint(self, load_dir, tag=None, load_module_strict=True, load_optimizer_states=True,
                        load_lr_scheduler_states=True):
        """Returns ``(path, client_state)`` like ``DeepSpeedEngine.load_checkpoint``
        (``deepspeed/runtime/engine.py:1925-1990``); the stage partition may differ from the
        one that wrote the checkpoint."""
        from . import checkpoint
        return checkpoint.load_checkpoint(self, load_dir, tag, load_optimizer_states, load_lr_scheduler_states)

    def eval_batch(self, *a, **k):
        raise PipelineError("eval_batch is outside the training-step path of this implementation")

    def forward(self, *a, **k):
        raise PipelineError("Only train_batch() is accessible in pipeline mode.")

    def backward(self, *a, **k):
        raise PipelineError("Only train_batch() is accessible in pipeline mode.")

    def step(self, *a, **k):
        raise PipelineError("Only train_batch() is accessible in pipeline mode.")

    # ------------------------------------------------------------------ executors
    def _exec_load_micro_batch(self, buffer_id):
        if self.pipe_buffers["label"][buffer_id] is not None or self.pipe_buffers["data"][buffer_id] is not None:
            return
        batch = self._next_batch()
        if self._shadow_ctx and self.rc_stream is not None:
            # a load that only the redundant forward consumes: its copies go to that stream, so the
            # forward is ordered behind them without waiting for the main stream's queued work
            with torch.cuda.stream(self.rc_stream):
                return self._place_micro_batch(batch, buffer_id)
        return self._place_micro_batch(batch, buffer_id)

    def _place_micro_batch(self, batch, buffer_id):
        if 0 in self.stage_ids or 0 in self.r_stage_ids:
            x = batch[0]
            if torch.is_tensor(x):
                x = x.to(self.device, non_blocking=True).detach()
                x.requires_grad = x.is_floating_point()
            else:
                x = tuple(t.to(self.device, non_blocking=True).detach() for t in x)
            self.pipe_buffers["data"][buffer_id] = x
        last = self.num_stages - 1
        if last in self.stage_ids or last in self.r_stage_ids:
            y = batch[1]
            if torch.is_tensor(y):
                y = y.to(self.device, non_blocking=True)
            elif isinstance(y, (tuple, list)):
                y = tuple(t.to(self.device, non_blocking=True).detach() for t in y)
            self.pipe_buffers["label"][buffer_id] = y

    def _is_shadow(self, stage_id):
        return stage_id in self.r_stage_ids and stage_id not in self.stage_ids

    def _exec_forward_pass(self, buffer_id, stage_id):
        out_key = f"output_{stage_id}"
        if stage_id != self.num_stages - 1 and self.pipe_buffers[out_key][buffer_id] is not None:
            return
        in_key = "data" if stage_id == 0 else f"input_{stage_id}"
        inputs = self.pipe_buffers[in_key][buffer_id]
        shadow = self._is_shadow(stage_id)
        if shadow and self.rc_stream is not None:
            # redundant computation: off the critical path, on the low-priority stream.  Its load
            # and its input hand-off were issued on that stream too (see _exec_load_micro_batch,
            # _exec_recv_activations), behind the event of this rank's own forward of the same
            # micro-batch - not behind the present end of the main stream, which holds later work
            if not self._shadow_ctx:
                # issued outside a redundant-work group (its inputs were produced on the main stream)
                self.rc_stream.wait_event(torch.cuda.current_stream().record_event())
            # the redundant forward may run many micro-batches later than it was issued: its
            # inputs must not go back to the main stream's allocator before it has read them
            for t in (inputs if isinstance(inputs, tuple) else (inputs,)):
                if torch.is_tensor(t) and t.is_cuda:
                    t.record_stream(self.rc_stream)
            label = self.pipe_buffers["label"][buffer_id] if stage_id == self.num_stages - 1 else None
            if torch.is_tensor(label) and label.is_cuda:
                label.record_stream(self.rc_stream)
            if self._config.rc_deferred and hasattr(self.transport, "idle_hook"):
                # issued layer by layer whenever the host finds the main stream idle (waiting for a
                # neighbour's message), the rest at the end of the batch: see _rc_pump
                self._rc_queue.append(self._rc_forward_chunks(inputs, label, buffer_id, stage_id))
            else:
                for _ in self._rc_forward_chunks(inputs, label, buffer_id, stage_id):
                    pass
        else:
            self._forward_stage(inputs, buffer_id, stage_id, retain=(not shadow) or self._config.rc_retain_graph)
            if self.rc_stream is not None and not shadow and self._inc(stage_id) in self.r_stage_ids:
                self._fwd_done[(stage_id, buffer_id)] = torch.cuda.current_stream().record_event()
        if stage_id == 0:
            self.pipe_buffers["data"][buffer_id] = None
        if stage_id == self.num_stages - 1:
            self.pipe_buffers["label"][buffer_id] = None

    def _rc_forward_chunks(self, inputs, label, buffer_id, stage_id):
        """A redundant forward as a generator: every ``next()`` issues one layer of the shadow
        stage on the redundant-computation stream; the last one stores the stage's output (or its
        loss).  Issuing it in pieces lets the host hand the GPU redundant work only while the own
        stage has nothing to run."""
        from . import lib as _lib
        retain = self._config.rc_retain_graph
        last = stage_id == self.num_stages - 1
        budget = -1 if self._config.rc_short_ctas else self._config.rc_max_ctas
        x = tuple(t.clone() for t in inputs) if isinstance(inputs, tuple) else inputs
        for f in self.module.func_buckets[stage_id]:
            with torch.cuda.stream(self.rc_stream), (torch.enable_grad() if retain else torch.no_grad()):
                _lib.GEMM_MAX_CTAS = budget     # SM budget of the redundant GEMMs (bb_gemm_desc.max_ctas)
                try:
                    x = f(x)
                finally:
                    _lib.GEMM_MAX_CTAS = 0
            yield
        with torch.cuda.stream(self.rc_stream), (torch.enable_grad() if retain else torch.no_grad()):
            if not last:
                self.pipe_buffers[f"output_{stage_id}"][buffer_id] = x
            else:
                self._losses[(buffer_id, stage_id)] = (self.loss_model(x, label)
                                                       if self._compute_loss and self.loss_model is not None else x)
            self._rc_event = self.rc_stream.record_event()
        yield

    def _rc_pump(self, everything=False, idle_for_s=0.0):
        """Issue one pending chunk of redundant work (or all of it).  Called by the transport while
        the host waits for a message and the main stream has drained, by the end of the batch and
        before anything that needs the redundant results."""
        if not everything:
            # a bounded number of chunks ahead of the GPU: whatever is already queued on the redundant
            # stream competes with the own stage's kernels once the awaited message arrives
            while self._rc_inflight and self._rc_inflight[0].query():
                self._rc_inflight.popleft()
            # a wait that has already lasted long is a pipeline bubble, not a hand-over gap: deeper queue
            allowed = self._config.rc_chunks_in_flight
            if idle_for_s > 0.0005:
                allowed = min(allowed + int(idle_for_s / 0.0005), 4 * allowed)
            if len(self._rc_inflight) >= allowed:
                return bool(self._rc_queue)
        while self._rc_queue:
            try:
                next(self._rc_queue[0])
            except StopIteration:
                self._rc_queue.popleft()
                continue
            self.instr_counts["rc_chunks_flushed" if everything else "rc_chunks_in_idle_time"] += 1
            if not everything:
                self._rc_inflight.append(self.rc_stream.record_event())
                return True
        return False

    def _forward_stage(self, inputs, buffer_id, stage_id, retain=True):
        ctx = torch.enable_grad() if retain else torch.no_grad()
        with ctx:
            x = tuple(t.clone() for t in inputs) if isinstance(inputs, tuple) else inputs
            outputs = self.module(x, stage_id=stage_id)
            if stage_id != self.num_stages - 1:
                self.pipe_buffers[f"output_{stage_id}"][buffer_id] = outputs
                return
            if self._compute_loss and self.loss_model is not None:
                loss = self.loss_model(outputs, self.pipe_buffers["label"][buffer_id])
            else:
                loss = outputs
        self._losses[(buffer_id, stage_id)] = loss
        if not self._is_shadow(stage_id):
            self.loss = loss
            if self.total_loss is None:
                self.total_loss = torch.zeros_like(loss.detach())
            self.total_loss += loss.detach()

    def _exec_backward_pass(self, buffer_id, stage_id):
        if stage_id == self.num_stages - 1:
            loss = self._losses.pop((buffer_id, stage_id), self.loss)
            # gradient accumulation: each micro-batch contributes loss / GAS
            (loss / self.micro_batches).backward()
        else:
            outputs = self.pipe_buffers[f"output_{stage_id}"][buffer_id]
            grads = self.grad_layer
            if isinstance(outputs, tuple):
                outs = [t for t in outputs if t.is_floating_point()]
                torch.autograd.backward(tensors=outs, grad_tensors=grads)
            else:
                torch.autograd.backward(tensors=(outputs,), grad_tensors=(grads,))
            if not self.eager_recovery and self._inc(stage_id) in self.r_stage_ids:
                # kept so the successor's forward can be replayed if it dies mid-batch
                self.pipe_buffers[f"output_{stage_id}"][buffer_id] = outputs.detach()
            else:
                self.pipe_buffers[f"output_{stage_id}"][buffer_id] = None
        self.arenas[stage_id].fold_autograd_grads()

    def _next_seq(self, kind, peer):
        self._seq[(kind, peer)] += 1
        return self._seq[(kind, peer)]

    def _exec_send_activations(self, buffer_id, stage_id):
        if self._inc(stage_id) in self.stage_ids:
            return
        dst = self._stage_rank(self.next_stage)
        try:
            if buffer_id >= 0:
                out = self.pipe_buffers[f"output_{stage_id}"][buffer_id]
                self.transport.send(out, dst, ACT, buffer_id, self._next_seq("sa", dst))
            else:
                self.transport.send_ping(dst, self._next_seq("sp", dst))
        except PeerTimeout as e:
            self.global_store.set(str(dst), "1")
            raise NextStageException(e)

    def _exec_recv_activations(self, buffer_id, stage_id):
        if self._dec(stage_id) in self.stage_ids or (self.eager_recovery and stage_id in self.r_stage_ids):
            if buffer_id >= 0 and self.pipe_buffers[f"input_{stage_id}"][buffer_id] is None:
                src = self.pipe_buffers[f"output_{self._dec(stage_id)}"][buffer_id]
                if self._shadow_ctx and self.rc_stream is not None and self._is_shadow(stage_id):
                    # hand-off to the redundant forward: the copy runs on its stream, as soon as this
                    # rank's own forward of the micro-batch has produced the source
                    ready = self._fwd_done.pop((self._dec(stage_id), buffer_id), None)
                    if ready is None:
                        ready = torch.cuda.current_stream().record_event()
                    self.rc_stream.wait_event(ready)
                    with torch.cuda.stream(self.rc_stream):
                        t = src.detach().clone()
                    src.record_stream(self.rc_stream)
                else:
                    t = src.detach().clone()
                t.requires_grad = True
                self.pipe_buffers[f"input_{stage_id}"][buffer_id] = t
            return
        src = self._stage_rank(self.prev_stage)
        try:
            if buffer_id >= 0:
                t = self.transport.recv(src, ACT, buffer_id, self._next_seq("ra", src))
                t.requires_grad = t.is_floating_point()
                self.pipe_buffers[f"input_{stage_id}"][buffer_id] = t
            else:
                self.transport.recv_ping(src, self._next_seq("rp", src))
        except PeerTimeout as e:
            self.global_store.set(str(src), "1")
            raise PrevStageException(e)

    def _exec_send_grads(self, buffer_id, stage_id):
        if self._dec(stage_id) in self.stage_ids:
            return
        key = f"input_grad_{stage_id}"
        stash = self.pipe_buffers.get(key)
        replay = stash is not None and stash[buffer_id] is not None
        if replay:
            grad = stash[buffer_id]
        else:
            inp = self.pipe_buffers[f"input_{stage_id}"][buffer_id]
            assert inp.grad is not None
            grad = inp.grad
        dst = self._stage_rank(self.prev_stage)
        try:
            self.transport.send(grad, dst, GRAD, buffer_id, self._next_seq("sg", dst))
        except PeerTimeout as e:
            self.global_store.set(str(dst), "1")
            raise PrevStageException(e)
        if self.redundancy_level > 0 and stage_id != 0:
            # keep the sent gradient until the end of the batch: if the receiver dies, whoever
            # takes over its stage asks for it again
            if key in self.pipe_buffers:
                self.pipe_buffers[key][buffer_id] = None if replay else grad.detach()
            self.pipe_buffers[f"input_{stage_id}"][buffer_id] = None
        else:
            self.pipe_buffers[f"input_{stage_id}"][buffer_id] = None

    def _exec_recv_grads(self, buffer_id, stage_id):
        if self._inc(stage_id) in self.stage_ids:
            self.grad_layer = self.pipe_buffers[f"input_{self._inc(stage_id)}"][buffer_id].grad
            return
        src = self._stage_rank(self.next_stage)
        try:
            self.grad_layer = self.transport.recv(src, GRAD, buffer_id, self._next_seq("rg", src))
        except PeerTimeout as e:
            self.global_store.set(str(src), "1")
            raise NextStageException(e)

    def _join_wgrad_stream(self):
        """Weight gradients are produced on a side stream by the sm_100a layers; everything that
        reads the gradient arena (all-reduce, optimizer, gradient capture) waits for it first."""
        if self.native:
            from .layers import wgrad_sync
            wgrad_sync(self.device)

    def _exec_reduce_grads(self, stage_id):
        """Average the stage's gradients over its data-parallel column: one all-reduce over
        the flat fp32 gradient arena, 1/dp folded into the optimizer kernel."""
        self._join_wgrad_stream()
        self._reduce_scale = getattr(self, "_reduce_scale", {})
        self._reduce_scale[stage_id] = 1.0
        if self.dp_world_size > 1 and self.dist is not None:
            pg = self.grid.get_data_parallel_group(stage_id)
            self.dist.all_reduce(self.arenas[stage_id].grad, group=pg)
            self._reduce_scale[stage_id] = 1.0 / self.dp_world_size

    def _exec_reduce_tied_grads(self):
        return

    def _exec_optimizer_step(self, lr_kwargs=None):
        self._join_wgrad_stream()
        scales = getattr(self, "_reduce_scale", {})
        if getattr(self, "capture_grads", False):
            self.last_grads = {sid: self.arenas[sid].grad.clone() * scales.get(sid, 1.0) for sid in self.stage_ids}
        for sid in self.stage_ids:
            a = self._adam
            self.arenas[sid].adam_step(lr=a["lr"], beta1=a["beta1"], beta2=a["beta2"], eps=a["eps"],
                                       weight_decay=a["weight_decay"], adam_w_mode=a["adam_w_mode"],
                                       bias_correction=a["bias_correction"], grad_scale=scales.get(sid, 1.0))
        if self.lr_scheduler is not None:
            self.lr_scheduler.step(**(lr_kwargs or {}))
        self.global_steps += 1
        self.global_samples += self.train_batch_size()
        self._sync_shadow_state()

    def _sync_shadow_state(self):
        """End of step: every live stage ships (weights, exp_avg, exp_avg_sq) to the rank that
        shadows it, and the shadow's working copy is refreshed."""
        # redundant forwards of this batch read the shadow's working copy: all of them are issued
        # before the refresh that follows on their stream
        self._rc_pump(everything=True)
        if self.redundancy_level == 0 or self.num_stages == 1 or not self._config.shadow_sync:
            return
        # after a failover the ring is broken at the dead rank: only intact pairs keep syncing
        send_to = self._shadow_holder_rank
        tensors_out = self.arenas[self.stage_id].state_tensors() if send_to is not None else []
        recv_from, tensors_in = None, []
        for sid in self.r_stage_ids:
            if sid in self.param_buffers and self._shadow_source_rank.get(sid) is not None:
                recv_from, tensors_in = self._shadow_source_rank[sid], self.param_buffers[sid].state_tensors()
        if send_to is None and recv_from is None:
            return
        if self.rc_stream is not None and self._lp_refreshed is not None:
            # the previous refresh (on the RC stream) reads the master copy this transfer overwrites
            torch.cuda.current_stream().wait_event(self._lp_refreshed)
            self._lp_refreshed = None
        try:
            self.transport.exchange_state(send_to, tensors_out, recv_from, tensors_in, self.global_steps)
        except PeerTimeout as e:
            # Transports deliver the three pieces all-or-nothing, so after a failed transfer the
            # shadow is whole but one step old; it is marked so that a later promotion is refused
            # rather than silently continued from stale state.  A failed send needs nothing here:
            # the holder of that shadow records the same on its side.
            if recv_from is not None and e.peer == recv_from:
                for sid in self.r_stage_ids:
                    if sid in self.param_buffers:
                        self._shadow_valid[sid] = False
                self.log(f"shadow state of stage(s) {self.r_stage_ids} not refreshed: {e}")
            return
        if recv_from is not None:
            for sid in self.r_stage_ids:
                if sid in self.param_buffers:
                    if self.rc_stream is not None:
                        # Redundant forwards of this step may still be queued on the low-priority
                        # stream and read the shadow's bf16 working copy; the fp32 state that just
                        # arrived is not read by them.  So the working copy is refreshed ON that
                        # stream, behind them, and the main stream never waits for redundant work.
                        self.rc_stream.wait_event(torch.cuda.current_stream().record_event())
                        with torch.cuda.stream(self.rc_stream):
                            self.param_buffers[sid].refresh_lp()
                            self._lp_refreshed = self.rc_stream.record_event()
                    else:
                        self.param_buffers[sid].refresh_lp()
                    self.param_buffers[sid].step_count = self.arenas[self.stage_id].step_count

    def _alive(self, rank):
        try:
            return _decode(self.global_store.get(str(rank))) != "1"
        except Exception:
            return True

    def _sends_before_redundant_work(self, step_cmds):
        """Execution order inside one step of an eager-RC stream.  The stream puts the successor's
        queued [load, receive, forward] in front of this stage's own instructions; issuing those
        ~50 launches takes the host a couple of milliseconds, during which this stage's finished
        activation (or gradient) would sit unsent and the neighbour would wait for it.  The sends
        of the step are therefore issued first, then the redundant work, then the rest in its
        emitted order.  (Sends are non-blocking store kernels; the emitted stream is unchanged.)"""
        last = -1
        for i, c in enumerate(step_cmds):
            sid = c.kwargs.get("stage_id") if hasattr(c, "kwargs") else None
            if sid is not None and sid in self.r_stage_ids and sid not in self.stage_ids \
                    and type(c) in (schedule.ForwardPass, schedule.RecvActivation):
                last = i
        if last < 0:
            return step_cmds, ()
        shadow, own = step_cmds[:last + 1], step_cmds[last + 1:]
        sends = [c for c in own if type(c) in (schedule.SendActivation, schedule.SendGrad)]
        rest = [c for c in own if type(c) not in (schedule.SendActivation, schedule.SendGrad)]
        return sends + shadow + rest, {id(c) for c in shadow}

    _INSTRUCTION_MAP = {
        schedule.OptimizerStep: _exec_optimizer_step,
        schedule.ReduceGrads: _exec_reduce_grads,
        schedule.ReduceTiedGrads: _exec_reduce_tied_grads,
        schedule.LoadMicroBatch: _exec_load_micro_batch,
        schedule.ForwardPass: _exec_forward_pass,
        schedule.BackwardPass: _exec_backward_pass,
        schedule.SendActivation: _exec_send_activations,
        schedule.RecvActivation: _exec_recv_activations,
        schedule.SendGrad: _exec_send_grads,
        schedule.RecvGrad: _exec_recv_grads,
    }

    def _exec_schedule(self, pipe_schedule, start_step=0, debug=False) -> Optional[Tuple[int, Exception]]:
        """Run the instruction stream; returns ``None`` or ``(step index, exception)``.  Errors
        are handled per step: communication comes before computation inside a step, so a step
        that failed in communication can be executed again."""
        steps = pipe_schedule if isinstance(pipe_schedule, list) else list(pipe_schedule)
        self._reserve_pipe_buffers(self.micro_batches)
        self.fwd_outputs = []
        for i, step_cmds in enumerate(steps):
            if i < start_step:
                continue
            if debug:
                print(f"[DEBUG Pipeline] Instructions in step {i}:", *step_cmds, sep=" ")
            if any(type(c) is schedule.ReduceGrads for c in step_cmds) and self.dp_world_size > 1:
                for rank in self.grid.current_dp_group:
                    if not self._alive(rank):
                        dp = self.grid._topo.get_coord(rank).data
                        msg = f"RANK {rank} FROM PIPELINE {dp} IN ALL-REDUCE GROUP FAILED. USING FALLBACK"
                        return i, AllReduceException(dp, f"{schedule.ReduceGrads}: {msg}")
            if any(type(c) is schedule.OptimizerStep for c in step_cmds):
                # The merged failover stream carries the dead stage's ReduceGrads *after* OptimizerStep
                # (reference quirk, schedule.py:417-421).  The stream is kept as emitted; the executor
                # runs every reduction of the step before the optimizer so that the promoted stage
                # steps on averaged gradients.
                reduces = [c for c in step_cmds if type(c) is schedule.ReduceGrads]
                rest = [c for c in step_cmds if type(c) is not schedule.ReduceGrads]
                k = next(i for i, c in enumerate(rest) if type(c) is schedule.OptimizerStep)
                step_cmds = rest[:k] + reduces + rest[k:]
            shadow_ids = ()
            if self.eager_recovery:
                step_cmds, shadow_ids = self._sends_before_redundant_work(step_cmds)
            for cmd in step_cmds:
                self._shadow_ctx = id(cmd) in shadow_ids
                try:
                    fn = self._INSTRUCTION_MAP.get(type(cmd))
                    if fn is None:
                        raise RuntimeError(f"{self.__class__.__name__} does not understand instruction {cmd!r}")
                    self.instr_counts[type(cmd).__name__] += 1
                    self._exec_instr = MethodType(fn, self)
                    self._exec_instr(**cmd.kwargs)
                except (NextStageException, PrevStageException, AllReduceException) as e:
                    msg = f"{type(cmd)}: {e}"
                    err = type(e)(e.src, msg) if hasattr(e, "src") else type(e)(msg)
                    return i, err
        return None
