"""Host logic of the pipeline engine on CPU ranks (gloo): schedules executed end to end,
redundant computation, shadow-state transfer and failover, checked against the
single-process oracle."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from oracle import gpt_ref  # noqa: E402

CFG = gpt_ref.RefConfig(layers=4, hidden=64, heads=4, ffn=128, seq=16, vocab=96)
MB, GAS, STEPS, LR = 2, 4, 5, 1e-3


def _oracle_losses():
    ref = gpt_ref.RefTrainer(CFG, seed=0, lr=LR, micro_batches=GAS)
    data = gpt_ref.synthetic_batches(CFG, MB, GAS, STEPS, seed=1)
    return [ref.train_batch(step) for step in data], ref


def _train(rank, world, store, stages, rc, eager, victim_step, victim_stage=None, ckpt_interval=0):
    """Body of one rank.  ``victim_step``: the rank of ``victim_stage`` (default: the last stage)
    announces its preemption so that it is gone from step ``victim_step`` on (None = no failure)."""
    import cpu_layers
    from bamboo_b200 import api
    from bamboo_b200.module import PipelineModule
    model = PipelineModule(cpu_layers.ref_layer_specs(CFG, 0), num_stages=stages, loss_fn=cpu_layers.ref_loss(CFG),
                           partition_method="uniform", device="cpu", activation_checkpoint_interval=ckpt_interval)
    config = {"train_micro_batch_size_per_gpu": MB, "gradient_accumulation_steps": GAS,
              "optimizer": {"type": "Adam", "params": {"lr": LR}}, "bamboo_b200": {"p2p_timeout_s": 20}}
    engine, *_ = api.initialize(model=model, config=config, redundancy_level=rc, eager_recovery=eager,
                                store=store if world > 1 else None)
    data = gpt_ref.synthetic_batches(CFG, MB, GAS, STEPS, seed=1)
    losses = []
    for step, batches in enumerate(data):
        if victim_step is not None and step == victim_step - 1 and rank == (stages - 1 if victim_stage is None else victim_stage):
            engine.announce_preemption()
        loss = engine.train_batch(data_iter=iter(batches))
        losses.append(float(loss))
    params = {sid: engine.arenas[sid].master.clone() for sid in engine.stage_ids}
    return {"losses": losses, "stage_ids": list(engine.stage_ids), "numel": {s: p.numel() for s, p in params.items()},
            "checksum": {s: float(p.double().sum()) for s, p in params.items()}, "counts": dict(engine.instr_counts)}


def test_single_stage_matches_oracle():
    want, ref = _oracle_losses()
    os.environ["BAMBOO_QUIET"] = "1"
    got = _train(0, 1, None, 1, 0, False, None)
    assert got["losses"] == pytest.approx(want, rel=1e-5)
    total = sum(float(p.detach().double().sum()) for p in ref.P.values())
    assert got["checksum"][0] == pytest.approx(total, rel=1e-6)


@pytest.mark.parametrize("interval", [1, 2])
def test_activation_checkpointing_matches_oracle(interval):
    """Recomputing every `interval` layers in the backward pass changes memory, not numbers
    (``PipelineModule.forward``, reference ``deepspeed/runtime/pipe/module.py:551-573``)."""
    want, _ = _oracle_losses()
    os.environ["BAMBOO_QUIET"] = "1"
    got = _train(0, 1, None, 1, 0, False, None, ckpt_interval=interval)
    assert got["losses"] == pytest.approx(want, rel=1e-5)


@pytest.mark.parametrize("rc,eager", [(0, False), (1, False), (1, True)])
def test_two_stage_pipeline_matches_oracle(rc, eager):
    from dist_utils import run_ranks
    want, _ = _oracle_losses()
    res = run_ranks(_train, 2, 2, rc, eager, None)
    assert res[1][0] == "ok" and res[0][0] == "ok"
    assert res[1][1]["losses"] == pytest.approx(want, rel=1e-5)
    assert res[0][1]["losses"] == [0] * STEPS          # non-last stages return 0
    if eager:
        # stage 0 ran its successor's forward once per micro-batch
        assert res[0][1]["counts"]["ForwardPass"] == 2 * GAS * STEPS


@pytest.mark.parametrize("eager", [False, True])
def test_failover_continues_the_same_trajectory(eager):
    """Stage 1 is preempted after step 3; stage 0 promotes its shadow copy and finishes the
    run alone - the losses must be those of an undisturbed run."""
    from dist_utils import run_ranks
    want, ref = _oracle_losses()
    res = run_ranks(_train, 2, 2, 1, eager, 3)
    assert res[1] == ("exit", 13)
    status, out = res[0]
    assert status == "ok"
    assert out["stage_ids"] == [0, 1]
    assert out["losses"][:3] == [0, 0, 0]
    assert out["losses"][3:] == pytest.approx(want[3:], rel=1e-5)
    total = sum(float(p.detach().double().sum()) for p in ref.P.values())
    assert sum(out["checksum"].values()) == pytest.approx(total, rel=1e-6)


@pytest.mark.parametrize("eager,victim", [(False, None), (True, None), (True, 3), (False, 1)])
def test_four_stage_pipeline(eager, victim):
    """Four stages on four CPU ranks with redundant computation; optionally one stage (the last
    one, or one in the middle whose neighbours on both sides must re-route) is preempted after
    step 2.  The survivors' losses are those of an undisturbed single-process run."""
    from dist_utils import run_ranks
    want, ref = _oracle_losses()
    res = run_ranks(_train, 4, 4, 1, eager, None if victim is None else 2, victim, timeout=300)
    last = 3 if victim != 3 else 2                    # the rank that ends up owning the last stage
    for r in range(4):
        if r == victim:
            assert res[r] == ("exit", 13)
        else:
            assert res[r][0] == "ok", res[r]
    losses = res[last][1]["losses"]
    if victim == 3:
        assert losses[:2] == [0, 0] and losses[2:] == pytest.approx(want[2:], rel=1e-5)
        assert res[2][1]["stage_ids"] == [2, 3]
    else:
        assert losses == pytest.approx(want, rel=1e-5)
    if victim == 1:
        assert res[0][1]["stage_ids"] == [0, 1]
    total = sum(float(p.detach().double().sum()) for p in ref.P.values())
    got = sum(sum(res[r][1]["checksum"].values()) for r in range(4) if r != victim)
    assert got == pytest.approx(total, rel=1e-6)


# ---------------------------------------------------------------------------------------------
# pipeline x data parallel grid (2 stages x 2 replicas on 4 CPU ranks)
def _train_grid(rank, world, store, stages, dp, rc, victim_rank, victim_step):
    import cpu_layers
    from bamboo_b200 import api
    from bamboo_b200.module import PipelineModule
    from bamboo_b200.topology import PipeDataParallelTopology
    topo = PipeDataParallelTopology(num_pp=stages, num_dp=dp)
    model = PipelineModule(cpu_layers.ref_layer_specs(CFG, 0), topology=topo, loss_fn=cpu_layers.ref_loss(CFG),
                           partition_method="uniform", device="cpu")
    config = {"train_micro_batch_size_per_gpu": MB, "gradient_accumulation_steps": GAS,
              "train_batch_size": MB * GAS * dp,
              "optimizer": {"type": "Adam", "params": {"lr": LR}}, "bamboo_b200": {"p2p_timeout_s": 20}}
    engine, *_ = api.initialize(model=model, config=config, redundancy_level=rc, store=store)
    replica = engine.grid.get_data_parallel_id()
    data = gpt_ref.synthetic_batches(CFG, MB, GAS * dp, STEPS, seed=1)
    losses = []
    for step, batches in enumerate(data):
        if victim_rank is not None and step == victim_step - 1 and rank == victim_rank:
            engine.announce_preemption()
        mine = batches[replica * GAS:(replica + 1) * GAS]        # each replica trains on its own slice
        losses.append(float(engine.train_batch(data_iter=iter(mine))))
    return {"losses": losses, "stage_ids": list(engine.stage_ids), "replica": replica,
            "checksum": {s: float(engine.arenas[s].master.double().sum()) for s in engine.stage_ids}}


def _oracle_grid(dp):
    """Data parallelism = gradient averaging = one big accumulation over all replicas' micro-batches."""
    ref = gpt_ref.RefTrainer(CFG, seed=0, lr=LR, micro_batches=GAS * dp)
    per_replica = []
    for batches in gpt_ref.synthetic_batches(CFG, MB, GAS * dp, STEPS, seed=1):
        with torch.no_grad():
            per_replica.append([sum(float(gpt_ref.forward_loss(CFG, ref.P, t, l)) for t, l in batches[r * GAS:(r + 1) * GAS]) / GAS
                                for r in range(dp)])
        ref.train_batch(batches)
    return per_replica, ref


def test_two_by_two_grid_averages_gradients_over_replicas():
    from dist_utils import run_ranks
    want, ref = _oracle_grid(2)
    res = run_ranks(_train_grid, 4, 2, 2, 0, None, None)
    for rank in (2, 3):                                           # last-stage ranks: rank = stage * dp + replica
        status, out = res[rank]
        assert status == "ok"
        assert out["losses"] == pytest.approx([w[out["replica"]] for w in want], rel=1e-5)
    total = sum(float(p.detach().double().sum()) for p in ref.P.values())
    assert res[0][1]["checksum"][0] + res[2][1]["checksum"][1] == pytest.approx(total, rel=1e-6)
    assert res[0][1]["checksum"] == res[1][1]["checksum"]        # replicas stay identical


def test_grid_failover_uses_the_fallback_data_parallel_group():
    """Rank 2 (stage 1 of replica 0) is preempted after step 3: rank 0 promotes its shadow of
    stage 1 and takes rank 2's seat in stage 1's all-reduce; rank 3 switches to the fallback group."""
    from dist_utils import run_ranks
    want, ref = _oracle_grid(2)
    res = run_ranks(_train_grid, 4, 2, 2, 1, 2, 3)
    assert res[2] == ("exit", 13)
    assert res[0][0] == "ok" and res[1][0] == "ok" and res[3][0] == "ok"
    assert res[0][1]["stage_ids"] == [0, 1]
    assert res[0][1]["losses"][3:] == pytest.approx([w[0] for w in want][3:], rel=1e-5)
    assert res[3][1]["losses"] == pytest.approx([w[1] for w in want], rel=1e-5)
    total = sum(float(p.detach().double().sum()) for p in ref.P.values())
    assert sum(res[0][1]["checksum"].values()) == pytest.approx(total, rel=1e-6)
    assert res[3][1]["checksum"][1] == pytest.approx(res[0][1]["checksum"][1], rel=1e-9)


# ---------------------------------------------------------------------------------------------
# unannounced death in the middle of a batch: detected through the transport, redo window
def _train_sudden_death(rank, world, store, die_in_step, die_at_backward):
    import cpu_layers
    from bamboo_b200 import api, engine as E
    from bamboo_b200.module import PipelineModule
    model = PipelineModule(cpu_layers.ref_layer_specs(CFG, 0), num_stages=2, loss_fn=cpu_layers.ref_loss(CFG),
                           partition_method="uniform", device="cpu")
    config = {"train_micro_batch_size_per_gpu": MB, "gradient_accumulation_steps": GAS,
              "optimizer": {"type": "Adam", "params": {"lr": LR}}, "bamboo_b200": {"p2p_timeout_s": 5}}
    engine, *_ = api.initialize(model=model, config=config, redundancy_level=1, eager_recovery=False, store=store)
    if rank == 1:
        calls = {"n": 0}
        orig = E.PipelineEngine._exec_backward_pass

        def dying_backward(self, buffer_id, stage_id):
            if self.global_steps == die_in_step:
                calls["n"] += 1
                if calls["n"] == die_at_backward:
                    os._exit(0)                  # no announcement, no clean-up: the process is just gone
            return orig(self, buffer_id, stage_id)
        E.PipelineEngine._exec_backward_pass = dying_backward
        E.PipelineEngine._INSTRUCTION_MAP[E.schedule.BackwardPass] = dying_backward
    data = gpt_ref.synthetic_batches(CFG, MB, GAS, STEPS, seed=1)
    losses = []
    for batches in data:
        losses.append(float(engine.train_batch(data_iter=iter(batches))))
    return {"losses": losses, "stage_ids": list(engine.stage_ids),
            "checksum": {s: float(engine.arenas[s].master.double().sum()) for s in engine.stage_ids}}


@pytest.mark.parametrize("die_at_backward", [1, 3])
def test_unannounced_death_mid_batch_is_recovered(die_at_backward):
    """Stage 1 vanishes during step 3 after some of its backward passes; stage 0 notices on its
    next receive, promotes its shadow, replays the dead stage's part of the batch and finishes
    the run with the oracle's losses."""
    from dist_utils import run_ranks
    want, ref = _oracle_losses()
    res = run_ranks(_train_sudden_death, 2, 3, die_at_backward)
    status, out = res[0]
    assert status == "ok", out
    assert out["stage_ids"] == [0, 1]
    assert out["losses"][3:] == pytest.approx(want[3:], rel=1e-5)
    total = sum(float(p.detach().double().sum()) for p in ref.P.values())
    assert sum(out["checksum"].values()) == pytest.approx(total, rel=1e-6)


# ---------------------------------------------------------------------------------------------
# the plumbing configuration at its stated size: 4-layer decoder, hidden 256, 4 heads, FFN 1024,
# seq 128, vocab 1024, fp32, micro-batch 4 x 4, Adam lr 1e-4, 5 steps, stage 1 preempted after
# step 3, redundant computation on; fp32 tolerance 1e-4
C1 = gpt_ref.RefConfig(layers=4, hidden=256, heads=4, ffn=1024, seq=128, vocab=1024)
C1_MB, C1_GAS, C1_STEPS, C1_LR = 4, 4, 5, 1e-4


def _train_c1(rank, world, store, eager):
    import cpu_layers
    from bamboo_b200 import api
    from bamboo_b200.module import PipelineModule
    model = PipelineModule(cpu_layers.ref_layer_specs(C1, 0), num_stages=2, loss_fn=cpu_layers.ref_loss(C1),
                           partition_method="uniform", device="cpu")
    config = {"train_micro_batch_size_per_gpu": C1_MB, "gradient_accumulation_steps": C1_GAS,
              "optimizer": {"type": "Adam", "params": {"lr": C1_LR}}, "bamboo_b200": {"p2p_timeout_s": 30}}
    engine, *_ = api.initialize(model=model, config=config, redundancy_level=1, eager_recovery=eager, store=store)
    engine.capture_grads = True
    losses, grad_norms = [], []
    for step, batches in enumerate(gpt_ref.synthetic_batches(C1, C1_MB, C1_GAS, C1_STEPS, seed=1)):
        if step == 2 and rank == 1:
            engine.announce_preemption()                  # gone from step 3 on
        losses.append(float(engine.train_batch(data_iter=iter(batches))))
        grad_norms.append(float(sum(g.double().pow(2).sum() for g in engine.last_grads.values()).sqrt()))
    return {"losses": losses, "grad_norms": grad_norms, "stage_ids": list(engine.stage_ids),
            "checksum": {s: float(engine.arenas[s].master.double().sum()) for s in engine.stage_ids}}


@pytest.mark.parametrize("eager", [False, True])
def test_plumbing_configuration_at_its_stated_size(eager):
    from dist_utils import run_ranks
    ref = gpt_ref.RefTrainer(C1, seed=0, lr=C1_LR, micro_batches=C1_GAS)
    want, want_norm = [], []
    for batches in gpt_ref.synthetic_batches(C1, C1_MB, C1_GAS, C1_STEPS, seed=1):
        want.append(ref.train_batch(batches))
        want_norm.append(float(sum(g.double().pow(2).sum() for g in ref.last_grads.values()).sqrt()))
    res = run_ranks(_train_c1, 2, eager, timeout=400)
    assert res[1] == ("exit", 13)
    status, out = res[0]
    assert status == "ok", out
    assert out["stage_ids"] == [0, 1]
    # stage 0 owns the loss only after it took stage 1 over (steps 3 and 4)
    assert out["losses"][3:] == pytest.approx(want[3:], rel=1e-4)
    # after the failover this rank holds every gradient of the model
    assert out["grad_norms"][3:] == pytest.approx(want_norm[3:], rel=1e-4)
    total = sum(float(p.detach().double().sum()) for p in ref.P.values())
    assert sum(out["checksum"].values()) == pytest.approx(total, rel=1e-6)


# ---------------------------------------------------------------------------------------------
# failure bookkeeping details
def test_concurrent_detectors_agree_on_the_earlier_step():
    """Both neighbours of a dead middle stage publish their step at the same moment with the
    default (lock-free) rendezvous stand-in: neither entry may be lost, both return the minimum."""
    import threading
    from types import SimpleNamespace
    from bamboo_b200.engine import LocalStore, PipelineEngine
    for trial in range(20):
        store = LocalStore()
        cfg = SimpleNamespace(p2p_timeout_s=5.0)
        out = {}
        barrier = threading.Barrier(2)

        def detect(rank, step, other):
            eng = SimpleNamespace(global_store=store, global_rank=rank, _config=cfg)
            barrier.wait()
            out[rank] = PipelineEngine._agree_failed_step(eng, 1, step, other)
        ts = [threading.Thread(target=detect, args=(0, 7, 2)), threading.Thread(target=detect, args=(2, 5, 0))]
        [t.start() for t in ts]
        [t.join() for t in ts]
        assert out == {0: 5, 2: 5}


def test_simultaneous_preemption_announcements_are_both_recorded():
    """Several members announce their preemption at the same moment: the shared record ends up with every
    entry (the read-extend-write of the record runs under a mutex kept in the store), and an entry of a step
    long past is dropped on the way."""
    import json
    import threading
    import time
    from types import SimpleNamespace
    from bamboo_b200.engine import LocalStore, PipelineEngine, store_mutex

    class SlowStore(LocalStore):
        """Widens the window between reading and writing the record, so that unprotected updates would collide."""
        def set(self, key, value):
            if key == "failures":
                time.sleep(0.005)
            super().set(key, value)

    for trial in range(3):
        store = SlowStore()
        store.set("failures", json.dumps({"7": 2}))
        start = threading.Barrier(4)

        def announce(rank):
            eng = SimpleNamespace(global_store=store, global_rank=rank, global_steps=5)
            start.wait()
            PipelineEngine.announce_preemption(eng)
        ts = [threading.Thread(target=announce, args=(r,)) for r in (1, 3, 4, 6)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        assert json.loads(store.get("failures")) == {"1": 6, "3": 6, "4": 6, "6": 6}
    # a holder that died without releasing delays the next member by the timeout, no longer
    store = LocalStore()
    store.add("m-ticket", 1)                                 # somebody took a ticket and never released
    t0 = time.time()
    with store_mutex(store, "m", timeout_s=0.3):
        pass
    assert 0.25 < time.time() - t0 < 2.0
    t0 = time.time()
    with store_mutex(store, "m", timeout_s=0.3):             # the counter was moved past the dead holder's ticket
        pass
    assert time.time() - t0 < 0.2


def test_lone_detector_keeps_its_own_step():
    from types import SimpleNamespace
    from bamboo_b200.engine import LocalStore, PipelineEngine
    eng = SimpleNamespace(global_store=LocalStore(), global_rank=0, _config=SimpleNamespace(p2p_timeout_s=0.2))
    assert PipelineEngine._agree_failed_step(eng, 1, 4, None) == 4
    assert PipelineEngine._agree_failed_step(eng, 1, 4, 2) == 4          # the other detector never shows up


def _partial_state_sender(rank, world, store):
    """Rank 1 ships one of three state pieces and then goes silent; rank 0 must keep its buffers."""
    import time
    import torch.distributed as dist
    from bamboo_b200.p2p import DistTransport, PeerTimeout
    tr = DistTransport(dist, timeout_s=2.0)
    if rank == 1:
        w = dist.isend(torch.full((8,), 5.0), 0, tag=3)
        w.wait()
        time.sleep(4.0)
        return "sent one piece"
    bufs = [torch.zeros(8), torch.ones(8), torch.full((8,), 2.0)]
    try:
        tr.exchange_state(None, [], 1, bufs, 1)
    except PeerTimeout as e:
        return {"peer": e.peer, "bufs": [b.tolist() for b in bufs]}
    return "no timeout"


def test_state_transfer_is_all_or_nothing():
    from dist_utils import run_ranks
    res = run_ranks(_partial_state_sender, 2)
    status, out = res[0]
    assert status == "ok" and out["peer"] == 1
    assert out["bufs"] == [[0.0] * 8, [1.0] * 8, [2.0] * 8]


def _stale_shadow(rank, world, store):
    import cpu_layers
    from bamboo_b200 import api
    from bamboo_b200.module import PipelineModule
    from bamboo_b200.p2p import PeerTimeout
    model = PipelineModule(cpu_layers.ref_layer_specs(CFG, 0), num_stages=2, loss_fn=cpu_layers.ref_loss(CFG),
                           partition_method="uniform", device="cpu")
    config = {"train_micro_batch_size_per_gpu": MB, "gradient_accumulation_steps": GAS,
              "optimizer": {"type": "Adam", "params": {"lr": LR}}, "bamboo_b200": {"p2p_timeout_s": 20}}
    engine, *_ = api.initialize(model=model, config=config, redundancy_level=1, store=store)
    data = gpt_ref.synthetic_batches(CFG, MB, GAS, 2, seed=1)
    engine.train_batch(data_iter=iter(data[0]))
    if rank == 0:
        real = engine.transport.exchange_state

        def failing(send_to, tensors_out, recv_from, tensors_in, seq):
            real(send_to, tensors_out, recv_from, tensors_in, seq)      # keeps the peer in step
            raise PeerTimeout(recv_from, "injected: the owner went silent during the transfer")
        engine.transport.exchange_state = failing
    engine.train_batch(data_iter=iter(data[1]))
    if rank != 0:
        return None
    valid = dict(engine._shadow_valid)
    try:
        engine._promote_next_stage()
        refused = False
    except RuntimeError as e:
        refused = "cannot be promoted" in str(e)
    return {"valid": valid, "refused": refused}


def test_failed_shadow_refresh_blocks_promotion():
    """A state transfer that timed out leaves the shadow one step behind: it is marked and a
    later promotion is refused instead of continuing from stale weights."""
    from dist_utils import run_ranks
    res = run_ranks(_stale_shadow, 2)
    status, out = res[0]
    assert status == "ok", out
    assert out["valid"] == {1: False} and out["refused"]


def test_four_by_two_grid_middle_stage_failover():
    """The GPT-6.7B configuration's failure case on a small model: 4 stages x 2 replicas (rank =
    stage * 2 + replica), replica-0 stage 2 (rank 4) is preempted after step 2.  Rank 2 promotes its
    shadow of stage 2 and takes rank 4's seat in that stage's all-reduce, rank 6 re-points its
    predecessor to rank 2, rank 5 switches to the fallback group; every survivor keeps the oracle's
    trajectory."""
    from dist_utils import run_ranks
    want, ref = _oracle_grid(2)
    res = run_ranks(_train_grid, 8, 4, 2, 1, 4, 2, timeout=400)
    assert res[4] == ("exit", 13)
    for r in (0, 1, 2, 3, 5, 6, 7):
        assert res[r][0] == "ok", res[r]
    assert res[2][1]["stage_ids"] == [1, 2]
    assert res[6][1]["losses"] == pytest.approx([w[0] for w in want], rel=1e-5)     # last stage of replica 0
    assert res[7][1]["losses"] == pytest.approx([w[1] for w in want], rel=1e-5)     # last stage of replica 1
    total = sum(float(p.detach().double().sum()) for p in ref.P.values())
    replica1 = sum(sum(res[r][1]["checksum"].values()) for r in (1, 3, 5, 7))
    replica0 = sum(sum(res[r][1]["checksum"].values()) for r in (0, 2, 6))
    assert replica1 == pytest.approx(total, rel=1e-6) and replica0 == pytest.approx(total, rel=1e-6)
