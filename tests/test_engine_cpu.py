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


def _train(rank, world, store, stages, rc, eager, victim_step):
    """Body of one rank.  ``victim_step``: the last stage's rank announces its preemption so
    that it is gone from step ``victim_step`` on (None = no failure)."""
    import cpu_layers
    from bamboo_b200 import api
    from bamboo_b200.module import PipelineModule
    model = PipelineModule(cpu_layers.ref_layer_specs(CFG, 0), num_stages=stages, loss_fn=cpu_layers.ref_loss(CFG),
                           partition_method="uniform", device="cpu")
    config = {"train_micro_batch_size_per_gpu": MB, "gradient_accumulation_steps": GAS,
              "optimizer": {"type": "Adam", "params": {"lr": LR}}, "bamboo_b200": {"p2p_timeout_s": 20}}
    engine, *_ = api.initialize(model=model, config=config, redundancy_level=rc, eager_recovery=eager,
                                store=store if world > 1 else None)
    data = gpt_ref.synthetic_batches(CFG, MB, GAS, STEPS, seed=1)
    losses = []
    for step, batches in enumerate(data):
        if victim_step is not None and step == victim_step - 1 and rank == stages - 1:
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
