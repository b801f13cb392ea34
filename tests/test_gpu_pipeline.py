"""Two pipeline stages on two GPUs: activations and gradients through the NVLink mailboxes,
eager redundant computation on the low-priority stream, shadow-state refresh, and an
announced preemption of stage 1 after step 3 - losses must follow the fp32 oracle
(bf16 tolerance 2e-2) before and after the failover.  Needs two GPUs; skipped otherwise."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from oracle import gpt_ref  # noqa: E402

pytestmark = pytest.mark.gpu
CFG = gpt_ref.RefConfig(layers=4, hidden=256, heads=4, ffn=1024, seq=128, vocab=1024)
MB, GAS, STEPS, LR = 4, 4, 5, 1e-4


def _train(rank, world, store, rc, eager, victim_step):
    from bamboo_b200 import api, lib, models
    from bamboo_b200.module import PipelineModule
    tc = models.TransformerConfig(layers=CFG.layers, hidden=CFG.hidden, heads=CFG.heads, ffn=CFG.ffn, seq=CFG.seq,
                                  vocab=CFG.vocab)
    model = PipelineModule(models.transformer_layer_specs(tc, 0), num_stages=world, loss_fn=models.transformer_loss(tc),
                           partition_method="type:TransformerBlock")
    config = {"train_micro_batch_size_per_gpu": MB, "gradient_accumulation_steps": GAS, "bf16": {"enabled": True},
              "optimizer": {"type": "Adam", "params": {"lr": LR}}, "bamboo_b200": {"p2p_timeout_s": 20}}
    engine, *_ = api.initialize(model=model, config=config, redundancy_level=rc, eager_recovery=eager, store=store)
    data = gpt_ref.synthetic_batches(CFG, MB, GAS, STEPS, seed=1)
    losses = []
    for step, batches in enumerate(data):
        if victim_step is not None and step == victim_step - 1 and rank == world - 1:
            engine.announce_preemption()
        losses.append(float(engine.train_batch(data_iter=iter(batches))))
    torch.cuda.synchronize()
    return {"losses": losses, "stage_ids": list(engine.stage_ids), "status": lib.read_status(),
            "transport": engine.transport.name}


def _oracle():
    ref = gpt_ref.RefTrainer(CFG, seed=0, lr=LR, micro_batches=GAS)
    return [ref.train_batch(s) for s in gpt_ref.synthetic_batches(CFG, MB, GAS, STEPS, seed=1)]


needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")


@needs2
@pytest.mark.parametrize("rc,eager", [(0, False), (1, False), (1, True)])
def test_two_stage_pipeline_over_mailboxes(rc, eager):
    from dist_utils import run_ranks
    want = _oracle()
    res = run_ranks(_train, 2, rc, eager, None, backend="nccl")
    assert res[0][0] == "ok" and res[1][0] == "ok"
    assert res[1][1]["transport"] == "mailbox" and res[1][1]["status"] == 0 and res[0][1]["status"] == 0
    assert res[1][1]["losses"] == pytest.approx(want, rel=2e-2)


@needs2
@pytest.mark.parametrize("eager", [False, True])
def test_failover_on_gpu_keeps_the_trajectory(eager):
    from dist_utils import run_ranks
    want = _oracle()
    res = run_ranks(_train, 2, 1, eager, 3, backend="nccl")
    assert res[1] == ("exit", 13)
    status, out = res[0]
    assert status == "ok" and out["stage_ids"] == [0, 1] and out["status"] == 0
    assert out["losses"][3:] == pytest.approx(want[3:], rel=2e-2)


def _train_dp(rank, world, store):
    """One stage, two replicas: the only collective is the NCCL all-reduce of the fp32 gradient arena."""
    from bamboo_b200 import api, lib, models
    from bamboo_b200.module import PipelineModule
    from bamboo_b200.topology import PipeDataParallelTopology
    tc = models.TransformerConfig(layers=CFG.layers, hidden=CFG.hidden, heads=CFG.heads, ffn=CFG.ffn, seq=CFG.seq,
                                  vocab=CFG.vocab)
    model = PipelineModule(models.transformer_layer_specs(tc, 0), topology=PipeDataParallelTopology(1, world),
                           loss_fn=models.transformer_loss(tc), partition_method="uniform")
    config = {"train_micro_batch_size_per_gpu": MB, "gradient_accumulation_steps": GAS,
              "train_batch_size": MB * GAS * world, "bf16": {"enabled": True},
              "optimizer": {"type": "Adam", "params": {"lr": LR}}}
    engine, *_ = api.initialize(model=model, config=config, store=store)
    data = gpt_ref.synthetic_batches(CFG, MB, GAS * world, 3, seed=1)
    losses = [float(engine.train_batch(data_iter=iter(b[rank * GAS:(rank + 1) * GAS]))) for b in data]
    torch.cuda.synchronize()
    return {"losses": losses, "checksum": float(engine.arenas[0].master.double().sum()), "status": lib.read_status()}


@needs2
def test_data_parallel_replicas_average_gradients():
    from dist_utils import run_ranks
    ref = gpt_ref.RefTrainer(CFG, seed=0, lr=LR, micro_batches=GAS * 2)
    want = []
    for batches in gpt_ref.synthetic_batches(CFG, MB, GAS * 2, 3, seed=1):
        with torch.no_grad():
            want.append([sum(float(gpt_ref.forward_loss(CFG, ref.P, t, l)) for t, l in batches[r * GAS:(r + 1) * GAS]) / GAS
                         for r in range(2)])
        ref.train_batch(batches)
    res = run_ranks(_train_dp, 2, backend="nccl")
    for r in range(2):
        assert res[r][0] == "ok" and res[r][1]["status"] == 0
        assert res[r][1]["losses"] == pytest.approx([w[r] for w in want], rel=2e-2)
    assert res[0][1]["checksum"] == res[1][1]["checksum"]          # replicas stay bit-identical
