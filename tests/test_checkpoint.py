"""Per-layer checkpoint format: file names, resume equivalence, and loading into a different
stage partition than the one that wrote the checkpoint (CPU ranks, gloo)."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from oracle import gpt_ref  # noqa: E402

CFG = gpt_ref.RefConfig(layers=4, hidden=64, heads=4, ffn=128, seq=16, vocab=96)
MB, GAS, LR = 2, 4, 1e-3


def _engine(stages, store, world):
    import cpu_layers
    from bamboo_b200 import api
    from bamboo_b200.module import PipelineModule
    os.environ["BAMBOO_QUIET"] = "1"
    model = PipelineModule(cpu_layers.ref_layer_specs(CFG, 0), num_stages=stages, loss_fn=cpu_layers.ref_loss(CFG),
                           partition_method="uniform", device="cpu")
    config = {"train_micro_batch_size_per_gpu": MB, "gradient_accumulation_steps": GAS,
              "optimizer": {"type": "Adam", "params": {"lr": LR}}, "bamboo_b200": {"p2p_timeout_s": 20}}
    engine, *_ = api.initialize(model=model, config=config, redundancy_level=1 if stages > 1 else 0,
                                store=store if world > 1 else None)
    return engine


def _write(rank, world, store, stages, ckpt):
    engine = _engine(stages, store, world)
    data = gpt_ref.synthetic_batches(CFG, MB, GAS, 3, seed=1)
    losses = [float(engine.train_batch(data_iter=iter(b))) for b in data[:2]]
    engine.save_checkpoint(ckpt, client_state={"note": "after two steps"})
    losses.append(float(engine.train_batch(data_iter=iter(data[2]))))
    return losses


def _resume(rank, world, store, stages, ckpt):
    engine = _engine(stages, store, world)
    path, client = engine.load_checkpoint(ckpt)
    data = gpt_ref.synthetic_batches(CFG, MB, GAS, 3, seed=1)
    return {"path": path, "client": client, "steps": engine.global_steps,
            "loss": float(engine.train_batch(data_iter=iter(data[2])))}


def test_single_stage_files_and_resume(tmp_path):
    ckpt = str(tmp_path / "ckpt")
    losses = _write(0, 1, None, 1, ckpt)
    assert open(os.path.join(ckpt, "latest")).read() == "global_step2"
    files = sorted(os.listdir(os.path.join(ckpt, "global_step2")))
    # layer list: embedding, 4 blocks, final LayerNorm, head = layers 00..06, one stage file
    assert files == [f"layer_{i:02d}-model_states.pt" for i in range(7)] + ["mp_rank_00_model_states.pt"]
    blk = torch.load(os.path.join(ckpt, "global_step2", "layer_01-model_states.pt"), weights_only=False)
    assert all(v.dtype == torch.float32 for v in blk.values()) and len(blk) == 12
    out = _resume(0, 1, None, 1, ckpt)
    assert out["steps"] == 2 and out["client"] == {"note": "after two steps"}
    assert out["loss"] == pytest.approx(losses[2], rel=1e-6)
    fresh = _engine(1, None, 1)
    assert fresh.load_checkpoint(str(tmp_path / "nothing_here")) == (None, None)


def test_two_stage_checkpoint_loads_into_one_stage(tmp_path):
    """Written by two pipeline stages (each its own layers and optimizer moments), resumed by a
    single stage: the third step continues the same trajectory."""
    from dist_utils import run_ranks
    ckpt = str(tmp_path / "ckpt")
    res = run_ranks(_write, 2, 2, ckpt)
    assert res[0][0] == "ok" and res[1][0] == "ok"
    want = res[1][1][2]                                   # the last stage reports the loss
    files = sorted(os.listdir(os.path.join(ckpt, "global_step2")))
    assert "mp_rank_00_model_states.pt" in files and "mp_rank_01_model_states.pt" in files
    assert sum(f.startswith("layer_") for f in files) == 7
    out = _resume(0, 1, None, 1, ckpt)
    assert out["loss"] == pytest.approx(want, rel=1e-5)
    # and back into two stages (shadow copies restart from the same state)
    res2 = run_ranks(_resume, 2, 2, ckpt)
    assert res2[1][1]["loss"] == pytest.approx(want, rel=1e-5)
