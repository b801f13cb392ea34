"""A Bamboo training script's imports and calls resolve against this repository: the four
statements of ``DeepSpeedExamples/pipeline_parallelism/transformer.py:21-23,67,241,274`` of the
reference, then one ``train_batch`` through the names they bind."""
import argparse
import os

import torch
from torch import nn


def test_reference_script_statements_resolve():
    import deepspeed
    from deepspeed.pipe import PipelineModule
    from deepspeed.runtime.pipe.topology import ProcessTopology, PipeDataParallelTopology

    parser = deepspeed.add_config_arguments(argparse.ArgumentParser())
    args = parser.parse_args(["--deepspeed"])
    assert args.deepspeed and args.deepspeed_config is None
    assert callable(deepspeed.init_distributed) and callable(deepspeed.initialize)
    assert issubclass(PipeDataParallelTopology, ProcessTopology)
    from bamboo_b200 import module, topology
    assert PipelineModule is module.PipelineModule and PipeDataParallelTopology is topology.PipeDataParallelTopology
    # names other scripts of the reference use
    import deepspeed.runtime.utils as ds_utils
    from deepspeed.runtime.pipe.schedule import TrainSchedule
    from deepspeed.pipe import LayerSpec, TiedLayerSpec  # noqa: F401
    ds_utils.set_random_seed(7)
    assert ds_utils.partition_uniform(10, 2) == [0, 5, 10]
    assert len(list(TrainSchedule(micro_batches=4, stages=2, stage_id=0))) == 10


def test_train_batch_through_the_deepspeed_names():
    import deepspeed
    from deepspeed.pipe import PipelineModule
    os.environ["BAMBOO_QUIET"] = "1"
    torch.manual_seed(0)
    layers = [nn.Linear(8, 16), nn.Tanh(), nn.Linear(16, 8)]
    model = PipelineModule(layers=layers, loss_fn=nn.MSELoss(), num_stages=1, partition_method="uniform", device="cpu")
    x = torch.randn(4, 8)
    data = [(x, torch.zeros(4, 8))] * 4
    engine, _, _, _ = deepspeed.initialize(args=None, model=model,
                                           model_parameters=[p for p in model.parameters() if p.requires_grad],
                                           config={"train_micro_batch_size_per_gpu": 4, "gradient_accumulation_steps": 2,
                                                   "optimizer": {"type": "Adam", "params": {"lr": 1e-2}}},
                                           redundancy_level=0, eager_recovery=False)
    first = float(engine.train_batch(data_iter=iter(data)))
    second = float(engine.train_batch(data_iter=iter(data)))
    assert engine.global_steps == 2 and second < first
    for call in (engine.forward, engine.backward, engine.step):
        try:
            call()
            raise AssertionError("expected PipelineError")
        except deepspeed.PipelineError:
            pass
