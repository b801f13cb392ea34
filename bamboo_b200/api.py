"""The ``deepspeed`` entry points a Bamboo training script calls.

``initialize`` keeps the signature of the reference (``deepspeed/__init__.py:61-168``,
including Bamboo's ``redundancy_level``, ``sync_save`` and ``eager_recovery``) and returns
``(engine, optimizer, training_dataloader, lr_scheduler)``; ``init_distributed`` keeps
Bamboo's ``store=`` argument (``deepspeed/utils/distributed.py:14-68``);
``add_config_arguments`` adds ``--deepspeed`` / ``--deepspeed_config``
(``deepspeed/__init__.py:222-235``).
"""
import os
from datetime import timedelta

import torch

from .config import PipeConfig
from .engine import PipelineEngine
from .module import PipelineModule


def init_distributed(dist_backend="nccl", auto_mpi_discovery=True, distributed_port=29500, verbose=True,
                     timeout=timedelta(minutes=30), init_method=None, rank=-1, store=None, world_size=-1):
    import torch.distributed as dist
    if dist.is_initialized():
        return
    kw = dict(backend=dist_backend, timeout=timeout)
    if store is not None:
        kw.update(store=store, rank=rank, world_size=world_size)
    else:
        if init_method is not None:
            kw["init_method"] = init_method
        if rank >= 0:
            kw["rank"] = rank
        if world_size > 0:
            kw["world_size"] = world_size
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(distributed_port))
    if dist_backend == "nccl" and torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group(**kw)


def add_config_arguments(parser):
    group = parser.add_argument_group("DeepSpeed", "DeepSpeed configurations")
    group.add_argument("--deepspeed", default=False, action="store_true",
                       help="Enable DeepSpeed (helper flag for user code, no impact on DeepSpeed backend)")
    group.add_argument("--deepspeed_config", default=None, type=str, help="DeepSpeed json configuration file.")
    group.add_argument("--deepscale", default=False, action="store_true", help="Deprecated enable flag")
    group.add_argument("--deepscale_config", default=None, type=str, help="Deprecated config file")
    group.add_argument("--deepspeed_mpi", default=False, action="store_true", help="MPI discovery (ignored)")
    return parser


def initialize(args=None, model=None, optimizer=None, model_parameters=None, training_data=None, lr_scheduler=None,
               mpu=None, dist_init_required=None, collate_fn=None, config=None, config_params=None,
               redundancy_level=0, sync_save=False, eager_recovery=False, rdzv_handler=None, store=None,
               transport=None):
    """Build the engine for ``model``.  Only pipeline models are on this implementation's
    path; anything else is refused."""
    assert model is not None, "deepspeed.initialize requires a model"
    if not isinstance(model, PipelineModule):
        raise NotImplementedError("this implementation covers the PipelineModule / train_batch path only")
    if optimizer is not None:
        raise NotImplementedError("client optimizers are not supported: configure Adam/AdamW in the JSON config; "
                                  "the step runs as one fused kernel over the stage's parameter arena")
    cfg = config if config is not None else config_params
    if cfg is None and args is not None:
        cfg = getattr(args, "deepspeed_config", None) or getattr(args, "deepscale_config", None)
    dp = model._grid.data_parallel_size
    engine = PipelineEngine(model, PipeConfig(cfg, dp), redundancy_level=redundancy_level, sync_save=sync_save,
                            eager_recovery=eager_recovery, training_data=training_data, collate_fn=collate_fn,
                            rdzv_handler=rdzv_handler, store=store, transport=transport, lr_scheduler=lr_scheduler)
    return engine, engine.optimizer, engine.training_dataloader, engine.lr_scheduler
