"""Import surface of DeepSpeed as Bamboo's training scripts use it, served by ``bamboo_b200``.

A script written against the reference keeps its imports (``import deepspeed``,
``from deepspeed.pipe import PipelineModule``, ``from deepspeed.runtime.pipe.topology import
PipeDataParallelTopology``; e.g. ``DeepSpeedExamples/pipeline_parallelism/transformer.py:21-23``)
and its calls (``deepspeed.init_distributed(backend, rank=, world_size=, store=)``,
``deepspeed.add_config_arguments(parser)``, ``deepspeed.initialize(..., redundancy_level=,
eager_recovery=)``, ``deepspeed/__init__.py:61-168,222-235`` of the reference).  Only the
pipeline-parallel ``train_batch`` path exists behind these names; everything else raises.
"""
from bamboo_b200.api import add_config_arguments, init_distributed, initialize
from bamboo_b200.config import DeepSpeedConfigError
from bamboo_b200.engine import PipelineEngine, PipelineError
from bamboo_b200.module import PipelineModule

from . import pipe, runtime, utils  # noqa: F401  (sub-packages reachable as attributes)

__version__ = "0.5.2+bamboo_b200"
__version_major__, __version_minor__, __version_patch__ = 0, 5, 2

__all__ = ["initialize", "init_distributed", "add_config_arguments", "PipelineEngine", "PipelineModule",
           "PipelineError", "DeepSpeedConfigError"]
