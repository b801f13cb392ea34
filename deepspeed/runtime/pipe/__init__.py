"""``deepspeed.runtime.pipe`` (reference ``deepspeed/runtime/pipe/__init__.py``)."""
from bamboo_b200.module import LayerSpec, PipelineModule, TiedLayerSpec

from . import engine, module, schedule, topology  # noqa: F401
from .topology import ProcessTopology

__all__ = ["PipelineModule", "LayerSpec", "TiedLayerSpec", "ProcessTopology"]
