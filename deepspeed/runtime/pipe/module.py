"""``deepspeed.runtime.pipe.module`` (reference ``deepspeed/runtime/pipe/module.py``)."""
from bamboo_b200.engine import PipelineError
from bamboo_b200.module import LayerSpec, PipelineModule, TiedLayerSpec

__all__ = ["PipelineModule", "LayerSpec", "TiedLayerSpec", "PipelineError"]
