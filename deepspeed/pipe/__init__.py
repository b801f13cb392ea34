"""``from deepspeed.pipe import PipelineModule, LayerSpec, TiedLayerSpec`` (reference:
``deepspeed/pipe/__init__.py``)."""
from bamboo_b200.module import LayerSpec, PipelineModule, TiedLayerSpec

__all__ = ["PipelineModule", "LayerSpec", "TiedLayerSpec"]
