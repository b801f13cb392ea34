"""``deepspeed.runtime.pipe.topology`` (reference ``deepspeed/runtime/pipe/topology.py``)."""
from bamboo_b200.topology import (GlobalInfo, PipeDataParallelTopology, PipelineParallelGrid,
                                  PipeModelDataParallelTopology, ProcessTopology)

__all__ = ["ProcessTopology", "PipeDataParallelTopology", "PipeModelDataParallelTopology", "PipelineParallelGrid",
           "GlobalInfo"]
