"""``deepspeed.runtime.pipe.engine`` (reference ``deepspeed/runtime/pipe/engine.py``)."""
from bamboo_b200.engine import (AllReduceException, NextStageException, PipelineEngine, PipelineError,
                                PrevStageException)

__all__ = ["PipelineEngine", "PipelineError", "NextStageException", "PrevStageException", "AllReduceException"]
