"""bamboo_b200: B200-native pipeline-parallel training step with redundant computation.

The package mirrors the part of Bamboo (patched DeepSpeed 0.5.2) that sits on the
``PipelineEngine.train_batch`` path.  Host logic is Python; every stage-compute,
optimizer and inter-stage transfer kernel is hand-written CUDA for sm_100a reached
through the C ABI declared in ``include/bamboo_b200.h``.
"""
__version__ = "0.1.0"
