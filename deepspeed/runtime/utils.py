"""``deepspeed.runtime.utils``: the helpers pipeline scripts and ``PipelineModule`` use
(reference ``deepspeed/runtime/utils.py:51-61,470-551``)."""
import random

import torch

from bamboo_b200.partition import partition_balanced, partition_uniform

__all__ = ["set_random_seed", "partition_uniform", "partition_balanced"]


def set_random_seed(seed):
    """Seed ``random``, ``numpy`` and ``torch`` alike."""
    import numpy
    random.seed(seed)
    numpy.random.seed(seed)
    torch.manual_seed(seed)
