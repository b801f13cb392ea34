"""``deepspeed.utils.distributed`` (reference ``deepspeed/utils/distributed.py``)."""
from bamboo_b200.api import init_distributed

__all__ = ["init_distributed"]
