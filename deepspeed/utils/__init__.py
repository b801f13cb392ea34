"""``deepspeed.utils``: ``init_distributed`` with Bamboo's ``store=`` argument (reference
``deepspeed/utils/distributed.py:14-68``)."""
from . import distributed  # noqa: F401
from .distributed import init_distributed

__all__ = ["init_distributed"]
