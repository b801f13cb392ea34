"""``deepspeed.runtime``: the pipeline sub-package and the partition / seeding helpers."""
from . import pipe, utils  # noqa: F401
