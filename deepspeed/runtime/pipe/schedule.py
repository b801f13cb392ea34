"""``deepspeed.runtime.pipe.schedule`` (reference ``deepspeed/runtime/pipe/schedule.py``)."""
from bamboo_b200.schedule import *  # noqa: F401,F403
from bamboo_b200 import schedule as _s

__all__ = [n for n in dir(_s) if not n.startswith("_")]
