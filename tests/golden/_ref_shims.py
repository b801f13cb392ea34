"""Shims that let the upstream Bamboo/DeepSpeed sources import under a modern torch.

Used only by the golden-vector generator and by optional cross-checks in the test
suite when a checkout of the reference is present; never by the product package.
"""
import collections.abc
import math
import os
import sys
import types


def install(reference_root):
    """Register stub modules and put the reference packages on sys.path."""
    if "torch._six" not in sys.modules:
        six = types.ModuleType("torch._six")
        six.inf = math.inf
        six.string_classes = (str,)
        six.container_abcs = collections.abc
        sys.modules["torch._six"] = six
    if "tensorboardX" not in sys.modules:
        tbx = types.ModuleType("tensorboardX")

        class SummaryWriter:  # no-op writer
            def __init__(self, *a, **k):
                pass

            def add_scalar(self, *a, **k):
                pass

            def flush(self):
                pass

        tbx.SummaryWriter = SummaryWriter
        sys.modules["tensorboardX"] = tbx
    if "colorama" not in sys.modules:
        col = types.ModuleType("colorama")

        class _Blank:
            def __getattr__(self, name):
                return ""

        col.Fore = _Blank()
        col.Style = _Blank()
        col.Back = _Blank()
        col.init = lambda *a, **k: None
        sys.modules["colorama"] = col
    if "etcd" not in sys.modules:
        et = types.ModuleType("etcd")
        for name in ("EtcdKeyNotFound", "EtcdAlreadyExist", "EtcdCompareFailed",
                     "EtcdWatchTimedOut", "EtcdEventIndexCleared", "EtcdException",
                     "EtcdConnectionFailed"):
            setattr(et, name, type(name, (Exception,), {}))
        et.Client = type("Client", (), {})
        et.Lock = type("Lock", (), {})
        et.EtcdResult = type("EtcdResult", (), {})
        sys.modules["etcd"] = et
    for p in (os.path.join(reference_root, "external", "deepspeed"), reference_root):
        if p not in sys.path:
            sys.path.insert(0, p)
