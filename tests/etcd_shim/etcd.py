"""Stands where ``import etcd`` would find python-etcd, for processes started by the launcher tests:
``Client(host, port, ...)`` connects to the in-process stand-in (tests/fake_etcd.py) served at that address."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import fake_etcd  # noqa: E402
from fake_etcd import (EtcdAlreadyExist, EtcdCompareFailed, EtcdEventIndexCleared, EtcdException, EtcdKeyNotFound,  # noqa: E402,F401
                       EtcdNotFile, EtcdResult, EtcdWatchTimedOut, Lock)


def Client(host, port, **_options):
    return fake_etcd.connect((host, int(port)))
