import gzip
import json
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def golden_schedules():
    with gzip.open(os.path.join(GOLDEN, "schedules.json.gz"), "rb") as f:
        return json.loads(f.read().decode())


@pytest.fixture(scope="session")
def golden_partition():
    with open(os.path.join(GOLDEN, "partition.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def golden_topology():
    with open(os.path.join(GOLDEN, "topology.json")) as f:
        return json.load(f)
