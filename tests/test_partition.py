"""Partition and redundancy maps against answers computed by the reference
(tests/golden/partition.json, tests/golden/topology.json) plus the known-answer
vectors of the reference's own unit tests (tests/unit/test_partition.py:121-154)."""
from bamboo_b200.partition import (get_redundant_stage_ids, get_redundant_user_stage_ids,
                                   partition_balanced, partition_uniform)


def test_uniform_golden(golden_partition):
    for key, want in golden_partition["uniform"].items():
        n, p = map(int, key.split(","))
        assert partition_uniform(n, p) == want, key


def test_balanced_golden(golden_partition):
    assert len(golden_partition["balanced"]) >= 200
    for case in golden_partition["balanced"]:
        assert partition_balanced(case["weights"], case["parts"]) == case["answer"], case


def test_reference_known_answers():
    # same vectors as the reference's test_int_balanced / test_float_balanced / test_float_midheavy
    assert partition_balanced([0, 1, 2, 3, 3, 3], 4) == [0, 3, 4, 5, 6]
    assert partition_balanced([0., 1.1, 1.9, 3., 3., 3.], 4) == [0, 3, 4, 5, 6]
    assert partition_balanced([0., 1.1, 30, 3.], 3) == [0, 2, 3, 4]
    # short inputs fall back to one item per part
    assert partition_balanced([5], 3) == [0, 1, 1, 1]
    assert partition_uniform(0, 2) == [0, 0, 0]


def test_redundancy_maps(golden_topology):
    for row in golden_topology["redundancy"]:
        assert get_redundant_stage_ids(row["level"], row["stage"], row["stages"]) == row["shadows"]
        assert get_redundant_user_stage_ids(row["level"], row["stage"], row["stages"]) == row["shadowed_by"]
