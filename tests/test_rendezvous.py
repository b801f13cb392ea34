"""The etcd rendezvous handler against traces of the reference's own handler.

``tests/golden/rendezvous.json`` was written by ``tests/golden/gen_rendezvous_golden.py``, which
runs ``project_pactum/rendezvous/etcd.py`` of the reference (imported in place) on the in-process
etcd of ``tests/fake_etcd.py``.  The same scenarios run here with ``bamboo_b200.rendezvous``:
results, seat assignment, reconfiguration decisions and the whole etcd key space must be equal."""
import json
import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import fake_etcd  # noqa: E402
import rendezvous_scenarios as sc  # noqa: E402


def make_impl(client, run_id, min_nodes, max_nodes):
    from bamboo_b200.rendezvous import EtcdRendezvous
    return EtcdRendezvous(client, sc.PREFIX, run_id, min_nodes, max_nodes, timeout=60, last_call_timeout=1,
                          etcd_module=fake_etcd)


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(HERE, "golden", "rendezvous.json")) as f:
        return json.load(f)


@pytest.mark.parametrize("name", sorted(sc.SCENARIOS))
def test_scenario_matches_reference_trace(name, golden):
    got = sc.scrub(sc.SCENARIOS[name](make_impl))
    want = golden[name]
    assert sorted(got) == sorted(want)
    for key in want:
        assert got[key] == want[key], key


def test_known_answers_of_the_seat_assignment(golden):
    """Human-checkable part of the golden file: 2 x 2 grid, pipeline-major seats in rank order."""
    keys = golden["fresh_2x2"]["keys"]
    for r, seat in enumerate([[0, 0], [0, 1], [1, 0], [1, 1]]):
        assert json.loads(keys[f"/rdzv/v_1/rank_{r}_coordinates"]) == [seat]
    final = json.loads(keys["/rdzv/active_version"])
    assert final["status"] == "final" and final["num_pipelines"] == "2" and final["num_stages"] == "2"
    assert json.loads(keys["/rdzv/previous_state"])["version"] == "1"
    odd = golden["fresh_5_members_2_stages"]["keys"]
    assert json.loads(odd["/rdzv/v_1/rank_4_coordinates"]) == []          # no seat for the fifth member


def test_etcd_store_round_trip():
    from bamboo_b200.rendezvous import EtcdStore
    client = fake_etcd.Client()
    store = EtcdStore(client, "/kv", etcd_module=fake_etcd)
    assert not store.check(["a"])
    store.set("a", b"\x00\x01binary")
    assert store.check(["a"]) and store.get("a") == b"\x00\x01binary"
    assert store.add("n", 2) == 2 and store.add("n", 3) == 5
    assert store.get("n") == b"5"


def test_engine_talks_to_the_handler():
    """A one-stage engine driven through the handler: the rendezvous supplies the grid seat and
    the step counter; every ``train_batch`` records the cluster status and one reconfiguration
    decision per global step in etcd (reference ``pipe/engine.py:1068-1112``)."""
    import torch
    from torch import nn
    import bamboo_b200.engine as E
    from bamboo_b200.module import PipelineModule
    from bamboo_b200.rendezvous import create_rdzv_handler
    os.environ["BAMBOO_QUIET"] = "1"
    server = fake_etcd.Server()
    client = fake_etcd.Client(server)
    client.write(f"{sc.PREFIX}/run_solo/rdzv/default_pipelines", "1")
    handler = create_rdzv_handler(client, "solo", 1, 1, prefix=sc.PREFIX, last_call_timeout=1, etcd_module=fake_etcd)
    store, rank, world, pipelines, stages, decision = handler.next_rendezvous()
    assert (rank, world, pipelines, stages) == (0, 1, 1, 1)
    assert [tuple(g) for g in decision] == [(0, [], [[0, 0]])]
    store.set("hello", "x")
    assert store.get("hello") == b"x"
    torch.manual_seed(0)
    model = PipelineModule(layers=[nn.Linear(4, 4)], loss_fn=nn.MSELoss(), num_stages=1, partition_method="uniform",
                           device="cpu")
    engine = E.PipelineEngine(model, {"train_micro_batch_size_per_gpu": 2, "gradient_accumulation_steps": 1,
                                      "optimizer": {"type": "Adam", "params": {"lr": 1e-2}}}, rdzv_handler=handler)
    assert engine.coordinates == [[0, 0]] and engine.global_steps == 0
    data = [(torch.ones(2, 4), torch.zeros(2, 4))]
    engine.train_batch(data_iter=iter(data))
    engine.train_batch(data_iter=iter(data))
    keys = server.dump()
    root = f"{sc.PREFIX}/run_solo/rdzv"
    assert json.loads(keys[f"{root}/cluster_status"]) == "train"
    assert json.loads(keys[f"{root}/global_steps_0"]) is False and json.loads(keys[f"{root}/global_steps_1"]) is False
    assert json.loads(keys[f"{root}/current_step"]) == 1
    handler.stop_keep_alive()
