"""Bench lines -> the cost simulator's constants (step time per grid, failover slowdown)."""
import json
from types import SimpleNamespace

import pytest


def _line(par, ms, rc="eager", batch=128, failover=None, rc_off_ms=None, model="gpt2-medium"):
    d = {"metric": "tokens/sec", "ms_per_step": ms,
         "config": {"workload": f"{model} (24 layers) pipeline step", "parallelism": par, "rc": rc, "global_batch": batch}}
    if failover:
        d["failover"] = failover
    if rc_off_ms:
        d["rc_off"] = {"ms_per_step": rc_off_ms}
    return d


def test_constants_and_install():
    from bamboo_b200 import simulation
    lines = [_line("pp1", 445.0, rc="off"),
             json.dumps(_line("pp4", 157.0, rc_off_ms=140.6,
                              failover={"post_failover_step_s": 0.236, "normal_step_s": 0.157, "pause_s": 0.19})),
             _line("pp4dp2", 2121.7, batch=128, model="gpt-6.7b",
                   failover={"post_failover_step_s": 3.267, "normal_step_s": 2.1217, "pause_s": 1.74}),
             {"impl": "reference", "ms_per_step": 1.0}]
    c = simulation.constants_from_bench(lines)
    assert c["step_delta_ms"]["gpt2-medium"] == {(1, 4): 157.0}
    assert c["step_delta_rc_off_ms"]["gpt2-medium"] == {(1, 1): 445.0, (1, 4): 140.6}
    assert c["step_delta_ms"]["gpt-6.7b"] == {(2, 4): 2121.7}
    assert c["fallback_slowdown"]["gpt2-medium"][(1, 4)] == pytest.approx(1.503, rel=1e-3)
    assert c["failover_pause_ms"]["gpt-6.7b"][(2, 4)] == pytest.approx(1740.0)
    sim = SimpleNamespace(num_pipelines=2, num_stages=4, step_delta=None, fallback_slowdown=1.5, samples_per_step=32)
    simulation.install(sim, c, "gpt-6.7b")
    sim.simulate_step_delta()
    assert sim.step_delta == 2121.7 and sim.fallback_slowdown == pytest.approx(1.54, rel=1e-2) and sim.samples_per_step == 128
    sim.num_pipelines = 3
    with pytest.raises(NotImplementedError):
        sim.simulate_step_delta()
