"""Bench lines -> the cost simulator's constants (step time per grid, failover slowdown)."""
import json
from types import SimpleNamespace

import pytest


def _line(par, ms, rc="eager", batch=128, failover=None, rc_off_ms=None, model="gpt2-medium"):
    d = {"metric": "tokens/sec", "ms_per_step": ms,
         "config": {"workload": f"{model} (24 layers) pipeline step, micro-batch 8 x 16", "parallelism": par, "rc": rc,
                    "global_batch": batch}}
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
    assert sim.step_delta == 2122 and sim.fallback_slowdown == pytest.approx(1.54, rel=1e-2) and sim.samples_per_step == 128
    sim.num_pipelines = 3
    with pytest.raises(NotImplementedError):
        sim.simulate_step_delta()


def test_prediction_for_grids_that_were_not_measured():
    from bamboo_b200 import simulation
    c = simulation.constants_from_bench([_line("pp4", 152.0), _line("pp8", 92.0), _line("pp2", 300.0), _line("pp2dp2", 306.0)])
    assert c["micro_batches"]["gpt2-medium"][(1, 4)] == 16
    assert simulation.predict_step_ms(c, "gpt2-medium", 1, 4) == 152.0                      # measured
    slot = 152.0 / 19
    assert simulation.predict_step_ms(c, "gpt2-medium", 2, 4) == pytest.approx(slot * (8 + 3) * 1.02)
    assert simulation.predict_step_ms(c, "gpt2-medium", 3, 8) == pytest.approx(92.0 / 23 * (6 + 7) * 1.02)
    assert simulation.predict_step_ms(c, "gpt2-medium", 2, 12) is None                      # no 12-stage run to scale from


# the reference checkout, when it lies beside this repository (or where BAMBOO_REFERENCE points)
import os as _os  # noqa: E402

_REFERENCE = _os.environ.get("BAMBOO_REFERENCE") or _os.path.join(
    _os.path.dirname(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__)))), "reference")
REFERENCE_SIMULATOR = _os.path.join(_REFERENCE, "project_pactum", "simulation", "simulator.py")


@pytest.mark.skipif(not _os.path.exists(REFERENCE_SIMULATOR), reason="reference checkout not present")
def test_reference_simulator_runs_on_measured_step_times():
    """The reference's own spot-market simulator, imported in place, replays a day with this implementation's numbers."""
    from bamboo_b200 import simulation
    lines = [_line("pp4", 152.0, failover={"post_failover_step_s": 0.2316, "normal_step_s": 0.1499, "pause_s": 0.146}),
             _line("pp8", 93.0), _line("pp2", 300.0), _line("pp2dp2", 306.0)]
    result, sim = simulation.run_reference_simulator(REFERENCE_SIMULATOR, lines, "gpt2-medium", hours=6, seed=3, stages_target=4,
                                                     capacity=16, removal_probability=0.05)
    assert sim.num_stages_target == 4 and sim.samples_per_step == 128
    assert sim.fallback_slowdown == pytest.approx(0.2316 / 0.1499)
    assert result.num_steps_complete > 1000                                 # 6 h at ~0.1-0.15 s per step, minus rendezvous time
    assert result.average_performance > 0 and result.average_cost > 0
    # the step time in force at the end is one of ours (measured 4-stage value or a prediction from it)
    assert 0 < sim.step_delta <= 152
