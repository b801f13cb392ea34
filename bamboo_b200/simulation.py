"""Measured step times for Bamboo's cost simulator.

The reference's simulator (``project_pactum/simulation/simulator.py``) replays spot-instance
traces against hard-coded per-model step times - ``*_simulate_step_delta`` set ``step_delta`` in
milliseconds from ``(num_pipelines, num_stages)`` (``:294-380``) - and one slowdown factor for a
pipeline that absorbed a failure (``fallback_slowdown = 1.5``, ``:192``).  This module turns the
JSON lines ``bench.py`` prints into those constants, and can install them on a simulator object,
so the simulator prices B200 runs with measured numbers instead of the published V100 ones.
"""
import json
import re
from typing import Dict, Iterable, Tuple


def _grid(line) -> Tuple[int, int]:
    """(pipelines, stages) of a bench line, from its ``config.parallelism`` ("pp4", "pp4dp2")."""
    m = re.fullmatch(r"pp(\d+)(?:dp(\d+))?", line["config"]["parallelism"])
    return int(m.group(2) or 1), int(m.group(1))


def constants_from_bench(lines: Iterable) -> Dict:
    """``lines``: bench.py JSON lines (dicts or strings).  Returns::

        {"step_delta_ms": {model: {(pipelines, stages): ms}},       # RC on, as the simulator assumes
         "step_delta_rc_off_ms": {model: {(pipelines, stages): ms}},
         "fallback_slowdown": {model: {(pipelines, stages): normal step / post-failover step ... inverted: >= 1}},
         "failover_pause_ms": {model: {(pipelines, stages): ms}},
         "samples_per_step": {model: {(pipelines, stages): global batch}},
         "micro_batches": {model: {(pipelines, stages): micro-batches per pipeline and step}}}
    """
    out = {"step_delta_ms": {}, "step_delta_rc_off_ms": {}, "fallback_slowdown": {}, "failover_pause_ms": {},
           "samples_per_step": {}, "micro_batches": {}}
    for line in lines:
        if isinstance(line, str):
            line = json.loads(line)
        if line.get("impl") == "reference":
            continue
        model = line["config"]["workload"].split(" ")[0]
        key = _grid(line)
        target = "step_delta_ms" if line["config"].get("rc", "off") != "off" else "step_delta_rc_off_ms"
        out[target].setdefault(model, {})[key] = float(line["ms_per_step"])
        out["samples_per_step"].setdefault(model, {})[key] = int(line["config"]["global_batch"])
        mb = re.search(r"micro-batch (\d+) x (\d+)", line["config"]["workload"])
        if mb:
            out["micro_batches"].setdefault(model, {})[key] = int(mb.group(2))
        if "rc_off" in line:
            out["step_delta_rc_off_ms"].setdefault(model, {})[key] = float(line["rc_off"]["ms_per_step"])
        fo = line.get("failover")
        if fo:
            out["fallback_slowdown"].setdefault(model, {})[key] = fo["post_failover_step_s"] / fo["normal_step_s"]
            out["failover_pause_ms"].setdefault(model, {})[key] = 1e3 * fo["pause_s"]
    return out


def predict_step_ms(constants: Dict, model: str, pipelines: int, stages: int, micro_batches_per_pipeline=None):
    """Step time of a grid that was not measured, from a measured single-pipeline run with the same number of
    stages: a 1F1B step lasts (M + S - 1) micro-batch slots, so one slot is ``ms / (M + S - 1)``; with ``p``
    pipelines sharing the step's micro-batches each runs ``ceil(M / p)`` of them.  The gradient all-reduce across
    replicas is added as the measured ratio of a (2, S') run to its (1, S') run when both exist, else nothing.
    ``None`` when no run with ``stages`` stages was measured."""
    table = constants["step_delta_ms"].get(model) or constants["step_delta_rc_off_ms"].get(model) or {}
    if (pipelines, stages) in table:
        return table[(pipelines, stages)]
    if (1, stages) not in table:
        return None
    per_pipe = constants["micro_batches"].get(model, {}).get((1, stages))
    if not per_pipe:
        return None
    slot = table[(1, stages)] / (per_pipe + stages - 1)
    mine = micro_batches_per_pipeline if micro_batches_per_pipeline is not None else -(-per_pipe // pipelines)
    ratio = 1.0
    for (p2, s2), ms2 in table.items():
        if p2 == 2 and (1, s2) in table:
            same_work = table[(1, s2)]                      # the bench keeps the work per pipeline fixed when replicas are added
            ratio = max(1.0, ms2 / same_work)
            break
    return slot * (mine + stages - 1) * (ratio if pipelines > 1 else 1.0)


def install(simulator, constants: Dict, model: str, stages_target=None):
    """Make ``simulator`` (an object with the reference simulator's attributes ``num_pipelines``,
    ``num_stages``, ``step_delta``, ``fallback_slowdown``, ``simulate_step_delta``, ``num_stages_target``,
    ``samples_per_step``) use the measured numbers of ``model``: ``simulate_step_delta`` then looks ``step_delta``
    up by the current grid (measured, else predicted by ``predict_step_ms``), ``fallback_slowdown`` becomes the mean
    measured slowdown, ``samples_per_step`` the measured global batch and ``num_stages_target`` the measured stage
    count (the largest one, or ``stages_target``)."""
    table = constants["step_delta_ms"].get(model) or constants["step_delta_rc_off_ms"][model]

    def simulate_step_delta():
        key = (simulator.num_pipelines, simulator.num_stages)
        ms = predict_step_ms(constants, model, *key)
        if ms is None:
            raise NotImplementedError(f"no measured step time for {model} on {key[0]} pipelines x {key[1]} stages")
        simulator.step_delta = int(round(ms)) if ms >= 1 else ms
    simulator.simulate_step_delta = simulate_step_delta
    slow = list((constants["fallback_slowdown"].get(model) or {}).values())
    if slow:
        simulator.fallback_slowdown = sum(slow) / len(slow)
    sizes = constants["samples_per_step"].get(model) or {}
    if sizes:
        simulator.samples_per_step = max(sizes.values())
    if hasattr(simulator, "num_stages_target") or stages_target is not None:
        simulator.num_stages_target = stages_target if stages_target is not None else max(s for _, s in table)
    return simulator


def load_reference_simulator(path):
    """The reference's ``project_pactum/simulation/simulator.py`` imported from where it lies (it needs only the
    standard library)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("_reference_simulator", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def run_reference_simulator(simulator_path, bench_lines, model, hours=24.0, seed=1, base_model="GPT-2", stages_target=None,
                            capacity=None, removal_probability=None):
    """Replays the reference's spot-market simulation with this implementation's measured step times.  ``base_model``
    picks the simulator's price / capacity preset that the measured numbers then override."""
    mod = load_reference_simulator(simulator_path)
    sim = mod.Simulator(seed=seed, start_hour=0, model=base_model, removal_probability=removal_probability)
    constants = constants_from_bench(bench_lines)
    install(sim, constants, model, stages_target)
    if capacity is not None:
        sim.spot_instance_desired_capacity = capacity
    return sim.simulate(duration=int(hours * 3600 * 1000)), sim


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser(description="run the reference's cost simulator on measured bench lines")
    ap.add_argument("--simulator", required=True, help="path of project_pactum/simulation/simulator.py")
    ap.add_argument("--bench-lines", required=True, help="file with one bench.py JSON line per measured grid")
    ap.add_argument("--model", default="gpt2-medium")
    ap.add_argument("--base-model", default="GPT-2")
    ap.add_argument("--hours", type=float, default=24.0)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--stages", type=int, default=None)
    ap.add_argument("--capacity", type=int, default=None)
    a = ap.parse_args()
    lines = [l for l in open(a.bench_lines) if l.strip().startswith("{")]
    result, _ = run_reference_simulator(a.simulator, lines, a.model, a.hours, a.seed, a.base_model, a.stages, a.capacity)
    print(result)
