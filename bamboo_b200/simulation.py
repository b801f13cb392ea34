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
         "samples_per_step": {model: {(pipelines, stages): global batch}}}
    """
    out = {"step_delta_ms": {}, "step_delta_rc_off_ms": {}, "fallback_slowdown": {}, "failover_pause_ms": {},
           "samples_per_step": {}}
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
        if "rc_off" in line:
            out["step_delta_rc_off_ms"].setdefault(model, {})[key] = float(line["rc_off"]["ms_per_step"])
        fo = line.get("failover")
        if fo:
            out["fallback_slowdown"].setdefault(model, {})[key] = fo["post_failover_step_s"] / fo["normal_step_s"]
            out["failover_pause_ms"].setdefault(model, {})[key] = 1e3 * fo["pause_s"]
    return out


def install(simulator, constants: Dict, model: str):
    """Make ``simulator`` (an object with the reference simulator's attributes ``num_pipelines``,
    ``num_stages``, ``step_delta``, ``fallback_slowdown``, ``simulate_step_delta``) use the measured
    numbers of ``model``: its ``simulate_step_delta`` then looks ``step_delta`` up by the current
    grid and ``fallback_slowdown`` becomes the mean measured slowdown."""
    table = constants["step_delta_ms"].get(model) or constants["step_delta_rc_off_ms"][model]

    def simulate_step_delta():
        key = (simulator.num_pipelines, simulator.num_stages)
        if key not in table:
            raise NotImplementedError(f"no measured step time for {model} on {key[0]} pipelines x {key[1]} stages")
        simulator.step_delta = table[key]
    simulator.simulate_step_delta = simulate_step_delta
    slow = list((constants["fallback_slowdown"].get(model) or {}).values())
    if slow:
        simulator.fallback_slowdown = sum(slow) / len(slow)
    sizes = constants["samples_per_step"].get(model) or {}
    if sizes:
        simulator.samples_per_step = max(sizes.values())
    return simulator
