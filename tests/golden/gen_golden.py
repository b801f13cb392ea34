"""Generate golden vectors by running the reference's own code in place.

Run where a checkout of uclasystem/bamboo is available:

    python tests/golden/gen_golden.py /path/to/bamboo

It imports (never copies) the reference's pipeline schedule generators, partition
helpers, topology tables and redundancy maps through the stubs in ``_ref_shims`` and
writes:

* ``schedules.json.gz`` - instruction streams (list of steps, each a list of
  ``repr(instruction)`` strings) for every stage of the (stages, micro_batches) pairs
  used by the benchmark configurations, for the plain, lazy-RC and eager-RC schedules
  and for every next-stage / prev-stage / all-reduce failover composition, including
  redo windows (``failed_step``/``curr_step`` > 0).  A composition on which the
  reference raises is recorded as ``{"raises": "<ExceptionType>"}``.
* ``partition.json`` - ``partition_uniform`` / ``partition_balanced`` answers.
* ``topology.json`` - rank/coordinate tables, communicator lists and fallback
  data-parallel groups.
"""
import gzip
import json
import os
import random
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import _ref_shims  # noqa: E402

GRID = [(1, 4), (2, 4), (2, 1), (3, 5), (4, 16), (8, 32), (4, 32), (4, 2), (5, 3)]
REDO = [(0, 0), (3, 5), (5, 5), (2, 7)]


def _dump(sched):
    try:
        return [[repr(c) for c in step] for step in sched]
    except Exception as e:  # the reference raises on some compositions
        return {"raises": type(e).__name__}


def gen_schedules(S):
    out = {}
    for stages, mb in GRID:
        def train(s):
            return S.TrainSchedule(micro_batches=mb, stages=stages, stage_id=s)

        def rc(mode, s):
            cls = S.LazyRecoverySchedule if mode == "lazy" else S.EagerRecoverySchedule
            return cls(train(s), train((s + 1) % stages))

        for s in range(stages):
            out[f"S{stages}M{mb}/train/stage{s}"] = _dump(train(s))
            if stages == 1:
                continue
            for mode in ("lazy", "eager"):
                out[f"S{stages}M{mb}/{mode}/stage{s}"] = _dump(rc(mode, s))
        if stages == 1:
            continue
        for victim in range(stages):
            pred = (victim - 1) % stages
            succ = (victim + 1) % stages
            for base in ("train", "lazy", "eager"):
                def own(s):
                    return train(s) if base == "train" else rc(base, s)
                for fs, cs in REDO:
                    if (fs, cs) != (0, 0) and (stages, mb) not in ((2, 4), (4, 16), (3, 5)):
                        continue
                    tag = f"S{stages}M{mb}/{base}/victim{victim}/f{fs}c{cs}"
                    out[f"{tag}/next_on_stage{pred}"] = _dump(
                        S.NextStageFailoverSchedule(own(pred), train(victim),
                                                    failed_step=fs, curr_step=cs))
                    out[f"{tag}/prev_on_stage{succ}"] = _dump(
                        S.PrevStageFailoverSchedule(train(victim), own(succ),
                                                    failed_step=fs, curr_step=cs))
                    out[f"{tag}/allreduce_on_stage{victim}"] = _dump(
                        S.AllReduceFailoverSchedule(own(victim),
                                                    [[] for _ in own(victim)],
                                                    failed_step=fs))
    return out


def gen_partition(U):
    rng = random.Random(1234)
    uni = {f"{n},{p}": U.partition_uniform(n, p)
           for n in range(0, 40) for p in range(1, 10)}
    bal = []
    for _ in range(200):
        n = rng.randint(1, 60)
        p = rng.randint(1, 12)
        if rng.random() < 0.5:
            w = [rng.randint(0, 20) for _ in range(n)]
        else:
            w = [round(rng.random() * 10, 3) for _ in range(n)]
        bal.append({"weights": w, "parts": p, "answer": U.partition_balanced(w, p)})
    # layer-weight vectors shaped like the benchmark models (embedding, blocks, norm, head)
    for layers, stages in ((24, 4), (24, 8), (32, 4), (4, 2)):
        w = [51_000_000] + [12_600_000] * layers + [2048, 51_000_000]
        bal.append({"weights": w, "parts": stages,
                    "answer": U.partition_balanced(w, stages)})
    return {"uniform": uni, "balanced": bal}


def gen_topology(T, R):
    out = {"grids": [], "redundancy": []}
    for pp, dp in ((1, 1), (2, 1), (4, 1), (8, 1), (4, 2), (2, 4), (3, 3)):
        topo = T.PipeDataParallelTopology(num_pp=pp, num_dp=dp)
        world = topo.world_size()
        entry = {
            "pp": pp, "dp": dp,
            "coords": [list(topo.get_coord(r)) for r in range(world)],
            "pipe_lists": topo.get_axis_comm_lists("pipe"),
            "data_lists": topo.get_axis_comm_lists("data"),
            "axis_pipe0": topo.get_axis_list("pipe", 0),
            "match_data0": topo.filter_match(data=0),
            "rank_repr": [topo.get_rank_repr(r, omit_axes=[]) for r in range(world)],
        }
        # fallback data-parallel groups (PipelineParallelGrid.init_fallback_group maths,
        # evaluated without creating process groups)
        fb = {}
        for ranks in topo.get_axis_comm_lists("data"):
            for rank in ranks:
                coord = topo.get_coord(rank)
                f_coord = coord._replace(pipe=(coord.pipe - 1) % pp)
                f_rank = topo.get_rank(**f_coord._asdict())
                fb[str(rank)] = [r if r != rank else f_rank for r in ranks]
        entry["fallback"] = fb
        out["grids"].append(entry)
    for level in (0, 1):
        for stages in (1, 2, 4, 8):
            for s in range(stages):
                out["redundancy"].append({
                    "level": level, "stages": stages, "stage": s,
                    "shadows": R.get_redundant_stage_ids(level, s, stages),
                    "shadowed_by": R.get_redundant_user_stage_ids(level, s, stages)})
    return out


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BAMBOO_REFERENCE")
    if not ref:
        sys.exit("usage: gen_golden.py <path of the reference checkout>  (or set BAMBOO_REFERENCE)")
    _ref_shims.install(ref)
    from deepspeed.runtime.pipe import schedule as S, topology as T, redundancy as R
    from deepspeed.runtime import utils as U

    sched = gen_schedules(S)
    with gzip.GzipFile(os.path.join(HERE, "schedules.json.gz"), "wb", mtime=0) as f:
        f.write(json.dumps(sched, sort_keys=True).encode())
    with open(os.path.join(HERE, "partition.json"), "w") as f:
        json.dump(gen_partition(U), f)
    with open(os.path.join(HERE, "topology.json"), "w") as f:
        json.dump(gen_topology(T, R), f)
    n_raise = sum(1 for v in sched.values() if isinstance(v, dict))
    print(f"{len(sched)} streams ({n_raise} raise in the reference)")


if __name__ == "__main__":
    main()
