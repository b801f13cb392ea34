"""A member that absorbed a failed neighbour's stage is itself preempted: before it leaves, the state of both
of its stages moves to a member that stays, the job re-forms with newcomers, and training continues on the
oracle's trajectory (reference ``save_shadow_node_state``, ``pipe/engine.py:660-727`` + ``:1129-1164``).

Three members run one 3-stage pipeline; the middle one leaves after step 0 (its predecessor takes stage 1
over from its shadow copy); two newcomers arrive and wait; the predecessor - now holding stages 0 and 1, of
which stage 1 has no shadow any more - announces its own preemption for step 3.  At step 3 the rendezvous
decides to reconfigure, the leaving member hands both stages to the survivor, the survivor and the two
newcomers form the new pipeline and the newcomers fetch their layers from the survivor."""
import json
import os
import sys
import time
import traceback

import pytest
import torch
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from oracle import gpt_ref  # noqa: E402

CFG = gpt_ref.RefConfig(layers=4, hidden=32, heads=2, ffn=64, seq=8, vocab=48)
MB, GAS, LR, STEPS = 2, 2, 1e-3, 6
MIDDLE_LEAVES_AT, LOADED_LEAVES_AT = 1, 3
PREFIX, RUN = "/torchelastic/p2p", "handover"


def _newcomers_wait(client, n):
    """True once ``n`` newcomers wait on the final round - or the round is already gone or being re-formed: another
    member saw them first, went on into the step and took the decision."""
    try:
        state = json.loads(client.get(f"{PREFIX}/run_{RUN}/rdzv/active_version").value)
    except Exception:
        return True
    return state.get("status") != "final" or state.get("num_workers_waiting", 0) >= n


def _member(idx, address, late, queue):
    try:
        import fake_etcd
        import cpu_layers
        import torch.distributed as dist
        from bamboo_b200 import api
        from bamboo_b200.module import PipelineModule
        from bamboo_b200.rendezvous import create_rdzv_handler
        from bamboo_b200.topology import PipeDataParallelTopology
        os.environ.update(BAMBOO_QUIET="1", MASTER_ADDR="127.0.0.1")
        torch.set_num_threads(1)
        client = fake_etcd.connect(address)
        if late:
            while True:                                  # arrive once the first failover is over
                try:
                    if json.loads(client.get(f"{PREFIX}/run_{RUN}/rdzv/current_step").value) >= MIDDLE_LEAVES_AT:
                        break
                except Exception:
                    pass
                time.sleep(0.05)
        handler = create_rdzv_handler(client, RUN, 3, 5, prefix=PREFIX, timeout=120, last_call_timeout=2, etcd_module=fake_etcd)
        store, rank, world, pipelines, stages, decision = handler.next_rendezvous()
        first_rank = rank
        dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
        topo = PipeDataParallelTopology(num_pp=stages, num_dp=pipelines, custom_mapping=decision)
        model = PipelineModule(cpu_layers.ref_layer_specs(CFG, 0), topology=topo, loss_fn=cpu_layers.ref_loss(CFG),
                               partition_method="uniform", device="cpu")
        config = {"train_micro_batch_size_per_gpu": MB, "gradient_accumulation_steps": GAS,
                  "optimizer": {"type": "Adam", "params": {"lr": LR}}, "bamboo_b200": {"p2p_timeout_s": 60}}
        engine, *_ = api.initialize(model=model, config=config, redundancy_level=1, rdzv_handler=handler)
        data = gpt_ref.synthetic_batches(CFG, MB, GAS, STEPS, seed=1)
        record = []
        while engine.global_steps < STEPS:
            step = engine.global_steps
            if not late and first_rank == 1 and step == MIDDLE_LEAVES_AT - 1:
                engine.announce_preemption()
            if not late and first_rank == 0 and step == LOADED_LEAVES_AT - 1:
                engine.announce_preemption()
            if not late and step == LOADED_LEAVES_AT:
                # the step at which the job re-forms is fixed by the test: both newcomers are waiting by then
                while not _newcomers_wait(client, 2):
                    time.sleep(0.05)
            loss = float(engine.train_batch(data_iter=iter(data[step])))
            record.append({"step": step, "stages": list(engine.stage_ids), "loss": loss, "rank": engine.global_rank,
                           "last": engine.stage_ids[-1] == engine.num_stages - 1})
        handler.stop_keep_alive()
        queue.put((idx, "ok", {"record": record, "first_rank": first_rank if not late else None,
                               "checksum": sum(float(engine.arenas[s].master.double().sum()) for s in engine.stage_ids)}))
    except SystemExit as e:
        queue.put((idx, "exit", e.code))
    except BaseException:
        queue.put((idx, "error", traceback.format_exc()))


def test_state_of_a_leaving_two_stage_member_survives():
    import fake_etcd
    mgr, address = fake_etcd.start_shared_server()
    fake_etcd.connect(address).write(f"{PREFIX}/run_{RUN}/rdzv/default_pipelines", "3")
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_member, args=(i, address, i >= 3, queue)) for i in range(5)]
    try:
        for p in procs:
            p.start()
        results = {}
        deadline = time.monotonic() + 400
        while len(results) < 5 and time.monotonic() < deadline:
            try:
                idx, status, payload = queue.get(timeout=1.0)
                results[idx] = (status, payload)
            except Exception:
                pass
        assert len(results) == 5, f"members {sorted(set(range(5)) - set(results))} did not finish: {results}"
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
        mgr.shutdown()
    exits = sorted(payload for status, payload in results.values() if status == "exit")
    assert exits == [13, 13], results                      # the middle member, then the member that held two stages
    done = [payload for status, payload in results.values() if status == "ok"]
    assert len(done) == 3, results
    ref = gpt_ref.RefTrainer(CFG, seed=0, lr=LR, micro_batches=GAS)
    data = gpt_ref.synthetic_batches(CFG, MB, GAS, STEPS, seed=1)
    want = [ref.train_batch(data[s]) for s in range(STEPS)]
    seen = {}
    for out in done:
        for rec in out["record"]:
            if rec["last"]:
                seen[rec["step"]] = rec["loss"]
    # every step's loss was reported by whoever owned the last stage at that step, and it is the oracle's
    assert sorted(seen) == list(range(STEPS))
    assert [seen[s] for s in range(STEPS)] == pytest.approx(want, rel=1e-5)
    # the three final members hold the whole model, bit for bit the oracle's sum
    total = sum(float(p.detach().double().sum()) for p in ref.P.values())
    assert sum(out["checksum"] for out in done) == pytest.approx(total, rel=1e-6)
    survivor = [out for out in done if out["first_rank"] == 2][0]
    assert [r["step"] for r in survivor["record"]] == list(range(STEPS))
