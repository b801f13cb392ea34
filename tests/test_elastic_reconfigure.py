"""Elastic re-formation of a running job on CPU ranks: two members train one 2-stage pipeline;
two more arrive and wait; the rendezvous decides to reconfigure; all four re-join, the process
group and the pipeline module are rebuilt for a 2 x 2 grid, the newcomers fetch their stages'
layers and Adam moments from the old members, and training continues on the oracle's trajectory
(now averaging gradients over two replicas).  The members talk to one in-process etcd stand-in
served from a manager process."""
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

CFG = gpt_ref.RefConfig(layers=4, hidden=64, heads=4, ffn=128, seq=16, vocab=96)
MB, GAS, LR, STEPS, GROW_AT = 2, 2, 1e-3, 4, 2
PREFIX, RUN = "/torchelastic/p2p", "elastic"


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
            # newcomers show up while the first two run the step before the one at which the job is to
            # grow (the decision of a step records its number as rdzv/current_step)
            while True:
                try:
                    if json.loads(client.get(f"{PREFIX}/run_{RUN}/rdzv/current_step").value) >= GROW_AT - 1:
                        break
                except Exception:
                    pass
                time.sleep(0.05)
        handler = create_rdzv_handler(client, RUN, 2, 4, prefix=PREFIX, timeout=120, last_call_timeout=2,
                                      etcd_module=fake_etcd)
        store, rank, world, pipelines, stages, decision = handler.next_rendezvous()
        dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
        topo = PipeDataParallelTopology(num_pp=stages, num_dp=pipelines, custom_mapping=decision)
        model = PipelineModule(cpu_layers.ref_layer_specs(CFG, 0), topology=topo, loss_fn=cpu_layers.ref_loss(CFG),
                               partition_method="uniform", device="cpu")
        config = {"train_micro_batch_size_per_gpu": MB, "gradient_accumulation_steps": GAS,
                  "optimizer": {"type": "Adam", "params": {"lr": LR}}, "bamboo_b200": {"p2p_timeout_s": 60}}
        engine, *_ = api.initialize(model=model, config=config, redundancy_level=1, rdzv_handler=handler)
        data = gpt_ref.synthetic_batches(CFG, MB, GAS * 2, STEPS, seed=1)
        record = []
        while engine.global_steps < STEPS:
            step = engine.global_steps
            if step == GROW_AT and not late and engine.dp_world_size == 1:
                while not _newcomers_wait(client, 2):            # the step at which the job grows is fixed by the test
                    time.sleep(0.05)
            batches = data[step]
            # micro-batches of a step are dealt to the replicas in blocks; a replica learns its id only
            # inside train_batch when the grid changes, so it is handed an iterator that looks it up late
            def feed(step_batches=batches):
                r = engine.grid.get_data_parallel_id()
                yield from step_batches[r * GAS:(r + 1) * GAS]
            loss = float(engine.train_batch(data_iter=feed()))
            record.append({"step": step, "dp": engine.dp_world_size, "replica": engine.grid.get_data_parallel_id(),
                           "stage": engine.stage_id, "loss": loss, "rank": engine.global_rank})
        out = {"record": record, "stage": engine.stage_id, "replica": engine.grid.get_data_parallel_id(),
               "checksum": float(engine.arenas[engine.stage_id].master.double().sum()),
               "received_s": engine.timers.get("layer_transfer_s")}
        handler.stop_keep_alive()
        queue.put((idx, "ok", out))
    except SystemExit as e:
        queue.put((idx, "exit", e.code))
    except BaseException:
        queue.put((idx, "error", traceback.format_exc()))


def test_job_grows_from_one_pipeline_to_two():
    import fake_etcd
    mgr, address = fake_etcd.start_shared_server()
    # what the launcher publishes before any member joins: the number of stages of a pipeline
    fake_etcd.connect(address).write(f"{PREFIX}/run_{RUN}/rdzv/default_pipelines", "2")
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_member, args=(i, address, i >= 2, queue)) for i in range(4)]
    try:
        for p in procs:
            p.start()
        results = {}
        deadline = time.monotonic() + 300
        while len(results) < 4 and time.monotonic() < deadline:
            try:
                idx, status, payload = queue.get(timeout=1.0)
                results[idx] = (status, payload)
            except Exception:
                pass
        assert len(results) == 4, f"members {sorted(set(range(4)) - set(results))} did not finish"
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
        mgr.shutdown()
    for idx, (status, payload) in results.items():
        assert status == "ok", payload

    # oracle: steps before the growth use GAS micro-batches, afterwards 2 x GAS (two replicas averaged)
    ref = gpt_ref.RefTrainer(CFG, seed=0, lr=LR, micro_batches=GAS)
    data = gpt_ref.synthetic_batches(CFG, MB, GAS * 2, STEPS, seed=1)
    want = {}
    for step in range(STEPS):
        dp = 1 if step < GROW_AT else 2
        used = data[step][:GAS * dp]
        with torch.no_grad():
            for r in range(dp):
                want[(step, r)] = sum(float(gpt_ref.forward_loss(CFG, ref.P, t, l)) for t, l in used[r * GAS:(r + 1) * GAS]) / GAS
        ref.micro_batches = GAS * dp
        ref.train_batch(used)
    seen = set()
    for idx, (_, out) in results.items():
        for rec in out["record"]:
            assert rec["dp"] == (1 if rec["step"] < GROW_AT else 2), rec
            if rec["stage"] == 1:                       # the last stage reports the loss
                assert rec["loss"] == pytest.approx(want[(rec["step"], rec["replica"])], rel=1e-5), rec
                seen.add((rec["step"], rec["replica"]))
    assert seen == set(want)
    # members that arrived late received their stage's layers; final weights are the oracle's
    late = [results[i][1] for i in (2, 3)]
    assert all(o["received_s"] is not None for o in late)
    total = sum(float(p.detach().double().sum()) for p in ref.P.values())
    by_seat = {(o["replica"], o["stage"]): o["checksum"] for _, (s, o) in results.items()}
    assert len(by_seat) == 4
    for replica in (0, 1):
        assert by_seat[(replica, 0)] + by_seat[(replica, 1)] == pytest.approx(total, rel=1e-6)
