"""Elastic growth of a running job on GPUs: one member trains a one-stage model alone; a second member
arrives and waits; the rendezvous decides to reconfigure; both re-join, the NCCL process group is rebuilt
for two replicas, the newcomer fetches every layer and its Adam moments from the old member over NCCL
send / recv, and training continues on the oracle's trajectory with the gradients averaged over the two
replicas (bf16 tolerance).  The members talk to the in-process etcd stand-in served from a manager process.
Needs two GPUs; skipped otherwise."""
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

pytestmark = pytest.mark.gpu
CFG = gpt_ref.RefConfig(layers=2, hidden=256, heads=4, ffn=1024, seq=128, vocab=1024)
MB, GAS, LR, STEPS, GROW_AT = 2, 2, 1e-4, 4, 2
PREFIX, RUN = "/torchelastic/p2p", "gpu-elastic"


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
        import torch.distributed as dist
        from bamboo_b200 import api, lib, models
        from bamboo_b200.module import PipelineModule
        from bamboo_b200.rendezvous import create_rdzv_handler
        from bamboo_b200.topology import PipeDataParallelTopology
        os.environ.update(BAMBOO_QUIET="1", MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0",
                          LOCAL_RANK=str(idx))        # the GPU of a worker is the one its launcher names
        torch.cuda.set_device(idx)
        client = fake_etcd.connect(address)
        if late:
            while True:
                try:
                    if json.loads(client.get(f"{PREFIX}/run_{RUN}/rdzv/current_step").value) >= GROW_AT - 1:
                        break
                except Exception:
                    pass
                time.sleep(0.05)
        handler = create_rdzv_handler(client, RUN, 1, 2, prefix=PREFIX, timeout=120, last_call_timeout=2, etcd_module=fake_etcd)
        store, rank, world, pipelines, stages, decision = handler.next_rendezvous()
        dist.init_process_group("nccl", store=store, rank=rank, world_size=world)
        topo = PipeDataParallelTopology(num_pp=stages, num_dp=pipelines, custom_mapping=decision)
        tc = models.TransformerConfig(layers=CFG.layers, hidden=CFG.hidden, heads=CFG.heads, ffn=CFG.ffn, seq=CFG.seq, vocab=CFG.vocab)
        model = PipelineModule(models.transformer_layer_specs(tc, 0), topology=topo, loss_fn=models.transformer_loss(tc),
                               partition_method="uniform")
        config = {"train_micro_batch_size_per_gpu": MB, "gradient_accumulation_steps": GAS, "bf16": {"enabled": True},
                  "optimizer": {"type": "Adam", "params": {"lr": LR}}, "bamboo_b200": {"p2p_timeout_s": 60}}
        engine, *_ = api.initialize(model=model, config=config, redundancy_level=0, rdzv_handler=handler)
        data = gpt_ref.synthetic_batches(CFG, MB, GAS * 2, STEPS, seed=1)
        record = []
        while engine.global_steps < STEPS:
            step = engine.global_steps
            if step == GROW_AT and not late and engine.dp_world_size == 1:
                while not _newcomers_wait(client, 1):                # the step at which the job grows is fixed by the test
                    time.sleep(0.05)
            batches = data[step]

            def feed(step_batches=batches):
                r = engine.grid.get_data_parallel_id()
                yield from step_batches[r * GAS:(r + 1) * GAS]
            loss = float(engine.train_batch(data_iter=feed()))
            record.append({"step": step, "dp": engine.dp_world_size, "replica": engine.grid.get_data_parallel_id(), "loss": loss})
        torch.cuda.synchronize()
        out = {"record": record, "status": lib.read_status(),
               "checksum": float(engine.arenas[engine.stage_id].master.double().sum()),
               "received_s": engine.timers.get("layer_transfer_s")}
        handler.stop_keep_alive()
        dist.destroy_process_group()
        queue.put((idx, "ok", out))
    except SystemExit as e:
        queue.put((idx, "exit", e.code))
    except BaseException:
        queue.put((idx, "error", traceback.format_exc()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_job_grows_from_one_replica_to_two_on_gpus():
    import fake_etcd
    mgr, address = fake_etcd.start_shared_server()
    fake_etcd.connect(address).write(f"{PREFIX}/run_{RUN}/rdzv/default_pipelines", "1")     # one stage per pipeline
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_member, args=(i, address, i >= 1, queue)) for i in range(2)]
    try:
        for p in procs:
            p.start()
        results = {}
        deadline = time.monotonic() + 300
        while len(results) < 2 and time.monotonic() < deadline:
            try:
                idx, status, payload = queue.get(timeout=1.0)
                results[idx] = (status, payload)
            except Exception:
                pass
        assert len(results) == 2, f"members {sorted(set(range(2)) - set(results))} did not finish: {results}"
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
        mgr.shutdown()
    for idx, (status, payload) in results.items():
        assert status == "ok", payload
        assert payload["status"] == 0
    # oracle: GAS micro-batches per step before the growth, 2 x GAS afterwards (two replicas averaged)
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
            assert rec["loss"] == pytest.approx(want[(rec["step"], rec["replica"])], rel=2e-2), rec
            seen.add((rec["step"], rec["replica"]))
    assert seen == set(want)
    # both replicas hold the same weights at the end, and the newcomer received them over the wire
    assert results[0][1]["checksum"] == pytest.approx(results[1][1]["checksum"], rel=1e-6)
    assert results[1][1]["received_s"] is not None
