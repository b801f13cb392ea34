"""The launcher -> worker environment contract (project_pactum/run/api.py:322-332, agent/api.py:342-362;
consumed by deepspeed/runtime/engine.py:152-184): a worker started with PROJECT_PACTUM_ENABLED builds its
rendezvous handler and its etcd-backed bookkeeping store from the environment alone."""
import json
import os
import sys
import time
import traceback
import types

import pytest
import torch
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from oracle import gpt_ref  # noqa: E402

CFG = gpt_ref.RefConfig(layers=2, hidden=32, heads=2, ffn=64, seq=8, vocab=48)
MB, GAS, LR, STEPS = 2, 2, 1e-3, 2
PREFIX, RUN = "/torchelastic/p2p", "envjob"


def test_endpoint_and_environment_parsing():
    import fake_etcd
    from bamboo_b200 import rendezvous as R
    assert R.parse_endpoint("10.0.0.7:4001") == ("10.0.0.7", 4001)
    assert R.parse_endpoint("etcd.local") == ("etcd.local", 2379)
    assert R.parse_endpoint("[::1]:2380") == ("::1", 2380)
    with pytest.raises(ValueError):
        R.parse_endpoint("host:port")
    assert R.handler_from_env({}) is None
    with pytest.raises(KeyError):
        R.handler_from_env({"PROJECT_PACTUM_ENABLED": "1", "PROJECT_PACTUM_ENDPOINT": "h:1"})
    env = {"PROJECT_PACTUM_ENABLED": "1", "PROJECT_PACTUM_ENDPOINT": "h:1", "PROJECT_PACTUM_RUN_ID": "r7",
           "PROJECT_PACTUM_MIN_NODES": "2", "PROJECT_PACTUM_MAX_NODES": "6",
           "PROJECT_PACTUM_RDZV_CONFIGS": json.dumps({"timeout": 17, "last_call_timeout": 30, "etcd_prefix": "/custom"})}
    handler = R.handler_from_env(env, etcd_module=fake_etcd, client=fake_etcd.Client())
    impl = handler._rdzv_impl
    assert (impl._run_id, impl._num_min_workers, impl._num_max_workers) == ("r7", 2, 6)
    assert impl._timeout == 17 and impl._last_call_timeout == 2      # a worker's last call is 2 s whatever the launcher used
    assert impl.get_path("/rdzv/x").startswith("/custom/run_r7")
    with pytest.raises(ValueError):
        R.create_etcd_client("h:1", {"protocol": "ftp"}, etcd_module=fake_etcd)
    assert R.grid_from_env({}) is None
    assert R.grid_from_env({"PROJECT_PACTUM_NUM_PIPELINES": "2", "PROJECT_PACTUM_NUM_STAGES": "4",
                            "PROJECT_PACTUM_COORDINATES": "[[1, 3]]"}) == (2, 4, [[1, 3]])


def _etcd_shim():
    """A module that stands where `import etcd` would find python-etcd: its Client(host, port, ...) connects to the
    stand-in served at that address."""
    import fake_etcd
    shim = types.ModuleType("etcd")
    for name in dir(fake_etcd):
        if name.startswith("Etcd") or name == "Lock":
            setattr(shim, name, getattr(fake_etcd, name))
    shim.Client = lambda host, port, **_options: fake_etcd.connect((host, port))
    return shim


def _worker(idx, address, queue):
    try:
        import fake_etcd
        import cpu_layers
        import torch.distributed as dist
        from bamboo_b200 import api
        from bamboo_b200.module import PipelineModule
        from bamboo_b200.rendezvous import EtcdRendezvousHandler, EtcdStore, create_rdzv_handler
        from bamboo_b200.topology import PipeDataParallelTopology
        os.environ.update(BAMBOO_QUIET="1", MASTER_ADDR="127.0.0.1")
        torch.set_num_threads(1)
        # ---- what the node agent does: rendezvous, then environment for the worker it starts
        agent = create_rdzv_handler(fake_etcd.connect(address), RUN, 2, 2, prefix=PREFIX, timeout=60, last_call_timeout=2,
                                    etcd_module=fake_etcd)
        store, rank, world, pipelines, stages, decision = agent.next_rendezvous()
        mine = [info for info in decision if info.rank == rank][0]
        os.environ.update({
            "PROJECT_PACTUM_ENABLED": "1", "PROJECT_PACTUM_ENDPOINT": f"{address[0]}:{address[1]}", "PROJECT_PACTUM_RUN_ID": RUN,
            "PROJECT_PACTUM_MIN_NODES": "2", "PROJECT_PACTUM_MAX_NODES": "2",
            "PROJECT_PACTUM_RDZV_CONFIGS": json.dumps({"timeout": 60, "etcd_prefix": PREFIX}),
            "PROJECT_PACTUM_MAX_PIPE_PARALLEL_SIZE": "2", "PROJECT_PACTUM_DEFAULT_PIPELINE_SIZE": "2",
            "PROJECT_PACTUM_NUM_PIPELINES": str(pipelines), "PROJECT_PACTUM_NUM_STAGES": str(stages),
            "PROJECT_PACTUM_COORDINATES": json.dumps(mine.active_coordinates)})
        # ---- the worker: no handler, no store passed in
        sys.modules["etcd"] = _etcd_shim()
        dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
        from bamboo_b200.rendezvous import grid_from_env
        num_dp, num_pp, coords = grid_from_env()
        topo = PipeDataParallelTopology(num_pp=num_pp, num_dp=num_dp, custom_mapping=decision)
        model = PipelineModule(cpu_layers.ref_layer_specs(CFG, 0), topology=topo, loss_fn=cpu_layers.ref_loss(CFG),
                               partition_method="uniform", device="cpu")
        config = {"train_micro_batch_size_per_gpu": MB, "gradient_accumulation_steps": GAS,
                  "optimizer": {"type": "Adam", "params": {"lr": LR}}, "bamboo_b200": {"p2p_timeout_s": 60}}
        engine, *_ = api.initialize(model=model, config=config, redundancy_level=1)
        assert isinstance(engine.rdzv_handler, EtcdRendezvousHandler) and isinstance(engine.global_store, EtcdStore)
        assert engine.max_pipe_parallel_size == "2" and engine.join is False
        assert [list(c) for c in coords] == engine.coordinates
        data = gpt_ref.synthetic_batches(CFG, MB, GAS, STEPS, seed=1)
        losses = [float(engine.train_batch(data_iter=iter(data[s]))) for s in range(STEPS)]
        engine.rdzv_handler.stop_keep_alive()
        agent.stop_keep_alive()
        queue.put((idx, "ok", {"stage": engine.stage_id, "losses": losses, "rank": rank}))
    except SystemExit as e:
        queue.put((idx, "exit", e.code))
    except BaseException:
        queue.put((idx, "error", traceback.format_exc()))


def test_workers_configure_themselves_from_the_environment():
    import fake_etcd
    mgr, address = fake_etcd.start_shared_server()
    client = fake_etcd.connect(address)
    client.write(f"{PREFIX}/run_{RUN}/rdzv/default_pipelines", "2")
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(i, address, queue)) for i in range(2)]
    try:
        for p in procs:
            p.start()
        results = {}
        deadline = time.monotonic() + 240
        while len(results) < 2 and time.monotonic() < deadline:
            try:
                idx, status, payload = queue.get(timeout=1.0)
                results[idx] = (status, payload)
            except Exception:
                pass
        assert len(results) == 2, f"workers {sorted(set(range(2)) - set(results))} did not finish"
        for idx, (status, payload) in results.items():
            assert status == "ok", payload
        # the bookkeeping keys live in etcd under the rendezvous version's kv directory (values base64, as the store writes them)
        version = json.loads(client.get(f"{PREFIX}/run_{RUN}/rdzv/active_version").value)["version"]
        kv = client.get(f"{PREFIX}/run_{RUN}/rdzv/v_{version}/kv")
        names = {child.key.rsplit("/", 1)[-1] for child in kv.children}
        assert len(names) >= 3, names                     # rank flags "0", "1" and "failures"
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
        mgr.shutdown()
    ref = gpt_ref.RefTrainer(CFG, seed=0, lr=LR, micro_batches=GAS)
    data = gpt_ref.synthetic_batches(CFG, MB, GAS, STEPS, seed=1)
    want = [ref.train_batch(data[s]) for s in range(STEPS)]
    last = [payload for _, (status, payload) in results.items() if payload["stage"] == 1][0]
    assert last["losses"] == pytest.approx(want, rel=1e-5)
