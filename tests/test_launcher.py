"""Launcher CLI and node agent (`python -m bamboo_b200.run`), the counterpart of the reference's
`project_pactum.run` (flags run/__init__.py:23-218, launch run/api.py:252-383, agent agent/api.py:46-397)."""
import json
import os
import subprocess
import sys
import time

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, HERE)
from oracle import gpt_ref  # noqa: E402


def test_command_line_as_the_reference_launcher_takes_it():
    from bamboo_b200 import run
    argv = ["--project-pactum", "--rdzv_backend=etcd-v2", "--rdzv_endpoint=10.0.0.5:2379", "--rdzv_id=job42", "--nnodes=4:16",
            "--nproc_per_node=1", "--rdzv_conf", "timeout=900,last_call_timeout=5", "--max-pipe-parallel-size", "8", "-dps", "4",
            "--max_restarts", "3", "--monitor_interval", "2", "train.py", "--deepspeed_config", "ds.json", "-r", "1"]
    args = run.parse(argv)
    assert args.training_script == "train.py" and args.training_script_args == ["--deepspeed_config", "ds.json", "-r", "1"]
    config, cmd, cmd_args = run.config_from_args(args)
    assert (config.min_nodes, config.max_nodes, config.nproc_per_node) == (4, 16, 1)
    assert (config.rdzv_backend, config.rdzv_endpoint, config.run_id) == ("etcd-v2", "10.0.0.5:2379", "job42")
    assert config.rdzv_configs == {"timeout": "900", "last_call_timeout": "5"}
    assert (config.project_pactum, config.max_pipe_parallel_size, config.default_num_stages) == (True, 8, 4)
    assert (config.max_restarts, config.monitor_interval) == (3, 2.0)
    assert cmd == sys.executable and cmd_args == ["-u", "train.py", "--deepspeed_config", "ds.json", "-r", "1"]
    # module / no-python forms, single node count, static backend endpoint from master address and port
    args = run.parse(["--nnodes", "2", "-m", "--master_addr", "n0", "--master_port", "1234", "pkg.train"])
    config, cmd, cmd_args = run.config_from_args(args)
    assert (config.min_nodes, config.max_nodes, config.rdzv_endpoint, config.rdzv_configs) == (2, 2, "n0:1234", {"rank": 0})
    assert cmd_args == ["-u", "-m", "pkg.train"]
    config, cmd, cmd_args = run.config_from_args(run.parse(["--no_python", "./a.out", "x"]))
    assert cmd == "./a.out" and cmd_args == ["x"]
    with pytest.raises(ValueError):
        run.config_from_args(run.parse(["--no_python", "-m", "mod"]))
    with pytest.raises(ValueError):
        run.parse_rdzv_conf("timeout")
    with pytest.raises(NotImplementedError):
        run.launch_agent(run.LaunchConfig(1, 1, 1), "x", [])


def test_agent_environment_and_preemption_forwarding(tmp_path):
    """The variables a worker gets, and a termination request (operator's SIGTERM or a spot notice) reaching the worker."""
    import fake_etcd
    from bamboo_b200 import run
    from bamboo_b200.rendezvous import create_rdzv_handler
    client = fake_etcd.Client()
    handler = create_rdzv_handler(client, "solo", 1, 1, timeout=30, last_call_timeout=1, etcd_module=fake_etcd)
    handler.write("/rdzv/default_pipelines", 1)
    marker = tmp_path / "got_sigterm"
    script = tmp_path / "sleeper.py"
    script.write_text("import signal, sys, time\n"
                      f"def h(s, f):\n    open({str(marker)!r}, 'w').write('1'); sys.exit(13)\n"
                      "signal.signal(signal.SIGTERM, h)\n"
                      "time.sleep(120)\n")
    fired = {"n": 0}

    def notice():
        fired["n"] += 1
        return fired["n"] >= 3                              # the third poll reports the preemption notice
    config = run.LaunchConfig(1, 1, 1, run_id="solo", monitor_interval=0.2, max_restarts=2, project_pactum=True)
    agent = run.NodeAgent(config, handler, sys.executable, ["-u", str(script)], extra_env={"PROJECT_PACTUM_ENABLED": "1"},
                          notice_source=notice, notice_interval=0.3, master_addr="127.0.0.1")
    result = agent.run()
    handler.stop_keep_alive()
    assert marker.exists()
    assert (result.state, result.exitcode, result.restarts) == ("FAILED", 13, 0)     # a drained worker is not restarted
    env = agent.last_env
    assert (env["RANK"], env["WORLD_SIZE"], env["LOCAL_RANK"], env["MASTER_ADDR"]) == ("0", "1", "0", "127.0.0.1")
    assert (env["PROJECT_PACTUM_NUM_PIPELINES"], env["PROJECT_PACTUM_NUM_STAGES"]) == ("1", "1")
    assert json.loads(env["PROJECT_PACTUM_COORDINATES"]) == [[0, 0]]
    assert env["NCCL_ASYNC_ERROR_HANDLING"] == "1" and env["TORCHELASTIC_RUN_ID"] == "solo" and env["PROJECT_PACTUM_ENABLED"] == "1"
    # several GPUs on a node: one agent per GPU, told which one through its environment
    os.environ["BAMBOO_AGENT_LOCAL_RANK"] = "5"
    try:
        other = run.NodeAgent(config, handler, sys.executable, [], master_addr="127.0.0.1")
        assert other.worker_env(3, 8, 2, 4, [[1, 1]], "127.0.0.1", 29500, 0)["LOCAL_RANK"] == "5"
    finally:
        del os.environ["BAMBOO_AGENT_LOCAL_RANK"]


@pytest.mark.parametrize("standby_once", [False, True])
def test_two_nodes_launched_from_the_command_line(tmp_path, standby_once):
    """Two launcher processes (one per 'node') rendezvous through etcd, start one worker each with nothing but the
    environment, the workers train a 2-stage pipeline on the oracle's trajectory.  With `standby_once` the first workers
    withdraw the rendezvous version and end with 125, as in a reconfiguration: both agents go through another rendezvous
    round and start new workers, no restart is used up."""
    import fake_etcd
    mgr, address = fake_etcd.start_shared_server()
    out = tmp_path / "out"
    out.mkdir()
    env = dict(os.environ)
    env.update({"PYTHONPATH": os.pathsep.join([os.path.join(HERE, "etcd_shim"), ROOT, env.get("PYTHONPATH", "")]),
                "LAUNCHER_TEST_OUT": str(out), "BAMBOO_AGENT_MASTER_ADDR": "127.0.0.1", "BAMBOO_SPOT_NOTICES": "0",
                "OMP_NUM_THREADS": "1"})
    if standby_once:
        env["LAUNCHER_TEST_STANDBY_ONCE"] = "1"
    cmd = [sys.executable, "-m", "bamboo_b200.run", "--project-pactum", "--rdzv_backend", "etcd-v2",
           "--rdzv_endpoint", f"{address[0]}:{address[1]}", "--rdzv_id", "cli", "--nnodes", "2:2", "--default-num-stages", "2",
           "--max-pipe-parallel-size", "2", "--monitor_interval", "0.5", "--rdzv_conf", "timeout=120,last_call_timeout=2",
           "--log_dir", str(tmp_path / "logs"), os.path.join(HERE, "launcher_worker.py")]
    procs = []
    try:
        for node in ("a", "b"):
            procs.append(subprocess.Popen(cmd, env=dict(env, LAUNCHER_TEST_NODE=node), cwd=ROOT, stdout=subprocess.PIPE,
                                          stderr=subprocess.STDOUT, text=True))
        deadline = time.monotonic() + 300
        outs = []
        for p in procs:
            try:
                o, _ = p.communicate(timeout=max(1.0, deadline - time.monotonic()))
            except subprocess.TimeoutExpired:
                p.kill()
                o, _ = p.communicate()
            outs.append(o)
        logs = "\n".join(outs) + "\n".join(open(os.path.join(tmp_path, "logs", f)).read()[-2000:]
                                          for f in sorted(os.listdir(tmp_path / "logs"))) if (tmp_path / "logs").exists() else ""
        assert [p.returncode for p in procs] == [0, 0], logs
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        mgr.shutdown()
    results = [json.load(open(out / f"rank{r}.json")) for r in range(2)]
    cfg = gpt_ref.RefConfig(layers=2, hidden=32, heads=2, ffn=64, seq=8, vocab=48)
    ref = gpt_ref.RefTrainer(cfg, seed=0, lr=1e-3, micro_batches=2)
    data = gpt_ref.synthetic_batches(cfg, 2, 2, 2, seed=1)
    want = [ref.train_batch(data[s]) for s in range(2)]
    last = [r for r in results if r["stage"] == 1][0]
    assert last["losses"] == pytest.approx(want, rel=1e-5)
    for r in results:
        assert r["blocking_wait"] == "1" and r["store"] == "EtcdStore" and r["restart"] == "0"
        assert r["coords"] == [[0, r["stage"]]]
    if standby_once:
        assert (out / "standby_once_a").exists() and (out / "standby_once_b").exists()
