"""Launcher and node agent: ``python -m bamboo_b200.run [flags] training_script [script args]``.

Command line, environment handed to the workers and etcd keys are those of the reference's
``project_pactum.run`` (flags: ``project_pactum/run/__init__.py:23-218``; launch:
``project_pactum/run/api.py:252-383``; agent: ``project_pactum/agent/api.py:46-397``), so job scripts
and tooling written for it keep working.  The agent itself is written from scratch for one worker per
node (the reference asserts ``nproc_per_node == 1``): it does not build on torchelastic's agent
classes, it runs the worker as a child process and watches it.

One agent runs per node:

1. rendezvous through the etcd handler until this node holds a seat (a node without coordinates
   waits for the next round);
2. the node of rank 0 publishes the master address / port in the rendezvous store, the others read it;
3. the worker is started with the torchelastic variables (``RANK``, ``WORLD_SIZE``, ``MASTER_*`` ...),
   the grid variables ``PROJECT_PACTUM_NUM_PIPELINES / NUM_STAGES / COORDINATES`` and the job description
   ``PROJECT_PACTUM_ENABLED / ENDPOINT / RUN_ID / MIN_NODES / MAX_NODES / RDZV_CONFIGS /
   MAX_PIPE_PARALLEL_SIZE / DEFAULT_PIPELINE_SIZE`` and ``NCCL_BLOCKING_WAIT=1``;
4. every ``monitor_interval`` seconds the worker is polled: exit code 0 ends the agent; 125 ("put me on
   standby / re-form the job") starts over at 1 without using up a restart; any other failure starts over
   while restarts remain; new nodes that wait do NOT restart a healthy worker (the engine re-forms the job
   itself at the next step boundary);
   On a node with several GPUs one agent runs per GPU, each with ``BAMBOO_AGENT_LOCAL_RANK=<gpu index>`` in
   its environment (the worker's ``LOCAL_RANK``; default 0, the reference's one-GPU nodes);
5. SIGTERM to the agent - sent by the operator or by the spot-notice poller - is passed on to the worker,
   whose engine then announces its preemption and leaves between steps.
"""
import argparse
import dataclasses
import json
import os
import signal
import socket
import subprocess
import sys
import threading
import time
import uuid
from typing import Callable, Dict, List, Optional, Tuple

from . import rendezvous as _rdzv

EXIT_STANDBY = 125          # worker: this node holds no seat any more / wants the job re-formed
EXIT_PREEMPTED = 13         # worker: left because its node is going away


# ------------------------------------------------------------------------------------------ command line
class _Env(argparse.Action):
    """Default from the environment variable ``PET_<DEST>`` (as torchrun's flags)."""

    def __init__(self, dest, default=None, required=False, **kw):
        default = os.environ.get(f"PET_{dest.upper()}", default)
        super().__init__(dest=dest, default=default, required=False, **kw)

    def __call__(self, parser, namespace, values, option_string=None):
        setattr(namespace, self.dest, values)


class _CheckEnv(argparse.Action):
    """Boolean flag, on when given or when ``PET_<DEST>=1``."""

    def __init__(self, dest, default=False, **kw):
        default = bool(int(os.environ.get(f"PET_{dest.upper()}", "1" if default else "0")))
        super().__init__(dest=dest, const=True, default=default, nargs=0, **kw)

    def __call__(self, parser, namespace, values, option_string=None):
        setattr(namespace, self.dest, self.const)


def parse(argv):
    p = argparse.ArgumentParser(prog="bamboo_b200.run", description="launcher of an elastic pipeline-parallel job")
    p.add_argument("--project-pactum", action="store_true")
    p.add_argument("--max-pipe-parallel-size", type=int)
    p.add_argument("--default-num-stages", "-dps", type=int)
    p.add_argument("--nnodes", action=_Env, type=str, default="1:1")
    p.add_argument("--nproc_per_node", action=_Env, type=str, default="1")
    p.add_argument("--rdzv_backend", action=_Env, type=str, default="static")
    p.add_argument("--rdzv_endpoint", action=_Env, type=str, default="")
    p.add_argument("--rdzv_id", action=_Env, type=str, default="none")
    p.add_argument("--rdzv_conf", action=_Env, type=str, default="")
    p.add_argument("--standalone", action=_CheckEnv)
    p.add_argument("--max_restarts", action=_Env, type=int, default=0)
    p.add_argument("--monitor_interval", action=_Env, type=float, default=5)
    p.add_argument("--start_method", action=_Env, type=str, default="spawn", choices=["spawn", "fork", "forkserver"])
    p.add_argument("--role", action=_Env, type=str, default="default")
    p.add_argument("-m", "--module", action=_CheckEnv)
    p.add_argument("--no_python", action=_CheckEnv)
    p.add_argument("--run_path", action=_CheckEnv)
    p.add_argument("--log_dir", action=_Env, type=str, default=None)
    p.add_argument("-r", "--redirects", action=_Env, type=str, default="0")
    p.add_argument("-t", "--tee", action=_Env, type=str, default="0")
    p.add_argument("--node_rank", action=_Env, type=int, default=0)
    p.add_argument("--master_addr", action=_Env, type=str, default="127.0.0.1")
    p.add_argument("--master_port", action=_Env, type=int, default=29500)
    p.add_argument("--use_env", default=True, action="store_true")
    p.add_argument("training_script", type=str)
    p.add_argument("training_script_args", nargs=argparse.REMAINDER)
    args = p.parse_args(argv)
    for name in ("max_restarts", "node_rank", "master_port"):          # values that came from the environment are strings
        setattr(args, name, int(getattr(args, name)))
    args.monitor_interval = float(args.monitor_interval)
    return args


@dataclasses.dataclass
class LaunchConfig:
    min_nodes: int
    max_nodes: int
    nproc_per_node: int
    run_id: str = ""
    role: str = "default"
    rdzv_endpoint: str = ""
    rdzv_backend: str = "etcd"
    rdzv_configs: Dict = dataclasses.field(default_factory=dict)
    max_restarts: int = 0
    monitor_interval: float = 5.0
    start_method: str = "spawn"
    log_dir: Optional[str] = None
    project_pactum: bool = False
    max_pipe_parallel_size: int = 2
    default_num_stages: int = 2


def parse_min_max_nnodes(text):
    parts = str(text).split(":")
    if len(parts) == 1:
        return int(parts[0]), int(parts[0])
    if len(parts) == 2:
        return int(parts[0]), int(parts[1])
    raise RuntimeError(f'nnodes={text} is not in "MIN:MAX" format')


def parse_rdzv_conf(text):
    """``key1=value1,key2=value2`` -> dict (values stay strings, as torchelastic leaves them)"""
    out = {}
    for item in filter(None, (s.strip() for s in (text or "").split(","))):
        key, sep, value = item.partition("=")
        if not sep or not key.strip() or not value.strip():
            raise ValueError("The rendezvous configuration string must be in format <key1>=<value1>,...,<keyN>=<valueN>.")
        out[key.strip()] = value.strip()
    return out


def config_from_args(args) -> Tuple[LaunchConfig, str, List[str]]:
    min_nodes, max_nodes = parse_min_max_nnodes(args.nnodes)
    assert 0 < min_nodes <= max_nodes
    assert args.max_restarts >= 0
    nproc = int(args.nproc_per_node)
    configs = parse_rdzv_conf(args.rdzv_conf)
    if args.rdzv_backend == "static":
        configs["rank"] = args.node_rank
        endpoint = args.rdzv_endpoint or f"{args.master_addr}:{args.master_port}"
    else:
        endpoint = args.rdzv_endpoint
    config = LaunchConfig(min_nodes=min_nodes, max_nodes=max_nodes, nproc_per_node=nproc, run_id=args.rdzv_id, role=args.role,
                          rdzv_endpoint=endpoint, rdzv_backend=args.rdzv_backend, rdzv_configs=configs,
                          max_restarts=args.max_restarts, monitor_interval=args.monitor_interval, start_method=args.start_method,
                          log_dir=args.log_dir, project_pactum=args.project_pactum,
                          max_pipe_parallel_size=args.max_pipe_parallel_size, default_num_stages=args.default_num_stages)
    cmd_args: List[str] = []
    if not args.no_python:
        cmd = sys.executable
        cmd_args.append("-u")
        if args.module:
            cmd_args.append("-m")
        cmd_args.append(args.training_script)
    else:
        if args.module:
            raise ValueError("Don't use both the '--no_python' flag and the '--module' flag at the same time.")
        cmd = args.training_script
    cmd_args.extend(args.training_script_args)
    return config, cmd, cmd_args


# ------------------------------------------------------------------------------------------ spot notices
def ec2_spot_notice(timeout=2.0) -> bool:
    """True once the EC2 instance metadata service announces that this spot instance will be reclaimed
    (the reference polls the same endpoint, ``project_pactum/agent/get_notices.py``)."""
    import urllib.error
    import urllib.request
    base = "http://169.254.169.254/latest"
    try:
        req = urllib.request.Request(f"{base}/api/token", method="PUT", headers={"X-aws-ec2-metadata-token-ttl-seconds": "21600"})
        token = urllib.request.urlopen(req, timeout=timeout).read().decode()
        req = urllib.request.Request(f"{base}/meta-data/spot/instance-action", headers={"X-aws-ec2-metadata-token": token})
        return urllib.request.urlopen(req, timeout=timeout).status == 200
    except (urllib.error.URLError, OSError, ValueError):
        return False


# ------------------------------------------------------------------------------------------ the agent
@dataclasses.dataclass
class RunResult:
    state: str                       # "SUCCEEDED" | "FAILED"
    exitcode: int = 0
    restarts: int = 0
    rounds: int = 0                  # rendezvous rounds this agent took part in


class NodeAgent:
    def __init__(self, config: LaunchConfig, handler, cmd: str, cmd_args: List[str], extra_env: Optional[Dict[str, str]] = None,
                 notice_source: Optional[Callable[[], bool]] = None, notice_interval: float = 3.0, master_addr: Optional[str] = None,
                 master_port: Optional[int] = None, log=None):
        assert config.nproc_per_node == 1, "one worker per node"
        self.config, self.handler, self.cmd, self.cmd_args = config, handler, cmd, list(cmd_args)
        self.extra_env = dict(extra_env or {})
        self.master_addr, self.master_port = master_addr, master_port
        # one agent per node in the reference (one GPU per node); on a multi-GPU node one agent runs per GPU
        # and BAMBOO_AGENT_LOCAL_RANK names the GPU of this agent's worker
        self.local_rank = str(int(os.environ.get("BAMBOO_AGENT_LOCAL_RANK", "0")))
        self._remaining_restarts = config.max_restarts
        self._proc: Optional[subprocess.Popen] = None
        self._draining = False
        self._log = log or (lambda msg: print(f"[agent {os.getpid()}] {msg}", file=sys.stderr, flush=True))
        self.rounds = 0
        self.last_env: Dict[str, str] = {}
        try:
            signal.signal(signal.SIGTERM, self._drain)
        except ValueError:
            pass                         # not the main thread (tests): drain() is called directly
        if notice_source is not None:
            threading.Thread(target=self._watch_notices, args=(notice_source, notice_interval), daemon=True).start()

    # ---- preemption
    def _watch_notices(self, source, interval):
        while not self._draining:
            try:
                if source():
                    self._log("preemption notice: draining the worker")
                    self._drain()
                    return
            except Exception as e:  # noqa: BLE001 - a broken poller must not take the agent down
                self._log(f"notice poller: {e!r}")
            time.sleep(interval)

    def _drain(self, signum=None, frame=None):
        """Pass the termination on to the worker: its engine announces the preemption and leaves between steps."""
        self._draining = True
        proc = self._proc
        if proc is not None and proc.poll() is None:
            proc.send_signal(signal.SIGTERM)

    # ---- one round
    def _rendezvous(self):
        while True:
            store, rank, world, pipelines, stages, decision = self.handler.next_rendezvous()
            self.rounds += 1
            coords = []
            for info in decision:
                if info.rank == rank:
                    coords = info.active_coordinates
            if len(coords) != 0:                      # a node without a seat does not start a worker: next round
                return store, rank, world, pipelines, stages, decision, coords

    def _master(self, store, rank):
        if rank == 0:
            addr = self.master_addr or os.environ.get("BAMBOO_AGENT_MASTER_ADDR") or socket.getfqdn()
            port = self.master_port
            if not port:
                with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
                    s.bind(("", 0))
                    port = s.getsockname()[1]
            store.set("MASTER_ADDR", addr.encode())
            store.set("MASTER_PORT", str(port).encode())
        addr = store.get("MASTER_ADDR")
        port = store.get("MASTER_PORT")
        dec = lambda v: v.decode() if isinstance(v, (bytes, bytearray)) else str(v)  # noqa: E731
        return dec(addr), int(dec(port))

    def worker_env(self, rank, world, pipelines, stages, coords, master_addr, master_port, restart_count) -> Dict[str, str]:
        env = {
            "LOCAL_RANK": self.local_rank, "RANK": str(rank), "GROUP_RANK": str(rank), "ROLE_RANK": str(rank), "ROLE_NAME": self.config.role,
            "LOCAL_WORLD_SIZE": "1", "WORLD_SIZE": str(world), "GROUP_WORLD_SIZE": str(world), "ROLE_WORLD_SIZE": str(world),
            "MASTER_ADDR": master_addr, "MASTER_PORT": str(master_port),
            "TORCHELASTIC_RESTART_COUNT": str(restart_count), "TORCHELASTIC_MAX_RESTARTS": str(self.config.max_restarts),
            "TORCHELASTIC_RUN_ID": str(self.config.run_id), "TORCHELASTIC_USE_AGENT_STORE": str(self.handler.get_backend() == "static"),
            "NCCL_ASYNC_ERROR_HANDLING": "1",
            "PROJECT_PACTUM_NUM_PIPELINES": str(pipelines), "PROJECT_PACTUM_NUM_STAGES": str(stages),
            "PROJECT_PACTUM_COORDINATES": json.dumps(coords),
        }
        if "OMP_NUM_THREADS" in os.environ:
            env["OMP_NUM_THREADS"] = os.environ["OMP_NUM_THREADS"]
        env.update(self.extra_env)
        return env

    def _start_worker(self):
        store, rank, world, pipelines, stages, decision, coords = self._rendezvous()
        addr, port = self._master(store, rank)
        restart_count = self.config.max_restarts - self._remaining_restarts
        self.last_env = self.worker_env(rank, world, pipelines, stages, coords, addr, port, restart_count)
        self._log(f"rendezvous complete: rank {rank} of {world}, grid {pipelines} x {stages}, coordinates {coords}, "
                  f"master {addr}:{port}, restart {restart_count}")
        env = dict(os.environ)
        env.update(self.last_env)
        out = None
        if self.config.log_dir:
            os.makedirs(self.config.log_dir, exist_ok=True)
            out = open(os.path.join(self.config.log_dir, f"{self.config.run_id}_rank{rank}_attempt{restart_count}_{self.rounds}.log"), "w")
        self._proc = subprocess.Popen([self.cmd] + self.cmd_args, env=env, stdout=out, stderr=subprocess.STDOUT if out else None)
        if out is not None:
            out.close()                                  # the child holds its own descriptor
        if self._draining:
            self._drain()

    def _stop_worker(self):
        proc = self._proc
        if proc is not None and proc.poll() is None:
            proc.terminate()
            try:
                proc.wait(timeout=30)
            except subprocess.TimeoutExpired:
                proc.kill()
        self._proc = None

    def run(self) -> RunResult:
        self._start_worker()
        while True:
            time.sleep(self.config.monitor_interval)
            code = self._proc.poll()
            if code is None:
                continue                                        # healthy; waiting nodes do not restart it
            restarts = self.config.max_restarts - self._remaining_restarts
            if code == 0:
                self._log("worker finished")
                return RunResult("SUCCEEDED", 0, restarts, self.rounds)
            if code == EXIT_STANDBY and not self._draining:
                self._log("worker asked for a new rendezvous (exit code 125)")
                self._start_worker()
                continue
            if self._remaining_restarts > 0 and not self._draining:
                self._log(f"worker failed with exit code {code}; {self._remaining_restarts}/{self.config.max_restarts} restarts left")
                self._remaining_restarts -= 1
                self._start_worker()
                continue
            self._log(f"worker ended with exit code {code}" + (" after a termination request" if self._draining else ""))
            return RunResult("FAILED", code, restarts, self.rounds)


# ------------------------------------------------------------------------------------------ launch
def launch_agent(config: LaunchConfig, cmd: str, cmd_args: List[str], etcd_module=None, client=None, notice_source=None,
                 master_addr=None, master_port=None) -> RunResult:
    if not config.run_id:
        config.run_id = str(uuid.uuid4().int)
    if not config.project_pactum:
        raise NotImplementedError("only elastic pipeline jobs are launched here (--project-pactum); "
                                  "use torchrun for anything else")
    assert config.rdzv_backend in ("etcd", "etcd-v2"), "the elastic launcher needs the etcd rendezvous backend"
    rdzv_cfg = dict(config.rdzv_configs)
    if client is None:
        client = _rdzv.create_etcd_client(config.rdzv_endpoint, rdzv_cfg, etcd_module)
    handler = _rdzv.create_rdzv_handler(client, config.run_id, config.min_nodes, config.max_nodes,
                                        prefix=rdzv_cfg.get("etcd_prefix", "/torchelastic/p2p"),
                                        timeout=int(rdzv_cfg.get("timeout", _rdzv.DEFAULT_TIMEOUT)),
                                        last_call_timeout=int(rdzv_cfg.get("last_call_timeout", _rdzv.DEFAULT_LAST_CALL_TIMEOUT)),
                                        etcd_module=etcd_module)
    handler.write("/rdzv/default_pipelines", config.default_num_stages)
    extra_env = {
        "PROJECT_PACTUM_ENABLED": "1", "PROJECT_PACTUM_ENDPOINT": config.rdzv_endpoint, "PROJECT_PACTUM_RUN_ID": str(config.run_id),
        "PROJECT_PACTUM_MIN_NODES": str(config.min_nodes), "PROJECT_PACTUM_MAX_NODES": str(config.max_nodes),
        "PROJECT_PACTUM_RDZV_CONFIGS": json.dumps(config.rdzv_configs),
        "PROJECT_PACTUM_MAX_PIPE_PARALLEL_SIZE": str(config.max_pipe_parallel_size),
        "PROJECT_PACTUM_DEFAULT_PIPELINE_SIZE": str(config.default_num_stages),
        "NCCL_BLOCKING_WAIT": "1",
    }
    agent = NodeAgent(config, handler, cmd, cmd_args, extra_env=extra_env, notice_source=notice_source,
                      master_addr=master_addr, master_port=master_port)
    try:
        return agent.run()
    finally:
        agent._stop_worker()
        try:
            handler.stop_keep_alive()
        except Exception:  # noqa: BLE001
            pass


def main(argv=None):
    args = parse(sys.argv[1:] if argv is None else argv)
    if args.standalone:
        raise NotImplementedError("--standalone: a single-node job needs no elastic launcher; run the script directly or with torchrun")
    config, cmd, cmd_args = config_from_args(args)
    # the spot-notice poller only makes sense on an EC2 instance; BAMBOO_SPOT_NOTICES=0 switches it off
    notices = ec2_spot_notice if os.environ.get("BAMBOO_SPOT_NOTICES", "1") != "0" else None
    result = launch_agent(config, cmd, cmd_args, notice_source=notices)
    return 0 if result.state == "SUCCEEDED" else (result.exitcode or 1)


if __name__ == "__main__":
    sys.exit(main())
