"""Etcd-backed rendezvous with Bamboo's grid bookkeeping, as the pipeline engine sees it.

Follows the observable behaviour (etcd keys, values, state transitions) of
``project_pactum/rendezvous/etcd.py`` of the reference - torch-elastic's etcd v2 rendezvous
(state ``setup -> joinable -> frozen -> final``, one compare-and-swap on ``active_version``
per transition, per-member keep-alive leases) extended with

* ``assign_coordinates`` (``:778-858``): when the last member confirms, every rank gets its
  ``(pipeline, stage)`` seat under ``rdzv/v_<version>/rank_<r>_coordinates`` and the final
  state is remembered as ``rdzv/previous_state``;
* ``get_global_decision`` (``:897-925``): the ``GlobalInfo(rank, previous_coordinates,
  active_coordinates)`` list ``PipeDataParallelTopology`` is built from;
* ``should_reconfigure`` / ``decide_reconfigure`` (``:1065-1155``): one decision per global step,
  agreed through ``rdzv/global_steps_<n>``, recorded as ``rdzv/current_step``;
* ``update_coordinates`` (``:860-870``): a rank that took a dead neighbour's stage over publishes
  both of its seats.

The engine calls ``write``, ``should_reconfigure``, ``get_global_decision``,
``get_current_step``, ``update_coordinates`` and ``create_lock`` on the handler
(``deepspeed/runtime/pipe/engine.py:1068-1112`` of the reference).

``client`` is a ``python-etcd`` client (``etcd.Client``) or anything with its methods;
``etcd_module`` supplies the matching exception classes and ``Lock`` (default: ``import etcd``).
The transitions are written here as one loop over a small compare-and-swap helper rather than
phase methods calling each other; keys and values are the reference's.
"""
import json
import re
import socket
import threading
import time
from datetime import timedelta

from .topology import GlobalInfo

# time-to-live of the ephemeral keys, seconds (reference: etcd.py:82-96)
SETUP_TTL = 5
FROZEN_TTL = 10
JOINABLE_EPHEMERAL_TTL = 10
WORKER_KEEPALIVE_TTL = 10
RUNID_SUBROOT_TTL = 7200
DEFAULT_TIMEOUT = 60
DEFAULT_LAST_CALL_TIMEOUT = 30


class TooFewNodesException(Exception):
    """Fewer members than one pipeline has stages."""


class RendezvousClosedError(Exception):
    pass


class RendezvousTimeoutError(Exception):
    pass


class _Retry(Exception):
    """The state moved under us; start over (``delay``: wait a second first)."""

    def __init__(self, delay=False):
        super().__init__()
        self.delay = delay


def _load_etcd():
    import etcd  # python-etcd
    return etcd


# ------------------------------------------------------------------------------------ key/value store
def _store_base():
    try:
        from torch.distributed import Store
        return Store
    except Exception:  # pragma: no cover - torch without distributed support
        return object


class EtcdStore(_store_base()):
    """The job's c10d store on the rendezvous' etcd directory ``rdzv/v_<version>/kv`` (what
    ``setup_kv_store`` returns, reference ``etcd.py:1466-1470``; key and value encoding of
    torch-elastic's ``EtcdStore``: base64 of the bytes, one etcd node per key)."""

    def __init__(self, client, prefix, etcd_module=None, timeout=timedelta(seconds=300)):
        super().__init__()
        self.client = client
        self.prefix = prefix if prefix.endswith("/") else prefix + "/"
        self._etcd = etcd_module or _load_etcd()
        self._timeout = timeout

    @staticmethod
    def _enc(v):
        from base64 import b64encode
        if isinstance(v, str):
            v = v.encode()
        return b64encode(bytes(v)).decode()

    @staticmethod
    def _dec(v):
        from base64 import b64decode
        return b64decode(v.encode())

    def set(self, key, value):
        self.client.set(key=self.prefix + self._enc(key), value=self._enc(value))

    def check(self, keys):
        for k in keys:
            try:
                self.client.get(self.prefix + self._enc(k))
            except self._etcd.EtcdKeyNotFound:
                return False
        return True

    def wait(self, keys, override_timeout=None):
        deadline = time.time() + (override_timeout or self._timeout).total_seconds()
        while not self.check(keys):
            if time.time() > deadline:
                raise LookupError(f"timeout waiting for keys {list(keys)} in the etcd store")
            time.sleep(0.02)

    def get(self, key):
        self.wait([key])
        return self._dec(self.client.get(self.prefix + self._enc(key)).value)

    def add(self, key, num):
        node_key = self.prefix + self._enc(key)
        try:
            self.client.write(key=node_key, value=self._enc(str(num)), prevExist=False)
            return int(num)
        except self._etcd.EtcdAlreadyExist:
            pass
        while True:
            node = self.client.get(node_key)
            new = self._enc(str(int(self._dec(node.value)) + int(num)))
            try:
                self.client.test_and_set(key=node_key, value=new, prev_value=node.value)
                return int(self._dec(new))
            except self._etcd.EtcdCompareFailed:
                time.sleep(0.01)

    def set_timeout(self, timeout):
        self._timeout = timeout


# ------------------------------------------------------------------------------------ rendezvous
class EtcdRendezvous:
    """One member's view of the rendezvous of a run (``run_id``) under ``prefix`` in etcd."""

    def __init__(self, client, prefix, run_id, num_min_workers, num_max_workers, timeout=DEFAULT_TIMEOUT,
                 last_call_timeout=DEFAULT_LAST_CALL_TIMEOUT, etcd_module=None):
        self.client = client
        self._etcd = etcd_module or _load_etcd()
        self._prefix = prefix if prefix.endswith("/") else prefix + "/"
        self._run_id = run_id
        self._num_min_workers, self._num_max_workers = num_min_workers, num_max_workers
        self._timeout, self._last_call_timeout = timeout, last_call_timeout
        self._lease_run_id_stop = None
        self._lease_this_rank_stop = None
        self._deadline = time.time() + timeout
        if self._prefix != "/":
            self._mkdir(self._prefix)
        self._mkdir(self.get_path(""), ttl=RUNID_SUBROOT_TTL)
        self._lease_run_id_stop = self._keep_alive(self.get_path(""), RUNID_SUBROOT_TTL)
        self._mkdir(self.get_path("/rdzv"))
        try:
            self.client.write(key=self.get_path("/rdzv/version_counter"), value="0", prevExist=False)
        except self._etcd.EtcdAlreadyExist:
            pass
        self.rank_pattern = re.compile(r".*/rdzv/v_(\d+)/rank_(\d+)")

    # ---- plumbing
    def get_path(self, path):
        if not path.startswith("/"):
            path = "/" + path
        return f"{self._prefix}run_{self._run_id}{path}"

    def _mkdir(self, full_path, ttl=None):
        try:
            self.client.write(key=full_path, value=None, dir=True, prevExist=False, ttl=ttl)
        except self._etcd.EtcdAlreadyExist:
            pass

    def _keep_alive(self, full_path, ttl):
        """Refresh an ephemeral key every ttl/2 seconds until told to stop or the key is gone."""
        stop = threading.Event()

        def worker():
            while True:
                try:
                    self.client.refresh(full_path, ttl=ttl)
                except (self._etcd.EtcdKeyNotFound, ConnectionRefusedError):
                    return
                if stop.wait(timeout=ttl / 2):
                    return
        threading.Thread(target=worker, daemon=True).start()
        return stop

    def stop_keep_alive(self):
        for ev in (self._lease_run_id_stop, self._lease_this_rank_stop):
            if ev is not None:
                ev.set()

    __del__ = stop_keep_alive

    def write(self, key, value):
        """Free-form status keys of the run (``/rdzv/cluster_status``, ``/rdzv/last_reconfig``);
        strings are stored JSON-quoted (reference ``etcd.py:451-455``)."""
        if isinstance(value, str):
            value = json.dumps(value)
        self.client.write(self.get_path(key), value)

    def get_rdzv_state(self):
        node = self.client.get(key=self.get_path("/rdzv/active_version"))
        return node, json.loads(node.value)

    def _cas_state(self, node, state, ttl=None):
        """Replace ``active_version`` if it still holds what ``node`` holds."""
        return self.client.test_and_set(key=self.get_path("/rdzv/active_version"), value=json.dumps(state),
                                        prev_value=node.value, ttl=ttl)

    def _wait_change(self, etcd_index, timeout=None):
        """Block until ``active_version`` changes (or the time is up) and read it again."""
        overall = max(self._deadline - time.time(), 0.0) + 1.0
        timeout = overall if timeout is None else min(timeout, overall)
        try:
            self.client.watch(self.get_path("/rdzv/active_version"), index=etcd_index, timeout=timeout)
        except (self._etcd.EtcdEventIndexCleared, self._etcd.EtcdWatchTimedOut):
            pass
        if time.time() > self._deadline:
            raise RendezvousTimeoutError()
        return self.get_rdzv_state()

    @staticmethod
    def _cas_delay():
        import random
        time.sleep(random.uniform(0, 0.1))

    # ---- the barrier: setup -> joinable -> frozen -> final
    def rendezvous_barrier(self, previous_global_rank=-1):
        """Blocks until this member is part of a final rendezvous.  Returns
        ``(version, rank, world_size, num_pipelines, num_stages)``."""
        self._deadline = time.time() + self._timeout
        while True:
            if time.time() > self._deadline:
                raise RendezvousTimeoutError()
            try:
                if self._lease_this_rank_stop is not None:
                    self._lease_this_rank_stop.set()        # disown the lease of an earlier round
                return self._attempt(previous_global_rank)
            except _Retry as r:
                if r.delay:
                    time.sleep(1)
            except (RendezvousTimeoutError, RendezvousClosedError):
                raise
            except Exception:
                # like the reference, anything else (a key that vanished, too few members for one
                # pipeline) is retried after a pause until the deadline
                time.sleep(1)

    def _attempt(self, previous_global_rank):
        try:
            node = self._create_round()
            state = json.loads(node.value)
        except self._etcd.EtcdAlreadyExist:
            node, state = self.get_rdzv_state()
        status = state["status"]
        if status == "closed":
            raise RendezvousClosedError()
        if status == "final":
            # a complete rendezvous exists: count ourselves as waiting and watch for its end
            self._announce_waiting(state["version"])
            self._wait_until_not_final(state["version"])
            raise _Retry()
        if status != "joinable":
            self._wait_change(node.etcd_index + 1)
            raise _Retry(delay=True)

        version = state["version"]
        node, rank = self._join(version)
        state = json.loads(node.value)
        if rank == self._num_min_workers - 1 and state["status"] == "joinable":
            # the member that completed the minimum keeps the door open for the last-call period
            self._last_call(version, time.time() + self._last_call_timeout)
        node, state = self.get_rdzv_state()
        while not (state["status"] == "frozen" and state["version"] == version):
            if not (state["status"] == "joinable" and state["version"] == version):
                raise _Retry(delay=True)
            node, state = self._wait_change(node.etcd_index + 1)

        self._confirm(version, rank, previous_global_rank)
        node, state = self.get_rdzv_state()
        while not (state["status"] == "final" and state["version"] == version):
            if not (state["status"] == "frozen" and state["version"] == version):
                raise _Retry(delay=True)
            node, state = self._wait_change(node.etcd_index + 1)
        json.loads(self.client.get(self.get_path(f"rdzv/v_{version}/rank_{rank}_coordinates")).value)
        return state["version"], rank, len(state["participants"]), int(state["num_pipelines"]), int(state["num_stages"])

    def _create_round(self):
        """A new version: ephemeral ``{"status": "setup"}``, bump the counter, make the version's
        directory, publish ``joinable``."""
        node = self.client.write(key=self.get_path("/rdzv/active_version"), value=json.dumps({"status": "setup"}),
                                 prevExist=False, ttl=SETUP_TTL)
        try:
            counter = self.client.get(self.get_path("/rdzv/version_counter"))
            counter.value = str(int(counter.value) + 1)
            self.client.update(counter)
        except (self._etcd.EtcdKeyNotFound, self._etcd.EtcdCompareFailed):
            raise RuntimeError("Unexpected state of EtcdRendezvousHandler, worker needs to die.")
        self.client.write(key=self.get_path(f"/rdzv/v_{counter.value}"), value=None, dir=True, prevExist=False)
        return self._cas_state(node, {"status": "joinable", "version": counter.value, "participants": []})

    def _join(self, version):
        while True:
            self._cas_delay()
            node, state = self.get_rdzv_state()
            if state["status"] != "joinable":
                raise _Retry(delay=True)
            if state["version"] != version:
                raise _Retry()
            assert len(state["participants"]) < self._num_max_workers
            rank = len(state["participants"])
            state["participants"].append(rank)
            ttl = None
            if len(state["participants"]) == self._num_max_workers:
                state["status"], state["keep_alives"], ttl = "frozen", [], FROZEN_TTL
            elif len(state["participants"]) >= self._num_min_workers:
                ttl = JOINABLE_EPHEMERAL_TTL
            try:
                return self._cas_state(node, state, ttl=ttl), rank
            except self._etcd.EtcdCompareFailed:
                continue

    def _last_call(self, version, deadline):
        node, state = self.get_rdzv_state()
        while True:
            if state["status"] == "frozen" and state["version"] == version:
                return
            if state["status"] != "joinable" or state["version"] != version:
                raise _Retry(delay=True)
            try:
                if time.time() >= deadline:
                    state["status"], state["keep_alives"] = "frozen", []
                    self._cas_state(node, state, ttl=FROZEN_TTL)
                    return
                # refresh the TTL of the unchanged state, then sleep until something happens
                node = self.client.test_and_set(key=self.get_path("/rdzv/active_version"), value=node.value,
                                                prev_value=node.value, ttl=JOINABLE_EPHEMERAL_TTL)
                node, state = self._wait_change(node.etcd_index + 1,
                                                timeout=min(JOINABLE_EPHEMERAL_TTL / 2, deadline - time.time() + 1.0))
            except self._etcd.EtcdCompareFailed:
                self._cas_delay()
                node, state = self.get_rdzv_state()

    def _confirm(self, version, rank, previous_global_rank):
        """Lease key ``rank_<r>`` (value: the rank this member had in the previous round), its
        address, and our name on the keep-alive list; the last one to confirm assigns the seats
        and makes the round final."""
        while True:
            self._cas_delay()
            node, state = self.get_rdzv_state()
            if state["status"] != "frozen" or state["version"] != version:
                raise _Retry()
            lease_key = self.get_path(f"/rdzv/v_{version}/rank_{rank}")
            self.client.set(lease_key, value=str(previous_global_rank), ttl=WORKER_KEEPALIVE_TTL)
            try:
                my_ip = socket.gethostbyname(socket.gethostname())
            except OSError:
                my_ip = "127.0.0.1"
            self.client.set(self.get_path(f"/rdzv/v_{version}/rank_{rank}_ip"), value=str(my_ip), ttl=None)
            state["keep_alives"].append(lease_key)
            final = len(state["keep_alives"]) == len(state["participants"])
            if final:
                state["status"], state["num_workers_waiting"] = "final", 0
                self.assign_coordinates(version, state)
            try:
                node = self._cas_state(node, state, ttl=None if final else FROZEN_TTL)
                self._lease_this_rank_stop = self._keep_alive(lease_key, WORKER_KEEPALIVE_TTL)
                return node
            except self._etcd.EtcdCompareFailed:
                continue

    def _announce_waiting(self, version):
        while True:
            self._cas_delay()
            node, state = self.get_rdzv_state()
            if state["status"] != "final" or state["version"] != version:
                raise _Retry()
            state["num_workers_waiting"] += 1
            try:
                return self._cas_state(node, state)
            except self._etcd.EtcdCompareFailed:
                continue

    def _wait_until_not_final(self, version):
        """A final round is never torn down because a member died (failures are absorbed by
        redundancy); we only wait for somebody to delete or change it."""
        while True:
            try:
                node, state = self.get_rdzv_state()
            except self._etcd.EtcdKeyNotFound:
                return
            if state["status"] != "final" or state["version"] != version:
                return
            try:
                self.client.watch(key=self.get_path("/rdzv"), index=node.etcd_index + 1, recursive=True,
                                  timeout=max(self._deadline - time.time(), 0.0) + 1.0)
            except (self._etcd.EtcdEventIndexCleared, self._etcd.EtcdWatchTimedOut):
                pass
            if time.time() > self._deadline:
                raise RendezvousTimeoutError()

    def set_closed(self):
        while True:
            node, state = self.get_rdzv_state()
            if state["status"] == "closed":
                return
            state["status"] = "closed"
            try:
                self._cas_state(node, state)
                return
            except self._etcd.EtcdCompareFailed:
                self._cas_delay()

    # ---- seats in the pipeline x replica grid
    def get_rank_coordinates_for_version(self, state, version, previous_version=None):
        """``{rank(str): [[pipeline, stage], ...]}`` of the members whose lease is alive.  With
        ``previous_version`` the seats are those the member held in that earlier round (its
        lease key stores the rank it had then; -1 = newcomer, skipped)."""
        alive = {ch.key for ch in self.client.get(self.get_path(f"/rdzv/v_{version}")).children}
        out = {}
        for key in state["keep_alives"]:
            if key.endswith("_coordinates") or key not in alive:
                continue
            rank = self.rank_pattern.match(key).group(2)
            if previous_version is not None:
                try:
                    previous_rank = self.client.get(key).value
                except Exception:
                    continue
                if int(previous_rank) < 0:
                    continue
                path = self.get_path(f"rdzv/v_{previous_version}/rank_{previous_rank}_coordinates")
            else:
                path = self.get_path(f"rdzv/v_{version}/rank_{rank}_coordinates")
            out[rank] = json.loads(self.client.get(path).value)
        return out

    def assign_coordinates(self, version, state):
        """Seats for a round that is about to become final.  The number of stages is the run's
        ``rdzv/default_pipelines`` value (sic: the key holds the stage count), the number of
        pipelines what the members fill; ranks beyond ``pipelines x stages`` get no seat.  Seats
        are handed out in rank order, pipeline-major; a member keeps its previous seat only when
        the grid is unchanged AND square (the reference compares the stage count with the previous
        *pipeline* count, ``etcd.py:831``) - kept as is, since the stored keys are the contract."""
        n = len(state["participants"])
        prev_key = self.get_path("/rdzv/previous_state")
        try:
            previous = json.loads(self.client.get(prev_key).value)
        except Exception:
            previous = None
        if previous:
            held = self.get_rank_coordinates_for_version(state, version, previous_version=previous["version"])
            previous_version = previous["version"]
        else:
            held, previous_version = {}, "-1"
        num_stages = json.loads(self.client.get(self.get_path("/rdzv/default_pipelines")).value)
        num_pipelines = n // num_stages
        if n < num_stages:
            raise TooFewNodesException()
        state["previous_version"] = previous_version
        state["num_pipelines"], state["num_stages"] = str(num_pipelines), str(num_stages)
        prev_pipelines = int(previous["num_pipelines"]) if previous else 0
        free = [(i // num_stages, i % num_stages) for i in range(num_pipelines * num_stages)]
        seats = {}
        if num_pipelines == prev_pipelines and num_stages == prev_pipelines:
            for rank, coords in held.items():
                if coords:
                    seat = coords[0]
                    free.remove(tuple(seat) if tuple(seat) in free else seat)
                    seats[rank] = [seat]
        for seat in free:
            for r in range(n):
                if str(r) not in seats:
                    seats[str(r)] = [seat]
                    break
        for r in range(n):
            seats.setdefault(str(r), [])
        for rank, coords in seats.items():
            self.client.set(self.get_path(f"rdzv/v_{version}/rank_{rank}_coordinates"), value=json.dumps(coords), ttl=None)
        self.client.set(prev_key, value=json.dumps(state), ttl=None)

    def update_coordinates(self, rank, coordinates):
        _, state = self.get_rdzv_state()
        self.update_coordinates_for_version(state["version"], rank, coordinates)

    def update_coordinates_for_version(self, version, rank, coordinates):
        node = self.client.get(self.get_path(f"/rdzv/v_{version}/rank_{rank}_coordinates"))
        node.value = json.dumps(coordinates)
        self.client.update(node)

    def previous_version_exists(self):
        _, state = self.get_rdzv_state()
        return int(state["previous_version"]) > 0

    def get_previous_state(self):
        return json.loads(self.client.get(self.get_path("/rdzv/previous_state")).value)

    def create_lock(self, lock_name):
        return self._etcd.Lock(self.client, lock_name)

    def get_current_step(self):
        try:
            return json.loads(self.client.get(self.get_path("/rdzv/current_step")).value)
        except self._etcd.EtcdKeyNotFound:
            return 0

    def get_global_decision(self):
        _, state = self.get_rdzv_state()
        version, previous_version = state["version"], state["previous_version"]
        before = {} if int(previous_version) < 0 else \
            self.get_rank_coordinates_for_version(state, version, previous_version=previous_version)
        now = self.get_rank_coordinates_for_version(state, version)
        return [GlobalInfo(rank=int(rank), previous_coordinates=before.get(rank, []), active_coordinates=coords)
                for rank, coords in now.items()]

    # ---- reconfiguration decision, one per global step
    def should_reconfigure(self, global_steps, failures):
        key = self.get_path(f"/rdzv/global_steps_{global_steps}")
        while True:
            try:
                node, state = self.get_rdzv_state()
            except Exception:
                return True                                  # no rendezvous: everybody re-joins
            if state["status"] != "final":
                return True
            try:
                return json.loads(self.client.get(key).value)   # somebody already decided for this step
            except self._etcd.EtcdKeyNotFound:
                pass
            try:
                return self.decide_reconfigure(global_steps, key, failures, node, state)
            except Exception:
                continue                                     # lost the race for the key: read it next time

    def decide_reconfigure(self, global_step, global_steps_key, failures, active_version, state):
        """Reconfigure when a member holds more than two seats, when a member holding two (it
        already absorbed a failure) is announced to be preempted at this step, or when the
        waiting members would make one more whole pipeline."""
        decision = False
        overloaded = 0
        waiting = int(state["num_workers_waiting"])
        for rank, coords in self.get_rank_coordinates_for_version(state, state["version"]).items():
            if len(coords) > 2:
                decision = True
                break
            if len(coords) == 2:
                if failures.get(str(rank), -1) == global_step:
                    decision = True
                    break
                overloaded += 1
        try:
            pipelines, stages = int(state["num_pipelines"]), int(state["num_stages"])
            active = pipelines * stages - overloaded
            if (active + waiting - overloaded) // stages > pipelines:
                decision = True
        except Exception:
            pass
        self.client.write(global_steps_key, value=json.dumps(decision), prevExist=False)
        if decision:
            self.client.delete(key=self.get_path("/rdzv/active_version"), prevValue=active_version.value)
        self.client.write(self.get_path("/rdzv/current_step"), global_step)
        return decision

    def setup_kv_store(self, version):
        path = self.get_path(f"/rdzv/v_{version}/kv")
        self._mkdir(path)
        return EtcdStore(self.client, path, etcd_module=self._etcd)


class EtcdRendezvousHandler:
    """What the launcher and the engine hold (reference ``EtcdRendezvousHandler``,
    ``etcd.py:134-378``): ``next_rendezvous`` for the agent, the bookkeeping calls for the engine."""

    def __init__(self, rdzv_impl):
        self._rdzv_impl = rdzv_impl

    def get_backend(self):
        return "etcd"

    def next_rendezvous(self, previous_global_rank=-1):
        """Returns ``(store, rank, world_size, num_pipelines, num_stages, global_decision)``;
        ``world_size`` counts the members that hold a seat."""
        if isinstance(previous_global_rank, str):
            previous_global_rank = int(previous_global_rank)
        version, rank, _, num_pipelines, num_stages = self._rdzv_impl.rendezvous_barrier(previous_global_rank)
        decision = self._rdzv_impl.get_global_decision()
        world_size = len([info for info in decision if len(info.active_coordinates) != 0])
        return self._rdzv_impl.setup_kv_store(version), rank, world_size, num_pipelines, num_stages, decision

    def setup_kv_store(self):
        _, state = self._rdzv_impl.get_rdzv_state()
        return self._rdzv_impl.setup_kv_store(state["version"])

    def write(self, key, value):
        self._rdzv_impl.write(key, value)

    def should_reconfigure(self, global_steps, failures={}):
        return self._rdzv_impl.should_reconfigure(global_steps, failures) if self._rdzv_impl is not None else False

    def get_global_decision(self):
        return self._rdzv_impl.get_global_decision()

    def get_current_step(self):
        return self._rdzv_impl.get_current_step()

    def create_lock(self, lock_name):
        return self._rdzv_impl.create_lock(lock_name)

    def stop_keep_alive(self):
        self._rdzv_impl.stop_keep_alive()

    def update_coordinates(self, rank, coordinates):
        self._rdzv_impl.update_coordinates(rank, coordinates)

    def update_coordinates_for_version(self, version, rank, coordinates):
        self._rdzv_impl.update_coordinates_for_version(version, rank, coordinates)

    def previous_version_exists(self):
        return self._rdzv_impl.previous_version_exists()

    def get_previous_state(self):
        return self._rdzv_impl.get_previous_state()

    def get_current_state(self):
        return self._rdzv_impl.get_rdzv_state()[1]

    def get_rank_coordinates_for_version(self, state, version):
        return self._rdzv_impl.get_rank_coordinates_for_version(state, version)

    def is_closed(self):
        try:
            return self._rdzv_impl.get_rdzv_state()[1]["status"] == "closed"
        except self._rdzv_impl._etcd.EtcdKeyNotFound:
            return False

    def set_closed(self):
        self._rdzv_impl.set_closed()

    def num_nodes_waiting(self):
        try:
            state = self._rdzv_impl.get_rdzv_state()[1]
            if state["status"] == "final":
                return state["num_workers_waiting"]
        except self._rdzv_impl._etcd.EtcdKeyNotFound:
            pass
        return 0

    def get_run_id(self):
        return self._rdzv_impl._run_id

    def shutdown(self):
        try:
            self.set_closed()
            return True
        except Exception:
            return False


def create_rdzv_handler(client, run_id, min_nodes, max_nodes, prefix="/torchelastic/p2p", timeout=DEFAULT_TIMEOUT,
                        last_call_timeout=DEFAULT_LAST_CALL_TIMEOUT, etcd_module=None):
    """Handler over an existing etcd client (the reference builds the client from
    ``RendezvousParameters``: endpoint, protocol, certificates, ``etcd.py:1472-1574``)."""
    return EtcdRendezvousHandler(EtcdRendezvous(client, prefix, run_id, min_nodes, max_nodes, timeout, last_call_timeout,
                                                etcd_module=etcd_module))


# ---------------------------------------------------------------------------------- environment contract
# The launcher hands the job's rendezvous to every worker through the environment
# (project_pactum/run/api.py:322-332); the reference engine builds its handler from it
# (deepspeed/runtime/engine.py:152-184).  Same variables, same defaults here.
ENV_ENABLED = "PROJECT_PACTUM_ENABLED"
ENV_KEYS = ("PROJECT_PACTUM_ENDPOINT", "PROJECT_PACTUM_RUN_ID", "PROJECT_PACTUM_MIN_NODES", "PROJECT_PACTUM_MAX_NODES",
            "PROJECT_PACTUM_RDZV_CONFIGS")


def parse_endpoint(endpoint, default_port=2379):
    """``host[:port]`` / ``[v6 host]:port`` -> (host, port)"""
    endpoint = endpoint.strip()
    if not endpoint:
        return "localhost", default_port
    if endpoint.startswith("["):
        host, _, rest = endpoint[1:].partition("]")
        port = rest[1:] if rest.startswith(":") else ""
    elif endpoint.count(":") == 1:
        host, _, port = endpoint.partition(":")
    else:
        host, port = endpoint, ""
    if port and not port.isdigit():
        raise ValueError(f"The port number of the rendezvous endpoint '{endpoint}' must be an integer between 0 and 65536.")
    return host, (int(port) if port else default_port)


def create_etcd_client(endpoint, config, etcd_module=None):
    """python-etcd client for ``endpoint`` with the launcher's options (``protocol``, ``cert`` / ``key``,
    ``cacert``: reference ``_create_etcd_client``, ``etcd.py:1472-1503``)."""
    if etcd_module is None:
        try:
            import etcd as etcd_module
        except ImportError as e:
            raise RuntimeError("the etcd rendezvous needs the python-etcd package (module `etcd`)") from e
    host, port = parse_endpoint(endpoint)
    protocol = config.get("protocol") or "http"
    if protocol not in ("http", "https"):
        raise ValueError("The etcd protocol must be HTTP or HTTPS.")
    cert = config.get("cert")
    if cert is not None and config.get("key") is not None:
        cert = (cert, config.get("key"))
    return etcd_module.Client(host, port, protocol=protocol, cert=cert, ca_cert=config.get("cacert"), allow_reconnect=True)


def handler_from_env(environ=None, etcd_module=None, client=None):
    """The worker's rendezvous handler as the launcher described it in the environment, or None when
    the job was not started by the launcher (``PROJECT_PACTUM_ENABLED`` absent).  ``last_call_timeout`` is
    2 s inside a worker, whatever the launcher's own value, like the reference."""
    import os
    environ = os.environ if environ is None else environ
    if ENV_ENABLED not in environ:
        return None
    missing = [k for k in ENV_KEYS if k not in environ]
    if missing:
        raise KeyError(f"{ENV_ENABLED} is set but {', '.join(missing)} missing from the environment")
    config = json.loads(environ["PROJECT_PACTUM_RDZV_CONFIGS"])
    config["last_call_timeout"] = 2
    if client is None:
        client = create_etcd_client(environ["PROJECT_PACTUM_ENDPOINT"], config, etcd_module)
    return create_rdzv_handler(client, environ["PROJECT_PACTUM_RUN_ID"], int(environ["PROJECT_PACTUM_MIN_NODES"]),
                               int(environ["PROJECT_PACTUM_MAX_NODES"]), prefix=config.get("etcd_prefix", "/torchelastic/p2p"),
                               timeout=int(config.get("timeout", DEFAULT_TIMEOUT)),
                               last_call_timeout=int(config["last_call_timeout"]), etcd_module=etcd_module)


def grid_from_env(environ=None):
    """(num_pipelines, num_stages, coordinates) that the node agent gave this worker
    (``PROJECT_PACTUM_NUM_PIPELINES / NUM_STAGES / COORDINATES``, agent/api.py:342-362), or None."""
    import os
    environ = os.environ if environ is None else environ
    if "PROJECT_PACTUM_NUM_PIPELINES" not in environ or "PROJECT_PACTUM_NUM_STAGES" not in environ:
        return None
    coords = json.loads(environ.get("PROJECT_PACTUM_COORDINATES", "[]"))
    return int(environ["PROJECT_PACTUM_NUM_PIPELINES"]), int(environ["PROJECT_PACTUM_NUM_STAGES"]), coords

