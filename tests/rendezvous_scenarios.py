"""Rendezvous scenarios run against the in-process etcd (tests/fake_etcd.py).  The same functions
drive this repository's handler and - in the golden generator - the reference's
``EtcdRendezvous``; each returns a JSON-able trace (results + the final etcd key space) that must
be identical for both."""
import json
import re
import threading
import time

PREFIX = "/torchelastic/p2p"


def _normalise(dump, run_id):
    """Key space without host-specific entries (addresses) and with TTL leases kept as values."""
    out = {}
    root = f"{PREFIX}/run_{run_id}"
    for k, v in dump.items():
        if k.endswith("_ip"):
            continue
        if k.endswith("/active_version") or k.endswith("/previous_state"):
            # members confirm in the order their threads happen to run: the list is a set
            st = json.loads(v)
            if isinstance(st, dict) and "keep_alives" in st:
                st["keep_alives"] = sorted(st["keep_alives"])
            v = json.dumps(st, sort_keys=True)
        out[k[len(root):] if k.startswith(root) else k] = v
    return out


def _state(server_dump, run_id):
    v = server_dump.get(f"{PREFIX}/run_{run_id}/rdzv/active_version")
    return json.loads(v) if v else None


def join_members(make_impl, server, run_id, n, num_stages, previous_ranks=None, min_nodes=None, max_nodes=None):
    """``n`` members join one after the other (so rank i is the i-th joiner); returns their results."""
    from fake_etcd import Client
    boot = Client(server)
    # the launcher publishes the stage count before anybody joins (key name as in the reference)
    impls = [make_impl(Client(server), run_id, min_nodes or n, max_nodes or n) for _ in range(n)]
    boot.write(f"{PREFIX}/run_{run_id}/rdzv/default_pipelines", json.dumps(num_stages))
    results = [None] * n
    errors = []

    def member(i):
        try:
            prev = -1 if previous_ranks is None else previous_ranks[i]
            results[i] = impls[i].rendezvous_barrier(prev)
        except BaseException as e:  # noqa: BLE001
            errors.append(repr(e))

    threads = []
    for i in range(n):
        t = threading.Thread(target=member, args=(i,), daemon=True)
        t.start()
        threads.append(t)
        # wait until this member is on the participants list before the next one starts
        deadline = time.time() + 20
        while time.time() < deadline:
            st = _state(server.dump(), run_id)
            if st and (len(st.get("participants", [])) > i or st.get("status") in ("frozen", "final")):
                break
            time.sleep(0.01)
    for t in threads:
        t.join(timeout=60)
    assert not errors, errors
    return impls, [list(r) for r in results]


def scenario_fresh_grid(make_impl, n=4, num_stages=2, run_id="fresh"):
    """A first rendezvous: seats are handed out in rank order, pipeline-major."""
    from fake_etcd import Server
    server = Server()
    impls, results = join_members(make_impl, server, run_id, n, num_stages)
    decision = sorted((int(g.rank), g.previous_coordinates, g.active_coordinates) for g in impls[0].get_global_decision())
    trace = {"results": sorted(results), "decision": [list(d) for d in decision],
             "current_step": impls[0].get_current_step(), "keys": _normalise(server.dump(), run_id)}
    for im in impls:
        im.stop_keep_alive()
    return trace


def scenario_reconfigure_decisions(make_impl, run_id="decide"):
    """Decisions of ``should_reconfigure`` on a 2 x 2 grid: nothing to do; a member that holds two
    seats (it absorbed a failure) stays until it is itself announced to fail; enough waiting
    members for one more pipeline."""
    from fake_etcd import Client, Server
    server = Server()
    impls, _ = join_members(make_impl, server, run_id, 4, 2)
    a, b = impls[0], impls[1]
    out = {}
    out["step0_quiet"] = [a.should_reconfigure(0, {}), b.should_reconfigure(0, {})]
    # rank 0 took over stage 1 of pipeline 0 from rank 1
    a.update_coordinates(0, [[0, 0], [0, 1]])
    a.update_coordinates(1, [])
    out["step1_overloaded_alive"] = [a.should_reconfigure(1, {"1": 1}), b.should_reconfigure(1, {"1": 1})]
    out["step_after_1"] = a.get_current_step()
    keys_before = _normalise(server.dump(), run_id)
    out["step2_overloaded_preempted"] = [a.should_reconfigure(2, {"0": 2}), b.should_reconfigure(2, {"0": 2})]
    out["active_version_deleted"] = f"{PREFIX}/run_{run_id}/rdzv/active_version" not in server.dump()
    out["without_rendezvous"] = a.should_reconfigure(3, {})
    out["keys_before_reconfigure"] = keys_before
    out["keys_after"] = _normalise(server.dump(), run_id)
    for im in impls:
        im.stop_keep_alive()
    return out


def scenario_waiting_members_make_a_pipeline(make_impl, run_id="grow"):
    """Two members run one 2-stage pipeline; two more arrive and wait; the next decision is to
    reconfigure, and the following rendezvous seats four members, the old ones first."""
    from fake_etcd import Client, Server
    server = Server()
    impls, first = join_members(make_impl, server, run_id, 2, 2, min_nodes=2, max_nodes=2)
    out = {"first": sorted(first)}
    out["quiet"] = impls[0].should_reconfigure(0, {})
    st = _state(server.dump(), run_id)
    st["num_workers_waiting"] = 2                      # what two late members' announcements amount to
    Client(server).write(f"{PREFIX}/run_{run_id}/rdzv/active_version", json.dumps(st))
    out["grow"] = impls[0].should_reconfigure(1, {})
    for im in impls:
        im.stop_keep_alive()
    # everybody re-joins: the two old members (previous ranks 0, 1) and two newcomers (-1)
    impls2, second = join_members(make_impl, server, run_id, 4, 2, previous_ranks=[0, 1, -1, -1])
    out["second"] = sorted(second)
    decision = sorted((int(g.rank), g.previous_coordinates, g.active_coordinates) for g in impls2[0].get_global_decision())
    out["decision"] = [list(d) for d in decision]
    out["keys"] = _normalise(server.dump(), run_id)
    for im in impls2:
        im.stop_keep_alive()
    return out


SCENARIOS = {
    "fresh_2x2": lambda mk: scenario_fresh_grid(mk, 4, 2, "fresh"),
    "fresh_5_members_2_stages": lambda mk: scenario_fresh_grid(mk, 5, 2, "odd"),
    "fresh_8_members_4_stages": lambda mk: scenario_fresh_grid(mk, 8, 4, "c5"),
    "decisions": scenario_reconfigure_decisions,
    "grow": scenario_waiting_members_make_a_pipeline,
}


def scrub(trace):
    """JSON round trip (tuples -> lists) and removal of values that differ from run to run."""
    text = json.dumps(trace, sort_keys=True)
    text = re.sub(r'"rank_(\d+)_ip": "[^"]*"', r'"rank_\1_ip": ""', text)
    return json.loads(text)
