"""Generate ``rendezvous.json``: traces of the reference's own etcd rendezvous
(``project_pactum/rendezvous/etcd.py``, imported in place, never copied) on the in-process etcd
of ``tests/fake_etcd.py``, for the scenarios of ``tests/rendezvous_scenarios.py``.

    python tests/golden/gen_rendezvous_golden.py /path/to/bamboo
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
TESTS = os.path.dirname(HERE)
sys.path.insert(0, HERE)
sys.path.insert(0, TESTS)
import fake_etcd  # noqa: E402

sys.modules["etcd"] = fake_etcd            # the reference does `import etcd`
import _ref_shims  # noqa: E402


def main(reference_root):
    _ref_shims.install(reference_root)
    import logging
    logging.disable(logging.CRITICAL)
    from project_pactum.rendezvous import etcd as ref
    import rendezvous_scenarios as sc

    def make_impl(client, run_id, min_nodes, max_nodes):
        return ref.EtcdRendezvous(client, sc.PREFIX, run_id, min_nodes, max_nodes, timeout=60, last_call_timeout=1)

    out = {name: sc.scrub(fn(make_impl)) for name, fn in sc.SCENARIOS.items()}
    with open(os.path.join(HERE, "rendezvous.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("wrote", len(out), "scenarios")


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BAMBOO_REFERENCE")
    if not root:
        sys.exit(f"usage: {os.path.basename(__file__)} <path of the reference checkout>  (or set BAMBOO_REFERENCE)")
    main(root)
