"""Generate ``reconfigure.json``: the reference's layer-transfer plans
(``PipelineEngine.get_recv_decisions`` / ``get_send_decisions``,
``deepspeed/runtime/pipe/engine.py:574-628``, imported in place) for a set of re-partitions.

    python tests/golden/gen_reconfigure_golden.py /path/to/bamboo
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import _ref_shims  # noqa: E402

# (name, old_parts, new_parts, [(rank, previous_coordinates, active_coordinates), ...])
CASES = [
    ("grow_1x2_to_2x2", [0, 3, 7], [0, 3, 7],
     [(0, [[0, 0]], [[0, 0]]), (1, [[0, 1]], [[0, 1]]), (2, [], [[1, 0]]), (3, [], [[1, 1]])]),
    ("survivor_with_two_stages_hands_one_back", [0, 3, 7], [0, 3, 7],
     [(0, [[0, 0], [0, 1]], [[0, 0]]), (1, [], [[0, 1]])]),
    ("two_stages_to_four", [0, 4, 8], [0, 2, 4, 6, 8],
     [(0, [[0, 0]], [[0, 0]]), (1, [[0, 1]], [[0, 1]]), (2, [], [[0, 2]]), (3, [], [[0, 3]])]),
    ("four_stages_to_two", [0, 2, 4, 6, 8], [0, 4, 8],
     [(0, [[0, 0]], [[0, 0]]), (1, [[0, 1]], []), (2, [[0, 2]], [[0, 1]]), (3, [[0, 3]], [])]),
    ("shifted_boundaries_2x4", [0, 13, 26, 37, 51], [0, 14, 27, 40, 51],
     [(r, [[r // 4, r % 4]], [[r // 4, r % 4]]) for r in range(8)]),
    ("seats_rotate", [0, 5, 10, 15], [0, 5, 10, 15],
     [(0, [[0, 0]], [[0, 1]]), (1, [[0, 1]], [[0, 2]]), (2, [[0, 2]], [[0, 0]])]),
]


def main(reference_root):
    _ref_shims.install(reference_root)
    from deepspeed.runtime.pipe.engine import PipelineEngine
    import collections
    GlobalInfo = collections.namedtuple("GlobalInfo", ["rank", "previous_coordinates", "active_coordinates"])
    out = {}
    for name, old, new, infos in CASES:
        decisions = [GlobalInfo(rank=r, previous_coordinates=p, active_coordinates=a) for r, p, a in infos]
        recv = PipelineEngine.get_recv_decisions(None, old, new, decisions)
        send = PipelineEngine.get_send_decisions(None, recv)
        out[name] = {"old_parts": old, "new_parts": new, "decisions": [list(i) for i in infos],
                     "recv": {str(r): {str(s): sorted(l) for s, l in d.items()} for r, d in recv.items()},
                     "send": {str(r): {str(s): sorted(l) for s, l in d.items()} for r, d in send.items()}}
    with open(os.path.join(HERE, "reconfigure.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("wrote", len(out), "cases")


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BAMBOO_REFERENCE")
    if not root:
        sys.exit(f"usage: {os.path.basename(__file__)} <path of the reference checkout>  (or set BAMBOO_REFERENCE)")
    main(root)
