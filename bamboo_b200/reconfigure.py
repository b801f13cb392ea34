"""Re-partitioning a running job after a re-rendezvous: who sends which layers to whom, and the
wire format of a layer's weights and Adam moments.

Follows ``deepspeed/runtime/pipe/engine.py`` of the reference: ``get_recv_decisions`` /
``get_send_decisions`` (``:574-628``), ``transfer_layers`` (``:515-534``: ranks take turns in rank
order, the rank whose turn it is sends, everybody else receives from it if they expect anything),
``send_layers`` / ``recv_layers`` (``:893-1003``: per peer two flat tensors - all parameters of the
moved layers, then per parameter ``exp_avg`` and ``exp_avg_sq``).

A layer's state here is ``(params: {name: tensor}, moments: [{"exp_avg": t, "exp_avg_sq": t}, ...])``
keyed by the layer's global index, the same shape the reference passes around (``state[idx][0]``,
``state[idx][1]``); ``ParamArena`` slices provide it without copies.
"""
from typing import Dict, Iterable, List, Sequence, Set

import torch

STATE_KEYS = ("exp_avg", "exp_avg_sq")


def get_recv_decisions(old_parts: Sequence[int], new_parts: Sequence[int], global_decisions) -> Dict[int, Dict[int, Set[int]]]:
    """``{rank: {source_rank: {layer indices}}}``: a seated rank needs the layers of its new stage
    minus those it already held (the span of its previous seats); each missing layer is fetched from
    the first rank, in decision order, whose previous seats covered it."""
    held = {}
    for info in global_decisions:
        if info.previous_coordinates:
            stages = [s for _, s in info.previous_coordinates]
            held[info.rank] = set(range(old_parts[min(stages)], old_parts[max(stages) + 1]))
    out: Dict[int, Dict[int, Set[int]]] = {}
    for info in global_decisions:
        if not info.active_coordinates:
            continue
        stage = info.active_coordinates[0][1]
        needed = set(range(new_parts[stage], new_parts[stage + 1])) - held.get(info.rank, set())
        sources: Dict[int, Set[int]] = {}
        for other in global_decisions:
            if other.rank not in held:
                continue
            common = needed & held[other.rank]
            if not common:
                continue
            sources[other.rank] = common
            needed -= common
            if not needed:
                break
        out[info.rank] = sources
        assert not needed, f"nobody holds layers {sorted(needed)} that rank {info.rank} needs"
    return out


def get_send_decisions(recv_decisions: Dict[int, Dict[int, Set[int]]]) -> Dict[int, Dict[int, Set[int]]]:
    """The same plan seen from the senders: ``{rank: {destination_rank: {layer indices}}}``."""
    out: Dict[int, Dict[int, Set[int]]] = {}
    for dst, sources in recv_decisions.items():
        for src, layers in sources.items():
            out.setdefault(src, {})[dst] = layers
    return out


def pack_layers(state, layer_idxs: Iterable[int]):
    """(flat parameters, flat moments) of the given layers, in index order and parameter order."""
    params: List[torch.Tensor] = []
    moments: List[torch.Tensor] = []
    for idx in sorted(layer_idxs):
        layer_params, layer_moments = state[idx]
        params += [t.reshape(-1) for t in layer_params.values()]
        for m in layer_moments:
            moments += [m[k].reshape(-1) for k in STATE_KEYS]
    cat = lambda ts: torch.cat(ts) if ts else torch.empty(0)  # noqa: E731
    return cat(params), cat(moments)


def unpack_layers(flat_params, flat_moments, layer_idxs: Iterable[int], shapes):
    """Inverse of ``pack_layers``; ``shapes[idx]`` = ``{name: shape}`` of layer ``idx``'s parameters
    (the receiver builds the layer from its spec to know them, as the reference does)."""
    out = {}
    po = mo = 0
    for idx in sorted(layer_idxs):
        layer_params, layer_moments = {}, []
        for name, shape in shapes[idx].items():
            n = 1
            for d in shape:
                n *= d
            layer_params[name] = flat_params[po:po + n].view(shape)
            po += n
        for name, shape in shapes[idx].items():
            n = 1
            for d in shape:
                n *= d
            m = {}
            for k in STATE_KEYS:
                m[k] = flat_moments[mo:mo + n].view(shape)
                mo += n
            layer_moments.append(m)
        out[idx] = [layer_params, layer_moments]
    assert po == flat_params.numel() and mo == flat_moments.numel(), "layer transfer: size mismatch"
    return out


def transfer_layers(dist, my_rank, world_size, recv_decisions, send_decisions, state, shapes, device="cpu"):
    """Move layers between ranks according to the plan.  Ranks take turns in rank order: on its turn
    a rank sends to each destination (ascending layer order, one (params, moments) pair per
    destination); on another rank's turn a rank receives if it expects layers from it.  Returns
    the received ``{layer index: [params, moments]}``."""
    mine_out = send_decisions.get(my_rank, {})
    mine_in = recv_decisions.get(my_rank, {})
    received = {}
    for turn in range(world_size):
        if turn == my_rank:
            for dst, layers in mine_out.items():
                layers = [i for i in layers if i in state]          # layers without parameters carry no state
                if not layers:
                    continue
                p, m = pack_layers(state, layers)
                dist.send(p.to(device).contiguous(), dst=dst)
                dist.send(m.to(device).contiguous(), dst=dst)
        elif turn in mine_in and any(i in shapes for i in mine_in[turn]):
            layers = sorted(i for i in mine_in[turn] if i in shapes)
            n = sum(_numel(s) for idx in layers for s in shapes[idx].values())
            p = torch.empty(n, dtype=torch.float32, device=device)
            m = torch.empty(2 * n, dtype=torch.float32, device=device)
            dist.recv(p, src=turn)
            dist.recv(m, src=turn)
            received.update(unpack_layers(p, m, layers, shapes))
    return received


def _numel(shape):
    n = 1
    for d in shape:
        n *= d
    return n
