"""Per-layer checkpoints of a pipeline engine, in the reference's on-disk layout.

    <save_dir>/latest                                  text file holding the newest tag
    <save_dir>/<tag>/layer_XX-model_states.pt          one file per layer of the layer list
    <save_dir>/<tag>/mp_rank_SS_model_states.pt        one file per pipeline stage: optimizer
                                                       state, scheduler, step counters

Reference: ``PipelineModule.ckpt_layer_path / save_state_dict / load_state_dir``
(``deepspeed/runtime/pipe/module.py:786-849``), ``DeepSpeedEngine.save_checkpoint`` /
``_save_checkpoint`` / ``_get_ckpt_name`` (``deepspeed/runtime/engine.py:2197-2253,2390-2417,
1902-1920``), ``PipelineEngine.module_state_dict`` (``deepspeed/runtime/pipe/engine.py:2288-2320``).
Because the model is stored by LAYER, a checkpoint written by S stages loads into any other
partition of the same layer list.  The reference keeps the optimizer state per rank; here every
moment is additionally keyed by its parameter name (``"<layer>.<param>"``), so that it follows
its layer to whichever stage owns it after a re-partition.  Values are the fp32 master weights.
"""
import glob
import os
from collections import OrderedDict

import torch


def layer_path(ckpt_dir, layer_key):
    key = f"{int(layer_key):02d}" if str(layer_key).isdigit() else str(layer_key)
    return os.path.join(ckpt_dir, f"layer_{key}-model_states.pt")


def stage_path(ckpt_dir, stage_id):
    return os.path.join(ckpt_dir, f"mp_rank_{stage_id:02d}_model_states.pt")


def _named_slices(engine, arena, stage_id):
    names = [n for n, _ in engine.module.get_named_param(stage_id)]
    assert len(names) == len(arena.params), "arena and stage disagree on the parameter list"
    for name, (i, off, n) in zip(names, arena.named_slices()):
        yield name, off, n, arena.params[i].shape


def save_checkpoint(engine, save_dir, tag=None, client_state=None, save_latest=True):
    """Every rank calls this.  Replica 0 of each stage writes the stage's layers and state; rank 0
    writes ``latest`` after all ranks are through."""
    tag = str(tag if tag is not None else f"global_step{engine.global_steps}")
    ckpt_dir = os.path.join(save_dir, tag)
    os.makedirs(ckpt_dir, exist_ok=True)
    if engine.device.type == "cuda":
        torch.cuda.synchronize(engine.device)
    if engine.grid.get_data_parallel_id() == 0:
        for sid in engine.stage_ids:
            arena = engine.arenas[sid]
            layers, by_name = OrderedDict(), OrderedDict()
            for name, off, n, shape in _named_slices(engine, arena, sid):
                layer_key, pname = name.split(".", 1)
                layers.setdefault(layer_key, OrderedDict())[pname] = arena.master[off:off + n].view(shape).detach().cpu().clone()
                by_name[name] = {"step": arena.step_count,
                                 "exp_avg": arena.exp_avg[off:off + n].view(shape).detach().cpu().clone(),
                                 "exp_avg_sq": arena.exp_avg_sq[off:off + n].view(shape).detach().cpu().clone()}
            for layer_key, sd in layers.items():
                torch.save(sd, layer_path(ckpt_dir, layer_key))
            names = list(by_name)
            optimizer = {"state": {i: by_name[n] for i, n in enumerate(names)},
                         "param_groups": [dict(engine._adam, params=list(range(len(names))))],
                         "param_names": names, "state_by_name": by_name}
            state = dict(module=None, optimizer=optimizer,
                         lr_scheduler=engine.lr_scheduler.state_dict() if engine.lr_scheduler is not None else None,
                         global_steps=engine.global_steps, global_samples=engine.global_samples,
                         dp_world_size=engine.dp_world_size, mp_world_size=engine.num_stages, stage_id=sid,
                         parts=list(engine.module.parts))
            state.update(client_state or {})
            torch.save(state, stage_path(ckpt_dir, sid))
    if engine.dist is not None and engine.world_size > 1:
        engine.dist.barrier()
    if save_latest and engine.global_rank == 0:
        with open(os.path.join(save_dir, "latest"), "w") as fd:
            fd.write(tag)
    return True


def load_checkpoint(engine, load_dir, tag=None, load_optimizer_states=True, load_lr_scheduler_states=True):
    """Loads the layers this rank owns (and the ones it shadows) from ``<load_dir>/<tag>``;
    returns ``(checkpoint directory, client state)`` or ``(None, None)`` when there is none."""
    if tag is None:
        latest = os.path.join(load_dir, "latest")
        if not os.path.isfile(latest):
            return None, None
        with open(latest) as fd:
            tag = fd.read().strip()
    ckpt_dir = os.path.join(load_dir, str(tag))
    stage_files = sorted(glob.glob(os.path.join(ckpt_dir, "mp_rank_*_model_states.pt")))
    if not stage_files:
        return None, None
    stage_states = [torch.load(f, map_location="cpu", weights_only=False) for f in stage_files]
    moments = {}
    for st in stage_states:
        moments.update(st["optimizer"]["state_by_name"])

    def fill(arena, stage_id, with_moments):
        layer_cache = {}
        with torch.no_grad():
            for name, off, n, shape in _named_slices(engine, arena, stage_id):
                layer_key, pname = name.split(".", 1)
                if layer_key not in layer_cache:
                    layer_cache[layer_key] = torch.load(layer_path(ckpt_dir, layer_key), map_location="cpu", weights_only=False)
                arena.master[off:off + n].copy_(layer_cache[layer_key][pname].reshape(-1))
                if with_moments and arena.exp_avg is not None and name in moments:
                    arena.exp_avg[off:off + n].copy_(moments[name]["exp_avg"].reshape(-1))
                    arena.exp_avg_sq[off:off + n].copy_(moments[name]["exp_avg_sq"].reshape(-1))
                    arena.step_count = int(moments[name]["step"])
        arena.refresh_lp()

    for sid in engine.stage_ids:
        fill(engine.arenas[sid], sid, load_optimizer_states)
    for sid in engine.r_stage_ids:                       # the shadow copies restart from the same state
        if sid in engine.param_buffers:
            fill(engine.param_buffers[sid], sid, load_optimizer_states)
    head = stage_states[0]
    engine.global_steps = int(head["global_steps"])
    engine.global_samples = int(head["global_samples"])
    if load_lr_scheduler_states and engine.lr_scheduler is not None and head.get("lr_scheduler") is not None:
        engine.lr_scheduler.load_state_dict(head["lr_scheduler"])
    reserved = {"module", "optimizer", "lr_scheduler", "global_steps", "global_samples", "dp_world_size", "mp_world_size",
                "stage_id", "parts"}
    client = {k: v for k, v in head.items() if k not in reserved}
    if engine.dist is not None and engine.world_size > 1:
        engine.dist.barrier()
    return ckpt_dir, client
