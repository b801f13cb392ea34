"""PipelineModule: a layer list partitioned into pipeline stages.

Keeps the constructor and the methods the training scripts and the engine use in Bamboo's
patched DeepSpeed (``deepspeed/runtime/pipe/module.py``): ``LayerSpec`` (``:31-76``),
``TiedLayerSpec`` (``:79-90``), ``PipelineModule(layers, num_stages, topology, loss_fn,
seed_layers, seed_fn, base_seed, partition_method, custom_partitions,
activation_checkpoint_interval, activation_checkpoint_func)`` (``:95-106``),
``forward(input, stage_id)`` (``:516-574``), ``build_layers(stage_id, buffer)``
(``:262-332``, also used to materialise a shadow copy of another stage),
``get_named_param`` / ``allocate_param`` (``:219-260``), ``parts`` from the
``uniform | parameters | type:regex | custom`` partition methods (``:576-635``).

Stage bookkeeping is explicit here: every stage built on this rank (its own, a shadow,
or one it took over) is a ``StageLayers`` record holding its modules and callables.
"""
import os
import re
from typing import Callable, Dict, Iterable, List, Optional

import torch
from torch import nn

from .partition import partition_balanced, partition_uniform
from .topology import PipeDataParallelTopology, PipelineParallelGrid


class LayerSpec:
    """Deferred layer construction: ``LayerSpec(Cls, *args, **kwargs).build()``."""

    def __init__(self, typename, *module_args, **module_kwargs):
        if not issubclass(typename, nn.Module):
            raise RuntimeError("LayerSpec only supports torch.nn.Module types.")
        self.typename = typename
        self.module_args = module_args
        self.module_kwargs = module_kwargs
        self.global_rank = int(os.environ.get("RANK", 0))

    def __repr__(self):
        args = ", ".join([repr(a) for a in self.module_args] + [f"{k}={v!r}" for k, v in self.module_kwargs.items()])
        return f"{self.typename.__name__}({args})"

    def build(self, log=False):
        if log:
            print(f"RANK={self.global_rank} building {self!r}")
        return self.typename(*self.module_args, **self.module_kwargs)


class TiedLayerSpec(LayerSpec):
    def __init__(self, key, typename, *module_args, forward_fn=None, tied_weight_attr="weight", **module_kwargs):
        super().__init__(typename, *module_args, **module_kwargs)
        self.key = key
        self.forward_fn = forward_fn
        self.tied_weight_attr = tied_weight_attr


class StageLayers:
    """The layers of one pipeline stage as built on this rank."""

    def __init__(self, stage_id):
        self.stage_id = stage_id
        self.funcs: List[Callable] = []
        self.modules: Dict[str, nn.Module] = {}

    def named_parameters(self):
        for name, mod in self.modules.items():
            for n, p in mod.named_parameters():
                if p.requires_grad:
                    yield f"{name}.{n}", p

    def parameters(self):
        return [p for _, p in self.named_parameters()]


def _resolve_device():
    if torch.cuda.is_available():
        return torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    return torch.device("cpu")


class PipelineModule(nn.Module):
    def __init__(self, layers, num_stages=None, topology=None, loss_fn=None, seed_layers=False, seed_fn=None,
                 base_seed=1234, partition_method="parameters", custom_partitions=(), activation_checkpoint_interval=0,
                 activation_checkpoint_func=None, device=None):
        super().__init__()
        if num_stages is None and topology is None:
            raise RuntimeError("must provide num_stages or topology")
        import torch.distributed as dist
        initialised = dist.is_available() and dist.is_initialized()
        self.global_rank = dist.get_rank() if initialised else 0
        self.world_size = dist.get_world_size() if initialised else 1
        self.local_rank = int(os.environ.get("LOCAL_RANK", 0))
        self.device = torch.device(device) if device is not None else _resolve_device()
        self.micro_offset = 0
        self.loss_fn = loss_fn
        self.seed_layers, self.seed_fn, self.base_seed = seed_layers, seed_fn, base_seed

        if topology is not None:
            self._topo = topology
            self.num_stages = topology.get_dim("pipe")
        else:
            if self.world_size % num_stages != 0:
                raise RuntimeError(f"num_stages ({num_stages}) must divide distributed world size ({self.world_size})")
            self.num_stages = num_stages
            self._topo = PipeDataParallelTopology(num_pp=num_stages, num_dp=self.world_size // num_stages)
        self._grid = PipelineParallelGrid(topology=self._topo, global_rank=self.global_rank, world_size=self.world_size)
        self.stage_id = self._topo.get_coord(self.global_rank).pipe

        self.partition_method = partition_method
        self._layer_specs = list(layers)
        self._num_layers = len(self._layer_specs)
        self.parts: List[int] = []
        self._partition_layers(method=partition_method, partitions=list(custom_partitions))

        self.tied_modules = nn.ModuleDict()
        self.tied_weight_attrs = {}
        self.stages: Dict[int, StageLayers] = {}
        self.param_name_buckets: Dict[int, List[str]] = {}
        self.func_buckets: Dict[int, List[Callable]] = {}
        self.build_layers(self.stage_id)
        self.activation_checkpoint_interval = activation_checkpoint_interval
        self.activation_checkpoint_func = activation_checkpoint_func

    # ------------------------------------------------------------------ partitioning
    def _count_layer_params(self):
        counts = [0] * len(self._layer_specs)
        for i, layer in enumerate(self._layer_specs):
            mod = layer.build() if isinstance(layer, LayerSpec) else layer
            if isinstance(mod, nn.Module):
                counts[i] = sum(p.numel() for p in mod.parameters() if p.requires_grad)
        return counts

    def _find_layer_type(self, layername):
        rx = re.compile(layername, re.IGNORECASE)
        hits = []
        for i, layer in enumerate(self._layer_specs):
            if isinstance(layer, LayerSpec):
                name = layer.typename.__name__
            elif isinstance(layer, nn.Module):
                name = layer.__class__.__name__
            else:
                name = getattr(layer, "__name__", None)
            if name is not None and rx.search(name):
                hits.append(i)
        if not hits:
            raise ValueError(f"Partitioning '{layername}' found no valid layers to partition.")
        return hits

    def _compute_parts(self, method, num_stages, partitions=None):
        method = method.lower()
        if method == "custom":
            assert partitions, "Required customized partitions"
            return list(partitions)
        if method == "uniform":
            return partition_uniform(num_items=len(self._layer_specs), num_parts=num_stages)
        if method == "parameters":
            return partition_balanced(weights=self._count_layer_params(), num_parts=num_stages)
        if method.startswith("type:"):
            weights = [0] * len(self._layer_specs)
            for i in self._find_layer_type(method.split(":")[1]):
                weights[i] = 1
            return partition_balanced(weights=weights, num_parts=num_stages)
        raise NotImplementedError(f"Partitioning method {method} not implemented.")

    def _partition_layers(self, method="uniform", partitions=None):
        self.parts = self._compute_parts(method, self._topo.get_dim("pipe"), partitions)
        self._local_start, self._local_stop = self.parts[self.stage_id], self.parts[self.stage_id + 1]

    def get_new_partition(self, new_num_stages):
        return self._compute_parts(self.partition_method, new_num_stages)

    # ------------------------------------------------------------------ building stages
    def build_layers(self, stage_id, buffer=None):
        """Instantiate the layers of ``stage_id`` on this rank's device.  ``buffer`` maps
        parameter names to tensors that overwrite the freshly built parameters (promotion
        of a shadow copy)."""
        start, stop = self.parts[stage_id], self.parts[stage_id + 1]
        stage = StageLayers(stage_id)
        for idx in range(start, stop):
            layer = self._layer_specs[idx]
            if self.seed_layers:
                (self.seed_fn or torch.manual_seed)(self.base_seed + idx)
            name = str(idx)
            if isinstance(layer, PipelineModule):
                raise NotImplementedError("RECURSIVE BUILD NOT YET IMPLEMENTED")
            if isinstance(layer, TiedLayerSpec):
                if layer.key not in self.tied_modules:
                    self.tied_modules[layer.key] = layer.build().to(self.device)
                    self.tied_weight_attrs[layer.key] = layer.tied_weight_attr
                mod = self.tied_modules[layer.key]
                stage.funcs.append(mod if layer.forward_fn is None else _bind(layer.forward_fn, mod))
                stage.modules.setdefault(f"tied_{layer.key}", mod)
            elif isinstance(layer, (LayerSpec, nn.Module)):
                mod = layer.build() if isinstance(layer, LayerSpec) else layer
                mod = mod.to(self.device)
                stage.funcs.append(mod)
                stage.modules[name] = mod
                if name not in self._modules:
                    self.add_module(name, mod)
            else:
                stage.funcs.append(layer)  # plain callable
        names = [n for n, _ in stage.named_parameters()]
        if buffer is not None:
            with torch.no_grad():
                for n, p in stage.named_parameters():
                    if n in buffer:
                        p.copy_(buffer[n])
        self.stages[stage_id] = stage
        self.func_buckets[stage_id] = stage.funcs
        self.param_name_buckets[stage_id] = names
        return names

    def get_named_param(self, stage_id):
        yield from self.stages[stage_id].named_parameters()

    def stage_parameters(self, stage_id):
        return self.stages[stage_id].parameters()

    def allocate_param(self, stage_id, param_buffer, device="cpu"):
        """Zero buffers shaped like the parameters of ``stage_id`` (lazy shadow copy)."""
        start, stop = self.parts[stage_id], self.parts[stage_id + 1]
        names = []
        for idx in range(start, stop):
            layer = self._layer_specs[idx]
            mod = layer.build() if isinstance(layer, LayerSpec) else layer
            if not isinstance(mod, nn.Module):
                continue
            for n, p in mod.named_parameters():
                if p.requires_grad:
                    param_buffer[f"{idx}.{n}"] = torch.zeros_like(p, device=device)
                    names.append(f"{idx}.{n}")
        self.param_name_buckets.setdefault(stage_id, names)
        return names

    # ------------------------------------------------------------------ forward
    def forward(self, forward_input, stage_id=None):
        stage_id = self.stage_id if stage_id is None else stage_id
        funcs = self.func_buckets.get(stage_id)
        if funcs is None:
            raise Exception(f"Unregistered stage id {stage_id}")
        self.micro_offset += 1

        def run(lo, hi):
            def body(*inputs):
                x = inputs[0] if len(inputs) == 1 else inputs
                for f in funcs[lo:hi]:
                    x = f(x)
                return x
            return body

        k = self.activation_checkpoint_interval
        if not k:
            return run(0, len(funcs))(forward_input)
        ckpt = self.activation_checkpoint_func
        if ckpt is None:
            from torch.utils.checkpoint import checkpoint as _ckpt
            # non-reentrant: the first segment of stage 0 takes integer tokens (nothing that
            # requires grad goes in), which the reentrant form cannot differentiate through
            ckpt = lambda fn, *a: _ckpt(fn, *a, use_reentrant=False)  # noqa: E731
        x = forward_input
        for lo in range(0, len(funcs), k):
            hi = min(lo + k, len(funcs))
            args = x if isinstance(x, tuple) else (x,)
            has_params = any(isinstance(f, nn.Module) and any(True for _ in f.parameters()) for f in funcs[lo:hi])
            x = ckpt(run(lo, hi), *args) if has_params else run(lo, hi)(*args)
        return x

    def topology(self):
        return self._topo

    def mpu(self):
        return self._grid

    def num_pipeline_stages(self):
        return self._topo.get_dim("pipe")


def _bind(fn, mod):
    def call(x):
        return fn(mod, x)
    return call
