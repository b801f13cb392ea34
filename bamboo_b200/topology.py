"""Process topology: (pipe, data) coordinates <-> global ranks, and the pipeline grid.

Keeps the interface of Bamboo's patched DeepSpeed topology module
(``deepspeed/runtime/pipe/topology.py``): ``ProcessTopology`` (``:13-237``, including the
rendezvous-driven ``custom_mapping`` of ``:49-59`` and ``modify_mapping`` of ``:61-64`` used
when a rank takes over a dead neighbour's coordinate), ``PipeDataParallelTopology``
(``:255-263``) and ``PipelineParallelGrid`` (``:272-519``).

Differences by design: the grid only creates the process groups the training step
really uses - one data-parallel group per stage column plus the pre-built fallback groups
that swap a dead rank for its pipeline predecessor (``init_fallback_group``, ``:382-399``).
The reference's per-rank singleton groups, pipe groups and p2p group storm are gone:
inter-stage traffic does not use collectives here.
"""
from collections import namedtuple
from itertools import product
from typing import Dict, List, Optional

GlobalInfo = namedtuple("GlobalInfo", ["rank", "previous_coordinates", "active_coordinates"])


class ProcessTopology:
    """Row-major map from named n-d coordinates to linear ranks (first axis slowest)."""

    def __init__(self, axes, dims, custom_mapping=None):
        self.axes = list(axes)
        self.dims = list(dims)
        self.ProcessCoord = namedtuple("ProcessCoord", axes)
        self.mapping: Dict[tuple, int] = {}
        if custom_mapping is None:
            for rank, coord in enumerate(product(*[range(d) for d in self.dims])):
                self.mapping[self.ProcessCoord(*coord)] = rank
        else:
            # rendezvous decision: each rank owns a list of [pipeline, stage] coordinates;
            # only the first one places it in the grid (standby ranks own none)
            for info in custom_mapping:
                if len(info.active_coordinates) == 0:
                    continue
                dp_id, stage = info.active_coordinates[0][0], info.active_coordinates[0][1]
                self.mapping[self.ProcessCoord(data=dp_id, pipe=stage)] = info.rank

    def modify_mapping(self, rank, **axes):
        self.mapping[self.ProcessCoord(**{a: axes.get(a) for a in self.axes})] = rank

    def get_rank(self, **coord_kwargs):
        if len(coord_kwargs) != len(self.axes):
            raise ValueError("get_rank() does not support slices. Use filter_match())")
        key = self.ProcessCoord(**coord_kwargs)
        assert key in self.mapping, f"key {coord_kwargs} invalid"
        return self.mapping[key]

    def get_axis_names(self):
        return self.axes

    def get_rank_repr(self, rank, omit_axes=("data", "pipe"), inner_sep="_", outer_sep="-"):
        omit = frozenset(omit_axes)
        coord = self.get_coord(rank)
        return outer_sep.join(f"{a}{inner_sep}{getattr(coord, a):02d}" for a in self.axes if a not in omit)

    def get_dim(self, axis):
        return self.dims[self.axes.index(axis)] if axis in self.axes else 0

    def get_coord(self, rank):
        # after a failover one rank may own two coordinates; the first inserted wins
        for coord, r in self.mapping.items():
            if r == rank:
                return coord
        raise ValueError(f"rank {rank} not found in topology.")

    def get_axis_comm_lists(self, axis):
        if axis not in self.axes:
            return []
        others = [a for a in self.axes if a != axis]
        lists = []
        for fixed in product(*[range(self.get_dim(a)) for a in others]):
            keys = dict(zip(others, fixed))
            lists.append([self.mapping[self.ProcessCoord(**keys, **{axis: i})] for i in range(self.get_dim(axis))])
        return lists

    def filter_match(self, **filter_kwargs):
        return [r for c, r in self.mapping.items() if all(getattr(c, k) == v for k, v in filter_kwargs.items())]

    def get_axis_list(self, axis, idx):
        pos = self.axes.index(axis)
        return [r for c, r in self.mapping.items() if c[pos] == idx]

    def world_size(self):
        return len(self.mapping)

    def __str__(self):
        return str(self.mapping)


def _prime_factors(n):
    if n <= 0:
        raise ValueError("Values must be strictly positive.")
    out, f = [], 2
    while n != 1:
        if n % f == 0:
            out.append(f)
            n //= f
        else:
            f += 1
    return out


class PipeDataParallelTopology(ProcessTopology):
    """axes = ['pipe', 'data']: rank = stage * num_dp + replica unless the rendezvous says otherwise."""

    def __init__(self, num_pp, num_dp, custom_mapping=None):
        super().__init__(axes=["pipe", "data"], dims=[num_pp, num_dp], custom_mapping=custom_mapping)


class PipeModelDataParallelTopology(ProcessTopology):
    def __init__(self, num_pp, num_mp, num_dp):
        super().__init__(axes=["pipe", "data", "model"], dims=[num_pp, num_dp, num_mp])


class PipelineParallelGrid:
    """This rank's place in the (stage, replica) grid plus its data-parallel groups.

    ``dist`` is the ``torch.distributed`` module (or a stand-in with ``new_group``); when it
    is ``None`` or not initialised no process groups are created (single-process use and
    unit tests) and group getters return ``None``.
    """

    def __init__(self, topology=None, process_group=None, global_rank=None, world_size=None, dist=None):
        if dist is None:
            import torch.distributed as _dist
            dist = _dist if (_dist.is_available() and _dist.is_initialized()) else None
        self._dist = dist
        self.global_rank = global_rank if global_rank is not None else (dist.get_rank() if dist else 0)
        self.world_size = world_size if world_size is not None else (dist.get_world_size() if dist else 1)
        if topology is None:
            num_pp = num_dp = 1
            for i, prime in enumerate(_prime_factors(self.world_size)):
                if i % 2 == 0:
                    num_pp *= prime
                else:
                    num_dp *= prime
            topology = PipeDataParallelTopology(num_dp=num_dp, num_pp=num_pp)
        self._topo = topology
        self.data_parallel_size = max(topology.get_dim("data"), 1)
        self.pipe_parallel_size = max(topology.get_dim("pipe"), 1)
        self.model_parallel_size = max(topology.get_dim("model"), 1)
        self.slice_parallel_size = self.model_parallel_size
        assert self._is_grid_valid(), "Invalid Grid"
        self.stage_id = self.get_stage_id()
        self.data_parallel_id = self.get_data_parallel_id()
        self.is_first_stage = self.stage_id == 0
        self.is_last_stage = self.stage_id == self.pipe_parallel_size - 1

        # data-parallel columns: same stage across pipelines
        self.dp_groups: List[List[int]] = topology.get_axis_comm_lists("data")
        self.dp_group: List[int] = []
        self.dp_proc_groups = {}
        self.dp_fallback_proc_groups = {}
        for ranks in self.dp_groups:
            pg = self._new_group(ranks)
            if self.global_rank in ranks:
                self.dp_group = ranks
                self.dp_proc_groups = {self.stage_id: pg}
        self.current_dp_group = self.dp_group
        self.dp_fallback_groups: Dict[int, List[int]] = {}

        self.pipe_groups = topology.get_axis_comm_lists("pipe")
        self.pp_group = next((g for g in self.pipe_groups if self.global_rank in g), [])
        self.p2p_groups = self._build_p2p_groups()
        self.p2p_matrix = {r: [i for i in comm if i != r] for comm in self.pipe_groups for r in comm}

    def _new_group(self, ranks):
        if self._dist is None or len(ranks) <= 1:
            return None
        return self._dist.new_group(ranks=list(ranks))

    def init_fallback_group(self, redundancy_level):
        """For every rank of every stage column, pre-build the group in which that rank is
        replaced by its pipeline predecessor (who holds its shadow weights)."""
        assert redundancy_level == 1
        self.dp_fallback_groups = {}
        for stage, ranks in enumerate(self.dp_groups):
            for pipeline, rank in enumerate(ranks):
                coord = self._topo.get_coord(rank)
                f_rank = self._topo.get_rank(**coord._replace(pipe=self._dec_stage(coord.pipe))._asdict())
                f_ranks = [r if r != rank else f_rank for r in ranks]
                group = self._new_group(f_ranks)
                if self.global_rank == f_rank:
                    self.dp_proc_groups[stage] = group
                if self.global_rank in ranks:
                    self.dp_fallback_groups[rank] = f_ranks
                    self.dp_fallback_proc_groups[pipeline] = group

    def set_fallback_group(self, src):
        if src not in self.dp_fallback_proc_groups:
            raise RuntimeError(f"Can not find fallback group for source {src}")
        self.dp_proc_groups[self.stage_id] = self.dp_fallback_proc_groups[src]

    def _inc_stage(self, s):
        return (s + 1) % self.pipe_parallel_size

    def _dec_stage(self, s):
        return (s - 1) % self.pipe_parallel_size

    def get_stage_id(self):
        return self._topo.get_coord(rank=self.global_rank).pipe

    def get_data_parallel_id(self):
        return self._topo.get_coord(rank=self.global_rank).data

    def _build_p2p_groups(self):
        out = []
        for rank in range(self.world_size):
            for comm in self.pipe_groups:
                if rank in comm:
                    out.append([rank, comm[(comm.index(rank) + 1) % self.pipe_parallel_size]])
                    break
        return out

    def _is_grid_valid(self):
        n = 1
        for ax in self._topo.get_axis_names():
            n *= self._topo.get_dim(ax)
        return n == self.world_size

    def stage_to_global(self, stage_id, **kwargs):
        me = self._topo.get_coord(self.global_rank)
        return self._topo.get_rank(**me._replace(pipe=stage_id, **kwargs)._asdict())

    def topology(self):
        return self._topo

    # mpu-style accessors
    def get_global_rank(self):
        return self.global_rank

    def get_pipe_parallel_rank(self):
        return self.get_stage_id()

    def get_pipe_parallel_world_size(self):
        return self.pipe_parallel_size

    def get_pipe_parallel_group(self):
        return None

    def get_data_parallel_rank(self):
        return self.data_parallel_id

    def get_data_parallel_world_size(self):
        return self.data_parallel_size

    def get_data_parallel_group(self, stage_id=None):
        stage_id = self.stage_id if stage_id is None else stage_id
        if stage_id not in self.dp_proc_groups:
            raise RuntimeError(f"Can not find group for stage {stage_id}")
        return self.dp_proc_groups[stage_id]

    def get_model_parallel_rank(self):
        return self.get_stage_id()

    def get_model_parallel_world_size(self):
        return self.pipe_parallel_size

    def get_model_parallel_group(self):
        return None

    def get_slice_parallel_rank(self):
        return 0

    def get_slice_parallel_world_size(self):
        return self.slice_parallel_size

    def get_slice_parallel_group(self):
        return None
