"""Topology tables against the reference's answers (tests/golden/topology.json) and the
known answers of its unit tests (tests/unit/test_topology.py:13-160)."""
from bamboo_b200.topology import (GlobalInfo, PipeDataParallelTopology, PipelineParallelGrid, ProcessTopology,
                                  _prime_factors)


def test_golden_grids(golden_topology):
    for g in golden_topology["grids"]:
        topo = PipeDataParallelTopology(num_pp=g["pp"], num_dp=g["dp"])
        world = topo.world_size()
        assert world == g["pp"] * g["dp"]
        assert [list(topo.get_coord(r)) for r in range(world)] == g["coords"]
        assert topo.get_axis_comm_lists("pipe") == g["pipe_lists"]
        assert topo.get_axis_comm_lists("data") == g["data_lists"]
        assert topo.get_axis_list("pipe", 0) == g["axis_pipe0"]
        assert topo.filter_match(data=0) == g["match_data0"]
        assert [topo.get_rank_repr(r, omit_axes=[]) for r in range(world)] == g["rank_repr"]
        for rank in range(world):
            grid = PipelineParallelGrid(topology=PipeDataParallelTopology(g["pp"], g["dp"]), global_rank=rank,
                                        world_size=world, dist=None)
            grid._dist = None
            grid.init_fallback_group(1)
            for r, ranks in grid.dp_fallback_groups.items():
                assert ranks == g["fallback"][str(r)]


def test_reference_known_answers():
    topo = ProcessTopology(axes=["row", "col"], dims=[2, 2])
    assert topo.get_rank(row=0, col=1) == 1 and topo.get_rank(row=1, col=0) == 2
    assert topo.get_axis_list(axis="row", idx=0) == [0, 1] and topo.get_axis_list(axis="col", idx=1) == [1, 3]
    topo = ProcessTopology(axes=["pipe", "data", "model"], dims=[2, 2, 2])
    assert topo.get_axis_comm_lists("pipe") == [[0, 4], [1, 5], [2, 6], [3, 7]]
    assert topo.get_axis_comm_lists("data") == [[0, 2], [1, 3], [4, 6], [5, 7]]
    assert topo.get_axis_comm_lists("model") == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert topo.get_axis_comm_lists("jeff") == []
    assert topo.filter_match(pipe=0, data=1) == [2, 3]
    assert topo.get_rank_repr(rank=3, omit_axes=["pipe"]) == "data_01-model_01"
    assert _prime_factors(12) == [2, 2, 3]


def test_custom_mapping_and_failover_remap():
    decision = [GlobalInfo(5, [], [[0, 0]]), GlobalInfo(2, [], [[0, 1]]), GlobalInfo(7, [], [])]
    topo = PipeDataParallelTopology(num_pp=2, num_dp=1, custom_mapping=decision)
    assert topo.get_rank(pipe=0, data=0) == 5 and topo.get_rank(pipe=1, data=0) == 2
    assert topo.world_size() == 2
    topo.modify_mapping(rank=5, pipe=1, data=0)          # rank 5 takes over stage 1
    assert topo.get_rank(pipe=1, data=0) == 5
    assert topo.get_coord(5).pipe == 0                    # first coordinate wins


def test_grid_roles():
    topo = PipeDataParallelTopology(num_pp=4, num_dp=2)
    grid = PipelineParallelGrid(topology=topo, global_rank=5, world_size=8)
    assert grid.get_stage_id() == 2 and grid.get_data_parallel_id() == 1
    assert grid.stage_to_global(3) == 7 and grid.dp_group == [4, 5]
    assert grid.p2p_groups[6] == [6, 0]
