"""Cartesian topology arithmetic: coordinates, axis subgroups, balanced ranges, ownership, fail-closed checks.
Golden values are the ones the reference asserts for the same shapes (eredu-core/src/topology.rs:609-697)."""
import pytest

from eredu_b200.parallel.context import ParallelContext
from eredu_b200.parallel.topology import ParallelTopology, balanced_contiguous_range


def test_rank_22_of_a_2x3x2x2_world():
    topo = ParallelTopology(data=2, pipeline=3, tensor=2, expert=2)
    assert topo.world_size == 24
    assert topo.coordinates(22) == {"data": 1, "pipeline": 2, "tensor": 1, "expert": 0}
    assert topo.rank_for(**topo.coordinates(22)) == 22
    assert topo.axis_members(22, "tensor") == [20, 22]
    assert topo.axis_members(22, "pipeline") == [14, 18, 22]
    assert topo.axis_members(22, "expert") == [22, 23]
    assert topo.axis_members(22, "data") == [10, 22]
    assert topo.pipeline_predecessor(22) == 18 and topo.pipeline_successor(22) is None
    assert not topo.owns_embedding(22) and topo.owns_output_head(22)
    assert topo.layer_range(22, 7) == (5, 7)
    assert topo.expert_range(22, 5) == (0, 3)
    assert topo.sampling_rank(22) == 20            # last stage, tensor 0, expert 0 of the same replica


def test_rank_mapping_round_trips_on_every_axis():
    topo = ParallelTopology(data=2, pipeline=2, tensor=3, expert=2)
    for rank in range(topo.world_size):
        c = topo.coordinates(rank)
        assert topo.rank_for(**c) == rank
        for axis in ("tensor", "pipeline", "expert", "data"):
            members = topo.axis_members(rank, axis)
            assert members[c[axis]] == rank and len(members) == getattr(topo, axis)


def test_expert_axis_over_the_tensor_ranks():
    topo = ParallelTopology(pipeline=2, tensor=4, expert=4, expert_over_tensor=True)
    assert topo.world_size == 8
    assert topo.coordinates(6) == {"data": 0, "pipeline": 1, "tensor": 2, "expert": 2}
    assert topo.axis_members(6, "tensor") == topo.axis_members(6, "expert") == [4, 5, 6, 7]
    assert topo.expert_range(6, 10) == (6, 8)
    with pytest.raises(ValueError):
        topo.rank_for(0, 0, 1, 2)
    with pytest.raises(ValueError):
        ParallelTopology(tensor=4, expert=2, expert_over_tensor=True)


def test_balanced_ranges_and_preflight():
    assert [balanced_contiguous_range(8, 3, i) for i in range(3)] == [(0, 3), (3, 6), (6, 8)]
    assert balanced_contiguous_range(2, 3, 2) == (2, 2)
    with pytest.raises(ValueError):
        balanced_contiguous_range(8, 3, 3)
    with pytest.raises(ValueError):
        ParallelTopology(tensor=0)
    topo = ParallelTopology(pipeline=4, tensor=8)
    assert topo.preflight(n_layers=32, n_heads=32, n_kv_heads=8) == []
    assert topo.preflight(n_layers=32, n_heads=32, n_kv_heads=2) == []          # kv heads replicate over 8 ranks
    issues = ParallelTopology(pipeline=4, tensor=3, expert=9).preflight(n_layers=2, n_heads=32, n_kv_heads=8, n_experts=8)
    assert len(issues) == 4


def test_data_axis_is_declared_but_fails_closed():
    topo = ParallelTopology(data=2, tensor=2)
    assert any("data parallelism" in i for i in topo.preflight(4, 4, 4))
    with pytest.raises(ValueError, match="data parallelism"):
        ParallelContext(topo, 0)
    assert ParallelContext(ParallelTopology(tensor=2), 1).tp_rank == 1
