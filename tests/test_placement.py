"""Placement of execution-group DAGs on pipeline stages: balanced ownership, routes derived from ownership, static
tensor roles, payload contracts, validation, concurrency rules (the cases of placement.rs's own tests, in spirit)."""
import pytest

from eredu_b200.parallel.placement import (ActiveSubgroup, ConcurrencyPolicy, GroupRequest, HIDDEN, PayloadSchema, PlacedExecutionDag,
                                           PlacementError, TOKENS, decoder_placement, multimodal_placement)


def test_decoder_over_four_stages():
    dag = decoder_placement(30, 4)
    dec = dag.group("decoder")
    assert dec.owners == [(0, (0, 8)), (1, (8, 16)), (2, (16, 23)), (3, (23, 30))]
    assert dag.static_owner("embedding") == 0 and dag.static_owner("output_head") == 3 and dag.static_owner("final_norm") == 3
    assert [(r.from_pp_rank, r.to_pp_rank) for r in dag.routes] == [(0, 1), (1, 2), (2, 3)]
    assert all(r.payload == HIDDEN and r.from_group == r.to_group == "decoder" for r in dag.routes)
    assert [r.from_pp_rank for r in dag.routes_into(2)] == [1] and [r.to_pp_rank for r in dag.routes_out_of(2)] == [3]
    assert dec.local_units(2) == (16, 23) and dec.local_units(7) is None
    # fewer layers than stages: trailing stages own nothing and carry no route
    small = decoder_placement(2, 4)
    assert small.group("decoder").owners == [(0, (0, 1)), (1, (1, 2))] and len(small.routes) == 1
    assert small.static_owner("output_head") == 1


def test_multimodal_dag_routes_follow_ownership_not_adjacency():
    dag = multimodal_placement(24, 3, vision_blocks=12, audio_blocks=6, encoder_stages=[2, 1])
    order = [dag.groups[i].id for i in dag.execution_order]
    assert order.index("vision_encoder") < order.index("vision_projector") < order.index("assembly") < order.index("decoder")
    vis = dag.group("vision_encoder")
    assert vis.owners == [(2, (0, 6)), (1, (6, 12))] and vis.merge_destination == 1
    routes = {(r.from_group, r.to_group): r.pp_path for r in dag.routes}
    assert routes[("vision_encoder", "vision_encoder")] == (2, 1)            # 2 -> 1: path order, not rank order
    assert routes[("vision_encoder", "vision_projector")] == (1,)            # same owner: no transfer
    assert routes[("vision_projector", "assembly")] == (1, 0)
    assert routes[("assembly", "decoder")] == (0,)
    # text-only requests skip the optional groups; a request with an image runs the vision ones
    assert [g.id for g in dag.local_groups(1)] == ["decoder"]
    assert [g.id for g in dag.local_groups(1, media_present=("vision_encoder", "vision_projector"))] == \
        ["vision_encoder", "vision_projector", "decoder"]
    assert [g.id for g in dag.local_groups(0)] == ["assembly", "decoder"]
    s = dag.summary()
    assert s["output"] == "decoder" and len(s["groups"]) == 6
    # two encoders that share a stage: collectives must be submitted in one order under tensor parallelism
    assert dag.concurrency_compatibility("vision_encoder", "audio_encoder", ConcurrencyPolicy(tensor_parallel_size=2)) == \
        ("collective_ordering", [1, 2])
    assert dag.concurrency_compatibility("vision_encoder", "audio_encoder", ConcurrencyPolicy()) is None
    assert dag.concurrency_compatibility("vision_encoder", "audio_encoder", ConcurrencyPolicy(rank_local_streams=False))[0] == "shared_rank_backend"
    assert dag.concurrency_compatibility("vision_encoder", "audio_encoder", ConcurrencyPolicy(shared_residency_window=True))[0] == "shared_residency_window"
    assert dag.concurrency_compatibility("vision_projector", "assembly", ConcurrencyPolicy(tensor_parallel_size=8)) is None


def req(gid, deps=(), path=(0,), inp=TOKENS, out=HIDDEN, **kw):
    return GroupRequest(gid, kw.pop("kind", "decoder"), kw.pop("units", 4), list(path), inp, out, dependencies=list(deps), **kw)


def test_validation_fails_closed():
    with pytest.raises(PlacementError, match="at least one"):
        PlacedExecutionDag.plan(0, [req("a")], "a")
    with pytest.raises(PlacementError, match="unique"):
        PlacedExecutionDag.plan(1, [req("a"), req("a")], "a")
    with pytest.raises(PlacementError, match="not declared"):
        PlacedExecutionDag.plan(1, [req("a")], "b")
    with pytest.raises(PlacementError, match="undeclared"):
        PlacedExecutionDag.plan(1, [req("a", deps=["ghost"])], "a")
    with pytest.raises(PlacementError, match="cycle"):
        PlacedExecutionDag.plan(1, [req("a", deps=["b"], inp=HIDDEN), req("b", deps=["a"], inp=HIDDEN)], "a")
    with pytest.raises(PlacementError, match="outside"):
        PlacedExecutionDag.plan(2, [req("a", path=(0, 2))], "a")
    with pytest.raises(PlacementError, match="twice"):
        PlacedExecutionDag.plan(2, [req("a", path=(1, 1))], "a")
    with pytest.raises(PlacementError, match="payload mismatch"):
        PlacedExecutionDag.plan(2, [req("a"), req("b", deps=["a"], inp=TOKENS)], "b")
    with pytest.raises(PlacementError, match="two owners"):
        PlacedExecutionDag.plan(2, [req("a", first_owner_static_roles=["embedding"]),
                                    req("b", deps=["a"], inp=HIDDEN, path=(1,), first_owner_static_roles=["embedding"])], "b")
    with pytest.raises(PlacementError, match="merge destination"):
        PlacedExecutionDag.plan(2, [req("a", merge_destination=5)], "a")
    with pytest.raises(PlacementError, match="kind"):
        PlacedExecutionDag.plan(1, [req("a", kind="mystery")], "a")
    with pytest.raises(PlacementError, match="fields"):
        PlacedExecutionDag.plan(1, [req("a", out=PayloadSchema("empty", ()))], "a")
    ok = PlacedExecutionDag.plan(2, [req("a", path=(1,), active=ActiveSubgroup(False, False)),
                                     req("b", deps=["a"], inp=HIDDEN, path=(0, 1), merge_destination=0)], "b")
    assert ok.group("b").merge_destination == 0 and ok.routes[-1].pp_path == (1, 0)
