"""Typed tensor-parallel plan: roles, member shardings, logical ranges with replication, segmented members, rank-selective
reads, validation; and that the dense decoder's loader cuts exactly what the plan says."""
import dataclasses

import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.parallel.planner import (MemberSharding, ParallelPlan, ParameterGroupSpec, ParameterMemberSpec, ParameterRole,
                                         PlanError, attention_groups, dense_decoder_plan, feed_forward_group)


def cfg_small(**kw):
    return dataclasses.replace(C.tiny_llama(), hidden_size=64, num_attention_heads=8, num_key_value_heads=2, head_dim=8,
                               intermediate_size=96, vocab_size=120, num_hidden_layers=2, **kw)


def test_heads_split_and_kv_heads_replicate_over_consecutive_ranks():
    cfg = cfg_small()
    plan = ParallelPlan(4)
    q, kv = attention_groups(cfg, 4, "a.")
    plan.add(q)
    plan.add(kv)
    assert kv.replication == 2 and q.replication == 1 and q.role is ParameterRole.ATTENTION_HEADS
    assert [plan.ranges("a.q_proj.weight", r) for r in range(4)] == [[(0, 16)], [(16, 32)], [(32, 48)], [(48, 64)]]
    assert [plan.ranges("a.k_proj.weight", r) for r in range(4)] == [[(0, 8)], [(0, 8)], [(8, 16)], [(8, 16)]]
    assert plan.ranges("a.o_proj.weight", 2) == [(32, 48)] and plan.local_shape("a.o_proj.weight", 2) == (64, 16)
    assert plan.coverage("a.q_proj.weight") and plan.coverage("a.k_proj.weight") and plan.coverage("a.o_proj.weight")
    w = torch.arange(64 * 64, dtype=torch.float32).view(64, 64)
    assert torch.equal(plan.select("a.o_proj.weight", w, 1), w[:, 16:32])
    with pytest.raises(PlanError):
        attention_groups(cfg, 3, "b.")                       # 8 heads over 3 ranks
    with pytest.raises(PlanError):
        attention_groups(dataclasses.replace(cfg, num_key_value_heads=3, num_attention_heads=12), 4, "c.")


def test_fused_and_segmented_members():
    cfg = cfg_small()
    plan = ParallelPlan(2)
    plan.add(feed_forward_group(cfg, "m.", fused_gate_up=True))
    assert plan.ranges("m.gate_up_proj.weight", 1) == [(48, 96), (144, 192)] and plan.ranges("m.down_proj.weight", 1) == [(48, 96)]
    assert plan.local_shape("m.gate_up_proj.weight", 0) == (96, 64) and plan.coverage("m.gate_up_proj.weight")
    # independently partitioned segments of unequal width (balanced ranges inside each)
    plan.add(ParameterGroupSpec("conv", ParameterRole.SEGMENTED, [
        ParameterMemberSpec("c.in_proj.weight", (10 + 7, 4), MemberSharding.segmented(0, [(0, 10), (10, 17)]))]))
    assert plan.ranges("c.in_proj.weight", 0) == [(0, 5), (10, 14)] and plan.ranges("c.in_proj.weight", 1) == [(5, 10), (14, 17)]
    assert plan.coverage("c.in_proj.weight")
    uneven = ParallelPlan(3)
    uneven.add(ParameterGroupSpec("vocab", ParameterRole.VOCABULARY, [
        ParameterMemberSpec("head", (10, 4), MemberSharding.partitioned(0))], extent=10, balanced=True))
    assert [uneven.ranges("head", r) for r in range(3)] == [[(0, 4)], [(4, 7)], [(7, 10)]]
    strict = ParallelPlan(3)
    strict.add(ParameterGroupSpec("vocab", ParameterRole.VOCABULARY, [
        ParameterMemberSpec("head", (10, 4), MemberSharding.partitioned(0))], extent=10))
    with pytest.raises(ValueError, match="evenly"):
        strict.ranges("head", 0)


def test_validation_fails_closed():
    plan = ParallelPlan(2)
    g = ParameterGroupSpec("x", ParameterRole.CHANNELS, [ParameterMemberSpec("t", (8, 4), MemberSharding.partitioned(0))], extent=8)
    plan.add(g)
    with pytest.raises(PlanError, match="planned twice"):
        plan.add(ParameterGroupSpec("y", ParameterRole.CHANNELS, [ParameterMemberSpec("t", (8, 4), MemberSharding.equal(0))]))
    for bad in (ParameterMemberSpec("u", (8, 4), MemberSharding.partitioned(2)),                 # axis outside the shape
                ParameterMemberSpec("u", (9, 4), MemberSharding.partitioned(0)),                 # extent mismatch
                ParameterMemberSpec("u", (9, 4), MemberSharding.equal(0)),                       # not divisible
                ParameterMemberSpec("u", (16, 4), MemberSharding.partitioned_segments(0, [(0, 8), (4, 12)])),   # overlap
                ParameterMemberSpec("u", (16, 4), MemberSharding.partitioned_segments(0, [(0, 6), (8, 16)]))):  # short segment
        with pytest.raises(PlanError):
            ParallelPlan(2).add(ParameterGroupSpec("z", ParameterRole.CHANNELS, [bad], extent=8))
    with pytest.raises(PlanError, match="not part"):
        plan.ranges("missing", 0)
    with pytest.raises(PlanError, match="shape"):
        plan.select("t", torch.zeros(4, 4), 0)


def test_rank_selective_reads_touch_only_the_owned_rows():
    class Source:
        def __init__(self, tensors):
            self.t, self.row_reads, self.full_reads = tensors, [], []

        def get(self, name):
            self.full_reads.append(name)
            return self.t[name]

        def get_rows(self, name, a, b):
            self.row_reads.append((name, a, b))
            return self.t[name][a:b]

    cfg = cfg_small(tie_word_embeddings=False)
    plan = dense_decoder_plan(cfg, 2, has=lambda n: n == "lm_head.weight")
    g = torch.Generator().manual_seed(0)
    tensors = {m.name: torch.randn(*m.shape, generator=g) for grp in plan.groups for m in grp.members}
    src = Source(tensors)
    p = "model.layers.1."
    up = plan.read(p + "mlp.up_proj.weight", src, 1)
    down = plan.read(p + "mlp.down_proj.weight", src, 1)
    head = plan.read("lm_head.weight", src, 0)
    norm = plan.read(p + "input_layernorm.weight", src, 1)
    assert torch.equal(up, tensors[p + "mlp.up_proj.weight"][48:]) and torch.equal(down, tensors[p + "mlp.down_proj.weight"][:, 48:])
    assert torch.equal(head, tensors["lm_head.weight"][:60]) and norm is tensors[p + "input_layernorm.weight"]
    assert src.row_reads == [(p + "mlp.up_proj.weight", 48, 96), ("lm_head.weight", 0, 60)]
    assert src.full_reads == [p + "mlp.down_proj.weight", p + "input_layernorm.weight"]       # column shards need the rows whole
    roles = {grp["role"] for grp in plan.summary()}
    assert {"attention_heads", "feed_forward_intermediate", "vocabulary", "replicated"} <= roles
    assert all(plan.coverage(m.name) for grp in plan.groups for m in grp.members)


def test_the_loader_cuts_what_the_plan_says():
    from eredu_b200.models.llama import build_from_tensors, random_state
    from eredu_b200.parallel.context import ParallelContext
    from eredu_b200.parallel.topology import ParallelTopology

    cfg = dataclasses.replace(C.tiny_llama(), num_key_value_heads=2)
    sd = random_state(cfg, seed=0, std=0.05)
    tp = 4
    plan = dense_decoder_plan(cfg, tp)
    D, nq = cfg.head_dim, cfg.num_attention_heads
    for rank in range(tp):
        par = ParallelContext(ParallelTopology(tensor=tp), rank)
        model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, par)
        lw = model.layers[1]
        p = "model.layers.1."
        q = plan.select(p + "self_attn.q_proj.weight", sd[p + "self_attn.q_proj.weight"], rank)
        k = plan.select(p + "self_attn.k_proj.weight", sd[p + "self_attn.k_proj.weight"], rank)
        v = plan.select(p + "self_attn.v_proj.weight", sd[p + "self_attn.v_proj.weight"], rank)
        assert torch.equal(lw.wqkv, torch.cat((q, k, v), 0)) and q.shape[0] == nq // tp * D and k.shape[0] == D
        assert torch.equal(lw.wo, plan.select(p + "self_attn.o_proj.weight", sd[p + "self_attn.o_proj.weight"], rank))
        gu = torch.cat((plan.select(p + "mlp.gate_proj.weight", sd[p + "mlp.gate_proj.weight"], rank),
                        plan.select(p + "mlp.up_proj.weight", sd[p + "mlp.up_proj.weight"], rank)), 0)
        assert torch.equal(lw.w_gate_up, gu)
        assert torch.equal(lw.w_down, plan.select(p + "mlp.down_proj.weight", sd[p + "mlp.down_proj.weight"], rank))
