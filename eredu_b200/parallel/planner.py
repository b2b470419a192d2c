"""Typed tensor-parallel plan: which slice of which checkpoint tensor a rank materialises.

Counterpart of the reference's planner (``ParameterRole`` / ``MemberSharding`` / ``ParameterGroupSpec`` /
``ParallelPlanBuilder``, eredu/src/backend/mlx/runtime/distributed/parallel.rs:138-330, and the rank-selective reads of
runtime/distributed/topology.rs:822-926). A *group* is one logical domain (the query heads, the feed-forward channels,
the vocabulary, ...) split once into per-rank ranges; its *members* are the physical tensors that carry that domain on
one of their axes, possibly several times (a fused gate|up matrix) or in units larger than one index (a head is
``head_dim`` rows). Nothing depends on tensor names: every member states its axis and its mapping explicitly.

``plan.ranges(member, rank)`` gives the index ranges along the member's axis; ``plan.select(member, tensor, rank)``
cuts a tensor; ``plan.read(member, source, rank)`` reads only the needed rows when the partitioned axis is the first one
and the source can read row ranges (``get_rows``), so a rank never touches the bytes of another rank's shard.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Optional

from .topology import balanced_contiguous_range


class ParameterRole(Enum):
    REPLICATED = "replicated"
    COLUMN_PROJECTION = "column_projection"              # output features are rank-local
    ROW_PROJECTION = "row_projection"                    # input features are rank-local, the output is reduced
    VOCABULARY = "vocabulary"
    ATTENTION_HEADS = "attention_heads"
    FEED_FORWARD_INTERMEDIATE = "feed_forward_intermediate"
    EXPERT_INTERMEDIATE = "expert_intermediate"
    CHANNELS = "channels"                                # state-space, convolution or recurrent channels
    SEGMENTED = "segmented"                              # a fused tensor of independently partitioned segments


@dataclass(frozen=True)
class MemberSharding:
    """``kind``: replicated | equal | balanced | partitioned | partitioned_segments | segmented.

    * equal / balanced: the axis itself is split (evenly, or into balanced contiguous ranges);
    * partitioned: the group's logical partition mapped onto the axis (``unit`` indices per logical element);
    * partitioned_segments: every segment of the axis carries the whole logical domain (gate | up);
    * segmented: every segment is partitioned on its own (balanced), results concatenated in segment order."""
    kind: str = "replicated"
    axis: int = 0
    segments: tuple = ()
    unit: int = 1

    @staticmethod
    def replicated():
        return MemberSharding()

    @staticmethod
    def equal(axis: int):
        return MemberSharding("equal", axis)

    @staticmethod
    def balanced(axis: int):
        return MemberSharding("balanced", axis)

    @staticmethod
    def partitioned(axis: int, unit: int = 1):
        return MemberSharding("partitioned", axis, (), unit)

    @staticmethod
    def partitioned_segments(axis: int, segments, unit: int = 1):
        return MemberSharding("partitioned_segments", axis, tuple((int(a), int(b)) for a, b in segments), unit)

    @staticmethod
    def segmented(axis: int, segments):
        return MemberSharding("segmented", axis, tuple((int(a), int(b)) for a, b in segments))


@dataclass(frozen=True)
class ParameterMemberSpec:
    name: str
    shape: tuple
    sharding: MemberSharding


@dataclass
class ParameterGroupSpec:
    """``extent``: size of the logical domain (heads, channels, vocabulary entries); ``replication``: consecutive ranks
    that share one logical range (KV heads when there are fewer of them than ranks); ``balanced``: allow uneven
    contiguous ranges instead of requiring ``extent % parts == 0``."""
    logical_name: str
    role: ParameterRole
    members: list
    extent: int = 0
    replication: int = 1
    balanced: bool = False

    def logical_range(self, rank: int, tp: int) -> tuple[int, int]:
        if self.role is ParameterRole.REPLICATED or self.extent == 0:
            return (0, self.extent)
        if tp % self.replication != 0:
            raise ValueError(f"{self.logical_name}: replication {self.replication} does not divide {tp} ranks")
        parts = tp // self.replication
        index = rank // self.replication
        if not self.balanced and self.extent % parts != 0:
            raise ValueError(f"{self.logical_name}: {self.extent} logical elements do not split evenly over {parts} parts")
        return balanced_contiguous_range(self.extent, parts, index)


class PlanError(ValueError):
    pass


@dataclass
class ParallelPlan:
    tp: int
    groups: list = field(default_factory=list)
    _members: dict = field(default_factory=dict)

    # ------------------------------------------------------------------ construction
    def add(self, group: ParameterGroupSpec) -> ParameterGroupSpec:
        for m in group.members:
            if m.name in self._members:
                raise PlanError(f"parameter {m.name} is planned twice ({self._members[m.name][0].logical_name}, {group.logical_name})")
            self._validate(group, m)
            self._members[m.name] = (group, m)
        self.groups.append(group)
        return group

    def _validate(self, g: ParameterGroupSpec, m: ParameterMemberSpec) -> None:
        sh = m.sharding
        if sh.kind == "replicated":
            return
        if not (0 <= sh.axis < len(m.shape)):
            raise PlanError(f"{m.name}: axis {sh.axis} outside shape {tuple(m.shape)}")
        n = int(m.shape[sh.axis])
        if sh.kind in ("partitioned",) and g.extent * sh.unit != n:
            raise PlanError(f"{m.name}: axis {sh.axis} has {n} entries, the group {g.logical_name} spans {g.extent} x {sh.unit}")
        if sh.kind == "equal" and n % self.tp != 0:
            raise PlanError(f"{m.name}: {n} entries do not split into {self.tp} equal shards")
        if sh.kind in ("partitioned_segments", "segmented"):
            prev = 0
            for a, b in sh.segments:
                if a < prev or b <= a or b > n:
                    raise PlanError(f"{m.name}: segments must be ordered, non-empty, non-overlapping and inside the axis")
                prev = b
                if sh.kind == "partitioned_segments" and (b - a) != g.extent * sh.unit:
                    raise PlanError(f"{m.name}: segment [{a}, {b}) does not carry the whole domain of {g.logical_name}")

    # ------------------------------------------------------------------ queries
    def member(self, name: str):
        try:
            return self._members[name]
        except KeyError:
            raise PlanError(f"parameter {name} is not part of the plan") from None

    def ranges(self, name: str, rank: int) -> Optional[list]:
        """Index ranges along the member's axis for ``rank`` (None: the whole tensor, replicated)."""
        g, m = self.member(name)
        sh = m.sharding
        if sh.kind == "replicated":
            return None
        n = int(m.shape[sh.axis])
        if sh.kind == "equal":
            per = n // self.tp
            return [(rank * per, (rank + 1) * per)]
        if sh.kind == "balanced":
            return [balanced_contiguous_range(n, self.tp, rank)]
        if sh.kind == "segmented":
            out = []
            for a, b in sh.segments:
                lo, hi = balanced_contiguous_range(b - a, self.tp, rank)
                out.append((a + lo, a + hi))
            return out
        lo, hi = g.logical_range(rank, self.tp)
        if sh.kind == "partitioned":
            return [(lo * sh.unit, hi * sh.unit)]
        return [(a + lo * sh.unit, a + hi * sh.unit) for a, _ in sh.segments]          # partitioned_segments

    def local_shape(self, name: str, rank: int) -> tuple:
        g, m = self.member(name)
        r = self.ranges(name, rank)
        if r is None:
            return tuple(m.shape)
        shape = list(m.shape)
        shape[m.sharding.axis] = sum(b - a for a, b in r)
        return tuple(shape)

    def select(self, name: str, tensor, rank: int):
        import torch

        r = self.ranges(name, rank)
        if r is None:
            return tensor
        axis = self.member(name)[1].sharding.axis
        if tuple(tensor.shape) != tuple(self.member(name)[1].shape):
            raise PlanError(f"{name}: tensor has shape {tuple(tensor.shape)}, the plan expects {tuple(self.member(name)[1].shape)}")
        parts = [tensor.narrow(axis, a, b - a) for a, b in r]
        return parts[0] if len(parts) == 1 else torch.cat(parts, axis)

    def read(self, name: str, source, rank: int):
        """Materialise this rank's shard from ``source``. With the partitioned axis first and a source that reads row
        ranges (``get_rows``), only those rows are read; otherwise the tensor is read whole and cut."""
        import torch

        r = self.ranges(name, rank)
        get = source.get if hasattr(source, "get") else source
        if r is None:
            return get(name)
        axis = self.member(name)[1].sharding.axis
        if axis == 0 and hasattr(source, "get_rows"):
            parts = [source.get_rows(name, a, b) for a, b in r]
            return parts[0] if len(parts) == 1 else torch.cat(parts, 0)
        return self.select(name, get(name), rank)

    def coverage(self, name: str) -> bool:
        """True when the ranks' ranges tile the member exactly once per replication group (a sanity check for plans)."""
        g, m = self.member(name)
        if m.sharding.kind == "replicated":
            return True
        n = int(m.shape[m.sharding.axis])
        seen = [0] * n
        for rank in range(0, self.tp, g.replication if m.sharding.kind.startswith("partitioned") else 1):
            for a, b in self.ranges(name, rank):
                for i in range(a, b):
                    seen[i] += 1
        return all(c == 1 for c in seen)

    def summary(self) -> list:
        return [{"group": g.logical_name, "role": g.role.value, "extent": g.extent, "replication": g.replication,
                 "members": [{"name": m.name, "shape": list(m.shape), "sharding": m.sharding.kind, "axis": m.sharding.axis}
                             for m in g.members]} for g in self.groups]


# -------------------------------------------------------------------------------------------------------------------
# Plans of the dense decoder families (HF tensor names). Sparse blocks are planned by the expert-parallel code.

def attention_groups(cfg, tp: int, prefix: str, fused_qkv: bool = False, bias: bool = False) -> list:
    """Query heads split evenly; key / value heads split, or replicated over ``tp / n_kv`` consecutive ranks when there are
    fewer of them than ranks (a GQA group stays whole); the output projection follows the query heads on its inputs."""
    H, D = cfg.hidden_size, cfg.head_dim
    nq, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
    if nq % tp != 0:
        raise PlanError(f"{nq} attention heads do not split over {tp} ranks")
    if nkv % tp != 0 and tp % nkv != 0:
        raise PlanError(f"{nkv} key / value heads can neither be split nor replicated over {tp} ranks")
    rep = 1 if nkv % tp == 0 else tp // nkv
    q_members, kv_members = [], []
    if fused_qkv:
        # one tensor [q | k | v]: two groups cannot share a member, so the fused tensor is a segmented member of the query
        # group only when the KV heads split like the query heads; otherwise the loader splits it first
        raise PlanError("fused qkv tensors are split into q, k, v by the loader before planning")
    q_members.append(ParameterMemberSpec(prefix + "q_proj.weight", (nq * D, H), MemberSharding.partitioned(0, D)))
    q_members.append(ParameterMemberSpec(prefix + "o_proj.weight", (H, nq * D), MemberSharding.partitioned(1, D)))
    for n in ("k_proj", "v_proj"):
        kv_members.append(ParameterMemberSpec(prefix + n + ".weight", (nkv * D, H), MemberSharding.partitioned(0, D)))
    if bias:
        q_members.append(ParameterMemberSpec(prefix + "q_proj.bias", (nq * D,), MemberSharding.partitioned(0, D)))
        for n in ("k_proj", "v_proj"):
            kv_members.append(ParameterMemberSpec(prefix + n + ".bias", (nkv * D,), MemberSharding.partitioned(0, D)))
    return [ParameterGroupSpec(prefix + "query_heads", ParameterRole.ATTENTION_HEADS, q_members, extent=nq),
            ParameterGroupSpec(prefix + "kv_heads", ParameterRole.ATTENTION_HEADS, kv_members, extent=nkv, replication=rep)]


def feed_forward_group(cfg, prefix: str, fused_gate_up: bool = False, intermediate: Optional[int] = None) -> ParameterGroupSpec:
    H, I = cfg.hidden_size, int(intermediate or cfg.intermediate_size)
    if fused_gate_up:
        members = [ParameterMemberSpec(prefix + "gate_up_proj.weight", (2 * I, H),
                                       MemberSharding.partitioned_segments(0, [(0, I), (I, 2 * I)]))]
    else:
        members = [ParameterMemberSpec(prefix + "gate_proj.weight", (I, H), MemberSharding.partitioned(0)),
                   ParameterMemberSpec(prefix + "up_proj.weight", (I, H), MemberSharding.partitioned(0))]
    members.append(ParameterMemberSpec(prefix + "down_proj.weight", (H, I), MemberSharding.partitioned(1)))
    return ParameterGroupSpec(prefix + "intermediate", ParameterRole.FEED_FORWARD_INTERMEDIATE, members, extent=I)


def dense_decoder_plan(cfg, tp: int, has=None) -> ParallelPlan:
    """The plan of a Llama-style dense decoder. ``has(name)``: which optional tensors the checkpoint carries (biases, a
    fused gate_up, an untied head); without it the plain layout is assumed."""
    has = has or (lambda name: False)
    plan = ParallelPlan(tp)
    H, V = cfg.hidden_size, cfg.vocab_size
    replicated = [ParameterMemberSpec("model.embed_tokens.weight", (V, H), MemberSharding.replicated()),
                  ParameterMemberSpec("model.norm.weight", (H,), MemberSharding.replicated())]
    if has("lm_head.weight") and not cfg.tie_word_embeddings:
        if V % tp == 0:
            plan.add(ParameterGroupSpec("vocabulary", ParameterRole.VOCABULARY,
                                        [ParameterMemberSpec("lm_head.weight", (V, H), MemberSharding.partitioned(0))], extent=V))
        else:
            replicated.append(ParameterMemberSpec("lm_head.weight", (V, H), MemberSharding.replicated()))
    for li in range(cfg.num_hidden_layers):
        p = f"model.layers.{li}."
        for g in attention_groups(cfg, tp, p + "self_attn.", bias=has(p + "self_attn.q_proj.bias")):
            plan.add(g)
        plan.add(feed_forward_group(cfg, p + "mlp.", fused_gate_up=has(p + "mlp.gate_up_proj.weight")))
        replicated += [ParameterMemberSpec(p + "input_layernorm.weight", (H,), MemberSharding.replicated()),
                       ParameterMemberSpec(p + "post_attention_layernorm.weight", (H,), MemberSharding.replicated())]
    plan.add(ParameterGroupSpec("replicated", ParameterRole.REPLICATED, replicated))
    return plan
