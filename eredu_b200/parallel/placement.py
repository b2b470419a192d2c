"""Placement of execution-group DAGs on pipeline stages.

Counterpart of ``PlacedExecutionDag`` (eredu/src/backend/mlx/architectures/distributed/pipeline/placement.rs): a model is
a DAG of *execution groups* - the ordered decoder blocks, a vision or audio encoder, a projector, the assembly of
modality and text payloads - each with a number of ordered units, the pipeline coordinates that may own it, the
tensors its first / last owner keeps (embedding, final norm, head), the payload it consumes and produces, and a
residency / checkpoint binding. Planning balances every group's units over its rank path, derives every transfer from
ownership (inside a group: owner to next owner; between groups: the producer's merge destination to the consumer's first
owner), and validates the whole before any weight is read: unknown or cyclic dependencies, impossible coordinates,
payload contracts that do not match, static tensors with two owners. Nothing is inferred from numeric adjacency of
pipeline ranks.

``decoder_placement`` is the plan of a text decoder (one group over all stages), ``multimodal_placement`` adds encoder,
projector and assembly groups in front of it. ``PipelineRunner`` checks its stage's layers against the plan.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from .topology import balanced_contiguous_range

KINDS = ("decoder", "vision_encoder", "audio_encoder", "projector", "merger", "modality_finalization")


class PlacementError(ValueError):
    pass


@dataclass(frozen=True)
class PayloadField:
    name: str
    shape: tuple                 # symbolic: ("tokens", "hidden")
    optional: bool = False


@dataclass(frozen=True)
class PayloadSchema:
    id: str
    fields: tuple

    @staticmethod
    def of(schema_id: str, *fields) -> "PayloadSchema":
        return PayloadSchema(schema_id, tuple(f if isinstance(f, PayloadField) else PayloadField(f[0], tuple(f[1])) for f in fields))


@dataclass(frozen=True)
class ActiveSubgroup:
    tensor_parallel: bool = True
    expert_parallel: bool = False


@dataclass
class GroupRequest:
    """Planner input for one group. ``rank_path``: the pipeline coordinates allowed to own it, in order."""
    id: str
    kind: str
    unit_count: int
    rank_path: list
    input_schema: PayloadSchema
    output_schema: PayloadSchema
    dependencies: list = field(default_factory=list)
    active: ActiveSubgroup = ActiveSubgroup()
    first_owner_static_roles: list = field(default_factory=list)
    last_owner_static_roles: list = field(default_factory=list)
    merge_destination: Optional[int] = None
    residency_prefix: str = ""
    request_optional: bool = False       # absent request media skip the group (no leases, no transfers)
    checkpoint_group: str = ""


@dataclass
class PlacedGroup:
    id: str
    kind: str
    dependencies: list
    unit_count: int
    owners: list                 # [(pp_rank, (start, end))] in path order, empty ranges dropped
    active: ActiveSubgroup
    static_tensors: list         # [(role, pp_rank)]
    input_schema: PayloadSchema
    output_schema: PayloadSchema
    merge_destination: int
    residency_prefix: str
    request_optional: bool
    checkpoint_group: str

    def local_units(self, pp_rank: int):
        for r, rng in self.owners:
            if r == pp_rank:
                return rng
        return None

    def first_owner(self):
        return self.owners[0][0] if self.owners else None


@dataclass(frozen=True)
class Route:
    from_group: str
    to_group: str
    from_pp_rank: int
    to_pp_rank: int
    pp_path: tuple
    payload: PayloadSchema


@dataclass(frozen=True)
class ConcurrencyPolicy:
    rank_local_streams: bool = True
    shared_residency_window: bool = False
    tensor_parallel_size: int = 1
    expert_parallel_size: int = 1


class PlacedExecutionDag:
    def __init__(self, groups, routes, order, output):
        self.groups = groups
        self.routes = routes
        self.execution_order = order          # indices into groups, dependencies first
        self.output = output
        self._by_id = {g.id: i for i, g in enumerate(groups)}

    # ------------------------------------------------------------------ planning
    @classmethod
    def plan(cls, pipeline_stages: int, requests: list, output: str) -> "PlacedExecutionDag":
        if pipeline_stages < 1:
            raise PlacementError("a placed execution DAG needs at least one pipeline rank")
        ids = [r.id for r in requests]
        if len(set(ids)) != len(ids):
            raise PlacementError("execution group ids must be unique")
        if output not in ids:
            raise PlacementError(f"output group {output!r} is not declared")
        known = set(ids)
        for r in requests:
            if r.kind not in KINDS:
                raise PlacementError(f"execution group {r.id!r} has unknown kind {r.kind!r}")
            for d in r.dependencies:
                if d not in known:
                    raise PlacementError(f"execution group {r.id!r} depends on undeclared group {d!r}")
                if d == r.id:
                    raise PlacementError(f"execution group {r.id!r} depends on itself")
        order = cls._topological(requests)
        groups = []
        for r in requests:
            cls._check_path(r, pipeline_stages)
            cls._check_schema(r.id, "input", r.input_schema)
            cls._check_schema(r.id, "output", r.output_schema)
            owners = []
            for i, rank in enumerate(r.rank_path):
                a, b = balanced_contiguous_range(r.unit_count, len(r.rank_path), i)
                if b > a:
                    owners.append((rank, (a, b)))
            first = owners[0][0] if owners else r.rank_path[0]
            last = owners[-1][0] if owners else first
            merge = last if r.merge_destination is None else r.merge_destination
            if not (0 <= merge < pipeline_stages):
                raise PlacementError(f"execution group {r.id!r} has impossible merge destination {merge}")
            static, seen = [], set()
            for role, rank in [(x, first) for x in r.first_owner_static_roles] + [(x, last) for x in r.last_owner_static_roles]:
                if role in seen:
                    raise PlacementError(f"execution group {r.id!r} assigns static tensor role {role!r} twice")
                seen.add(role)
                static.append((role, rank))
            groups.append(PlacedGroup(r.id, r.kind, list(r.dependencies), r.unit_count, owners, r.active, static,
                                      r.input_schema, r.output_schema, merge, r.residency_prefix or r.id, r.request_optional,
                                      r.checkpoint_group or r.id))
        by_id = {g.id: g for g in groups}
        routes = []
        for g in groups:
            for (a, _), (b, _) in zip(g.owners, g.owners[1:]):
                routes.append(Route(g.id, g.id, a, b, (a, b), g.output_schema))
        for consumer in groups:
            to = consumer.first_owner()
            to = consumer.merge_destination if to is None else to
            for dep in consumer.dependencies:
                producer = by_id[dep]
                if producer.output_schema != consumer.input_schema:
                    raise PlacementError(f"payload mismatch: {producer.id!r} outputs {producer.output_schema.id!r}, "
                                         f"{consumer.id!r} expects {consumer.input_schema.id!r}")
                frm = producer.merge_destination
                routes.append(Route(producer.id, consumer.id, frm, to, (frm,) if frm == to else (frm, to), producer.output_schema))
        roles = {}
        for g in groups:
            for role, rank in g.static_tensors:
                if role in roles and roles[role] != (g.id, rank):
                    raise PlacementError(f"static tensor role {role!r} has two owners: {roles[role]} and {(g.id, rank)}")
                roles[role] = (g.id, rank)
        return cls(groups, routes, order, output)

    @staticmethod
    def _topological(requests) -> list:
        index = {r.id: i for i, r in enumerate(requests)}
        state, order = {}, []

        def visit(i, trail):
            s = state.get(i)
            if s == 2:
                return
            if s == 1:
                raise PlacementError("execution groups form a cycle: " + " -> ".join(trail + [requests[i].id]))
            state[i] = 1
            for d in requests[i].dependencies:
                visit(index[d], trail + [requests[i].id])
            state[i] = 2
            order.append(i)

        for i in range(len(requests)):
            visit(i, [])
        return order

    @staticmethod
    def _check_path(r: GroupRequest, stages: int) -> None:
        if not r.rank_path:
            raise PlacementError(f"execution group {r.id!r} has an empty rank path")
        if len(set(r.rank_path)) != len(r.rank_path):
            raise PlacementError(f"execution group {r.id!r} names a pipeline rank twice")
        for rank in r.rank_path:
            if not (0 <= rank < stages):
                raise PlacementError(f"execution group {r.id!r} names pipeline rank {rank} outside {stages} stages")
        if r.unit_count < 0:
            raise PlacementError(f"execution group {r.id!r} has a negative unit count")

    @staticmethod
    def _check_schema(gid: str, side: str, schema: PayloadSchema) -> None:
        if not schema.id.strip():
            raise PlacementError(f"execution group {gid!r} has an unnamed {side} payload")
        names = [f.name for f in schema.fields]
        if not names or len(set(names)) != len(names):
            raise PlacementError(f"execution group {gid!r}: {side} payload {schema.id!r} needs distinct, non-empty fields")

    # ------------------------------------------------------------------ queries
    def group(self, gid: str) -> Optional[PlacedGroup]:
        i = self._by_id.get(gid)
        return None if i is None else self.groups[i]

    def local_groups(self, pp_rank: int, media_present=()) -> list:
        """Groups with units on ``pp_rank`` in execution order; request-optional groups only when their modality is present."""
        out = []
        for i in self.execution_order:
            g = self.groups[i]
            if g.local_units(pp_rank) is None:
                continue
            if g.request_optional and g.kind not in media_present and g.id not in media_present:
                continue
            out.append(g)
        return out

    def routes_into(self, pp_rank: int) -> list:
        return [r for r in self.routes if r.to_pp_rank == pp_rank and r.from_pp_rank != pp_rank]

    def routes_out_of(self, pp_rank: int) -> list:
        return [r for r in self.routes if r.from_pp_rank == pp_rank and r.to_pp_rank != pp_rank]

    def static_owner(self, role: str):
        for g in self.groups:
            for r, rank in g.static_tensors:
                if r == role:
                    return rank
        return None

    def concurrency_compatibility(self, a: str, b: str, policy: ConcurrencyPolicy):
        """None when two dependency-free groups may run at the same time, else (reason, shared pipeline ranks)."""
        ga, gb = self.group(a), self.group(b)
        shared = sorted({r for r, _ in ga.owners} & {r for r, _ in gb.owners})
        if not shared:
            return None
        if not policy.rank_local_streams:
            return ("shared_rank_backend", shared)
        if policy.shared_residency_window and (ga.residency_prefix or gb.residency_prefix):
            return ("shared_residency_window", shared)
        collectives = (policy.tensor_parallel_size > 1 and ga.active.tensor_parallel and gb.active.tensor_parallel) or \
                      (policy.expert_parallel_size > 1 and ga.active.expert_parallel and gb.active.expert_parallel)
        if collectives:
            return ("collective_ordering", shared)      # every rank must submit the groups' collectives in the same order
        return None

    def summary(self) -> dict:
        return {"output": self.output,
                "groups": [{"id": g.id, "kind": g.kind, "units": g.unit_count, "owners": [[r, list(rng)] for r, rng in g.owners],
                            "static": [list(s) for s in g.static_tensors], "merge_destination": g.merge_destination}
                           for g in self.groups],
                "routes": [{"from": r.from_group, "to": r.to_group, "path": list(r.pp_path), "payload": r.payload.id}
                           for r in self.routes]}


HIDDEN = PayloadSchema.of("hidden_states", ("hidden", ("tokens", "hidden")))
TOKENS = PayloadSchema.of("token_ids", ("token_ids", ("tokens",)))


def decoder_placement(n_layers: int, pipeline_stages: int, sparse: bool = False) -> PlacedExecutionDag:
    """A text decoder: one group over all stages, the embedding on its first owner, final norm and head on its last."""
    req = GroupRequest("decoder", "decoder", n_layers, list(range(pipeline_stages)), TOKENS, HIDDEN,
                       active=ActiveSubgroup(True, sparse), first_owner_static_roles=["embedding"],
                       last_owner_static_roles=["final_norm", "output_head"], residency_prefix="layer", checkpoint_group="decoder")
    return PlacedExecutionDag.plan(pipeline_stages, [req], "decoder")


def multimodal_placement(n_layers: int, pipeline_stages: int, vision_blocks: int = 0, audio_blocks: int = 0,
                         encoder_stages: Optional[list] = None, sparse: bool = False) -> PlacedExecutionDag:
    """Encoders (on ``encoder_stages``, by default the first stage) feed projectors; an assembly group on the decoder's
    first stage merges modality rows into the token embeddings; the decoder follows over all stages."""
    enc = encoder_stages or [0]
    feats = PayloadSchema.of("modality_features", ("features", ("patches", "hidden")))
    merged = PayloadSchema.of("merged_embeddings", ("hidden", ("tokens", "hidden")))
    reqs, deps = [], []
    for name, kind, blocks in (("vision", "vision_encoder", vision_blocks), ("audio", "audio_encoder", audio_blocks)):
        if blocks <= 0:
            continue
        raw = PayloadSchema.of(f"{name}_input", (f"{name}_patches", ("patches", "patch_dim")))
        enc_out = PayloadSchema.of(f"{name}_states", ("states", ("patches", f"{name}_hidden")))
        reqs.append(GroupRequest(f"{name}_encoder", kind, blocks, list(enc), raw, enc_out, active=ActiveSubgroup(True, False),
                                 first_owner_static_roles=[f"{name}_patch_embedding"], residency_prefix=f"{name}_block",
                                 request_optional=True, checkpoint_group=f"{name}_tower"))
        reqs.append(GroupRequest(f"{name}_projector", "projector", 1, [enc[-1]], enc_out, feats, dependencies=[f"{name}_encoder"],
                                 active=ActiveSubgroup(True, False), request_optional=True, checkpoint_group=f"{name}_tower"))
        deps.append(f"{name}_projector")
    reqs.append(GroupRequest("assembly", "modality_finalization", 1, [0], feats, merged, dependencies=deps,
                             active=ActiveSubgroup(False, False), first_owner_static_roles=["embedding"]))
    reqs.append(GroupRequest("decoder", "decoder", n_layers, list(range(pipeline_stages)), merged, HIDDEN, dependencies=["assembly"],
                             active=ActiveSubgroup(True, sparse), last_owner_static_roles=["final_norm", "output_head"],
                             residency_prefix="layer", checkpoint_group="decoder"))
    return PlacedExecutionDag.plan(pipeline_stages, reqs, "decoder")
