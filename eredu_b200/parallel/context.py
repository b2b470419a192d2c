"""Per-rank view of the parallel topology, bound to process groups.

The counterpart of ``MlxParallelContext`` / ``ParallelRankTopology`` (eredu/src/backend/mlx/topology.rs:88,
eredu-core/src/topology.rs:195-387): coordinates, axis groups, layer / expert ranges and ownership
predicates for one rank. Groups are ``torch.distributed`` process groups (NCCL on GPUs, gloo on CPU).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from .topology import ParallelTopology, balanced_contiguous_range


@dataclass
class ParallelContext:
    topology: ParallelTopology
    rank: int
    tp_group: object = None
    pp_group: object = None
    ep_group: object = None
    world_group: object = None
    coords: dict = field(default_factory=dict)
    # which expert-parallel rank owns which routed expert: "balanced" (contiguous ranges), "round_robin" (expert e on rank
    # e mod ep), or an explicit owner per expert (ExpertAssignment, eredu/src/backend/mlx/runtime/distributed/expert.rs)
    expert_assignment: object = "balanced"

    def __post_init__(self):
        if self.topology.data != 1:
            # the axis is declared so that rank arithmetic stays stable, but no execution path replicates requests
            # over it: fail closed like the reference (eredu/src/backend/mlx/distributed.rs:139-144)
            raise ValueError("data parallelism is declared but unsupported: run one server per replica instead")
        self.coords = self.topology.coordinates(self.rank)

    @classmethod
    def single(cls) -> "ParallelContext":
        return cls(ParallelTopology(), 0)

    @classmethod
    def from_env(cls, topology: ParallelTopology, backend: Optional[str] = None) -> "ParallelContext":
        """Create the axis groups. Collective: every rank of the world calls it with the same topology, and the
        groups are created in identical order on every rank (runtime/distributed/topology.rs:63-135)."""
        import torch.distributed as dist

        assert dist.is_initialized(), "init torch.distributed first"
        rank, world = dist.get_rank(), dist.get_world_size()
        if world != topology.world_size:
            raise ValueError(f"world size {world} != topology world {topology.world_size}")
        ctx = cls(topology, rank, world_group=dist.group.WORLD)
        for axis, attr in (("tensor", "tp_group"), ("pipeline", "pp_group"), ("expert", "ep_group")):
            if axis == "expert" and topology.expert_over_tensor:
                continue
            seen = set()
            for r in range(world):
                members = tuple(topology.axis_members(r, axis))
                if members in seen:
                    continue
                seen.add(members)
                g = dist.new_group(list(members), backend=backend) if len(members) > 1 else None
                if rank in members:
                    setattr(ctx, attr, g)
        if topology.expert_over_tensor:
            ctx.ep_group = ctx.tp_group
        return ctx

    # ------------------------------------------------------------------ coordinates
    @property
    def tp_rank(self) -> int:
        return self.coords["tensor"]

    @property
    def tp_size(self) -> int:
        return self.topology.tensor

    @property
    def pp_rank(self) -> int:
        return self.coords["pipeline"]

    @property
    def pp_size(self) -> int:
        return self.topology.pipeline

    @property
    def ep_rank(self) -> int:
        return self.coords["expert"]

    @property
    def ep_size(self) -> int:
        return self.topology.expert

    def layer_range(self, n_layers: int) -> tuple[int, int]:
        return self.topology.layer_range(self.rank, n_layers)

    def expert_range(self, n_experts: int) -> tuple[int, int]:
        return self.topology.expert_range(self.rank, n_experts)

    def expert_order(self, n_experts: int) -> Optional[list]:
        """Checkpoint expert ids in execution order, or None for the identity. Execution ids are contiguous per rank
        (rank r runs execution ids ``expert_range``); a non-contiguous assignment is a renaming applied when the router
        rows and the expert banks are read, so routing, dispatch and combine kernels never see it. Every rank must own
        the same number of experts."""
        a = self.expert_assignment
        ep = self.ep_size
        if a == "balanced" or ep == 1:
            return None
        if a == "round_robin":
            owners = [e % ep for e in range(n_experts)]
        else:
            owners = [int(o) for o in a]
            if len(owners) != n_experts:
                raise ValueError(f"explicit expert assignment names {len(owners)} experts, the model has {n_experts}")
        if n_experts % ep != 0 or any(owners.count(r) != n_experts // ep for r in range(ep)):
            raise ValueError("every expert-parallel rank must own the same number of experts")
        return sorted(range(n_experts), key=lambda e: (owners[e], e))

    def owns_embedding(self) -> bool:
        return self.topology.owns_embedding(self.rank)

    def owns_output_head(self) -> bool:
        return self.topology.owns_output_head(self.rank)

    def is_sampling_rank(self) -> bool:
        return self.topology.sampling_rank(self.rank) == self.rank

    def attention_partition(self, n_heads: int, n_kv_heads: int) -> tuple[int, int, int]:
        """(local q heads, local kv heads, kv replication factor). A GQA group stays whole; when there are
        fewer kv heads than tensor ranks each kv head is replicated on ``tp / n_kv`` consecutive ranks."""
        tp = self.tp_size
        if n_heads % tp != 0:
            raise ValueError(f"{n_heads} heads not divisible by tp={tp}")
        if n_kv_heads % tp == 0:
            return n_heads // tp, n_kv_heads // tp, 1
        if tp % n_kv_heads == 0:
            return n_heads // tp, 1, tp // n_kv_heads
        raise ValueError(f"cannot place {n_kv_heads} kv heads on tp={tp}")
