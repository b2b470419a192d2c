"""Cartesian parallel topology: data x pipeline x tensor x expert.

Rank formula and helper semantics follow eredu-core/src/topology.rs:65-167,195-387,495-520:
``rank = ((data * PP + pp) * TP + tp) * EP + ep`` (expert axis minor), contiguous balanced layer and
expert ranges, first stage owns the embedding, last stage owns the output head.

Extension the reference cannot express (its world size is the product of all axes): ``expert_over_tensor``
lets the expert axis *reuse* the tensor axis' ranks, i.e. attention runs TP=n while the experts of the
same ranks run EP=n (Qwen3-30B-A3B on 8 GPUs: attention TP=8 + EP=8).
"""
from __future__ import annotations

from dataclasses import dataclass


def balanced_contiguous_range(total: int, parts: int, index: int) -> tuple[int, int]:
    """[start, end) of part `index` when `total` items are split into `parts` contiguous, balanced ranges
    (the first ``total % parts`` ranges get one extra item)."""
    if parts <= 0 or not (0 <= index < parts):
        raise ValueError("invalid partition")
    base, extra = divmod(total, parts)
    start = index * base + min(index, extra)
    return start, start + base + (1 if index < extra else 0)


@dataclass(frozen=True)
class ParallelTopology:
    data: int = 1
    pipeline: int = 1
    tensor: int = 1
    expert: int = 1
    expert_over_tensor: bool = False

    def __post_init__(self):
        for name in ("data", "pipeline", "tensor", "expert"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} parallel size must be >= 1")
        if self.expert_over_tensor and self.expert != self.tensor:
            raise ValueError("expert_over_tensor requires expert == tensor")

    @property
    def world_size(self) -> int:
        e = 1 if self.expert_over_tensor else self.expert
        return self.data * self.pipeline * self.tensor * e

    def coordinates(self, rank: int) -> dict:
        if not (0 <= rank < self.world_size):
            raise ValueError(f"rank {rank} outside world of {self.world_size}")
        if self.expert_over_tensor:
            tp = rank % self.tensor
            rest = rank // self.tensor
            ep = tp
        else:
            ep = rank % self.expert
            rest = rank // self.expert
            tp = rest % self.tensor
            rest //= self.tensor
        pp = rest % self.pipeline
        data = rest // self.pipeline
        return {"data": data, "pipeline": pp, "tensor": tp, "expert": ep}

    def rank_for(self, data: int, pipeline: int, tensor: int, expert: int) -> int:
        if self.expert_over_tensor:
            if expert != tensor:
                raise ValueError("expert coordinate aliases the tensor coordinate")
            return (data * self.pipeline + pipeline) * self.tensor + tensor
        return ((data * self.pipeline + pipeline) * self.tensor + tensor) * self.expert + expert

    def axis_members(self, rank: int, axis: str) -> list[int]:
        """World ranks that differ from `rank` only along `axis`, in axis order."""
        c = self.coordinates(rank)
        size = getattr(self, axis)
        out = []
        for i in range(size):
            cc = dict(c)
            cc[axis] = i
            if self.expert_over_tensor and axis in ("tensor", "expert"):
                cc["tensor"] = cc["expert"] = i
            out.append(self.rank_for(cc["data"], cc["pipeline"], cc["tensor"], cc["expert"]))
        return out

    def layer_range(self, rank: int, n_layers: int) -> tuple[int, int]:
        return balanced_contiguous_range(n_layers, self.pipeline, self.coordinates(rank)["pipeline"])

    def expert_range(self, rank: int, n_experts: int) -> tuple[int, int]:
        return balanced_contiguous_range(n_experts, self.expert, self.coordinates(rank)["expert"])

    def pipeline_predecessor(self, rank: int):
        c = self.coordinates(rank)
        if c["pipeline"] == 0:
            return None
        return self.rank_for(c["data"], c["pipeline"] - 1, c["tensor"], c["expert"])

    def pipeline_successor(self, rank: int):
        c = self.coordinates(rank)
        if c["pipeline"] == self.pipeline - 1:
            return None
        return self.rank_for(c["data"], c["pipeline"] + 1, c["tensor"], c["expert"])

    def owns_embedding(self, rank: int) -> bool:
        return self.coordinates(rank)["pipeline"] == 0

    def owns_output_head(self, rank: int) -> bool:
        return self.coordinates(rank)["pipeline"] == self.pipeline - 1

    def sampling_rank(self, rank: int) -> int:
        """The rank of this replica that samples: last stage, tensor 0, expert 0 (backend/mlx/distributed.rs:160-186)."""
        c = self.coordinates(rank)
        return self.rank_for(c["data"], self.pipeline - 1, 0, 0)

    def preflight(self, n_layers: int, n_heads: int, n_kv_heads: int, n_experts: int = 0) -> list[str]:
        """Problems that make the topology unusable for a model; empty = ok. Checked before any payload I/O."""
        issues = []
        if self.data != 1:
            issues.append("data parallelism is declared but unsupported (fails closed)")
        if self.pipeline > n_layers:
            issues.append(f"pipeline size {self.pipeline} exceeds {n_layers} layers")
        if n_heads % self.tensor != 0:
            issues.append(f"{n_heads} attention heads are not divisible by tensor size {self.tensor}")
        if n_kv_heads % self.tensor != 0 and self.tensor % n_kv_heads != 0:
            issues.append(f"{n_kv_heads} kv heads can neither be split nor replicated over tensor size {self.tensor}")
        if self.expert > 1 and n_experts and self.expert > n_experts:
            issues.append(f"expert size {self.expert} exceeds {n_experts} experts")
        return issues
