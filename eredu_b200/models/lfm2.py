"""LFM2 / LFM2.5 hybrid decoders: gated short convolutions interleaved with q/k-normalised GQA attention.

Architecture: eredu/src/backend/mlx/architectures/lfm2/model.rs (layer schedule :246-290, attention :800-840, short
convolution :853-914, dense SwiGLU ``w2(silu(w1 x) * w3 x)``); tensor names: architectures/lfm2/checkpoint.rs:89-190.
The block structure is the Llama one (pre-norm operator, pre-norm FFN), so the family runs on
:class:`eredu_b200.models.llama.CausalLM`; this module only translates the checkpoint's tensor names to the
canonical ones the builder asks for.
"""
from __future__ import annotations

import re

_LAYER = re.compile(r"^model\.layers\.(\d+)\.(.+)$")
_REST = {
    "input_layernorm.weight": "operator_norm.weight",
    "post_attention_layernorm.weight": "ffn_norm.weight",
    "self_attn.o_proj.weight": "self_attn.out_proj.weight",
    "self_attn.q_norm.weight": "self_attn.q_layernorm.weight",
    "self_attn.k_norm.weight": "self_attn.k_layernorm.weight",
    "mlp.gate_proj.weight": "feed_forward.w1.weight",
    "mlp.up_proj.weight": "feed_forward.w3.weight",
    "mlp.down_proj.weight": "feed_forward.w2.weight",
    "mlp.gate.weight": "feed_forward.gate.weight",
    "mlp.expert_bias": "feed_forward.expert_bias",
}
_EXPERT = re.compile(r"^mlp\.experts\.(\d+)\.(gate|up|down)_proj\.weight$")
_EXPERT_W = {"gate": "w1", "up": "w3", "down": "w2"}


def checkpoint_name(canonical: str) -> str:
    """Name of a canonical (Llama-style) tensor in an LFM2 checkpoint."""
    if canonical == "model.norm.weight":
        return "model.embedding_norm.weight"
    m = _LAYER.match(canonical)
    if not m:
        return canonical
    li, rest = m.group(1), m.group(2)
    if rest in _REST:
        rest = _REST[rest]
    else:
        e = _EXPERT.match(rest)
        if e:
            rest = f"feed_forward.experts.{e.group(1)}.{_EXPERT_W[e.group(2)]}.weight"
    return f"model.layers.{li}.{rest}"


def canonical_access(get, has):
    """Wrap a checkpoint's ``get`` / ``has`` so that canonical names resolve to the LFM2 ones (either spelling of a
    tensor is accepted, so re-exported checkpoints that already use Llama names keep working)."""

    def g(name):
        alt = checkpoint_name(name)
        return get(alt) if alt != name and has(alt) else get(name)

    def h(name):
        alt = checkpoint_name(name)
        return (alt != name and has(alt)) or has(name)

    return g, h


def to_checkpoint_names(state: dict) -> dict:
    """Rename a canonical state dict the way an LFM2 export names its tensors (used to write test checkpoints)."""
    return {checkpoint_name(k): v for k, v in state.items()}
