"""Artifact inspection, resource estimates, admission and the automatic execution planner.

Counterparts: eredu-core/src/artifact.rs:484-516 (header-only inspection, preparation policy), inspection.rs:10-260
(``ModelInspectionReport`` with issue codes and ``is_loadable``), capability.rs:107-560 (``estimate_runtime_state``:
KV bytes per token, admission), execution.rs:9-318 (``ExecutionPlan`` schema version 2: device, topology,
residency, weight transformation, expert cache, drafting, mapped shards) and automatic.rs:96-830
(``HardwareProfile``, ``ModelResourceProfile``, ``AutomaticPlanner::plan``).

The planner is written for one node of B200s (180 GB HBM3e each, every peer at full NVLink bandwidth through
NVSwitch): it prefers the smallest tensor-parallel degree whose shards, KV pool and workspace fit, puts experts on the
tensor ranks for sparse models, and only then falls back to load-time 4-bit weights and host-resident layers.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Optional

from ..models.config import DENSE_TYPES, MOE_TYPES, ModelConfig

EXECUTION_PLAN_SCHEMA_VERSION = 2
DEFAULT_MAX_MAPPED_SHARDS = 4
SUPPORTED_TYPES = DENSE_TYPES | {"qwen3_moe", "mixtral", "gpt_oss", "lfm2_moe", "qwen3_next", "qwen3_5", "qwen3_5_text", "qwen3_5_moe", "qwen3_5_moe_text", "nemotron_h", "deepseek_v3", "deepseek_v4", "inkling_mm_model", "muse_glimmer", "kimi_linear", "gemma4"}


# ---------------------------------------------------------------------------------------------- inspection
@dataclass
class InspectionIssue:
    code: str
    severity: str      # "error" | "warning" | "info"
    message: str


@dataclass
class ModelInspectionReport:
    path: str
    format: str                      # "safetensors" | "gguf"
    model_type: str
    config: Optional[ModelConfig]
    tensor_count: int = 0
    tensor_bytes: int = 0
    parameter_count: int = 0
    dtypes: dict = field(default_factory=dict)      # dtype / quant type -> bytes
    quantization: Optional[dict] = None
    has_tokenizer: bool = False
    issues: list = field(default_factory=list)
    text: dict = field(default_factory=dict)        # filled by api.inspection.inspect_text_model: readiness per text facility

    @property
    def is_loadable(self) -> bool:
        return not any(i.severity == "error" for i in self.issues)

    def to_dict(self) -> dict:
        d = asdict(self)
        d["config"] = asdict(self.config) if self.config is not None else None
        d["is_loadable"] = self.is_loadable
        return d


# Checkpoints of the realtime speech stack: not text-generation models, each has a loader of its own.
SPEECH_TYPES = {
    "moshi": ("eredu_b200.models.moshi.MoshiLm.load (temporal + depth transformers; runtime.realtime drives sessions)",
              ["decoder.model.embed_tokens.weight", "decoder.model.norm.weight", "depth_decoder.input_projections.weight",
               "depth_decoder.lm_heads.weight"]),
    "mimi": ("eredu_b200.codec.Mimi.load (streaming audio codec)",
             ["encoder.layers.0.conv.weight", "decoder.layers.0.conv.weight", "quantizer.semantic_residual_vector_quantizer.input_proj.weight",
              "quantizer.acoustic_residual_vector_quantizer.output_proj.weight"]),
}


def required_tensors(cfg: ModelConfig) -> list[tuple]:
    """Tensors whose absence makes a SafeTensors directory unloadable, as tuples of accepted spellings: the embedding,
    the final norm and the main input projection of the first layer's operator, under the family's own names."""
    if cfg.model_type in SPEECH_TYPES:
        return [(n,) for n in SPEECH_TYPES[cfg.model_type][1]]
    if cfg.model_type == "deepseek_v4":
        return [("embed.weight",), ("norm.weight",), ("layers.0.attn.wq_a.weight",), ("hc_head_fn",)]
    if cfg.model_type == "inkling_mm_model":
        return [("model.embed_tokens.weight", "model.llm.embed.weight"), ("model.norm.weight", "model.llm.norm.weight"),
                ("model.layers.0.self_attn.r_proj.weight", "model.llm.layers.0.attn.wr_du.weight")]
    p = "model.layers.0."
    kind = cfg.layer_types[0] if cfg.layer_types else "full_attention"
    if cfg.model_type == "nemotron_h":
        first = {"mamba": "mixer.in_proj.weight", "attention_only": "mixer.q_proj.weight", "mlp_only": "mixer.up_proj.weight",
                 "moe_only": "mixer.gate.weight"}[kind]
        names = [("model.embed_tokens.weight",), ("model.norm.weight",), (p + first,)]
        from ..models.nemotron_h import checkpoint_names

        return [tuple(n for a in alt for n in (checkpoint_names(a) + [a])) for alt in names]
    if kind == "conv":
        first = (p + "conv.in_proj.weight",)
    elif kind == "linear_attention":
        first = (p + "linear_attn.in_proj_qkvz.weight", p + "linear_attn.in_proj_qkv.weight")
    elif kind == "kda":
        first = (p + "self_attn.f_a_proj.weight",)
    elif cfg.is_mla:
        first = (p + "self_attn.kv_a_proj_with_mqa.weight",)
    else:
        first = (p + "self_attn.q_proj.weight", p + "self_attn.qkv_proj.weight")
    names = [("model.embed_tokens.weight",), ("model.norm.weight",), first]
    if cfg.model_type in ("lfm2", "lfm2_moe"):
        from ..models.lfm2 import checkpoint_name

        return [tuple(n for a in alt for n in (checkpoint_name(a), a)) for alt in names]
    return names


def inspect_artifact(path) -> ModelInspectionReport:
    """Header-only inspection: no tensor payload is read or mapped."""
    from ..formats.checkpoint import GGML_NAME
    from ..lib import _eredu_host as H

    path = Path(path)
    issues: list[InspectionIssue] = []
    if path.is_dir():
        if not (path / "config.json").exists():
            return ModelInspectionReport(str(path), "safetensors", "unknown", None,
                                         issues=[InspectionIssue("missing_config", "error", "config.json not found")])
        try:
            cfg = ModelConfig.from_pretrained(path)
        except Exception as e:    # the config names a family but its fields do not describe a loadable model
            return ModelInspectionReport(str(path), "safetensors", "unknown", None,
                                         issues=[InspectionIssue("invalid_config", "error", f"config.json: {e}")])
        try:
            store = H.SafetensorsStore(str(path), 1)
        except Exception as e:
            return ModelInspectionReport(str(path), "safetensors", cfg.model_type, cfg,
                                         issues=[InspectionIssue("unreadable_weights", "error", str(e))])
        rep = ModelInspectionReport(str(path), "safetensors", cfg.model_type, cfg, quantization=cfg.quantization,
                                    has_tokenizer=(path / "tokenizer.json").exists())
        itemsize = {"F32": 4, "F16": 2, "BF16": 2, "I32": 4, "U32": 4, "I64": 8, "U8": 1, "I8": 1, "F64": 8, "BOOL": 1,
                    "I16": 2, "U16": 2, "F8_E4M3": 1, "F8_E5M2": 1}
        keys = set(store.keys())
        for k in keys:
            info = store.info(k)
            n = 1
            for s in info["shape"]:
                n *= int(s)
            nb = n * itemsize.get(info["dtype"], 1)
            rep.tensor_count += 1
            rep.tensor_bytes += nb
            rep.dtypes[info["dtype"]] = rep.dtypes.get(info["dtype"], 0) + nb
            if not k.endswith((".scales", ".biases")):
                bits = (cfg.quantization or {}).get("bits") if (k[:-7] + ".scales") in keys and k.endswith(".weight") else None
                rep.parameter_count += n * (32 // int(bits)) if bits else n
        # a decoder stored next to towers (vision-language exports, Qwen3.5) sits under model.language_model.*
        def spellings(name):
            return (name, "model.language_model." + name[len("model."):]) if name.startswith("model.") else (name,)

        for alternatives in required_tensors(cfg):
            if not any(sp in keys for name in alternatives for sp in spellings(name)):
                issues.append(InspectionIssue("missing_tensor", "error", f"required tensor {alternatives[0]} is absent"))
        if cfg.model_type not in SPEECH_TYPES and not cfg.tie_word_embeddings and "lm_head.weight" not in keys:
            issues.append(InspectionIssue("missing_tensor", "error", "untied model without lm_head.weight"))
    elif path.is_file():
        try:
            reader = H.GgufReader(str(path))
        except Exception as e:
            return ModelInspectionReport(str(path), "gguf", "unknown", None,
                                         issues=[InspectionIssue("unreadable_gguf", "error", str(e))])
        md = reader.metadata() if callable(reader.metadata) else reader.metadata
        tensors = reader.tensors()
        names = {t["name"] if isinstance(t, dict) else t[0] for t in tensors}
        cfg = ModelConfig.from_gguf_metadata(md, "output.weight" in names)
        rep = ModelInspectionReport(str(path), "gguf", cfg.model_type, cfg, has_tokenizer="tokenizer.ggml.tokens" in md)
        for t in tensors:
            info = t if isinstance(t, dict) else {"name": t[0], "type": t[1], "shape": t[2], "nbytes": t[3]}
            n = 1
            for s in info["shape"]:
                n *= int(s)
            rep.tensor_count += 1
            rep.tensor_bytes += int(info.get("nbytes", 0))
            tname = GGML_NAME.get(int(info["type"]), f"type{info['type']}")
            rep.dtypes[tname] = rep.dtypes.get(tname, 0) + int(info.get("nbytes", 0))
            rep.parameter_count += n
        if "token_embd.weight" not in names:
            issues.append(InspectionIssue("missing_tensor", "error", "token_embd.weight is absent"))
    else:
        return ModelInspectionReport(str(path), "unknown", "unknown", None,
                                     issues=[InspectionIssue("not_found", "error", f"{path} does not exist")])
    if cfg.model_type in SPEECH_TYPES:
        issues.append(InspectionIssue("speech_model", "error", f"{cfg.model_type} is not a text-generation model: load it with "
                                      + SPEECH_TYPES[cfg.model_type][0]))
        rep.issues = issues
        return rep
    if cfg.model_type not in SUPPORTED_TYPES:
        sev = "error"
        issues.append(InspectionIssue("unsupported_architecture", sev, f"model type {cfg.model_type!r} has no adapter here"
                                      + (" (recognised sparse family)" if cfg.model_type in MOE_TYPES else "")))
    if cfg.head_dim not in (64, 128):
        issues.append(InspectionIssue("head_dim", "warning", f"head_dim {cfg.head_dim}: attention kernels cover 64 and 128; "
                                      "other sizes run the reference path"))
    if not rep.has_tokenizer:
        issues.append(InspectionIssue("no_tokenizer", "info", "no tokenizer found: only token-id APIs are available"))
    rep.issues = issues
    return rep


# ---------------------------------------------------------------------------------------------- resource profile
@dataclass
class ModelResourceProfile:
    weight_bytes: int                 # as stored in the checkpoint (or after the planned transformation)
    kv_bytes_per_token: int           # all layers, K and V, at the cache dtype
    layers: int
    sliding_layers: int = 0
    sliding_window: int = 0
    expert_bytes: int = 0             # part of weight_bytes that belongs to routed experts
    workspace_bytes: int = 2 << 30    # activations, logits, collective buffers, allocator slack
    state_bytes_per_sequence: int = 0  # hybrid models: fixed recurrent / convolution state of one sequence
    windowed_bytes_per_token: int = 0  # families whose layers differ in width: bytes kept per token only inside ``sliding_window``
    #                                    (then ``kv_bytes_per_token`` counts what grows with the whole context and ``sliding_layers`` is 0)


def estimate_runtime_state(cfg: ModelConfig, weight_bytes: Optional[int] = None, cache_dtype_bytes: int = 2) -> ModelResourceProfile:
    """KV bytes per token and static weight bytes of a decoder (``estimate_runtime_state``, capability.rs)."""
    H, D = cfg.hidden_size, cfg.head_dim
    L = cfg.num_hidden_layers
    family = _family_profile(cfg, weight_bytes, cache_dtype_bytes)
    if family is not None:
        return family
    # only softmax-attention layers keep K/V per token; convolution and gated-delta layers keep a fixed state
    stateful = [li for li in range(L) if cfg.layer_is_conv(li) or cfg.layer_has_recurrent_state(li)]
    attn_layers = sum(1 for li in range(L) if cfg.layer_has_kv(li))
    kv_tok = 2 * cfg.num_key_value_heads * D * cache_dtype_bytes * attn_layers
    if cfg.is_mla:   # one compressed latent + rotary key per token and layer, shared by the heads
        kv_tok = (cfg.kv_lora_rank + cfg.qk_rope_head_dim) * cache_dtype_bytes * attn_layers
    state = 0
    for li in stateful:
        if cfg.layer_is_conv(li):
            state += (cfg.conv_l_cache - 1) * H * cache_dtype_bytes
        elif cfg.layer_is_kda(li):
            P_ = cfg.linear_num_value_heads * cfg.linear_value_head_dim
            state += (cfg.linear_conv_kernel_dim - 1) * 3 * P_ * cache_dtype_bytes
            state += cfg.linear_num_value_heads * cfg.linear_value_head_dim ** 2 * 4
        elif cfg.layer_is_mamba(li):
            inter = cfg.mamba_num_heads * cfg.mamba_head_dim
            state += (cfg.mamba_conv_kernel - 1) * (inter + 2 * cfg.mamba_n_groups * cfg.ssm_state_size) * cache_dtype_bytes
            state += cfg.mamba_num_heads * cfg.mamba_head_dim * cfg.ssm_state_size * 4
        else:
            conv_dim = 2 * cfg.linear_num_key_heads * cfg.linear_key_head_dim + cfg.linear_num_value_heads * cfg.linear_value_head_dim
            state += (cfg.linear_conv_kernel_dim - 1) * conv_dim * cache_dtype_bytes
            state += cfg.linear_num_value_heads * cfg.linear_key_head_dim * cfg.linear_value_head_dim * 4
    attn = (cfg.num_attention_heads * D * H) * 2 + (cfg.num_key_value_heads * D * H) * 2
    dense_mlp = 3 * H * cfg.intermediate_size
    expert = 3 * H * cfg.moe_intermediate_size * cfg.num_experts if cfg.is_moe else 0
    moe_layers = sum(1 for li in range(L) if cfg.layer_is_moe(li))
    params = L * attn + (L - moe_layers) * dense_mlp + moe_layers * (expert + cfg.num_experts * H)
    params += cfg.vocab_size * H * (1 if cfg.tie_word_embeddings else 2)
    wb = weight_bytes if weight_bytes is not None else params * 2
    sliding = sum(1 for li in range(L) if cfg.layer_window(li) > 0)
    share = (moe_layers * expert) / max(1, params)
    return ModelResourceProfile(int(wb), int(kv_tok), max(1, attn_layers), sliding, int(cfg.sliding_window or 0),
                                int(wb * share), state_bytes_per_sequence=int(state))


def _family_profile(cfg: ModelConfig, weight_bytes, b: int):
    """Cache formulas of the families whose layers do not share one K/V width (per-family formulas of the reference's
    capability.rs): bytes that grow with the whole context, bytes kept only inside the window, fixed state."""
    L = cfg.num_hidden_layers
    H = cfg.hidden_size
    if cfg.model_type == "gemma4":
        from ..models.gemma4 import geometry

        grow = win = 0
        for sliding, D, nkv, k_eq_v, donor in geometry(cfg):
            if donor is not None:
                continue                                      # the KV-sharing tail reads an earlier layer's pages
            per = (1 if k_eq_v else 2) * nkv * D * b
            if sliding:
                win += per
            else:
                grow += per
        wb = weight_bytes if weight_bytes is not None else 0
        return ModelResourceProfile(int(wb), int(grow), L, 0, int(cfg.sliding_window or 0), 0, windowed_bytes_per_token=int(win))
    if cfg.model_type == "deepseek_v4":
        g = cfg.extra["deepseek_v4"]
        D, Di = int(g["head_dim"]), int(g["index_head_dim"])
        ratios = [int(r) for r in (g.get("compress_ratios") or [0] * L)][:L]
        win = L * D * b                                       # one shared key = value head per layer, inside the window
        grow = sum((D + (Di if r == 4 else 0)) * b / r for r in ratios if r)          # pooled streams: one token per r
        # open pooling windows and the overlap halves: at most 2 r rows of up to 2 D (+ 2 Di) fp32 values per layer
        state = sum(2 * r * (2 * D + (2 * Di if r == 4 else 0)) * 4 for r in ratios if r)
        wb = weight_bytes if weight_bytes is not None else 0
        return ModelResourceProfile(int(wb), int(grow), L, 0, int(g.get("sliding_window") or 128), 0,
                                    state_bytes_per_sequence=int(state), windowed_bytes_per_token=int(win))
    if cfg.model_type == "inkling_mm_model":
        from ..models.inkling import InklingConfig

        ic = InklingConfig.from_dict(cfg.extra["inkling"])
        grow = win = state = 0
        for li in range(L):
            hq, hkv, D = ic.heads(ic.local_layers[li])
            per = 2 * hkv * D * b
            if ic.local_layers[li]:
                win += per
            else:
                grow += per
            state += (ic.sconv_kernel_size - 1) * (2 * hkv * D + 2 * H) * 4          # four convolution tails per layer
        wb = weight_bytes if weight_bytes is not None else 0
        return ModelResourceProfile(int(wb), int(grow), L, 0, int(ic.sliding_window_size), 0, state_bytes_per_sequence=int(state),
                                    windowed_bytes_per_token=int(win))
    return None


def kv_bytes_for(profile: ModelResourceProfile, context: int, batch: int) -> int:
    """KV pool bytes for ``batch`` sequences of ``context`` tokens (sliding layers hold at most their window)."""
    per_layer = profile.kv_bytes_per_token // max(1, profile.layers)
    full = profile.layers - profile.sliding_layers
    tokens_sliding = min(context, profile.sliding_window) if profile.sliding_window else context
    if profile.windowed_bytes_per_token:
        return batch * (profile.kv_bytes_per_token * context + profile.windowed_bytes_per_token * tokens_sliding
                        + profile.state_bytes_per_sequence)
    return batch * (per_layer * (full * context + profile.sliding_layers * tokens_sliding) + profile.state_bytes_per_sequence)


@dataclass
class AdmissionDecision:
    admitted: bool
    reason: str = ""
    max_context: int = 0


def apply_admission_policy(profile: ModelResourceProfile, device_free_bytes: int, context: int, batch: int = 1,
                           tensor_parallel: int = 1) -> AdmissionDecision:
    """Refuse a request whose KV cache cannot fit next to the weights (fail before any payload I/O)."""
    free = device_free_bytes - profile.weight_bytes // tensor_parallel - profile.workspace_bytes
    need = kv_bytes_for(profile, context, batch) // tensor_parallel
    per_tok = max(1, profile.kv_bytes_per_token // tensor_parallel) * batch
    if free <= 0:
        return AdmissionDecision(False, "weights and workspace alone exceed the device budget", 0)
    if need > free:
        return AdmissionDecision(False, f"KV cache needs {need} bytes, {free} available", int(free // per_tok))
    return AdmissionDecision(True, "", int(free // per_tok))


# ---------------------------------------------------------------------------------------------- execution plan
@dataclass
class ExecutionPlan:
    device: dict                                   # {"backend": "cuda-sm100a", "device": "gpu:0"}
    topology: dict                                 # {"data": 1, "pipeline": 1, "tensor": n, "expert": n, "expert_over_tensor": bool}
    residency: dict                                # {"mode": "fully_resident"} | {"mode": "layerwise_host", ...}
    weight_transformation: dict                    # {"mode": "preserve_checkpoint"} | {"mode": "affine", "bits", "group_size"}
    max_mapped_shards: int = DEFAULT_MAX_MAPPED_SHARDS
    expert_cache: Optional[dict] = None
    drafting: dict = field(default_factory=lambda: {"mode": "disabled"})
    kv_cache: dict = field(default_factory=lambda: {"mode": "device", "block_size_tokens": 16})
    required_capabilities: dict = field(default_factory=lambda: {"exact_completion": True, "collectives": False,
                                                                 "transfers": False, "persistent_cache": False})
    schema_version: int = EXECUTION_PLAN_SCHEMA_VERSION
    rationale: list = field(default_factory=list)

    def validate(self) -> None:
        if self.schema_version != EXECUTION_PLAN_SCHEMA_VERSION:
            raise ValueError(f"execution plan schema {self.schema_version} (supported: {EXECUTION_PLAN_SCHEMA_VERSION})")
        if self.max_mapped_shards <= 0:
            raise ValueError("max_mapped_shards must be positive")
        if not str(self.device.get("backend", "")).strip() or not str(self.device.get("device", "")).strip():
            raise ValueError("device plan needs a backend and a device")
        for axis in ("data", "pipeline", "tensor", "expert"):
            if int(self.topology.get(axis, 1)) < 1:
                raise ValueError(f"{axis} parallel size must be >= 1")
        d = self.drafting
        if d.get("mode") in ("embedded", "external") and int(d.get("max_draft_tokens", 0)) <= 0:
            raise ValueError("drafting needs max_draft_tokens > 0")
        if d.get("mode") == "external" and not str(d.get("model", "")).strip():
            raise ValueError("external drafting needs a model")
        if self.residency.get("mode") not in ("fully_resident", "layerwise_host", "dense_disk_stream"):
            raise ValueError(f"unknown residency mode {self.residency.get('mode')!r}")
        if self.weight_transformation.get("mode") not in ("preserve_checkpoint", "affine", "mxfp4"):
            raise ValueError("unknown weight transformation")

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=1)

    @classmethod
    def from_json(cls, text: str) -> "ExecutionPlan":
        plan = cls(**json.loads(text))
        plan.validate()
        return plan


@dataclass
class HardwareProfile:
    device_count: int = 1
    device_memory_bytes: int = 180 * 10**9
    device_free_bytes: Optional[int] = None
    host_memory_bytes: int = 0
    peer_access: bool = True          # every GPU reaches every peer (NVSwitch)
    name: str = "NVIDIA B200"

    @classmethod
    def discover(cls) -> "HardwareProfile":
        from .telemetry import hardware_profile

        hp = hardware_profile("cuda:0")
        dev = hp.get("device", {})
        return cls(int(dev.get("device_count", 1) or 1), int(dev.get("memory_bytes", 0) or 0) or 180 * 10**9,
                   int(dev.get("free_bytes", 0) or 0) or None, int(hp["host"].get("memory_bytes", 0)), True,
                   str(dev.get("name", "cpu")))


class AutomaticPlanner:
    """Chooses topology, weight transformation and residency for a model on this node."""

    def __init__(self, hardware: HardwareProfile, memory_fraction: float = 0.92):
        self.hw = hardware
        self.fraction = memory_fraction

    def plan(self, cfg: ModelConfig, profile: ModelResourceProfile, context: int = 4096, batch: int = 1,
             draft_model: Optional[str] = None, allow_quantization: bool = True, prefer_devices: Optional[int] = None) -> ExecutionPlan:
        budget = int((self.hw.device_free_bytes or self.hw.device_memory_bytes) * self.fraction)
        why: list[str] = []

        def fits(weight_bytes: int, tp: int) -> bool:
            need = weight_bytes // tp + kv_bytes_for(profile, context, batch) // tp + profile.workspace_bytes
            return need <= budget

        degrees = [d for d in (1, 2, 4, 8) if d <= self.hw.device_count and cfg.num_attention_heads % d == 0
                   and (cfg.num_key_value_heads % d == 0 or d % cfg.num_key_value_heads == 0)]
        if prefer_devices:
            degrees = [d for d in degrees if d >= prefer_devices] or degrees
        transformation = {"mode": "preserve_checkpoint"}
        residency = {"mode": "fully_resident"}
        weight_bytes = profile.weight_bytes
        tp = next((d for d in degrees if fits(weight_bytes, d)), None)
        if tp is None and allow_quantization and not cfg.quantization:
            q_bytes = int(profile.weight_bytes * (4.5 / 16.0))   # 4-bit codes + bf16 scale and bias per 64
            tp = next((d for d in degrees if fits(q_bytes, d)), None)
            if tp is not None:
                transformation = {"mode": "affine", "bits": 4, "group_size": 64}
                weight_bytes = q_bytes
                why.append("bf16 weights do not fit at any tensor-parallel degree: load-time 4-bit (group 64)")
        if tp is None:
            tp = degrees[-1]
            layer_bytes = weight_bytes // max(1, profile.layers) // tp
            kv = kv_bytes_for(profile, context, batch) // tp
            window = max(1, int((budget - kv - profile.workspace_bytes) // max(1, layer_bytes)))
            residency = {"mode": "layerwise_host", "device_layer_window": min(window, profile.layers),
                         "device_budget_bytes": budget, "host_budget_bytes": self.hw.host_memory_bytes or None}
            why.append(f"weights exceed device memory even at tp={tp}: layers stay in pinned host memory, "
                       f"{residency['device_layer_window']} at a time on the device")
        else:
            why.append(f"smallest tensor-parallel degree that fits weights + KV ({context} tokens x {batch}) + workspace: {tp}")
        topo = {"data": 1, "pipeline": 1, "tensor": tp, "expert": tp if cfg.is_moe else 1,
                "expert_over_tensor": bool(cfg.is_moe and tp > 1)}
        if cfg.is_moe and tp > 1:
            why.append("sparse model: experts are spread over the tensor ranks (replicated tokens, one combine + all-reduce)")
        drafting = {"mode": "disabled"}
        if cfg.mtp_layers > 0 and tp == 1 and residency["mode"] == "fully_resident":
            drafting = {"mode": "embedded", "max_draft_tokens": 3, "lookahead": True, "adaptive_lookahead": True}
            why.append("the checkpoint carries its own prediction layer: it drafts 3 tokens per round")
        if draft_model:
            drafting = {"mode": "external", "model": draft_model, "placement": {"mode": "target"}, "max_draft_tokens": 4,
                        "lookahead": False, "adaptive_lookahead": False}
        plan = ExecutionPlan(device={"backend": "cuda-sm100a", "device": "gpu:0" if tp == 1 else f"gpu:0-{tp - 1}"},
                             topology=topo, residency=residency, weight_transformation=transformation, drafting=drafting,
                             required_capabilities={"exact_completion": True, "collectives": tp > 1,
                                                    "transfers": residency["mode"] != "fully_resident",
                                                    "persistent_cache": False},
                             rationale=why)
        plan.validate()
        return plan


# ---------------------------------------------------------------------------------------------------------------
# Candidate enumeration and feedback (eredu-cli/src/main.rs:1259-1505 base / benchmark candidates;
# eredu-core/src/automatic.rs:1185-1250 selection from prior telemetry)

def _plan_key(plan: "ExecutionPlan | dict") -> str:
    d = asdict(plan) if isinstance(plan, ExecutionPlan) else dict(plan)
    d.pop("rationale", None)
    return json.dumps(d, sort_keys=True)


def candidate_plans(heuristic: ExecutionPlan, cfg: ModelConfig, profile: ModelResourceProfile, hw: HardwareProfile,
                    context: int = 4096, batch: int = 1, memory_fraction: float = 0.92) -> list[ExecutionPlan]:
    """Plans worth timing for this model on one device of this node: fully resident (when it fits), layer window from
    pinned host memory (when the weights fit in host memory), dense streaming from disk; each bounded form also with
    the expert cache for sparse models; the heuristic plan last. Duplicates are dropped, order is stable."""
    device_budget = int((hw.device_free_bytes or hw.device_memory_bytes) * memory_fraction)
    host_budget = int(hw.host_memory_bytes * 0.8) if hw.host_memory_bytes else 0
    tp = int(heuristic.topology.get("tensor", 1))
    need = profile.weight_bytes // tp + kv_bytes_for(profile, context, batch) // tp + profile.workspace_bytes
    resident_fits = need <= device_budget
    layerwise_fits = host_budget == 0 or profile.weight_bytes // tp <= host_budget
    base = dict(device=dict(heuristic.device), topology=dict(heuristic.topology),
                weight_transformation=dict(heuristic.weight_transformation), max_mapped_shards=heuristic.max_mapped_shards)
    out, seen = [], set()

    def push(plan: ExecutionPlan):
        plan.validate()
        k = _plan_key(plan)
        if k not in seen:
            seen.add(k)
            out.append(plan)

    forms = []
    if resident_fits:
        forms.append(({"mode": "fully_resident"}, False, "fully resident"))
    if layerwise_fits:
        forms.append(({"mode": "layerwise_host", "device_layer_window": 1, "device_budget_bytes": device_budget,
                       "host_budget_bytes": host_budget or None}, True, "one layer at a time from pinned host memory"))
    forms.append(({"mode": "dense_disk_stream", "device_budget_bytes": device_budget, "host_budget_bytes": host_budget or None,
                   "host_lookahead": 2 if host_budget else 0, "background_queue": 2 if host_budget else 0}, True,
                  "dense layers streamed from disk"))
    embedded = heuristic.drafting.get("mode") == "embedded" or (cfg.mtp_layers > 0 and tp == 1)
    for residency, bounded, why in forms:
        caps = {"exact_completion": True, "collectives": tp > 1, "transfers": bounded, "persistent_cache": False}
        variants = [(None, why)]
        if bounded and cfg.is_moe:
            variants.append(({"eviction": "lru", "device_budget_bytes": device_budget // 2}, why + " + expert cache"))
        for ec, label in variants:
            push(ExecutionPlan(residency=residency, required_capabilities=caps, expert_cache=ec,
                               rationale=[f"candidate: {label}"], **base))
            if embedded and not bounded:     # the prediction layer is bound next to fully resident weights only
                push(ExecutionPlan(residency=residency, required_capabilities=caps, expert_cache=ec,
                                   drafting={"mode": "embedded", "max_draft_tokens": 3, "lookahead": True,
                                             "adaptive_lookahead": True},
                                   rationale=[f"candidate: {label} + embedded drafting"], **base))
    h = ExecutionPlan.from_json(heuristic.to_json())
    if h.drafting.get("mode") == "external":
        h.drafting = {"mode": "disabled"}      # an external draft model is the user's choice, not a candidate axis
    push(h)
    return out


def _median(xs: list) -> float:
    xs = sorted(xs)
    m = len(xs) // 2
    return xs[m] if len(xs) % 2 else 0.5 * (xs[m - 1] + xs[m])


def select_from_feedback(telemetry: list, model_type: str, tensor_bytes: int, device: str,
                         minimum_tokens: int = 1) -> Optional[tuple]:
    """Best plan among earlier runs of this model on this device: telemetry records (dicts as written by
    ``--telemetry-json``) are grouped by their execution plan, each group scored by the median decode rate (total
    rate when a run had no decode phase). Returns ``(plan, samples, median_rate)`` or None when nothing matches."""
    groups: dict[str, tuple] = {}
    for t in telemetry:
        p = (t.get("plan") or {})
        ep = p.get("execution_plan")
        if not ep or t.get("generated_tokens", 0) < minimum_tokens:
            continue
        if p.get("device") != device or p.get("model_type") not in (None, model_type):
            continue
        if p.get("tensor_bytes") not in (None, tensor_bytes) or ep.get("schema_version") != EXECUTION_PLAN_SCHEMA_VERSION:
            continue
        timing = t.get("timing") or {}
        rate = timing.get("decode_token_rate") or 0.0
        if not (isinstance(rate, (int, float)) and rate > 0 and rate == rate and rate != float("inf")):
            rate = timing.get("token_rate") or 0.0
        if not (isinstance(rate, (int, float)) and rate > 0 and rate == rate and rate != float("inf")):
            continue
        k = _plan_key(ep)
        groups.setdefault(k, (ep, []))[1].append(float(rate))
    best = None
    for ep, rates in groups.values():
        try:
            plan = ExecutionPlan.from_json(json.dumps(ep))
        except (ValueError, TypeError):
            continue
        med = _median(rates)
        if best is None or med > best[2]:
            best = (plan, len(rates), med)
    return best
