"""Model configuration: normalisation of Hugging Face ``config.json`` and GGUF metadata.

Defaults and field fall-backs follow the reference's Llama/Qwen config readers
(eredu-architectures/src/llama/config.rs:82-101,206-312,402-454; eredu/src/backend/mlx/architectures/qwen/dense.rs:99-127).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import Any

DENSE_TYPES = {"llama", "mistral", "qwen2", "qwen3", "phi3", "lfm2"}
MOE_TYPES = {"qwen3_moe", "mixtral", "gpt_oss", "deepseek_v3", "lfm2_moe", "nemotron_h", "qwen3_next", "qwen3_5_moe", "qwen3_5_moe_text"}
QWEN_HYBRID_TYPES = {"qwen3_next", "qwen3_5", "qwen3_5_moe", "qwen3_5_text", "qwen3_5_moe_text"}


@dataclass
class ModelConfig:
    model_type: str = "llama"
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    head_dim: int = 128
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: dict | None = None
    rope_traditional: bool = False  # interleaved pairs (GGUF / llama.cpp convention)
    partial_rotary_factor: float = 1.0
    max_position_embeddings: int = 2048
    tie_word_embeddings: bool = True
    attention_bias: bool = False
    mlp_bias: bool = False
    sliding_window: int | None = None
    layer_types: list[str] | None = None  # per-layer "full_attention" | "sliding_attention" | "conv" (LFM2)
    # Qwen3-Next / 3.5 hybrids: "linear_attention" layers are gated delta networks
    linear_conv_kernel_dim: int = 4
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    # DeepSeek-V3 multi-head latent attention (kv_lora_rank > 0 turns it on)
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # Nemotron-H: every layer is ONE mixer ("mamba" | "attention_only" | "mlp_only" | "moe_only" in layer_types)
    mamba_num_heads: int = 0
    mamba_head_dim: int = 0
    ssm_state_size: int = 0
    mamba_n_groups: int = 1
    mamba_conv_kernel: int = 4
    mamba_conv_bias: bool = True
    mamba_proj_bias: bool = False
    time_step_min: float = 0.001
    use_rope: bool = True            # Nemotron-H attention carries no positional rotation
    attn_output_gate: bool = False   # q_proj also produces a per-channel sigmoid gate of the attention output
    shared_expert_gate: bool = False  # the shared expert's output is scaled by sigmoid(x . w)
    conv_l_cache: int = 3    # LFM2 short-convolution kernel width
    conv_bias: bool = False  # LFM2: biases on the convolution and its two projections
    qk_norm: bool = False  # per-head q/k RMSNorm (Qwen3)
    norm_weight_offset: float = 0.0  # Gemma stores (w - 1)
    embedding_scale: float = 1.0
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    router_scoring: str = "softmax"  # softmax | sigmoid | sqrt_softplus | topk_softmax
    routed_scaling_factor: float = 1.0  # multiplies the routing weights after renormalisation
    n_group: int = 1        # group-limited routing: experts in n_group groups, only the topk_group best stay eligible
    topk_group: int = 1
    shared_expert_intermediate_size: int = 0
    decoder_sparse_step: int = 1
    mlp_only_layers: list[int] = field(default_factory=list)
    swiglu_limit: float = 0.0
    attention_sinks: bool = False
    # quantisation recorded in the checkpoint
    quantization: dict | None = None
    eos_token_id: Any = None
    bos_token_id: Any = None
    torch_dtype: str = "bfloat16"
    extra: dict = field(default_factory=dict)

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    @property
    def kv_cache_dims(self) -> tuple:
        """(heads, key width, value width) of one cached token per layer: MLA caches one shared latent + rotary key."""
        if self.is_mla:
            return 1, self.kv_lora_rank + self.qk_rope_head_dim, 1
        if self.model_type == "gemma4":      # one pool wide enough for both layer types; layers use a slice of it
            g = self.extra["gemma4"]
            d = max(self.head_dim, int(g.get("global_head_dim") or 0))
            n = max(self.num_key_value_heads, int(g.get("num_global_key_value_heads") or 0))
            return n, d, d
        return self.num_key_value_heads, self.head_dim, self.head_dim

    @property
    def rotary_dim(self) -> int:
        if self.is_mla:
            return self.qk_rope_head_dim
        r = int(self.head_dim * self.partial_rotary_factor)
        return r - (r % 2)

    @property
    def mtp_layers(self) -> int:
        """Number of checkpoint-embedded next-token prediction layers (Qwen3-Next ``mtp.*``, DeepSeek-V3 layer L)."""
        return int(self.extra.get("mtp_num_hidden_layers") or self.extra.get("num_nextn_predict_layers") or 0)

    def layer_is_moe(self, layer: int) -> bool:
        if self.model_type == "nemotron_h":
            return self.layer_types[layer] == "moe_only"
        if not self.is_moe or layer in self.mlp_only_layers:
            return False
        return (layer + 1) % max(1, self.decoder_sparse_step) == 0

    def layer_is_conv(self, layer: int) -> bool:
        """LFM2 hybrid schedule: the layer's operator is the gated short convolution instead of attention."""
        return self.layer_types is not None and self.layer_types[layer] == "conv"

    def layer_is_kda(self, layer: int) -> bool:
        return self.layer_types is not None and self.layer_types[layer] == "kda"

    def layer_is_linear_attention(self, layer: int) -> bool:
        """Qwen3-Next style schedule: the layer's operator is a gated delta network instead of softmax attention."""
        return self.layer_types is not None and self.layer_types[layer] == "linear_attention"

    def layer_is_mamba(self, layer: int) -> bool:
        return self.layer_types is not None and self.layer_types[layer] == "mamba"

    def layer_has_kv(self, layer: int) -> bool:
        """The layer appends K/V pages (softmax attention); every other operator keeps a fixed state or none."""
        if self.layer_types is None:
            return True
        if self.model_type == "gemma4":      # the KV-sharing tail reads an earlier layer's pages
            shared = int(self.extra["gemma4"].get("num_kv_shared_layers") or 0)
            return layer < self.num_hidden_layers - shared or shared == 0
        return self.layer_types[layer] in ("full_attention", "sliding_attention", "attention_only")

    def layer_has_recurrent_state(self, layer: int) -> bool:
        return self.layer_types is not None and self.layer_types[layer] in ("linear_attention", "mamba", "kda")

    @property
    def is_hybrid(self) -> bool:
        return self.layer_types is not None and any(t in ("conv", "linear_attention", "mamba", "kda") for t in self.layer_types)

    def layer_window(self, layer: int) -> int:
        if self.sliding_window is None or self.sliding_window <= 0:
            return 0
        if self.layer_types is not None:
            return self.sliding_window if self.layer_types[layer] == "sliding_attention" else 0
        return self.sliding_window

    def to_hf_dict(self) -> dict:
        d = {k: v for k, v in asdict(self).items() if k not in ("extra", "qk_norm", "rope_traditional",
                                                                "norm_weight_offset", "embedding_scale",
                                                                "router_scoring", "attention_sinks", "quantization",
                                                                "routed_scaling_factor", "n_group", "topk_group")}
        if self.n_group > 1:
            d["n_group"], d["topk_group"] = self.n_group, self.topk_group
        d["architectures"] = [{"llama": "LlamaForCausalLM", "mistral": "MistralForCausalLM",
                               "qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM",
                               "qwen3_moe": "Qwen3MoeForCausalLM", "mixtral": "MixtralForCausalLM", "phi3": "Phi3ForCausalLM",
                               "gpt_oss": "GptOssForCausalLM", "lfm2": "Lfm2ForCausalLM",
                               "lfm2_moe": "Lfm2MoeForCausalLM", "qwen3_next": "Qwen3NextForCausalLM",
                               "qwen3_5_moe": "Qwen3_5MoeForCausalLM"}.get(self.model_type, "LlamaForCausalLM")]
        for k in ("mamba_n_groups", "mamba_conv_kernel", "mamba_conv_bias", "use_rope"):
            d.pop(k, None)
        if self.model_type == "kimi_linear":
            d["linear_attn_config"] = {
                "kda_layers": [i + 1 for i, t in enumerate(self.layer_types) if t == "kda"],
                "full_attn_layers": [i + 1 for i, t in enumerate(self.layer_types) if t != "kda"],
                "num_heads": self.linear_num_value_heads, "head_dim": self.linear_value_head_dim,
                "short_conv_kernel_size": self.linear_conv_kernel_dim}
            d.pop("layer_types", None)
            dense = [i for i in range(self.num_hidden_layers) if i in self.mlp_only_layers]
            first = next((i for i in range(self.num_hidden_layers) if i not in dense), self.num_hidden_layers)
            d.update(mla_use_nope=True, num_experts_per_token=self.num_experts_per_tok, moe_renormalize=self.norm_topk_prob,
                     num_shared_experts=(self.shared_expert_intermediate_size // max(1, self.moe_intermediate_size)),
                     moe_router_activation_func=self.router_scoring, num_expert_group=self.n_group, topk_group=self.topk_group,
                     use_grouped_topk=self.n_group > 1, first_k_dense_replace=first, moe_layer_freq=1)
            d.pop("head_dim", None)
            d.pop("mlp_only_layers", None)
        if self.model_type == "deepseek_v3":
            d.update(n_routed_experts=self.num_experts, first_k_dense_replace=len(self.mlp_only_layers),
                     n_shared_experts=(self.shared_expert_intermediate_size // max(1, self.moe_intermediate_size)),
                     scoring_func=self.router_scoring, rope_interleave=self.rope_traditional, architectures=["DeepseekV3ForCausalLM"])
            d.pop("head_dim", None)
        elif self.model_type != "kimi_linear":
            for k in ("q_lora_rank", "kv_lora_rank", "qk_nope_head_dim", "qk_rope_head_dim", "v_head_dim"):
                d.pop(k, None)
        if self.model_type == "nemotron_h":
            inv = {"mamba": "M", "attention_only": "*", "mlp_only": "-", "moe_only": "E"}
            d["hybrid_override_pattern"] = "".join(inv[t] for t in self.layer_types)
            d.pop("layer_types", None)
            d.update(n_groups=self.mamba_n_groups, conv_kernel=self.mamba_conv_kernel, use_conv_bias=self.mamba_conv_bias,
                     layer_norm_epsilon=self.rms_norm_eps, n_routed_experts=self.num_experts,
                     moe_shared_expert_intermediate_size=self.shared_expert_intermediate_size, n_shared_experts=1,
                     num_experts_per_tok=self.num_experts_per_tok, moe_intermediate_size=self.moe_intermediate_size,
                     norm_topk_prob=self.norm_topk_prob)
        else:
            for k in ("mamba_num_heads", "mamba_head_dim", "ssm_state_size", "mamba_proj_bias", "time_step_min"):
                d.pop(k, None)
        if self.model_type not in QWEN_HYBRID_TYPES and self.model_type != "kimi_linear":
            for k in ("linear_conv_kernel_dim", "linear_key_head_dim", "linear_value_head_dim", "linear_num_key_heads",
                      "linear_num_value_heads"):
                d.pop(k, None)
        d.pop("shared_expert_gate", None)
        if not self.attn_output_gate:
            d.pop("attn_output_gate", None)
        if self.routed_scaling_factor != 1.0 or self.model_type == "lfm2_moe":
            d["routed_scaling_factor"] = self.routed_scaling_factor
        if self.model_type == "lfm2_moe":
            d["num_dense_layers"] = len(self.mlp_only_layers)
        if self.model_type in ("lfm2", "lfm2_moe"):
            d["norm_eps"] = self.rms_norm_eps
            d["conv_L_cache"] = d.pop("conv_l_cache")
            d["block_auto_adjust_ff_dim"] = False
        else:
            d.pop("conv_l_cache", None)
            d.pop("conv_bias", None)
        if not self.is_moe:
            for k in ("num_experts", "num_experts_per_tok", "moe_intermediate_size", "norm_topk_prob",
                      "shared_expert_intermediate_size", "decoder_sparse_step", "mlp_only_layers", "swiglu_limit"):
                d.pop(k, None)
        if self.quantization is not None:
            d["quantization"] = dict(self.quantization)
            d["quantization_config"] = dict(self.quantization)
        d.update(self.extra)
        return d

    # -------------------------------------------------------------------------------------- HF
    @classmethod
    def from_hf_dict(cls, d: dict) -> "ModelConfig":
        mt = d.get("model_type", "llama")
        if "text_config" in d and isinstance(d["text_config"], dict):
            outer = d
            inner = dict(d["text_config"])
            inner.setdefault("model_type", mt)
            for k in ("quantization", "quantization_config", "eos_token_id", "tie_word_embeddings"):
                if k in d and k not in inner:
                    inner[k] = d[k]
            d = inner
            mt = d.get("model_type", mt)
            # the language model of a vision-language checkpoint is its text family (text-only use of Qwen3-VL)
            mt = {"qwen3_vl_text": "qwen3", "qwen3_vl_moe_text": "qwen3_moe", "qwen3_vl": "qwen3", "qwen3_vl_moe": "qwen3_moe",
                  "gemma4_text": "gemma4", "muse_glimmer_text": "muse_glimmer"}.get(mt, mt)
            d["model_type"] = mt
            d["_language_model_prefix"] = True
            d["_vision"] = {k: outer[k] for k in ("vision_config", "image_token_id", "video_token_id", "boi_token_id", "eoi_token_id", "vision_start_token_id",
                                                  "vision_end_token_id", "audio_config", "audio_token_id", "boa_token_id", "eoa_token_id",
                                                  "eoa_token_index", "projector_hidden_size", "out_hidden_size") if k in outer}
        # Transformers >= 5 writes RoPE settings as one ``rope_parameters`` object (theta inside it; optionally one
        # object per layer type): fold it back into rope_theta / rope_scaling
        rp = d.get("rope_parameters")
        if isinstance(rp, dict) and rp:
            if "rope_type" not in rp and "rope_theta" not in rp and isinstance(next(iter(rp.values())), dict):
                rp = rp.get("full_attention") or next(iter(rp.values()))
            d = dict(d)
            if rp.get("rope_theta") is not None and d.get("rope_theta") is None:
                d["rope_theta"] = rp["rope_theta"]
            if d.get("rope_scaling") is None and (rp.get("rope_type", "default") not in ("default", None)
                                                  or "mrope_section" in rp):
                d["rope_scaling"] = {k: v for k, v in rp.items() if k != "rope_theta"}
            if rp.get("partial_rotary_factor") is not None and d.get("partial_rotary_factor") is None:
                d["partial_rotary_factor"] = rp["partial_rotary_factor"]
        if mt == "gemma4_text":
            mt = "gemma4"
            d = dict(d, model_type=mt)
        raw_rope_parameters = d.get("rope_parameters")
        heads = int(d.get("num_attention_heads", 32))
        hidden = int(d.get("hidden_size", 4096))
        kv = int(d.get("num_key_value_heads") or 0) or heads
        head_dim = int(d.get("head_dim") or 0) or hidden // heads
        cfg = cls(
            model_type=mt,
            vocab_size=int(d.get("vocab_size", 32000)),
            hidden_size=hidden,
            intermediate_size=int(d.get("intermediate_size", 4 * hidden)),
            num_hidden_layers=int(d.get("num_hidden_layers", 32)),
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-5 if mt in ("llama", "mistral") else 1e-6)),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=d.get("rope_scaling"),
            partial_rotary_factor=float(d.get("partial_rotary_factor", 1.0)),
            max_position_embeddings=int(d.get("max_position_embeddings", 2048)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", True)),
            attention_bias=bool(d.get("attention_bias", mt == "qwen2")),
            mlp_bias=bool(d.get("mlp_bias", False)),
            sliding_window=d.get("sliding_window") if d.get("use_sliding_window", mt == "mistral") or mt == "mistral"
            else None,
            layer_types=d.get("layer_types"),
            qk_norm=mt in ("qwen3", "qwen3_moe"),
            num_experts=int(d.get("num_experts", d.get("num_local_experts", 0)) or 0),
            num_experts_per_tok=int(d.get("num_experts_per_tok", 0) or 0),
            moe_intermediate_size=int(d.get("moe_intermediate_size", 0) or 0),
            norm_topk_prob=bool(d.get("norm_topk_prob", mt == "mixtral")),
            shared_expert_intermediate_size=int(d.get("shared_expert_intermediate_size", 0) or 0),
            decoder_sparse_step=int(d.get("decoder_sparse_step", 1) or 1),
            mlp_only_layers=list(d.get("mlp_only_layers", []) or []),
            swiglu_limit=float(d.get("swiglu_limit", 0.0) or 0.0),
            routed_scaling_factor=float(d.get("routed_scaling_factor", 1.0) or 1.0),
            n_group=int(d.get("n_group", 1) or 1),
            topk_group=int(d.get("topk_group", 1) or 1),
            quantization=d.get("quantization") or d.get("quantization_config"),
            eos_token_id=d.get("eos_token_id"),
            bos_token_id=d.get("bos_token_id"),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
        )
        if mt == "muse_glimmer":
            # eredu/src/backend/mlx/architectures/muse_glimmer/mod.rs:197-243: the family's own fields travel as a dict
            keys = ("post_norm_eps", "layer_types", "layer_rope_theta", "qk_scale_factor", "output_multiplier",
                    "final_logit_softcapping", "num_experts", "moe_intermediate_size", "num_experts_per_tok", "norm_topk_prob")
            for k in ("post_norm_eps", "layer_types", "layer_rope_theta", "qk_scale_factor", "output_multiplier", "final_logit_softcapping"):
                if d.get(k) is None:
                    raise ValueError(f"Muse-Glimmer text_config lacks {k}")
            if float(d["final_logit_softcapping"]) <= 0:
                raise ValueError("Muse-Glimmer final_logit_softcapping must be positive")
            cfg.extra["muse_glimmer"] = {k: d.get(k) for k in keys}
            cfg.sliding_window = d.get("sliding_window")
            cfg.layer_types = list(d["layer_types"])
            cfg.num_experts = 0
        if mt == "inkling_mm_model":
            # the family's own decoder reads the text fields from the raw dictionary (models/inkling.py)
            cfg.extra["inkling"] = {k: v for k, v in d.items() if not k.startswith("_")}
            cfg.num_experts = int(d.get("n_routed_experts") or 0)
        if mt == "deepseek_v4":
            # the family's own decoder reads its fields from the raw dictionary (models/deepseek_v4.py)
            cfg.extra["deepseek_v4"] = {k: v for k, v in d.items() if not k.startswith("_")}
            cfg.num_experts = int(d.get("n_routed_experts") or 0)
            cfg.num_key_value_heads = 1
        if mt == "gemma4":
            # eredu/src/backend/mlx/architectures/gemma4/model.rs:374-430: the family's own fields travel as a dict;
            # the generic fields describe the sliding layers
            keys = ("global_head_dim", "num_global_key_value_heads", "attention_k_eq_v", "num_kv_shared_layers",
                    "use_double_wide_mlp", "hidden_size_per_layer_input", "vocab_size_per_layer_input", "enable_moe_block",
                    "top_k_experts", "hidden_activation", "final_logit_softcapping", "use_bidirectional_attention",
                    "pad_token_id")
            cfg.extra["gemma4"] = {k: d.get(k) for k in keys}
            cfg.extra["gemma4"]["rope_parameters"] = raw_rope_parameters
            cfg.embedding_scale = float(cfg.hidden_size) ** 0.5
            cfg.sliding_window = d.get("sliding_window")
            cfg.rms_norm_eps = float(d.get("rms_norm_eps", 1e-6))
            cfg.tie_word_embeddings = bool(d.get("tie_word_embeddings", True))
            cfg.num_experts = int(d.get("num_experts") or 0) if d.get("enable_moe_block") else 0
            cfg.num_experts_per_tok = int(d.get("top_k_experts") or 0)
            cfg.rope_scaling = None
            if cfg.layer_types is None or len(cfg.layer_types) != cfg.num_hidden_layers:
                raise ValueError("Gemma 4 config needs one layer_types entry per layer")
            if (d.get("hidden_activation") or "gelu_pytorch_tanh") != "gelu_pytorch_tanh":
                raise ValueError("Gemma 4: only the gelu_pytorch_tanh activation is supported")
        if mt == "kimi_linear":
            # eredu/src/backend/mlx/architectures/kimi_linear/model.rs:160-235 (source keys), :330-450 (schedule)
            la = d.get("linear_attn_config") or {}
            kda = {int(i) - 1 for i in la.get("kda_layers", [])}                       # the lists are 1-based
            full = {int(i) - 1 for i in la.get("full_attn_layers", [])}
            L = cfg.num_hidden_layers
            if (kda | full) != set(range(L)) or (kda & full):
                raise ValueError("Kimi Linear kda_layers and full_attn_layers must partition the layers")
            cfg.layer_types = ["kda" if i in kda else "full_attention" for i in range(L)]
            cfg.linear_num_value_heads = cfg.linear_num_key_heads = int(la.get("num_heads", cfg.num_attention_heads))
            cfg.linear_value_head_dim = cfg.linear_key_head_dim = int(la.get("head_dim", cfg.head_dim))
            cfg.linear_conv_kernel_dim = int(la.get("short_conv_kernel_size", 4))
            if not bool(d.get("mla_use_nope", False)):
                raise ValueError("Kimi Linear currently requires mla_use_nope=true")
            cfg.use_rope = False
            cfg.q_lora_rank = int(d.get("q_lora_rank") or 0)
            cfg.kv_lora_rank = int(d.get("kv_lora_rank", 512))
            cfg.qk_nope_head_dim = int(d.get("qk_nope_head_dim", 128))
            cfg.qk_rope_head_dim = int(d.get("qk_rope_head_dim", 64))
            cfg.v_head_dim = int(d.get("v_head_dim", 128))
            cfg.head_dim = cfg.qk_nope_head_dim + cfg.qk_rope_head_dim
            cfg.num_key_value_heads = cfg.num_attention_heads
            cfg.num_experts_per_tok = int(d.get("num_experts_per_token", d.get("num_experts_per_tok", 0)) or 0)
            shared = int(d.get("num_shared_experts", d.get("n_shared_experts", 1)) or 0)
            cfg.shared_expert_intermediate_size = cfg.moe_intermediate_size * shared if cfg.num_experts else 0
            cfg.router_scoring = {"sigmoid": "sigmoid", "softmax": "softmax"}[d.get("moe_router_activation_func", "sigmoid")]
            cfg.norm_topk_prob = bool(d.get("moe_renormalize", True))
            if bool(d.get("use_grouped_topk", True)):
                cfg.n_group = int(d.get("num_expert_group", d.get("n_group", 1)) or 1)
                cfg.topk_group = int(d.get("topk_group", 1) or 1)
            first, freq = int(d.get("first_k_dense_replace", 0) or 0), int(d.get("moe_layer_freq", 1) or 1)
            cfg.mlp_only_layers = [i for i in range(L) if not (cfg.num_experts and i >= first and i % freq == 0)]
            cfg.decoder_sparse_step = 1
            cfg.tie_word_embeddings = bool(d.get("tie_word_embeddings", False))
        if mt == "deepseek_v3":
            # eredu/src/backend/mlx/architectures/deepseek_v3/model.rs:339-403: latent attention, dense-then-sparse
            # schedule, sigmoid router with correction bias and group-limited top-k, shared experts
            cfg.q_lora_rank = int(d.get("q_lora_rank") or 0)
            cfg.kv_lora_rank = int(d.get("kv_lora_rank", 512))
            cfg.qk_nope_head_dim = int(d.get("qk_nope_head_dim", 128))
            cfg.qk_rope_head_dim = int(d.get("qk_rope_head_dim", 64))
            cfg.v_head_dim = int(d.get("v_head_dim", 128))
            cfg.head_dim = cfg.qk_nope_head_dim + cfg.qk_rope_head_dim
            cfg.num_key_value_heads = cfg.num_attention_heads
            cfg.rope_traditional = bool(d.get("rope_interleave", False))
            cfg.num_experts = int(d.get("n_routed_experts", 0) or 0)
            cfg.mlp_only_layers = list(range(int(d.get("first_k_dense_replace", 0) or 0)))
            cfg.decoder_sparse_step = int(d.get("moe_layer_freq", 1) or 1)
            cfg.shared_expert_intermediate_size = cfg.moe_intermediate_size * int(d.get("n_shared_experts", 0) or 0)
            cfg.router_scoring = {"sigmoid": "sigmoid", "softmax": "softmax"}[d.get("scoring_func", "sigmoid")]
            cfg.norm_topk_prob = bool(d.get("norm_topk_prob", True))
            cfg.tie_word_embeddings = bool(d.get("tie_word_embeddings", False))
        if mt == "nemotron_h":
            # eredu/src/backend/mlx/architectures/nemotron_h/model.rs:74-90 (pattern markers), :100-245 (fields)
            marks = {"M": "mamba", "*": "attention_only", "-": "mlp_only", "E": "moe_only"}
            pattern = str(d.get("hybrid_override_pattern", "") or "")
            blocks = d.get("layers_block_type")
            if blocks:      # newer exports spell the schedule out as a list
                names = {"mamba": "mamba", "attention": "attention_only", "mlp": "mlp_only", "moe": "moe_only"}
                if any(b not in names for b in blocks):
                    raise ValueError(f"Nemotron-H layers_block_type has unknown entries: {sorted(set(blocks) - set(names))}")
                cfg.layer_types = [names[b] for b in blocks]
            elif pattern and all(ch in marks for ch in pattern):
                cfg.layer_types = [marks[ch] for ch in pattern]
            else:
                raise ValueError("Nemotron-H needs layers_block_type or a hybrid_override_pattern made of 'M', '*', '-' and 'E'")
            cfg.num_hidden_layers = len(cfg.layer_types)
            cfg.mamba_num_heads = int(d.get("mamba_num_heads", 128))
            cfg.mamba_head_dim = int(d.get("mamba_head_dim", 64))
            cfg.ssm_state_size = int(d.get("ssm_state_size", 128))
            cfg.mamba_n_groups = int(d.get("n_groups", 8))
            cfg.mamba_conv_kernel = int(d.get("conv_kernel", 4))
            cfg.mamba_conv_bias = bool(d.get("use_conv_bias", True))
            cfg.mamba_proj_bias = bool(d.get("mamba_proj_bias", d.get("use_bias", False)))
            cfg.time_step_min = float(d.get("time_step_min", 0.001))
            cfg.rms_norm_eps = float(d.get("layer_norm_epsilon", d.get("rms_norm_eps", 1e-5)))
            cfg.head_dim = int(d.get("head_dim") or d.get("attention_head_dim") or cfg.head_dim)
            cfg.use_rope = False
            cfg.tie_word_embeddings = bool(d.get("tie_word_embeddings", False))
            cfg.num_experts = int(d.get("n_routed_experts", 0) or 0)
            cfg.num_experts_per_tok = int(d.get("num_experts_per_tok", 0) or 0)
            cfg.moe_intermediate_size = int(d.get("moe_intermediate_size", 0) or 0)
            cfg.shared_expert_intermediate_size = (int(d.get("moe_shared_expert_intermediate_size", 0) or 0)
                                                   * max(1, int(d.get("n_shared_experts", 1) or 1))
                                                   if cfg.num_experts else 0)
            cfg.router_scoring = "sigmoid"
            cfg.norm_topk_prob = bool(d.get("norm_topk_prob", True))
        if mt in QWEN_HYBRID_TYPES:
            # eredu/src/backend/mlx/architectures/qwen/hybrid/qwen3_5.rs:254-323: three gated-delta layers per full
            # attention layer, zero-centred RMSNorm weights, gated attention output, 25 % rotary, gated shared expert
            cfg.qk_norm = True
            cfg.norm_weight_offset = 1.0
            cfg.attn_output_gate = bool(d.get("attn_output_gate", True))
            rp = d.get("rope_parameters") or {}
            cfg.partial_rotary_factor = float(rp.get("partial_rotary_factor", d.get("partial_rotary_factor", 0.25)))
            cfg.rope_theta = float(rp.get("rope_theta", d.get("rope_theta", 10000000.0)))
            for key in ("linear_conv_kernel_dim", "linear_key_head_dim", "linear_value_head_dim", "linear_num_key_heads",
                        "linear_num_value_heads"):
                if key in d:
                    setattr(cfg, key, int(d[key]))
            if cfg.layer_types is None:
                every = int(d.get("full_attention_interval", 4))
                cfg.layer_types = ["full_attention" if (i + 1) % every == 0 else "linear_attention"
                                   for i in range(cfg.num_hidden_layers)]
            if len(cfg.layer_types) != cfg.num_hidden_layers:
                raise ValueError("hybrid Qwen config needs one layer_types entry per layer")
            cfg.norm_topk_prob = bool(d.get("norm_topk_prob", True))
            cfg.shared_expert_gate = cfg.shared_expert_intermediate_size > 0
            cfg.tie_word_embeddings = bool(d.get("tie_word_embeddings", False))
        if mt in ("lfm2", "lfm2_moe"):
            # eredu/src/backend/mlx/architectures/lfm2/model.rs:193-418: hybrid schedule of gated short convolutions
            # and q/k-normalised GQA attention; dense FFN width optionally re-derived from block_ff_dim
            cfg.rms_norm_eps = float(d.get("norm_eps", 1e-5))
            rp = d.get("rope_parameters") or {}
            cfg.rope_theta = float(rp.get("rope_theta", d.get("rope_theta") or 1_000_000.0))
            cfg.tie_word_embeddings = bool(d.get("tie_word_embeddings", d.get("tie_embedding", True)))
            cfg.qk_norm = True
            cfg.conv_l_cache = int(d.get("conv_L_cache", 3))
            cfg.conv_bias = bool(d.get("conv_bias", False))
            if cfg.layer_types is None and d.get("full_attn_idxs") is not None:
                full = set(d["full_attn_idxs"])
                cfg.layer_types = ["full_attention" if i in full else "conv" for i in range(cfg.num_hidden_layers)]
            if cfg.layer_types is None or len(cfg.layer_types) != cfg.num_hidden_layers:
                raise ValueError("LFM2 config needs one layer_types entry per layer")
            if mt == "lfm2_moe":
                # model.rs:264-290,1010-1046: the first num_dense_layers layers keep the dense FFN, the others route
                # with a sigmoid router (optional selection bias), optional renormalisation and a routing scale
                cfg.router_scoring = "sigmoid"
                cfg.norm_topk_prob = bool(d.get("norm_topk_prob", False))
                cfg.routed_scaling_factor = float(d.get("routed_scaling_factor", 1.0))
                cfg.mlp_only_layers = list(range(int(d.get("num_dense_layers", 0) or 0)))
                cfg.extra["use_expert_bias"] = bool(d.get("use_expert_bias", False))
            if mt == "lfm2":
                size = int(d.get("block_ff_dim") or cfg.intermediate_size)
                if bool(d.get("block_auto_adjust_ff_dim", True)):
                    mult, of = float(d.get("block_ffn_dim_multiplier", 1.0)), int(d.get("block_multiple_of", 256))
                    size = int(mult * (2 * size // 3))
                    size = of * ((size + of - 1) // of)
                cfg.intermediate_size = size
        for key in ("mtp_num_hidden_layers", "num_nextn_predict_layers"):
            if int(d.get(key, 0) or 0) > 0:
                cfg.extra[key] = int(d[key])     # checkpoint-embedded prediction layers (drafting only; the decoder ignores them)
        if d.get("mtp_hybrid_override_pattern"):
            cfg.extra["mtp_hybrid_override_pattern"] = str(d["mtp_hybrid_override_pattern"])   # Nemotron-H: blocks of one prediction step
        if d.get("_language_model_prefix"):
            cfg.extra["language_model_prefix"] = True   # tensors live under model.language_model.* next to a vision tower
            if d.get("_vision", {}).get("vision_config") or d.get("_vision", {}).get("audio_config"):
                cfg.extra["vision"] = d["_vision"]           # towers next to the decoder: vision and / or audio
        if mt == "mixtral":
            cfg.moe_intermediate_size = cfg.moe_intermediate_size or cfg.intermediate_size
            cfg.router_scoring = "topk_softmax"
        if mt == "gpt_oss":
            # eredu/src/backend/mlx/architectures/gpt_oss/model.rs:64-170: every layer is sparse, top-k then softmax
            # over the selected logits, attention sinks and biases, alternating sliding / full layers, clamp 7.0
            cfg.num_experts = int(d.get("num_local_experts", cfg.num_experts) or cfg.num_experts)
            cfg.num_experts_per_tok = int(d.get("num_experts_per_tok", d.get("experts_per_token", 4)) or 4)
            cfg.moe_intermediate_size = cfg.moe_intermediate_size or cfg.intermediate_size
            cfg.router_scoring = "topk_softmax"
            cfg.norm_topk_prob = False
            cfg.attention_bias = bool(d.get("attention_bias", True))
            cfg.attention_sinks = True
            cfg.swiglu_limit = float(d.get("swiglu_limit", 7.0) or 7.0)
            cfg.sliding_window = d.get("sliding_window", cfg.sliding_window)
            cfg.tie_word_embeddings = bool(d.get("tie_word_embeddings", False))
        return cfg

    @classmethod
    def from_pretrained(cls, path: str | Path) -> "ModelConfig":
        with open(Path(path) / "config.json") as f:
            return cls.from_hf_dict(json.load(f))

    # -------------------------------------------------------------------------------------- GGUF
    @classmethod
    def from_gguf_metadata(cls, md: dict, has_output_weight: bool) -> "ModelConfig":
        arch = md.get("general.architecture", "llama")

        def g(key, default=None):
            return md.get(f"{arch}.{key}", default)

        hidden = int(g("embedding_length"))
        heads = int(g("attention.head_count"))
        kv = g("attention.head_count_kv", heads)
        if isinstance(kv, (list, tuple)):
            kv = kv[0]
        kv = int(kv) or heads
        head_dim = int(g("attention.key_length", hidden // heads))
        vocab = g("vocab_size")
        if vocab is None:
            vocab = len(md.get("tokenizer.ggml.tokens", [])) or 32000
        scaling = None
        st = g("rope.scaling.type")
        if st and st != "none":
            scaling = {"rope_type": st, "factor": float(g("rope.scaling.factor", 1.0)),
                       "original_max_position_embeddings": int(g("rope.scaling.original_context_length", 0) or 0)}
        model_type = {"llama": "llama", "qwen2": "qwen2", "qwen3": "qwen3", "qwen3moe": "qwen3_moe",
                      "mistral": "mistral"}.get(arch, arch)
        return cls(
            model_type=model_type,
            vocab_size=int(vocab),
            hidden_size=hidden,
            intermediate_size=int(g("feed_forward_length", 4 * hidden)),
            num_hidden_layers=int(g("block_count")),
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            rms_norm_eps=float(g("attention.layer_norm_rms_epsilon", 1e-5)),
            rope_theta=float(g("rope.freq_base", 10000.0)),
            rope_scaling=scaling,
            rope_traditional=model_type in ("llama", "mistral"),
            max_position_embeddings=int(g("context_length", 2048)),
            tie_word_embeddings=not has_output_weight,
            sliding_window=g("attention.sliding_window"),
            qk_norm=model_type in ("qwen3", "qwen3_moe"),
            attention_bias=model_type == "qwen2",
            num_experts=int(g("expert_count", 0) or 0),
            num_experts_per_tok=int(g("expert_used_count", 0) or 0),
            moe_intermediate_size=int(g("expert_feed_forward_length", 0) or 0),
            eos_token_id=md.get("tokenizer.ggml.eos_token_id"),
            bos_token_id=md.get("tokenizer.ggml.bos_token_id"),
        )


# Shapes named by the benchmark configurations.
def llama3_8b() -> ModelConfig:
    return ModelConfig(model_type="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                       num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                       rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192,
                       tie_word_embeddings=False)


def llama3_70b() -> ModelConfig:
    return ModelConfig(model_type="llama", vocab_size=128256, hidden_size=8192, intermediate_size=28672,
                       num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                       rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192,
                       tie_word_embeddings=False)


def qwen3_30b_a3b() -> ModelConfig:
    return ModelConfig(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                       num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                       rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=40960,
                       tie_word_embeddings=False, qk_norm=True, num_experts=128, num_experts_per_tok=8,
                       moe_intermediate_size=768, norm_topk_prob=True)


def tiny_llama() -> ModelConfig:
    return ModelConfig(model_type="llama", vocab_size=32000, hidden_size=256, intermediate_size=688,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                       rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=2048,
                       tie_word_embeddings=True, torch_dtype="float32")


def draft_llama_16l() -> ModelConfig:
    return ModelConfig(model_type="llama", vocab_size=128256, hidden_size=2048, intermediate_size=8192,
                       num_hidden_layers=16, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
                       rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192,
                       tie_word_embeddings=False)
