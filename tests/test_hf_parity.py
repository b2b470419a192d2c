"""Checkpoint parity against Hugging Face Transformers on CPU: a tiny randomly initialised model of each family is
written with ``save_pretrained`` and loaded here from that directory; last-position logits must agree. This checks the
reading of a real ``config.json``, the checkpoint tensor names and the block semantics against an implementation that
shares no code with this repository."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from eredu_b200.api import LoadedModel, ModelLoadOptions


def hf_model(cls_name, cfg_name, **kw):
    cfg_cls = getattr(transformers, cfg_name)
    cfg = cfg_cls(**kw)
    torch.manual_seed(0)
    model = getattr(transformers, cls_name)(cfg).eval().float()
    # random initialisers leave norms at one and some biases at zero: perturb everything so that no term is silent
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn(p.shape, generator=g) * 0.1)
    return model


def check(model, tmp_path, prompt_len=19, atol=2e-3, max_seq_len=64):
    model.save_pretrained(tmp_path, safe_serialization=True)
    vocab = getattr(model.config, "vocab_size", None) or model.config.text_config.vocab_size
    prompt = torch.randint(0, vocab, (prompt_len,), generator=torch.Generator().manual_seed(2)).tolist()
    with torch.no_grad():
        ref = model(torch.tensor([prompt])).logits[0, -1].float()
    from eredu_b200.runtime.plan import inspect_artifact

    report = inspect_artifact(tmp_path)            # header-only inspection agrees that this directory can be loaded
    assert report.is_loadable, [(i.code, i.message) for i in report.issues]
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=max_seq_len))
    got = lm.prefill_logits(prompt)
    err = float((got - ref).abs().max())
    assert err < atol * max(1.0, float(ref.abs().max())), err
    # a second, chunked pass through the engine (prefill in pieces + decode-shaped steps) agrees with the full pass
    seq = lm.engine.new_sequence(prompt[:-4], max_new_tokens=8)
    lm.engine.prefill_logits([seq])
    logits = None
    for t in prompt[-4:]:
        logits = lm.engine.step_logits(seq, t)
    lm.engine.release(seq)
    assert float((logits.float().cpu() - ref).abs().max()) < atol * max(1.0, float(ref.abs().max()))
    return lm


BASE = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, max_position_embeddings=128)


def test_llama(tmp_path):
    check(hf_model("LlamaForCausalLM", "LlamaConfig", **BASE, rope_theta=50000.0, tie_word_embeddings=False), tmp_path)


def test_llama3_rope_scaling(tmp_path):
    check(hf_model("LlamaForCausalLM", "LlamaConfig", **BASE, rope_scaling={
        "rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
        "original_max_position_embeddings": 32}), tmp_path, prompt_len=50)


def test_mistral_sliding_window(tmp_path):
    check(hf_model("MistralForCausalLM", "MistralConfig", **BASE, sliding_window=8), tmp_path, prompt_len=30)


def test_qwen2_bias(tmp_path):
    check(hf_model("Qwen2ForCausalLM", "Qwen2Config", **BASE), tmp_path)


def test_qwen3_qk_norm(tmp_path):
    check(hf_model("Qwen3ForCausalLM", "Qwen3Config", **BASE, head_dim=32), tmp_path)


def test_phi3_fused_projections(tmp_path):
    check(hf_model("Phi3ForCausalLM", "Phi3Config", **BASE, pad_token_id=0), tmp_path)


def test_qwen3_moe(tmp_path):
    check(hf_model("Qwen3MoeForCausalLM", "Qwen3MoeConfig", **BASE, head_dim=32, num_experts=8, num_experts_per_tok=2,
                   moe_intermediate_size=48, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[]), tmp_path)


def test_mixtral(tmp_path):
    check(hf_model("MixtralForCausalLM", "MixtralConfig", **BASE, num_local_experts=4, num_experts_per_tok=2), tmp_path)


def test_gpt_oss(tmp_path):
    m = hf_model("GptOssForCausalLM", "GptOssConfig", vocab_size=320, hidden_size=64, intermediate_size=64, num_hidden_layers=2,
                 num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_local_experts=4, num_experts_per_tok=2,
                 sliding_window=8, max_position_embeddings=128, layer_types=["sliding_attention", "full_attention"],
                 rope_scaling=None, rope_parameters={"rope_type": "default", "rope_theta": 10000.0})
    check(m, tmp_path, prompt_len=30)


def test_lfm2(tmp_path):
    m = hf_model("Lfm2ForCausalLM", "Lfm2Config", vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=4,
                 num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128, conv_L_cache=3, conv_bias=False,
                 layer_types=["conv", "conv", "full_attention", "conv"], block_auto_adjust_ff_dim=True, block_multiple_of=32,
                 block_ffn_dim_multiplier=1.0, pad_token_id=0)
    check(m, tmp_path)


def test_deepseek_v3(tmp_path):
    m = hf_model("DeepseekV3ForCausalLM", "DeepseekV3Config", vocab_size=320, hidden_size=64, intermediate_size=96,
                 moe_intermediate_size=32, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4, n_shared_experts=1,
                 n_routed_experts=8, routed_scaling_factor=2.5, kv_lora_rank=16, q_lora_rank=24, qk_rope_head_dim=8,
                 v_head_dim=16, qk_nope_head_dim=16, n_group=2, topk_group=1, num_experts_per_tok=2, first_k_dense_replace=1,
                 norm_topk_prob=True, max_position_embeddings=128)
    check(m, tmp_path)


def test_lfm2_moe(tmp_path):
    m = hf_model("Lfm2MoeForCausalLM", "Lfm2MoeConfig", vocab_size=320, hidden_size=64, intermediate_size=128,
                 moe_intermediate_size=32, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                 max_position_embeddings=128, conv_L_cache=3, conv_bias=False, num_dense_layers=1, num_experts=8,
                 num_experts_per_tok=2, use_expert_bias=True, routed_scaling_factor=1.5, norm_topk_prob=True,
                 layer_types=["conv", "conv", "full_attention", "conv"], pad_token_id=0)
    with torch.no_grad():
        for name, p in m.named_parameters():
            if name.endswith("expert_bias"):
                p.copy_(torch.randn(p.shape, generator=torch.Generator().manual_seed(3)))
        for name, b in m.named_buffers():
            if name.endswith("expert_bias"):
                b.copy_(torch.randn(b.shape, generator=torch.Generator().manual_seed(3)))
    check(m, tmp_path)


def test_qwen3_next(tmp_path):
    m = hf_model("Qwen3NextForCausalLM", "Qwen3NextConfig", vocab_size=320, hidden_size=64, intermediate_size=128,
                 num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32, max_position_embeddings=128,
                 linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=8, linear_num_key_heads=2,
                 linear_num_value_heads=4, decoder_sparse_step=1, moe_intermediate_size=32, shared_expert_intermediate_size=48,
                 num_experts_per_tok=2, num_experts=8, norm_topk_prob=True, mlp_only_layers=[],
                 layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"])
    check(m, tmp_path)


@pytest.mark.parametrize("sparse", [False, True])
def test_qwen3_5(tmp_path, sparse):
    """Qwen3.5: split gated-delta projections, dense or sparse feed-forward, decoder under ``model.language_model``."""
    common = dict(vocab_size=320, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                  max_position_embeddings=128, linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=8,
                  linear_num_key_heads=2, linear_num_value_heads=4,
                  layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"])
    if sparse:
        m = hf_model("Qwen3_5MoeForCausalLM", "Qwen3_5MoeTextConfig", moe_intermediate_size=32, shared_expert_intermediate_size=48,
                     num_experts_per_tok=2, num_experts=8, **common)
    else:
        m = hf_model("Qwen3_5ForCausalLM", "Qwen3_5TextConfig", intermediate_size=128, **common)
    check(m, tmp_path)


def test_nemotron_h(tmp_path):
    m = hf_model("NemotronHForCausalLM", "NemotronHConfig", vocab_size=320, hidden_size=64, intermediate_size=96,
                 num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=128,
                 layers_block_type=["mamba", "moe", "mamba", "attention", "moe"], mamba_num_heads=8, mamba_head_dim=8,
                 ssm_state_size=16, n_groups=2, conv_kernel=4, chunk_size=8, use_conv_bias=True, use_bias=False, mlp_bias=False,
                 attention_bias=False, n_routed_experts=8, n_shared_experts=1, moe_intermediate_size=32,
                 moe_shared_expert_intermediate_size=48, num_experts_per_tok=2, routed_scaling_factor=2.0, n_group=2,
                 topk_group=1, norm_topk_prob=True)
    check(m, tmp_path)


def test_yarn_linear_and_partial_rotary(tmp_path):
    check(hf_model("Qwen2ForCausalLM", "Qwen2Config", **BASE, rope_scaling={
        "rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32, "beta_fast": 32, "beta_slow": 1}),
        tmp_path / "yarn", prompt_len=60)
    check(hf_model("LlamaForCausalLM", "LlamaConfig", **BASE, rope_scaling={"rope_type": "linear", "factor": 2.0}),
          tmp_path / "linear", prompt_len=40)
    check(hf_model("Phi3ForCausalLM", "Phi3Config", **BASE, pad_token_id=0, partial_rotary_factor=0.5), tmp_path / "partial")
    check(hf_model("MistralForCausalLM", "MistralConfig", **BASE, head_dim=24, sliding_window=None), tmp_path / "headdim")


def test_qwen3_vl_text_path(tmp_path):
    cfg_cls = transformers.Qwen3VLConfig
    text = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=32, max_position_embeddings=128,
                rope_scaling={"rope_type": "default", "mrope_section": [8, 4, 4], "mrope_interleaved": True})
    vision = dict(depth=1, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4, spatial_merge_size=2,
                  temporal_patch_size=2, out_hidden_size=64, num_position_embeddings=16, deepstack_visual_indexes=[0])
    cfg = cfg_cls(text_config=text, vision_config=vision, tie_word_embeddings=False)
    torch.manual_seed(0)
    model = transformers.Qwen3VLForConditionalGeneration(cfg).eval().float()
    check(model, tmp_path)


G4 = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=6, num_attention_heads=4, num_key_value_heads=2,
          head_dim=16, global_head_dim=32, sliding_window=8, max_position_embeddings=128,
          layer_types=["sliding_attention", "sliding_attention", "full_attention"] * 2, pad_token_id=0)


@pytest.mark.parametrize("variant", ["plain", "shared_kv_ple", "k_eq_v", "moe"])
def test_gemma4_text(tmp_path, variant):
    kw = dict(G4, num_kv_shared_layers=0, hidden_size_per_layer_input=0, attention_k_eq_v=False, enable_moe_block=False)
    if variant == "shared_kv_ple":
        kw.update(num_kv_shared_layers=3, hidden_size_per_layer_input=8, vocab_size_per_layer_input=320, use_double_wide_mlp=True)
    if variant == "k_eq_v":
        kw.update(attention_k_eq_v=True, num_global_key_value_heads=1)
    if variant == "moe":
        kw.update(enable_moe_block=True, num_experts=4, top_k_experts=2, moe_intermediate_size=32)
    m = hf_model("Gemma4ForCausalLM", "Gemma4TextConfig", **kw)
    with torch.no_grad():
        for name, b in m.named_buffers():
            if name.endswith("layer_scalar"):
                b.fill_(0.9)
        for name, p in m.named_parameters():
            if name.endswith(("router.scale", "per_expert_scale")):
                p.add_(torch.randn(p.shape, generator=torch.Generator().manual_seed(5)) * 0.2)
    check(m, tmp_path, prompt_len=30)
