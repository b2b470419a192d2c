"""Config 1 of the benchmark set: a tiny Llama (2 layers, hidden 256, 4 q / 2 kv heads, head_dim 64, SwiGLU 688,
vocab 32000, tied embeddings, theta 1e4, eps 1e-5), fp32 on CPU, saved as a SafeTensors directory and as an F32
GGUF - both must give identical logits and identical 64 greedy tokens for a 32-token random prompt."""
import numpy as np
import torch

from eredu_b200.api import LoadedModel, ModelLoadOptions
from eredu_b200.formats import checkpoint as ck
from eredu_b200.models import config as C
from eredu_b200.models.llama import random_state
from eredu_b200.ops import SamplingParams

from reference_model import forward_logits, greedy


def _write_both(tmp_path, cfg, sd):
    st_dir = tmp_path / "st"
    ck.save_safetensors_checkpoint(st_dir, cfg, sd, torch.float32)
    gg = tmp_path / "model.gguf"
    ck.save_gguf_checkpoint(gg, cfg, sd, "F32")
    return st_dir, gg


def test_safetensors_and_f32_gguf_give_identical_logits_and_tokens(tmp_path):
    cfg = C.tiny_llama()
    sd = random_state(cfg, seed=0, std=0.02)
    st_dir, gg = _write_both(tmp_path, cfg, sd)
    opt = ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=128)
    a = LoadedModel.load(st_dir, opt)
    b = LoadedModel.load(gg, opt)
    assert a.config.tie_word_embeddings and b.config.tie_word_embeddings
    assert b.config.num_key_value_heads == 2 and b.config.head_dim == 64 and b.config.rope_theta == 10000.0
    prompt = np.random.default_rng(0).integers(0, cfg.vocab_size, 32).tolist()
    la, lb = a.prefill_logits(prompt), b.prefill_logits(prompt)
    assert torch.equal(la, lb)
    ref = forward_logits(cfg, sd, prompt)[-1]
    assert float((la - ref).abs().max()) < 1e-4
    ta = list(a.generate_tokens(prompt, SamplingParams(temperature=0.0), 64, stop_on_eos=False))
    tb = list(b.generate_tokens(prompt, SamplingParams(temperature=0.0), 64, stop_on_eos=False))
    assert ta == tb and len(ta) == 64
    assert ta[:16] == greedy(cfg, sd, prompt, 16)


def test_gguf_stores_llama_cpp_row_order(tmp_path):
    cfg = C.tiny_llama()
    sd = random_state(cfg, seed=1)
    _, gg = _write_both(tmp_path, cfg, sd)
    src = ck.GgufSource(gg)
    stored = torch.from_numpy(src.reader.dequantize("blk.0.attn_q.weight"))
    hf = sd["model.layers.0.self_attn.q_proj.weight"]
    assert not torch.equal(stored, hf)
    assert torch.equal(stored, ck.permute_qk_to_ggml(hf, cfg.num_attention_heads))
    assert torch.equal(src.get("model.layers.0.self_attn.q_proj.weight"), hf)
    assert torch.equal(src.get("model.layers.1.self_attn.k_proj.weight"), sd["model.layers.1.self_attn.k_proj.weight"])


def test_sharded_safetensors_and_name_translation(tmp_path):
    cfg = C.tiny_llama()
    sd = random_state(cfg, seed=2)
    ck.save_safetensors_checkpoint(tmp_path / "sh", cfg, sd, torch.float32, shard_bytes=4 << 20)
    src = ck.SafetensorsSource(tmp_path / "sh", mapped_shards=1)
    assert (tmp_path / "sh" / "model.safetensors.index.json").exists()
    for k, v in sd.items():
        assert torch.equal(src.get(k), v)
    assert torch.equal(src.get_rows("model.embed_tokens.weight", 100, 200), sd["model.embed_tokens.weight"][100:200])
    for k in sd:
        g = ck.hf_to_gguf_name(k)
        assert g is not None and ck.gguf_to_hf_name(g) == k
