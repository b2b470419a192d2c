"""The families that run as tensor operations around the GEMM kernels (DeepSeek-V4, Inkling, Muse-Glimmer, the Gemma 4
assistant) and the KV block tiers, on the GPU in bf16: same invariants as on the CPU, with tolerances for bf16."""
import json

import pytest
import torch

from eredu_b200.ops import SamplingParams

pytestmark = pytest.mark.gpu


def _close(a, b, tol):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-6)) < tol


def test_deepseek_v4_on_the_gpu_matches_its_cpu_run():
    from eredu_b200.models.deepseek_v4 import DeepseekV4Config, DeepseekV4Model
    from test_deepseek_v4 import v4_cfg, v4_state

    cfg = DeepseekV4Config.from_dict(v4_cfg(hidden_size=128, moe_intermediate_size=64, head_dim=32, qk_rope_head_dim=16, q_lora_rank=64,
                                            o_lora_rank=32, vocab_size=256, index_head_dim=16))
    sd = v4_state(cfg)
    cpu = DeepseekV4Model(cfg, sd.__getitem__, sd.__contains__)
    gpu = DeepseekV4Model(cfg, sd.__getitem__, sd.__contains__, "cuda", torch.bfloat16)
    tokens = torch.randint(0, 256, (29,), generator=torch.Generator().manual_seed(1)).tolist()
    want = cpu.forward(tokens, cpu.new_cache())
    cache = gpu.new_cache()
    got = gpu.forward(tokens[:13], cache)
    for t in tokens[13:]:
        got = gpu.forward([t], cache)
    assert _close(got, want, 0.08)


def test_inkling_on_the_gpu_matches_its_cpu_run():
    from eredu_b200.models.inkling import InklingConfig, InklingModel
    from test_inkling import ink_cfg, ink_state

    cfg = InklingConfig.from_dict(ink_cfg(hidden_size=128, head_dim=32, swa_head_dim=32, vocab_size=256, unpadded_vocab_size=250,
                                          intermediate_size=64, dense_intermediate_size=64, moe_intermediate_size=32, d_rel=8))
    sd = ink_state(cfg)
    cpu = InklingModel(cfg, sd.__getitem__, sd.__contains__)
    gpu = InklingModel(cfg, sd.__getitem__, sd.__contains__, "cuda", torch.bfloat16)
    tokens = torch.randint(0, 250, (23,), generator=torch.Generator().manual_seed(1)).tolist()
    want = cpu.forward(tokens, cpu.new_cache())
    cache = gpu.new_cache()
    got = gpu.forward(tokens[:10], cache)
    for t in tokens[10:]:
        got = gpu.forward([t], cache)
    assert _close(got, want, 0.08)


@pytest.mark.parametrize("head_dim", [16, 64])
def test_muse_glimmer_on_the_gpu_engine(tmp_path, head_dim, monkeypatch):
    """Head size 16 runs the tensor-operation attention, 64 the attention kernels (tcgen05 prefill, split-KV decode)."""
    import test_muse_glimmer as T
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from test_muse_glimmer import dense_reference, save, state

    sd = state(D=head_dim)
    save(tmp_path, sd, dict(T.TEXT, head_dim=head_dim))
    lm = LoadedModel.load(tmp_path, ModelLoadOptions(device="cuda", max_batch=2, max_seq_len=64))
    tokens = torch.randint(0, 200, (21,), generator=torch.Generator().manual_seed(1)).tolist()
    want = dense_reference(sd, tokens, D=head_dim)
    assert _close(lm.prefill_logits(tokens), want[-1], 0.08)
    seq = lm.engine.new_sequence(tokens[:9], max_new_tokens=16)           # prefill, then decode-shaped steps
    lm.engine.prefill_logits([seq])
    row = None
    for t in tokens[9:]:
        row = lm.engine.step_logits(seq, t)
    lm.engine.release(seq)
    assert _close(row, want[-1], 0.08)
    out = lm.generate([tokens[:9], tokens[4:17]], SamplingParams(temperature=0.0), 6)
    assert [len(o) for o in out] == [6, 6]
    from eredu_b200.ops import native

    native.check_status(torch.device("cuda", torch.cuda.current_device()))


def test_block_tiers_on_the_gpu_use_the_copy_stream(tmp_path):
    from eredu_b200.runtime.engine import Engine
    from eredu_b200.runtime.kv_cache import PAGE
    from test_block_tiers import conversations
    from test_prefix_reuse import model

    cfg, m = model("cuda", torch.bfloat16)
    sp = SamplingParams(temperature=0.0)
    convs = conversations(cfg, n=5)
    cold = Engine(m, max_batch=1, max_seq_len=96)
    want = [cold.generate([c + [7, 8, 9]], sp, 6)[0] for c in convs]
    probe = Engine(m, max_batch=1, max_seq_len=96, num_pages=11, prefix_cache=True)
    L, _, nkv, _, D = probe.kv.k.shape
    block = 2 * L * nkv * PAGE * D * probe.kv.k.element_size()
    eng = Engine(m, max_batch=1, max_seq_len=96, num_pages=11, prefix_cache=True, kv_host_tier_bytes=2 * block,
                 kv_disk_tier_dir=str(tmp_path / "kv"), kv_disk_tier_bytes=64 * block)
    assert eng.block_tiers is not None and eng.block_tiers.stream is not None
    for c in convs:
        eng.generate([c], sp, 4)
    st = eng.block_tiers.stats
    assert st["demoted"] > 0 and st["spilled"] > 0
    for i, c in enumerate(convs):
        assert eng.generate([c + [7, 8, 9]], sp, 6)[0] == want[i], i
    assert st["promoted_host"] + st["promoted_disk"] > 0


def test_gemma4_assistant_on_the_gpu(tmp_path):
    transformers = pytest.importorskip("transformers")
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.models.gemma4_assistant import Gemma4Assistant, Gemma4AssistantConfig
    from eredu_b200.runtime.speculative import Gemma4AssistantDecoder
    from test_gemma4_assistant import _split

    whole, ast, cfg = _split(tmp_path, False)
    lm = LoadedModel.load(tmp_path / "target", ModelLoadOptions(device="cuda", max_batch=2, max_seq_len=96))
    assistant = Gemma4Assistant(Gemma4AssistantConfig.from_dict(cfg), ast.__getitem__, ast.__contains__, lm.engine.model)
    prompts = [list(range(3, 20)), list(range(40, 52))]
    sp = SamplingParams(temperature=0.0)
    plain = lm.engine.generate(prompts, sp, 12)
    dec = Gemma4AssistantDecoder(lm.engine, assistant)
    got = dec.generate(prompts, sp, 12)
    # bf16 ties aside, speculation commits what plain decoding commits whatever the drafter proposes
    agree = sum(a == b for x, y in zip(got, plain) for a, b in zip(x, y))
    assert agree >= 20 and dec.stats.rounds > 0 and dec.stats.proposed == 3 * dec.stats.rounds


def test_muse_glimmer_vision_tower_on_the_gpu():
    """The tower in bf16 on the GPU (this repository's GEMMs, fused attention per window) against its fp32 CPU run."""
    from eredu_b200.models.muse_glimmer_vision import MuseGlimmerVision, MuseVisionConfig
    from test_muse_glimmer_vision import LANG, PROJ, VISION, tower_state

    sd = tower_state()
    cfg = MuseVisionConfig.from_dict(VISION, LANG, PROJ)
    cpu = MuseGlimmerVision(cfg, sd.__getitem__, sd.__contains__)
    gpu = MuseGlimmerVision(cfg, sd.__getitem__, sd.__contains__, "cuda", torch.bfloat16)
    grids = [(1, 8, 12), (2, 4, 6)]
    patches = torch.randn(96 + 48, 96, generator=torch.Generator().manual_seed(4))
    want, got = cpu(patches, grids), gpu(patches, grids)
    assert got.shape == want.shape == (24 + 12, LANG) and got.is_cuda
    assert _close(got, want, 0.06)


def test_unpaged_speculative_decoder_on_the_gpu():
    """Inkling in bf16 on the GPU with a one-layer draft: rounds run on the device (caches cloned and restored there) and
    every emitted token is the target's own choice at its position, so the output has the requested length and the
    first token equals plain generation's (later ones may differ where bf16 multi-token and single-token passes tie)."""
    from eredu_b200.models.inkling import InklingConfig, InklingModel
    from eredu_b200.runtime.unpaged import UnpagedEngine, UnpagedSpeculativeDecoder
    from test_inkling import ink_cfg, ink_state

    def engine(seed, **over):
        cfg = InklingConfig.from_dict(ink_cfg(hidden_size=64, head_dim=16, swa_head_dim=16, d_rel=8, **over))
        sd = ink_state(cfg, seed=seed)
        return UnpagedEngine(InklingModel(cfg, sd.__getitem__, sd.__contains__, "cuda", torch.bfloat16), max_seq_len=128)

    target, draft = engine(0), engine(1, num_hidden_layers=1, layer_types=["full_attention"], dense_mlp_idx=0)
    sp = SamplingParams(temperature=0.0)
    prompt = list(range(5, 19))
    want = target.generate([prompt], sp, 12)[0]
    spec = UnpagedSpeculativeDecoder(target, draft, k=3)
    got = spec.generate([prompt], sp, 12)[0]
    assert len(got) == 12 and got[0] == want[0]
    s = spec.stats.summary()
    assert s["rounds"] >= 3 and s["proposed"] >= s["accepted"]
