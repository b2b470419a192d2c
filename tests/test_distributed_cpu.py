"""Host-side logic of the parallel runtime on CPU ranks (gloo, world size 2 and 4): tensor-parallel sharding
(GQA groups, KV-head replication, vocabulary-parallel head) and pipeline stages reproduce the single-rank tokens."""
import pytest
import torch

from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.engine import Engine

from dist_util import run_ranks
from dist_worker import lfm2_cfg, moe_cfg, tiny_cfg


def _oracle(n_new, prompts_lens=(9, 33)):
    cfg = tiny_cfg(False)
    sd = random_state(cfg, seed=0, std=0.05)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in prompts_lens]
    return Engine(model, max_batch=4, max_seq_len=128).generate(prompts, SamplingParams(temperature=0.0), n_new)


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_matches_single_rank(world, tmp_path):
    # world 4 > 2 kv heads: every kv head is replicated on two ranks
    res = run_ranks("cpu_tp_nccl", world, tmp_path)
    want = _oracle(12)
    for r in res:
        assert r["tokens"] == want


@pytest.mark.parametrize("scenario,world", [("cpu_pp", 2), ("cpu_pp_tp2", 4)])
def test_pipeline_parallel_matches_single_rank(scenario, world, tmp_path):
    res = run_ranks(scenario, world, tmp_path)
    want = _oracle(10)
    for r in res:
        assert r["tokens"] == want


@pytest.mark.parametrize("scenario,world", [("cpu_pp_moe", 2), ("cpu_pp_tp2_moe", 4)])
def test_pipeline_with_expert_and_tensor_axes(scenario, world, tmp_path):
    """A sparse model over pipeline stages, and over pipeline x tensor ranks with the experts spread over the tensor
    ranks of every stage (three axes on four ranks): tokens equal the single-rank model's."""
    from eredu_b200.models.moe import make_moe_factory

    res = run_ranks(scenario, world, tmp_path)
    cfg = moe_cfg(False)
    sd = random_state(cfg, seed=0, std=0.08)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]
    want = Engine(model, max_batch=4, max_seq_len=128).generate(prompts, SamplingParams(temperature=0.0), 10)
    for r in res:
        assert r["tokens"] == want


def test_prompt_cache_under_pipeline_parallelism(tmp_path):
    """Each stage writes the K/V of its own layers under its own rank directory; a later request resumes from the
    saved prefix on both stages and generates the tokens of an uncached run."""
    res = run_ranks("cpu_pp_pcache", 2, tmp_path)
    want = _oracle(10)
    for rank, r in enumerate(res):
        assert r["tokens"] == want
        assert r["pcache_cached"] == 32 and r["pcache_tokens"] == want[1]
        assert r["pcache_dir"] == f"rank-pp{rank}-tp0-ep0"
    layers = [set(r["pcache_layers"]) for r in res]
    assert layers[0] and layers[1] and not layers[0] & layers[1]              # every layer on exactly one stage
    assert layers[0] | layers[1] == {0, 1}


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_over_tensor_ranks_matches_single_rank(world, tmp_path):
    """Attention tensor-parallel + experts expert-parallel on the same ranks (replicated tokens, partial expert
    outputs summed over the group) reproduce the single-rank MoE model's tokens."""
    from eredu_b200.models.moe import make_moe_factory

    res = run_ranks("cpu_ep_nccl", world, tmp_path)
    cfg = moe_cfg(False)
    sd = random_state(cfg, seed=0, std=0.08)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]
    want = Engine(model, max_batch=4, max_seq_len=128).generate(prompts, SamplingParams(temperature=0.0), 10)
    for r in res:
        assert r["tokens"] == want


@pytest.mark.parametrize("scenario", ["cpu_ep_robin_nccl", "cpu_ep_explicit_nccl", "cpu_ep_robin_a2a_nccl"])
def test_expert_assignments_other_than_contiguous_ranges(scenario, tmp_path):
    """Round-robin and explicit expert placement are a renaming applied at load (router rows and banks read in execution
    order): the tokens stay those of the single-rank model, with replicated tokens and with the all-to-all dispatch."""
    from eredu_b200.models.moe import make_moe_factory
    from eredu_b200.parallel.context import ParallelContext
    from eredu_b200.parallel.topology import ParallelTopology

    res = run_ranks(scenario, 2, tmp_path)
    cfg = moe_cfg(False)
    sd = random_state(cfg, seed=0, std=0.08)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]
    want = Engine(model, max_batch=4, max_seq_len=128).generate(prompts, SamplingParams(temperature=0.0), 10)
    for r in res:
        assert r["tokens"] == want
    ctx = ParallelContext(ParallelTopology(tensor=2, expert=2, expert_over_tensor=True), 1)
    ctx.expert_assignment = "round_robin"
    assert ctx.expert_order(8) == [0, 2, 4, 6, 1, 3, 5, 7] and ParallelContext(ctx.topology, 0).expert_order(8) is None
    ctx.expert_assignment = [0, 0, 0, 1, 1, 1, 1, 1]
    with pytest.raises(ValueError, match="same number"):
        ctx.expert_order(8)


@pytest.mark.parametrize("scenario,world", [("cpu_lfm2_tp_nccl", 2), ("cpu_lfm2_pp", 2)])
def test_hybrid_family_under_tensor_and_pipeline_parallelism(scenario, world, tmp_path):
    """LFM2: convolution channels and their recurrent state are split over the tensor ranks (row-parallel out_proj
    summed over the group); pipeline stages own the state of their own layers."""
    res = run_ranks(scenario, world, tmp_path)
    cfg = lfm2_cfg()
    sd = random_state(cfg, seed=0, std=0.08)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]
    n_new = 12 if "tp" in scenario else 10
    want = Engine(model, max_batch=4, max_seq_len=128).generate(prompts, SamplingParams(temperature=0.0), n_new)
    for r in res:
        assert r["tokens"] == want


def test_nemotron_h_over_tensor_and_expert_ranks(tmp_path):
    """Mamba mixers split by heads and groups (state, convolution and grouped norm local to a rank, output projection
    summed), attention by head, relu^2 MLP by rows, experts over the same two ranks."""
    from eredu_b200.models.moe import make_moe_factory
    from test_nemotron_h import nh_cfg, state_for

    res = run_ranks("cpu_nemo_ep_nccl", 2, tmp_path)
    cfg = nh_cfg()
    sd = state_for(cfg)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]
    want = Engine(model, max_batch=4, max_seq_len=128).generate(prompts, SamplingParams(temperature=0.0), 10)
    for r in res:
        assert r["tokens"] == want


@pytest.mark.parametrize("variant", ["k_eq_v_moe", "shared_kv_ple"])
def test_gemma4_tensor_parallel(variant, tmp_path, monkeypatch):
    """Gemma 4 on two ranks: query heads split, one replicated global key / value head, feed-forward and expert rows split,
    every row-parallel sum taken before its sandwich norm; tokens equal the single-rank run of the same checkpoint."""
    transformers = pytest.importorskip("transformers")
    from eredu_b200.api import LoadedModel, ModelLoadOptions

    kw = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=6, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, global_head_dim=32, sliding_window=8, max_position_embeddings=128, pad_token_id=0,
              layer_types=["sliding_attention", "sliding_attention", "full_attention"] * 2, num_kv_shared_layers=0,
              hidden_size_per_layer_input=0, attention_k_eq_v=False, enable_moe_block=False)
    if variant == "k_eq_v_moe":
        kw.update(attention_k_eq_v=True, num_global_key_value_heads=1, enable_moe_block=True, num_experts=4, top_k_experts=2,
                  moe_intermediate_size=32)
    else:
        kw.update(num_kv_shared_layers=3, hidden_size_per_layer_input=8, vocab_size_per_layer_input=320, use_double_wide_mlp=True)
    torch.manual_seed(0)
    m = transformers.Gemma4ForCausalLM(transformers.Gemma4TextConfig(**kw)).eval().float()
    with torch.no_grad():
        for _, p in m.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn(p.shape, generator=torch.Generator().manual_seed(1)) * 0.1)
    ckpt = tmp_path / "ckpt"
    m.save_pretrained(ckpt, safe_serialization=True)
    monkeypatch.setenv("EREDU_TEST_CKPT", str(ckpt))
    res = run_ranks("cpu_g4_tp_nccl", 2, tmp_path)
    lm = LoadedModel.load(ckpt, ModelLoadOptions(device="cpu", max_batch=4, max_seq_len=128))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, lm.config.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]
    want = lm.engine.generate(prompts, SamplingParams(temperature=0.0), 12)
    for r in res:
        assert r["tokens"] == want


@pytest.mark.parametrize("variant,world", [("dense", 2), ("routed", 4)])
def test_muse_glimmer_tensor_parallel(variant, world, tmp_path, monkeypatch):
    """Muse-Glimmer over tensor ranks: query heads and the output gate split, key / value heads split (two ranks) or
    replicated (four ranks, two heads), feed-forward and expert rows split, sums taken before the sandwich norms."""
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from test_muse_glimmer import save, state

    sd = state()
    if variant == "routed":
        gen = torch.Generator().manual_seed(9)
        for li in range(4):
            p = f"model.language_model.layers.{li}.mlp."
            for n in ("gate_proj", "up_proj", "down_proj"):
                del sd[p + n + ".weight"]
            sd[p + "gate.weight"] = torch.randn(6, 64, generator=gen) * 0.5
            sd[p + "experts.gate_up_proj"] = torch.randn(6, 64, 64, generator=gen) * 0.2
            sd[p + "experts.down_proj"] = torch.randn(6, 64, 32, generator=gen) * 0.2
        from test_muse_glimmer import TEXT

        text = dict(TEXT, num_experts=6, num_experts_per_tok=2, norm_topk_prob=True, moe_intermediate_size=32)
    else:
        from test_muse_glimmer import TEXT as text
    ckpt = tmp_path / "ckpt"
    ckpt.mkdir()
    save(ckpt, sd, text)
    monkeypatch.setenv("EREDU_TEST_CKPT", str(ckpt))
    res = run_ranks("cpu_ckpt_tp_nccl", world, tmp_path)
    lm = LoadedModel.load(ckpt, ModelLoadOptions(device="cpu", max_batch=4, max_seq_len=128))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, lm.config.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]
    want = lm.engine.generate(prompts, SamplingParams(temperature=0.0), 12)
    for r in res:
        assert r["tokens"] == want


@pytest.mark.parametrize("family", ["nemo", "qnext", "dsv3", "kimi"])
def test_hybrid_and_latent_families_under_pipeline_parallelism(family, tmp_path):
    """Two pipeline stages: every stage keeps the K/V pages and recurrent states of its own layers only, activations
    travel between the stages, tokens equal the single-rank run."""
    from eredu_b200.models.moe import make_moe_factory

    if family == "nemo":
        from test_nemotron_h import nh_cfg as make_cfg, state_for
    elif family == "qnext":
        from test_qwen_next import next_cfg as make_cfg, state_for
    elif family == "dsv3":
        from test_deepseek import ds_cfg as make_cfg, state_for
    else:
        from test_kimi_linear import kimi_cfg as make_cfg, state_for
    res = run_ranks(f"cpu_{family}_pp", 2, tmp_path)
    cfg = make_cfg()
    sd = state_for(cfg)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]
    want = Engine(model, max_batch=4, max_seq_len=128).generate(prompts, SamplingParams(temperature=0.0), 10)
    for r in res:
        assert r["tokens"] == want


def test_kimi_linear_over_tensor_and_expert_ranks(tmp_path):
    """KDA layers split by heads (convolution channels, decay and gate expansions, recurrent state local to a rank),
    latent attention by head, experts over the same two ranks."""
    from eredu_b200.models.moe import make_moe_factory
    from test_kimi_linear import kimi_cfg, state_for

    res = run_ranks("cpu_kimi_ep_nccl", 2, tmp_path)
    cfg = kimi_cfg()
    sd = state_for(cfg)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]
    want = Engine(model, max_batch=4, max_seq_len=128).generate(prompts, SamplingParams(temperature=0.0), 10)
    for r in res:
        assert r["tokens"] == want


def test_qwen_next_family_over_tensor_and_expert_ranks(tmp_path):
    """Gated-delta layers sharded by key-head group, gated attention by head, experts over the same two ranks."""
    from eredu_b200.models.moe import make_moe_factory
    from test_qwen_next import next_cfg, state_for

    res = run_ranks("cpu_qnext_ep_nccl", 2, tmp_path)
    cfg = next_cfg()
    sd = state_for(cfg)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]
    want = Engine(model, max_batch=4, max_seq_len=128).generate(prompts, SamplingParams(temperature=0.0), 10)
    for r in res:
        assert r["tokens"] == want


def test_deepseek_family_over_tensor_and_expert_ranks(tmp_path):
    """Latent attention with heads split over two ranks (replicated latent cache), experts over the same ranks."""
    from eredu_b200.models.moe import make_moe_factory
    from test_deepseek import ds_cfg, state_for

    res = run_ranks("cpu_dsv3_ep_nccl", 2, tmp_path)
    cfg = ds_cfg()
    sd = state_for(cfg)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]
    want = Engine(model, max_batch=4, max_seq_len=128).generate(prompts, SamplingParams(temperature=0.0), 10)
    for r in res:
        assert r["tokens"] == want


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_all_to_all_matches_single_rank(world, tmp_path):
    """Token-sharded expert parallelism on CPU ranks (gloo): every rank routes its own slice of the tokens, the routes
    travel to their expert's owner and back (count exchange, rows and ids forward, rows in reverse, all-gather of the
    finished token rows), and every rank ends with the tokens of the single-rank model."""
    from eredu_b200.models.moe import make_moe_factory
    from dist_worker import moe_cfg

    res = run_ranks("cpu_ep_a2a_nccl", world, tmp_path)
    cfg = moe_cfg(False)
    sd = random_state(cfg, seed=0, std=0.08)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32, moe_factory=make_moe_factory())
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33)]
    want = Engine(model, max_batch=4, max_seq_len=128).generate(prompts, SamplingParams(temperature=0.0), 10)
    for r in res:
        assert r["tokens"] == want and r["a2a_calls"] > 0

