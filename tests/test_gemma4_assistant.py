"""Gemma 4 assistant drafter.

Oracle for the block math: a Transformers Gemma 4 model whose last three layers share the K / V of earlier layers IS a
target (its first three layers) followed by an assistant (the shared-KV tail) when the assistant's input projection
selects the hidden half of its input. The drafter's first step must then give the Transformers model's last-position
logits. The speculative loop is checked for exactness (greedy output equals plain decoding) with every head form."""
import json

import pytest
import torch

transformers = pytest.importorskip("transformers")

from eredu_b200.api import LoadedModel, ModelLoadOptions
from eredu_b200.models.gemma4_assistant import Gemma4Assistant, Gemma4AssistantConfig, load_gemma4_assistant
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.speculative import Gemma4AssistantDecoder
from test_hf_parity import G4, hf_model


def _split(tmp_path, double_wide):
    kw = dict(G4, num_kv_shared_layers=3, hidden_size_per_layer_input=0, attention_k_eq_v=False, enable_moe_block=False,
              use_double_wide_mlp=double_wide)
    whole = hf_model("Gemma4ForCausalLM", "Gemma4TextConfig", **kw)
    with torch.no_grad():
        for name, b in whole.named_buffers():
            if name.endswith("layer_scalar"):
                b.fill_(0.9)
    sd = {k: v.detach().clone() for k, v in whole.state_dict().items()}
    # the target: layers 0..2 under their own names
    tkw = dict(kw, num_hidden_layers=3, layer_types=kw["layer_types"][:3], num_kv_shared_layers=0)
    target = transformers.Gemma4ForCausalLM(transformers.Gemma4TextConfig(**tkw)).eval().float()
    tsd = target.state_dict()
    target.load_state_dict({k: sd[k] for k in tsd if k in sd}, strict=False)
    target.save_pretrained(tmp_path / "target", safe_serialization=True)
    # the assistant: layers 3..5 renamed to 0..2, the whole model's norm and embedding, a selecting input projection
    H = kw["hidden_size"]
    ast = {}
    for k, v in sd.items():
        if k.startswith("model.layers."):
            li = int(k.split(".")[2])
            if li >= 3:
                ast[k.replace(f"model.layers.{li}.", f"model.layers.{li - 3}.")] = v
    ast["model.norm.weight"] = sd["model.norm.weight"]
    ast["model.embed_tokens.weight"] = sd["model.embed_tokens.weight"]
    ast["pre_projection.weight"] = torch.cat((torch.zeros(H, H), torch.eye(H)), 1)
    ast["post_projection.weight"] = torch.eye(H)
    text = transformers.Gemma4TextConfig(**dict(kw, num_hidden_layers=3, layer_types=kw["layer_types"][3:],
                                                num_kv_shared_layers=3)).to_dict()      # as a published config.json spells it
    return whole, ast, {"model_type": "gemma4_assistant", "backbone_hidden_size": H, "text_config": text, "block_size": 4,
                        "tie_word_embeddings": True}


@pytest.mark.parametrize("double_wide", [False, True])
def test_first_draft_step_is_the_shared_kv_tail_of_a_transformers_model(tmp_path, double_wide):
    whole, ast, cfg = _split(tmp_path, double_wide)
    lm = LoadedModel.load(tmp_path / "target", ModelLoadOptions(device="cpu", max_batch=2, max_seq_len=64))
    assistant = Gemma4Assistant(Gemma4AssistantConfig.from_dict(cfg), ast.__getitem__, ast.__contains__, lm.engine.model)
    dec = Gemma4AssistantDecoder(lm.engine, assistant)
    assert dec.k == 3
    prompts = [torch.randint(0, 320, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (30, 11)]   # 30 > window
    seqs = [lm.engine.new_sequence(p, SamplingParams(temperature=0.0), 8) for p in prompts]
    dec._prefill(seqs, [None, None])
    eng = lm.engine
    hidden = torch.cat([dec._pending_hidden[s.seq_id] for s in seqs])
    lens = torch.tensor([len(p) for p in prompts])
    logits, nxt = assistant.draft_step(torch.tensor([5, 7]), hidden, eng.kv, eng._block_table(seqs), lens, 0)
    for b, p in enumerate(prompts):
        with torch.no_grad():
            ref = whole(torch.tensor([p])).logits[0, -1].float()
        assert float((logits[b] - ref).abs().max()) < 2e-3 * max(1.0, float(ref.abs().max()))
    assert nxt.shape == (2, 64)
    # a later step moves the query position: on a sliding layer the oldest visible key drops out of the window
    w = next(w for w in assistant.layers if w["sliding"])
    q = torch.randn(1, 4, w["D"])
    a0 = assistant._attend(q, w, eng.kv, eng._block_table(seqs[:1]), lens[:1], lens[:1] - 1)
    a2 = assistant._attend(q, w, eng.kv, eng._block_table(seqs[:1]), lens[:1], lens[:1] + 1)
    assert not torch.allclose(a0, a2)
    for s in seqs:
        eng.release(s)


@pytest.mark.parametrize("head", ["tied", "lm_head", "ordered"])
def test_speculative_generation_with_the_assistant_is_exact(tmp_path, head):
    whole, ast, cfg = _split(tmp_path, False)
    g = torch.Generator().manual_seed(3)
    H, V = 64, 320
    ast["pre_projection.weight"] = torch.randn(H, 2 * H, generator=g) * 0.1
    ast["post_projection.weight"] = torch.randn(H, H, generator=g) * 0.1
    if head == "lm_head":
        cfg["tie_word_embeddings"] = False
        ast["lm_head.weight"] = torch.randn(V, H, generator=g) * 0.1
    if head == "ordered":
        cfg.update(use_ordered_embeddings=True, num_centroids=16, centroid_intermediate_top_k=4)
        ast["masked_embedding.centroids.weight"] = torch.randn(16, H, generator=g)
        ast["masked_embedding.token_ordering"] = torch.randperm(V, generator=g).to(torch.int32)
    from safetensors.torch import save_file

    (tmp_path / "assistant").mkdir()
    save_file({k: v.contiguous() for k, v in ast.items()}, str(tmp_path / "assistant" / "model.safetensors"))
    (tmp_path / "assistant" / "config.json").write_text(json.dumps(cfg))
    lm = LoadedModel.load(tmp_path / "target", ModelLoadOptions(device="cpu", max_batch=2, max_seq_len=96))
    lm.attach_assistant(tmp_path / "assistant")
    prompts = [list(range(3, 20)), list(range(40, 52))]
    sp = SamplingParams(temperature=0.0)
    plain = lm.engine.generate(prompts, sp, 20)
    dec = lm._mtp_decoder(None, 3)
    assert isinstance(dec, Gemma4AssistantDecoder)
    assert dec.generate(prompts, sp, 20) == plain
    assert dec.stats.rounds > 0 and dec.stats.proposed == 3 * dec.stats.rounds
    if head == "ordered":
        # only the tokens of the four best groups are evaluated; everything else sits one below the smallest of them
        h = torch.randn(1, H)
        logits = lm.assistant._logits(h)
        top = torch.topk(h @ ast["masked_embedding.centroids.weight"].t(), 4).indices[0]
        ids = ast["masked_embedding.token_ordering"].view(16, 20)[top].reshape(-1).long()
        want = h[0] @ ast["model.embed_tokens.weight"][ids].t()
        assert torch.allclose(logits[0, ids], want, atol=1e-5)
        rest = torch.ones(V, dtype=torch.bool)
        rest[ids] = False
        assert torch.allclose(logits[0, rest], (want.min() - 1.0).expand(int(rest.sum())))
    # stochastic rows run through the same loop
    out = dec.generate(prompts[:1], SamplingParams(temperature=0.8, top_p=0.9, seed=5), 12)
    assert len(out[0]) == 12


def test_assistant_refuses_a_mismatched_target(tmp_path):
    whole, ast, cfg = _split(tmp_path, False)
    lm = LoadedModel.load(tmp_path / "target", ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=32))
    bad = dict(cfg, backbone_hidden_size=128)
    with pytest.raises(ValueError, match="backbone width"):
        Gemma4Assistant(Gemma4AssistantConfig.from_dict(bad), ast.__getitem__, ast.__contains__, lm.engine.model)
    with pytest.raises(ValueError, match="text_config"):
        Gemma4AssistantConfig.from_dict({"model_type": "gemma4_assistant"})


def test_the_request_scheduler_drives_the_assistant(tmp_path):
    from eredu_b200.runtime.mtp_scheduler import MtpScheduler, MtpSchedulerOptions

    whole, ast, cfg = _split(tmp_path, False)
    g = torch.Generator().manual_seed(4)
    ast["pre_projection.weight"] = torch.randn(64, 128, generator=g) * 0.1
    lm = LoadedModel.load(tmp_path / "target", ModelLoadOptions(device="cpu", max_batch=4, max_seq_len=96))
    assistant = Gemma4Assistant(Gemma4AssistantConfig.from_dict(cfg), ast.__getitem__, ast.__contains__, lm.engine.model)
    prompts = [list(range(3, 20)), list(range(40, 52)), list(range(100, 109))]
    sp = SamplingParams(temperature=0.0)
    plain = lm.engine.generate(prompts, sp, 15)
    sched = MtpScheduler(Gemma4AssistantDecoder(lm.engine, assistant), MtpSchedulerOptions().with_lookahead(1))
    assert not sched.lookahead_possible                     # the assistant reads committed keys only
    for p in prompts:
        sched.submit(p, sp, 15)
    done = sched.finish()
    assert [r.token_ids for r in done.requests] == plain
