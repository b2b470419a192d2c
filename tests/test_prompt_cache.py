"""Prompt caches on disk: save -> load reproduces the tokens of an uncached run; every identity, hash or topology
mismatch is refused (CPU, tiny model)."""
import dataclasses
import json

import pytest
import torch

from eredu_b200.models import config as C
from eredu_b200.models.llama import build_from_tensors, random_state
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime import prompt_cache as PC
from eredu_b200.runtime.engine import Engine


def make_engine(seed=0, **over):
    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=512, **over)
    sd = random_state(cfg, seed=seed, std=0.05)
    model = build_from_tensors(cfg, sd.__getitem__, sd.__contains__, "cpu", torch.float32)
    return Engine(model, max_batch=2, max_seq_len=256)


def run(eng, seq, n):
    first = eng.prefill([seq])
    eng.start_decode([seq], first)
    out = [int(first[0])]
    for _ in range(n - 1):
        toks = eng.decode_step()
        eng.commit(toks)
        out.append(int(toks[0]))
    eng._decode_state = None
    return out


def test_round_trip_and_refusals(tmp_path):
    eng = make_engine()
    g = torch.Generator().manual_seed(1)
    prefix = torch.randint(0, 512, (75,), generator=g).tolist()
    tail = torch.randint(0, 512, (9,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0)
    s0 = eng.new_sequence(prefix + tail, sp, max_new_tokens=8)
    want = run(eng, s0, 6)
    eng.release(s0)

    s1 = eng.new_sequence(prefix, sp, max_new_tokens=4)
    eng.prefill([s1])
    d = PC.save_prompt_cache(eng, s1, tmp_path / "pc", "ckpt-A", block_tokens=32, namespace="unit")
    eng.release(s1)
    man = PC.open_prompt_cache(d)
    assert man.schema_version == 7 and man.total_prefix_tokens == 75 and man.prefix_sha256 == PC.sha256_tokens(prefix)
    assert len(man.blocks) == eng.cfg.num_hidden_layers * 3 and man.application_namespace == "unit"
    with pytest.raises(PC.PromptCacheError):
        PC.save_prompt_cache(eng, s1, tmp_path / "pc", "ckpt-A")  # kv_len 75 but exists, no replace

    eng2 = make_engine()
    s2 = PC.load_prompt_cache(eng2, d, prefix + tail, "ckpt-A", sp, max_new_tokens=8)
    assert s2.kv_len == 75
    assert run(eng2, s2, 6) == want
    # the whole request is cached: one token is still prefilled so that logits exist
    s3 = PC.load_prompt_cache(eng2, d, prefix, "ckpt-A", sp, max_new_tokens=8)
    assert s3.kv_len == 74

    with pytest.raises(PC.Incompatible):
        PC.load_prompt_cache(eng2, d, prefix + tail, "ckpt-B", sp, 8)
    with pytest.raises(PC.Incompatible):
        PC.load_prompt_cache(eng2, d, [1] + prefix[1:] + tail, "ckpt-A", sp, 8)
    with pytest.raises(PC.Incompatible):
        PC.load_prompt_cache(make_engine(rope_theta=12345.0), d, prefix + tail, "ckpt-A", sp, 8)
    with pytest.raises(PC.PromptCacheError):
        PC.open_prompt_cache(d, PC.PromptCacheTopology(tensor_parallel=(2, 1)))

    # corrupt one payload byte -> hash mismatch
    shard = d / "layer-0001.safetensors"
    raw = bytearray(shard.read_bytes())
    raw[-3] ^= 0x40
    shard.write_bytes(bytes(raw))
    free = eng2.kv.allocator.free_pages()
    with pytest.raises(PC.Corrupt):
        PC.load_prompt_cache(eng2, d, prefix + tail, "ckpt-A", sp, 8)
    assert eng2.kv.allocator.free_pages() == free  # pages of the failed load went back


def test_manifest_validation(tmp_path):
    eng = make_engine()
    s = eng.new_sequence(list(range(40)), max_new_tokens=4)
    eng.prefill([s])
    d = PC.save_prompt_cache(eng, s, tmp_path / "pc", "x", block_tokens=16)
    m = json.loads((d / "manifest.json").read_text())
    bad = dict(m, schema_version=6)
    (d / "manifest.json").write_text(json.dumps(bad))
    with pytest.raises(PC.UnsupportedSchema):
        PC.open_prompt_cache(d)
    bad = dict(m, blocks=m["blocks"][1:])
    (d / "manifest.json").write_text(json.dumps(bad))
    with pytest.raises(PC.Malformed):
        PC.open_prompt_cache(d)
    bad = json.loads(json.dumps(m))
    bad["blocks"][0]["shard"] = "../evil.safetensors"
    (d / "manifest.json").write_text(json.dumps(bad))
    with pytest.raises(PC.Malformed):
        PC.open_prompt_cache(d)
    bad = dict(m, prefix_sha256="zz")
    (d / "manifest.json").write_text(json.dumps(bad))
    with pytest.raises(PC.Malformed):
        PC.open_prompt_cache(d)
    # replace_existing publishes a fresh cache
    PC.save_prompt_cache(eng, s, tmp_path / "pc", "x", block_tokens=16, replace_existing=True)
    assert PC.open_prompt_cache(d).total_prefix_tokens == 40


@pytest.mark.parametrize("family", ["lfm2", "qwen3_next", "nemotron_h"])
def test_hybrid_models_persist_their_recurrent_state(family, tmp_path):
    """Convolution histories and recurrent matrices are stored as fixed-state tensors at the end of the prefix and come
    back into the new sequence's state slot."""
    from test_speculative import _hybrid

    cfg, model = _hybrid(family, 0)
    eng = Engine(model, max_batch=2, max_seq_len=160)
    g = torch.Generator().manual_seed(2)
    prefix = torch.randint(3, cfg.vocab_size, (41,), generator=g).tolist()
    tail = torch.randint(3, cfg.vocab_size, (7,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0)
    s0 = eng.new_sequence(prefix + tail, sp, max_new_tokens=8)
    want = run(eng, s0, 6)
    eng.release(s0)
    s1 = eng.new_sequence(prefix, sp, max_new_tokens=4)
    eng.prefill([s1])
    with pytest.raises(PC.PromptCacheError):
        PC.save_prompt_cache(eng, s1, tmp_path / "pc", "ckpt", prefix_tokens=32)     # states exist at length 41 only
    d = PC.save_prompt_cache(eng, s1, tmp_path / "pc", "ckpt", block_tokens=16)
    eng.release(s1)
    man = PC.open_prompt_cache(d)
    kinds = [l["kind"] for l in man.layer_layout]
    assert "recurrent" in kinds and "key_value" in kinds
    n_state = sum(len(l.get("fixed_state", [])) for l in man.layer_layout)
    assert len(man.state_tensors) == n_state > 0 and all(e["tokens"] == 41 for e in man.state_tensors)
    assert {b.global_layer for b in man.blocks} == {i for i, k in enumerate(kinds) if k == "key_value"}

    _, model2 = _hybrid(family, 0)
    eng2 = Engine(model2, max_batch=2, max_seq_len=160)
    busy = eng2.new_sequence([3, 4, 5], sp, max_new_tokens=4)          # occupies the first state slot / pages
    eng2.prefill([busy])
    s2 = PC.load_prompt_cache(eng2, d, prefix + tail, "ckpt", sp, max_new_tokens=8)
    assert s2.kv_len == 41 and run(eng2, s2, 6) == want
    with pytest.raises(PC.Incompatible):
        PC.load_prompt_cache(eng2, d, prefix, "ckpt", sp, 8)            # nothing left to prefill: no state for 40 tokens
    # a state entry that is missing, duplicated or taken elsewhere makes the manifest malformed
    mj = json.loads((d / "manifest.json").read_text())
    for damage in (lambda m: m["state_tensors"].pop(), lambda m: m["state_tensors"].append(dict(m["state_tensors"][0])),
                   lambda m: m["state_tensors"][0].__setitem__("tokens", 40)):
        bad = json.loads(json.dumps(mj))
        damage(bad)
        with pytest.raises(PC.Malformed):
            PC.PromptCacheManifest.from_json(json.dumps(bad)).validate()
    raw = bytearray((d / "state.safetensors").read_bytes())
    raw[-2] ^= 0x10
    (d / "state.safetensors").write_bytes(bytes(raw))
    with pytest.raises(PC.Corrupt):
        PC.load_prompt_cache(eng2, d, prefix + tail, "ckpt", sp, 8)
