"""Draft-and-verify decoding for targets on the unpaged engine: the output is token for token the plain generation, at
temperature 0 and above, with an unpaged draft (cache rolled back by value) and with a paged draft (rolled back by
length); a draft equal to the target is accepted in full."""
import pytest
import torch

from eredu_b200.models.inkling import InklingConfig, InklingModel
from eredu_b200.ops import SamplingParams
from eredu_b200.runtime.unpaged import UnpagedEngine, UnpagedSpeculativeDecoder
from test_inkling import ink_cfg, ink_state


def inkling(seed=0, **over):
    cfg = InklingConfig.from_dict(ink_cfg(**over))
    sd = ink_state(cfg, seed=seed)
    return UnpagedEngine(InklingModel(cfg, sd.__getitem__, sd.__contains__), max_seq_len=128)


@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_unpaged_draft_reproduces_plain_generation(temperature):
    target, draft = inkling(0), inkling(1, num_hidden_layers=1, layer_types=["full_attention"], dense_mlp_idx=0)
    sp = SamplingParams(temperature=temperature, top_p=0.95, seed=11)
    prompts = [list(range(5, 19)), [7, 3, 9]]
    want = target.generate(prompts, sp, 17)
    spec = UnpagedSpeculativeDecoder(target, draft, k=3)
    seen = []
    got = spec.generate(prompts, sp, 17, on_token=lambda i, t: seen.append((i, t)) and None)
    assert got == want and [t for i, t in seen if i == 1] == want[1]
    s = spec.stats.summary()
    assert s["rounds"] > 0 and s["proposed"] >= s["accepted"]
    # the target as its own draft: every proposal is accepted, a round emits k + 1 tokens
    own = UnpagedSpeculativeDecoder(target, inkling(0), k=3)
    assert own.generate(prompts[:1], sp, 12) == [want[0][:12]]
    assert own.stats.accepted == own.stats.proposed and own.stats.full_accept_rounds == own.stats.rounds


def test_paged_draft_and_stopping():
    from eredu_b200.models.config import ModelConfig
    from eredu_b200.models.llama import build_from_tensors, random_state
    from eredu_b200.runtime.engine import Engine

    target = inkling(0)
    vocab = target.cfg.vocab_size
    dcfg = ModelConfig.from_hf_dict({"model_type": "llama", "vocab_size": vocab, "hidden_size": 32, "intermediate_size": 64,
                                     "num_hidden_layers": 1, "num_attention_heads": 2, "num_key_value_heads": 1,
                                     "max_position_embeddings": 256})
    dsd = random_state(dcfg, seed=3, std=0.1)
    draft = Engine(build_from_tensors(dcfg, dsd.__getitem__, dsd.__contains__, "cpu", torch.float32), max_batch=2, max_seq_len=128)
    sp = SamplingParams(temperature=0.0)
    prompt = list(range(4, 15))
    want = target.generate([prompt], sp, 14)[0]
    spec = UnpagedSpeculativeDecoder(target, draft, k=4)
    assert spec.generate([prompt], sp, 14) == [want]
    # an end-of-sequence id inside an accepted run ends the output there
    eos = want[5]
    cut = want[:want.index(eos) + 1]
    assert spec.generate([prompt], sp, 14, eos_ids=(eos,)) == [cut] == target.generate([prompt], sp, 14, eos_ids=(eos,))
    with pytest.raises(ValueError, match="vocabulary"):
        UnpagedSpeculativeDecoder(target, inkling(0, vocab_size=64, unpadded_vocab_size=60), k=2)
