"""Probe records: logits at sampled prefill positions and along a teacher-forced decode, from this runtime and from
Hugging Face Transformers."""
from __future__ import annotations

import torch


def default_token_ids(vocab_size: int, length: int = 48, seed: int = 1729) -> list[int]:
    """Deterministic token ids (a repeated pattern with seeded variation) for checkpoints without a tokenizer."""
    g = torch.Generator().manual_seed(seed)
    base = torch.randint(3, max(4, vocab_size - 1), (12,), generator=g).tolist()
    ids = (base * (length // len(base) + 1))[:length]
    for i in range(5, length, 7):
        ids[i] = int(torch.randint(3, max(4, vocab_size - 1), (1,), generator=g))
    return ids


def _resolve(positions, n):
    out = []
    for p in positions:
        q = p if p >= 0 else n + p
        if 0 <= q < n and q not in out:
            out.append(q)
    return out


@torch.no_grad()
def probe_checkpoint(lm, token_ids, positions=(0, 7, -1), decode_steps: int = 16) -> dict:
    """``lm``: a :class:`eredu_b200.api.LoadedModel`. The last ``decode_steps`` tokens are fed one at a time after a
    prefill of the rest (teacher forcing); each of those steps is also recomputed by a full pass over its prefix."""
    from ..models.llama import ForwardBatch  # noqa: F401  (documented dependency: the engine's batch description)

    ids = [int(t) for t in token_ids]
    n_prefill = len(ids) - decode_steps
    if n_prefill < 1:
        raise ValueError("need at least one prompt token before the teacher-forced steps")
    eng = lm.engine
    rows = _resolve(positions, n_prefill)
    prefill = {}
    for r in rows:                                     # one pass per sampled row keeps the engine API small
        seq = eng.new_sequence(ids[:r + 1], max_new_tokens=1)
        prefill[r] = eng.feed_logits(seq, ids[:r + 1]).float().cpu()
        eng.release(seq)
    seq = eng.new_sequence(ids[:n_prefill], max_new_tokens=decode_steps + 1)
    eng.feed_logits(seq, ids[:n_prefill])
    decode = [eng.step_logits(seq, t).float().cpu() for t in ids[n_prefill:]]
    eng.release(seq)
    recompute = {}
    for i in (0, decode_steps - 1):
        if 0 <= i < decode_steps:
            s2 = eng.new_sequence(ids[:n_prefill + i + 1], max_new_tokens=1)
            recompute[i] = eng.feed_logits(s2, ids[:n_prefill + i + 1]).float().cpu()
            eng.release(s2)
    return {"token_ids": ids, "prefill": prefill, "decode": decode, "recompute": recompute}


@torch.no_grad()
def probe_reference(model, token_ids, positions=(0, 7, -1), decode_steps: int = 16) -> dict:
    """``model``: a Transformers causal LM (any device / dtype). One full forward gives every row."""
    ids = [int(t) for t in token_ids]
    n_prefill = len(ids) - decode_steps
    dev = next(model.parameters()).device
    logits = model(torch.tensor([ids], device=dev)).logits[0].float().cpu()
    rows = _resolve(positions, n_prefill)
    return {"token_ids": ids, "prefill": {r: logits[r] for r in rows},
            "decode": [logits[n_prefill + i] for i in range(decode_steps)], "recompute": {}}
