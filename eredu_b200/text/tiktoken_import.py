"""Import a rank-ordered tiktoken byte-BPE file (``tiktoken.model``: one ``base64(token bytes) rank`` pair per line)
as a fast ``tokenizers`` BPE tokenizer.

Counterpart of eredu-text/src/tiktoken.rs (the Kimi / K2 loader): the vocabulary is the ranked byte strings spelled in
the GPT-2 byte alphabet; the merge list is recovered by splitting every multi-byte token with the merges of lower rank
only - when exactly two parts remain, that pair is the merge that creates the token; special tokens come from
``tokenizer_config.json``'s ``added_tokens_decoder`` and must continue the id space.
"""
from __future__ import annotations

import base64
import json
from pathlib import Path

# Pre-tokenisation expression published with the Kimi-K2 tokenizer (Han runs, cased words with English contractions,
# digit groups of up to three, punctuation runs, newlines, trailing whitespace).
KIMI_K2_PATTERN = "|".join([
    r"[\p{Han}]+",
    r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}&&[^\p{Han}]]*[\p{Ll}\p{Lm}\p{Lo}\p{M}&&[^\p{Han}]]+(?i:'s|'t|'re|'ve|'m|'ll|'d)?",
    r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}&&[^\p{Han}]]+[\p{Ll}\p{Lm}\p{Lo}\p{M}&&[^\p{Han}]]*(?i:'s|'t|'re|'ve|'m|'ll|'d)?",
    r"\p{N}{1,3}",
    r" ?[^\s\p{L}\p{N}]+[\r\n]*",
    r"\s*[\r\n]+",
    r"\s+(?!\S)",
    r"\s+",
])


class TiktokenError(ValueError):
    pass


def read_ranks(path) -> list[bytes]:
    """Token bytes by rank; every rank from 0 to the largest must appear exactly once."""
    ranked: dict[int, bytes] = {}
    for n, line in enumerate(Path(path).read_text().splitlines(), 1):
        fields = line.split()
        if not fields:
            continue
        if len(fields) != 2:
            raise TiktokenError(f"line {n}: expected '<base64 token> <rank>'")
        try:
            token = base64.b64decode(fields[0], validate=True)
            rank = int(fields[1])
        except Exception as e:
            raise TiktokenError(f"line {n}: {e}") from None
        if not token:
            raise TiktokenError(f"line {n}: empty token")
        if rank < 0 or rank in ranked:
            raise TiktokenError(f"line {n}: duplicate or negative rank {rank}")
        ranked[rank] = token
    out = []
    for r in range(len(ranked)):
        if r not in ranked:
            raise TiktokenError(f"missing rank {r}")
        out.append(ranked[r])
    return out


def byte_alphabet() -> list[str]:
    """GPT-2 byte -> printable character table (the alphabet of byte-level BPE vocabularies)."""
    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    table = {b: chr(b) for b in keep}
    extra = 0
    for b in range(256):
        if b not in table:
            table[b] = chr(256 + extra)
            extra += 1
    return [table[b] for b in range(256)]


def _split_with_lower_ranks(ranks: dict, token: bytes, limit: int) -> list[bytes]:
    parts = [bytes([b]) for b in token]
    while len(parts) > 1:
        best = None
        for i in range(len(parts) - 1):
            r = ranks.get(parts[i] + parts[i + 1])
            if r is not None and r < limit and (best is None or r < best[0]):
                best = (r, i)
        if best is None:
            break
        i = best[1]
        parts[i:i + 2] = [parts[i] + parts[i + 1]]
    return parts


def build_tokenizer(ranked: list[bytes], pattern: str = KIMI_K2_PATTERN, special_tokens=()):
    """``tokenizers.Tokenizer`` for the ranked vocabulary. ``special_tokens``: (id, text) pairs continuing the ids."""
    from tokenizers import AddedToken, Regex, Tokenizer, decoders, models, pre_tokenizers

    alpha = byte_alphabet()
    spell = lambda bs: "".join(alpha[b] for b in bs)                                   # noqa: E731
    ranks = {tok: r for r, tok in enumerate(ranked)}
    vocab = {spell(tok): r for r, tok in enumerate(ranked)}
    if len(vocab) != len(ranked):
        raise TiktokenError("two ranks spell the same token")
    merges = []
    for r, tok in enumerate(ranked):
        if len(tok) > 1:
            parts = _split_with_lower_ranks(ranks, tok, r)
            if len(parts) == 2:
                merges.append((spell(parts[0]), spell(parts[1])))
    tk = Tokenizer(models.BPE(vocab=vocab, merges=merges))
    tk.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(pattern), behavior="isolated", invert=False),
        pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False),
    ])
    tk.decoder = decoders.ByteLevel()
    base = len(ranked)
    specials = sorted(special_tokens)
    for i, (tid, text) in enumerate(specials):
        if tid != base + i:
            raise TiktokenError(f"special token {text!r} has id {tid}, expected {base + i}: ids must continue the vocabulary")
    if specials:
        tk.add_special_tokens([AddedToken(text, special=True, normalized=False) for _, text in specials])
    return tk


def load_tiktoken_dir(path):
    """Tokenizer from a checkpoint directory holding ``tiktoken.model`` (+ ``tokenizer_config.json``)."""
    path = Path(path)
    ranked = read_ranks(path / "tiktoken.model")
    specials = []
    cfg_path = path / "tokenizer_config.json"
    if cfg_path.exists():
        cfg = json.loads(cfg_path.read_text())
        for tid, ent in (cfg.get("added_tokens_decoder") or {}).items():
            specials.append((int(tid), ent["content"] if isinstance(ent, dict) else str(ent)))
    return build_tokenizer(ranked, special_tokens=specials)
