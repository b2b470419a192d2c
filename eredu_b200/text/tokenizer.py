"""Tokenizers and their sidecar files.

* Hugging Face directories: ``tokenizer.json`` (+ ``tokenizer_config.json``, ``chat_template.jinja``,
  ``generation_config.json``, ``special_tokens_map.json``) - discovery rules of eredu/src/api/tokenizer.rs and
  api/metadata.rs (eredu/src/api/loaded.rs:637-709).
* GGUF files: a tokenizer rebuilt from ``tokenizer.ggml.*`` metadata (eredu-text/src/gguf.rs:31-90): byte-level BPE
  (``gpt2``) from tokens + merges, SentencePiece-style unigram (``llama``) from tokens + scores.
* ``TextDecoder``: incremental detokeniser that never emits half a UTF-8 sequence (eredu/src/api/portable.rs).
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional


@dataclass
class TokenizerBundle:
    tokenizer: object                      # tokenizers.Tokenizer
    chat_template: Optional[str] = None
    bos_token: Optional[str] = None
    eos_token: Optional[str] = None
    eos_ids: tuple = ()
    bos_id: Optional[int] = None
    add_bos: bool = False
    generation_config: dict = field(default_factory=dict)

    def encode(self, text: str, add_special_tokens: bool = True) -> list[int]:
        ids = self.tokenizer.encode(text, add_special_tokens=False).ids
        if add_special_tokens and self.add_bos and self.bos_id is not None and (not ids or ids[0] != self.bos_id):
            ids = [self.bos_id] + ids
        return ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return self.tokenizer.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def token_to_id(self, tok: str) -> Optional[int]:
        return self.tokenizer.token_to_id(tok)

    def vocab_size(self) -> int:
        return self.tokenizer.get_vocab_size(with_added_tokens=True)

    def fingerprint(self) -> str:
        """Stable hash of the vocabulary (prompt caches and constraint tables are keyed by it)."""
        vocab = sorted(self.tokenizer.get_vocab(with_added_tokens=True).items(), key=lambda kv: kv[1])
        h = hashlib.sha256()
        for tok, i in vocab:
            h.update(f"{i}\t{tok}\n".encode("utf-8", "surrogatepass"))
        return h.hexdigest()


def _token_text(v):
    if isinstance(v, dict):
        return v.get("content")
    return v


def _load_hf(path: Path) -> TokenizerBundle:
    from tokenizers import Tokenizer

    if (path / "tokenizer.json").exists():
        tok = Tokenizer.from_file(str(path / "tokenizer.json"))
    else:   # rank-ordered tiktoken vocabulary (Kimi): converted to the same fast byte-level BPE representation
        from .tiktoken_import import load_tiktoken_dir

        tok = load_tiktoken_dir(path)
    cfg = {}
    if (path / "tokenizer_config.json").exists():
        cfg = json.loads((path / "tokenizer_config.json").read_text())
    template = cfg.get("chat_template")
    if isinstance(template, list):  # named templates: [{"name": "default", "template": ...}, ...]
        named = {t.get("name"): t.get("template") for t in template}
        template = named.get("default") or next(iter(named.values()), None)
    for cand in ("chat_template.jinja", "chat_template.json"):
        f = path / cand
        if f.exists():
            text = f.read_text()
            template = json.loads(text).get("chat_template") if cand.endswith(".json") else text
            break
    gen = json.loads((path / "generation_config.json").read_text()) if (path / "generation_config.json").exists() else {}
    model_cfg = json.loads((path / "config.json").read_text()) if (path / "config.json").exists() else {}
    bos, eos = _token_text(cfg.get("bos_token")), _token_text(cfg.get("eos_token"))
    eos_ids: list[int] = []
    for source in (gen.get("eos_token_id"), model_cfg.get("eos_token_id")):
        if source is None:
            continue
        for e in (source if isinstance(source, list) else [source]):
            if e not in eos_ids:
                eos_ids.append(int(e))
    if eos is not None and tok.token_to_id(eos) is not None and tok.token_to_id(eos) not in eos_ids:
        eos_ids.append(tok.token_to_id(eos))
    return TokenizerBundle(tok, template, bos, eos, tuple(eos_ids), tok.token_to_id(bos) if bos else None,
                           bool(cfg.get("add_bos_token", False)), gen)


def _gguf_tokenizer(md: dict) -> TokenizerBundle:
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers

    tokens = md.get("tokenizer.ggml.tokens")
    if not tokens:
        raise ValueError("GGUF file carries no tokenizer")
    kind = md.get("tokenizer.ggml.model", "llama")
    types = md.get("tokenizer.ggml.token_type") or [1] * len(tokens)
    if kind == "gpt2":
        merges = [tuple(m.split(" ", 1)) for m in md.get("tokenizer.ggml.merges", [])]
        vocab = {t: i for i, t in enumerate(tokens)}
        tok = Tokenizer(models.BPE(vocab=vocab, merges=merges, fuse_unk=False))
        tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
        tok.decoder = decoders.ByteLevel()
    else:
        scores = md.get("tokenizer.ggml.scores") or [0.0] * len(tokens)
        unk = md.get("tokenizer.ggml.unknown_token_id", 0)
        tok = Tokenizer(models.Unigram([(t, float(s)) for t, s in zip(tokens, scores)], unk_id=int(unk), byte_fallback=True))
        tok.pre_tokenizer = pre_tokenizers.Metaspace(replacement="▁", prepend_scheme="first")
        tok.decoder = decoders.Sequence([decoders.Replace("▁", " "), decoders.ByteFallback(), decoders.Fuse(),
                                         decoders.Strip(" ", 1, 0)])
    special = [t for t, ty in zip(tokens, types) if ty in (3, 4)]  # control / user-defined
    if special:
        from tokenizers import AddedToken

        tok.add_special_tokens([AddedToken(t, special=True, normalized=False) for t in special])
    bos_id, eos_id = md.get("tokenizer.ggml.bos_token_id"), md.get("tokenizer.ggml.eos_token_id")
    eos_ids = [int(eos_id)] if eos_id is not None else []
    eot = md.get("tokenizer.ggml.eot_token_id")
    if eot is not None and int(eot) not in eos_ids:
        eos_ids.append(int(eot))
    return TokenizerBundle(tok, md.get("tokenizer.chat_template"),
                           tokens[bos_id] if bos_id is not None else None, tokens[eos_id] if eos_id is not None else None,
                           tuple(eos_ids), int(bos_id) if bos_id is not None else None,
                           bool(md.get("tokenizer.ggml.add_bos_token", kind != "gpt2")), {})


def load_tokenizer(path, source=None) -> TokenizerBundle:
    path = Path(path)
    if path.is_dir() and ((path / "tokenizer.json").exists() or (path / "tiktoken.model").exists()):
        return _load_hf(path)
    md = getattr(source, "metadata", None)
    if md is not None:
        return _gguf_tokenizer(md)
    if path.is_file() and (path.parent / "tokenizer.json").exists():
        return _load_hf(path.parent)
    raise FileNotFoundError(f"no tokenizer found for {path}")


class TextDecoder:
    """Incremental detokeniser: ``push(token_id)`` returns the newly completed text. Text is only released when
    it cannot change any more: a trailing replacement character (an incomplete UTF-8 sequence from byte tokens)
    is held back until the following tokens complete it."""

    def __init__(self, bundle: TokenizerBundle, skip_special_tokens: bool = True):
        self.bundle = bundle
        self.skip = skip_special_tokens
        self.ids: list[int] = []
        self.prefix_index = 0   # first token of the window that is re-decoded
        self.read_index = 0     # tokens before this index are fully emitted

    def push(self, token_id: int) -> str:
        self.ids.append(int(token_id))
        prev = self.bundle.decode(self.ids[self.prefix_index:self.read_index], self.skip)
        cur = self.bundle.decode(self.ids[self.prefix_index:], self.skip)
        if cur.endswith("�") or len(cur) <= len(prev):
            return ""
        out = cur[len(prev):]
        self.prefix_index = self.read_index
        self.read_index = len(self.ids)
        return out

    def flush(self) -> str:
        prev = self.bundle.decode(self.ids[self.prefix_index:self.read_index], self.skip)
        cur = self.bundle.decode(self.ids[self.prefix_index:], self.skip)
        self.read_index = len(self.ids)
        return cur[len(prev):] if len(cur) > len(prev) else ""
