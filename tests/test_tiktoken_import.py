"""tiktoken.model import: rank file validation, merge recovery, byte-exact agreement with the rank-ordered BPE."""
import base64
import json

import pytest

from eredu_b200.text.tiktoken_import import TiktokenError, build_tokenizer, byte_alphabet, load_tiktoken_dir, read_ranks
from eredu_b200.text.tokenizer import load_tokenizer


def toy_ranks():
    ranked = [bytes([b]) for b in range(256)]
    for tok in (b"th", b"he", b"in", b" t", b"the", b" th", b" the", b"er", b"ing", b"\xe4\xb8", b"\xe4\xb8\x96", b"  ",
                b"12", b"123", b"wor", b"ld", b"world", b" world", b"'s"):
        ranked.append(tok)
    return ranked


def write_model(path, ranked):
    path.write_text("\n".join(f"{base64.b64encode(t).decode()} {r}" for r, t in enumerate(ranked)) + "\n")


def rank_bpe(ranks, piece: bytes) -> list[int]:
    """tiktoken's algorithm: keep merging the adjacent pair whose concatenation has the lowest rank."""
    parts = [bytes([b]) for b in piece]
    while len(parts) > 1:
        best = None
        for i in range(len(parts) - 1):
            r = ranks.get(parts[i] + parts[i + 1])
            if r is not None and (best is None or r < best[0]):
                best = (r, i)
        if best is None:
            break
        parts[best[1]:best[1] + 2] = [parts[best[1]] + parts[best[1] + 1]]
    return [ranks[p] for p in parts]


def test_rank_file_validation(tmp_path):
    ranked = toy_ranks()
    f = tmp_path / "tiktoken.model"
    write_model(f, ranked)
    assert read_ranks(f) == ranked
    f.write_text("YQ== 0\nYg== 2\n")
    with pytest.raises(TiktokenError, match="missing rank 1"):
        read_ranks(f)
    f.write_text("YQ== 0\nYg== 0\n")
    with pytest.raises(TiktokenError, match="duplicate"):
        read_ranks(f)
    f.write_text("!!! 0\n")
    with pytest.raises(TiktokenError):
        read_ranks(f)
    alpha = byte_alphabet()
    assert len(set(alpha)) == 256 and alpha[ord("a")] == "a" and alpha[32] == "Ġ"


def test_imported_tokenizer_matches_rank_bpe(tmp_path):
    ranked = toy_ranks()
    ranks = {t: r for r, t in enumerate(ranked)}
    tk = build_tokenizer(ranked)
    for piece in (b"the", b" the", b"thing", b" world", b"other", b"ing", b"123"):
        ids = tk.encode(piece.decode()).ids
        assert ids == rank_bpe(ranks, piece), piece
    text = "the world's thing is in 世界 12345 other  things\n"
    enc = tk.encode(text)
    assert tk.decode(enc.ids) == text
    assert b"".join(ranked[i] for i in enc.ids).decode() == text


def test_directory_loader_with_special_tokens(tmp_path):
    ranked = toy_ranks()
    write_model(tmp_path / "tiktoken.model", ranked)
    n = len(ranked)
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({
        "added_tokens_decoder": {str(n): {"content": "<|im_end|>"}, str(n + 1): {"content": "<|im_user|>"}},
        "eos_token": "<|im_end|>", "chat_template": "{{ messages[0].content }}"}))
    tk = load_tiktoken_dir(tmp_path)
    assert tk.token_to_id("<|im_end|>") == n and tk.encode("the<|im_user|>").ids[-1] == n + 1
    b = load_tokenizer(tmp_path)
    assert n in b.eos_ids and b.chat_template and b.decode(b.encode("the thing")) == "the thing"
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"added_tokens_decoder": {str(n + 5): {"content": "<x>"}}}))
    with pytest.raises(TiktokenError, match="continue the vocabulary"):
        load_tiktoken_dir(tmp_path)
