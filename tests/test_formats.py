"""GGUF / SafeTensors codecs and quantisers (host C++ runtime) against byte-exact oracle vectors and round trips."""
import json
import os

import numpy as np
import pytest
import torch

from eredu_b200.lib import _eredu_host as H

FIX = os.path.join(os.path.dirname(__file__), "fixtures")


def _parse_field(field):
    name, shape, dtype, hexdata = field.split(":")
    shape = json.loads(shape)
    raw = bytes.fromhex(hexdata)
    dt = {"Uint32": "<u4", "Float16": "<f2", "Float32": "<f4"}[dtype]
    return name, np.frombuffer(raw, dtype=dt).reshape(shape)


def _oracle_cases():
    with open(os.path.join(FIX, "mlx-v0.32.0.oracle")) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            parts = line.split("|")
            yield int(parts[0]), bytes.fromhex(parts[1]), dict(_parse_field(p) for p in parts[2:])


@pytest.mark.parametrize("code,raw,fields", list(_oracle_cases()), ids=lambda v: str(v) if isinstance(v, int) else "")
def test_affine_conversion_matches_oracle_bytes(code, raw, fields):
    """Raw GGML blocks -> packed u32 / f16 scales / f16 biases must be byte-exact."""
    w = fields["oracle.weight"]
    if w.dtype != np.uint32:  # Q5_0 / Q5_1 in this fixture: dense f16 expectation
        rows, cols = w.shape
        ours = H.ggml_dequantize(code, raw, rows * cols).reshape(rows, cols)
        assert np.all(np.abs(ours - w.astype(np.float32)) <= 4 * np.spacing(np.abs(w)).astype(np.float32) + 1e-6)
        return
    deq = fields["oracle.dequantized"].astype(np.float32)
    rows, cols = deq.shape
    ours = H.ggml_dequantize(code, raw, rows * cols).reshape(rows, cols)
    # the fixture's dequantised values come from the affine form (f16 scales / biases): the direct block decode
    # differs by the f16 rounding of scale * 2^bits
    assert np.all(np.abs(ours - deq) <= 0.02 * np.abs(deq) + 0.02 * np.abs(deq).max() / 16 + 1e-6)
    w = fields["oracle.weight"]
    if w.dtype == np.uint32:
        packed, scales, biases, bits, group = H.ggml_to_affine(code, raw, rows, cols)
        assert packed.tobytes() == w.tobytes()
        assert scales.tobytes() == fields["oracle.scales"].view(np.uint16).tobytes()
        assert biases.tobytes() == fields["oracle.biases"].view(np.uint16).tobytes()
        # the fixture dequantises in f16 arithmetic (scale * q rounded to f16, then + bias): reproduce it exactly
        q = H.unpack_codes(packed, bits).astype(np.float16)
        f16 = np.repeat(scales.view(np.float16), group, 1) * q + np.repeat(biases.view(np.float16), group, 1)
        assert np.array_equal(f16.astype(np.float32), deq)


def test_gguf_round_trip_with_metadata_and_shapes(tmp_path):
    rng = np.random.default_rng(0)
    w = H.GgufWriter(32)
    w.add_metadata("general.architecture", "llama")
    w.add_metadata("llama.block_count", 2)
    w.add_metadata("llama.rope.freq_base", 10000.0)
    w.add_metadata("tokenizer.ggml.tokens", ["a", "b", "<s>"])
    w.add_metadata("llama.attention.head_count_kv", [2, 2], "i32")
    w.add_metadata("flag", True)
    a = rng.standard_normal((6, 64)).astype(np.float32)
    b = rng.standard_normal((4, 256)).astype(np.float32)
    w.add_tensor("a", [6, 64], 0, a)
    w.add_tensor("b.q8", [4, 256], 8, np.frombuffer(H.ggml_quantize(8, b), dtype=np.uint8))
    w.add_tensor("b.q4k", [4, 256], 12, np.frombuffer(H.ggml_quantize(12, b), dtype=np.uint8))
    w.add_tensor("b.q6k", [4, 256], 14, np.frombuffer(H.ggml_quantize(14, b), dtype=np.uint8))
    path = str(tmp_path / "m.gguf")
    w.write(path)
    r = H.GgufReader(path)
    md = r.metadata
    assert md["general.architecture"] == "llama" and md["llama.block_count"] == 2 and md["flag"] is True
    assert md["tokenizer.ggml.tokens"] == ["a", "b", "<s>"] and md["llama.attention.head_count_kv"] == [2, 2]
    assert r.version == 3 and not r.big_endian
    infos = {t["name"]: t for t in r.tensors()}
    assert infos["a"]["shape"] == [6, 64] and infos["b.q4k"]["type_name"] == "Q4_K"
    assert np.array_equal(r.dequantize("a"), a)
    for name, tol in (("b.q8", 0.02), ("b.q4k", 0.2), ("b.q6k", 0.06)):
        d = r.dequantize(name)
        assert d.shape == (4, 256)
        assert np.abs(d - b).max() < tol * np.abs(b).max(), name
    packed, scales, biases, bits, group = r.to_affine("b.q4k")
    assert (bits, group) == (4, 32) and packed.shape == (4, 32)
    back = H.affine_dequantize(packed, scales.view(np.float16).astype(np.float32),
                               biases.view(np.float16).astype(np.float32), bits, group)
    assert np.abs(back - r.dequantize("b.q4k")).max() < 2e-2


def test_gguf_sharded_set(tmp_path):
    for i in (1, 2):
        w = H.GgufWriter()
        w.add_metadata("general.architecture", "llama")
        w.add_metadata("split.no", i - 1, "u16")
        w.add_metadata("split.count", 2, "u16")
        w.add_metadata("split.tensors.count", 2, "i32")
        w.add_tensor(f"t{i}", [2, 32], 0, np.full((2, 32), float(i), dtype=np.float32))
        w.write(str(tmp_path / f"m-{i:05d}-of-00002.gguf"))
    r = H.GgufReader(str(tmp_path / "m-00001-of-00002.gguf"))
    assert r.shard_count == 2 and r.has("t1") and r.has("t2")
    assert float(r.dequantize("t2")[0, 0]) == 2.0


def test_gguf_rejects_malformed(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGUX" + b"\0" * 64)
    with pytest.raises(RuntimeError):
        H.GgufReader(str(p))
    p.write_bytes(b"GGUF" + (3).to_bytes(4, "little") + (1 << 40).to_bytes(8, "little") + b"\0" * 8)
    with pytest.raises(RuntimeError):
        H.GgufReader(str(p))


def test_safetensors_store_round_trip_and_bounded_mapping(tmp_path):
    rng = np.random.default_rng(1)
    files = {}
    weight_map = {}
    for s in range(6):
        name = f"model-{s + 1:05d}-of-00006.safetensors"
        a = rng.standard_normal((8, 16)).astype(np.float32)
        b = rng.integers(0, 2 ** 16, (4, 8)).astype(np.uint16)
        H.write_safetensors(str(tmp_path / name), [(f"a{s}", "F32", [8, 16], a), (f"b{s}", "BF16", [4, 8], b)],
                            {"format": "pt"})
        files[s] = (a, b)
        weight_map[f"a{s}"] = name
        weight_map[f"b{s}"] = name
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    st = H.SafetensorsStore(str(tmp_path), 2)
    assert sorted(st.keys()) == sorted(weight_map)
    assert st.diagnostics()["mapped_shards"] == 0  # header-only inspection maps nothing
    views = []
    for s in range(6):
        a = st.tensor(f"a{s}")
        assert np.array_equal(a, files[s][0]) and not a.flags.writeable
        assert st.info(f"b{s}")["dtype"] == "BF16"
        assert np.array_equal(st.tensor(f"b{s}"), files[s][1])
        views.append(a)
    d = st.diagnostics()
    assert d["mapped_shards"] == 2 and d["map_events"] == 6 and d["unmap_events"] == 4
    assert np.array_equal(views[0], files[0][0])  # evicted from the cache, still valid while referenced
    assert np.array_equal(st.rows("a3", 2, 5), files[3][0][2:5])
    assert st.metadata(0)["format"] == "pt"
    # compatible with the reference python implementation when it is installed
    try:
        from safetensors.numpy import load_file
    except Exception:
        return
    H.write_safetensors(str(tmp_path / "plain.safetensors"), [("a0", "F32", [8, 16], files[0][0])], {})
    ref = load_file(str(tmp_path / "plain.safetensors"))
    assert np.array_equal(ref["a0"], files[0][0])


@pytest.mark.parametrize("bits,group", [(4, 64), (8, 32), (3, 32), (6, 16), (2, 16), (5, 128), (4, 32)])
def test_affine_quantize_round_trip(bits, group):
    rng = np.random.default_rng(bits * 100 + group)
    w = (rng.standard_normal((16, 256)) * 0.05).astype(np.float32)
    packed, scales, biases = H.affine_quantize(w, bits, group, "bf16")
    assert packed.shape == (16, 256 * bits // 32) and scales.shape == (16, 256 // group)
    back = H.affine_dequantize(packed, scales, biases, bits, group)
    step = (w.reshape(16, -1, group).max(-1) - w.reshape(16, -1, group).min(-1)) / (2 ** bits - 1)
    err = np.abs(back - w).reshape(16, -1, group).max(-1)
    # edge-anchored scales can push the far extreme one code past the grid: at most ~one step
    span = w.reshape(16, -1, group).max(-1) - w.reshape(16, -1, group).min(-1)
    assert np.all(err <= 1.05 * step + 2.0 ** -7 * span + 1e-6)  # + bf16 rounding of the stored scale
    assert np.mean(err <= 0.6 * step + 2e-3 * np.abs(w).max()) > 0.5
    # the larger-magnitude extreme of every group is represented (almost) exactly
    wg = w.reshape(16, -1, group)
    edge = np.where(np.abs(wg.min(-1)) > np.abs(wg.max(-1)), wg.min(-1), wg.max(-1))
    bg = back.reshape(16, -1, group)
    rep = np.where(np.abs(wg.min(-1)) > np.abs(wg.max(-1)), bg.min(-1), bg.max(-1))
    assert np.all(np.abs(rep - edge) <= 1e-2 * np.abs(edge) + 1e-6)


def test_mxfp4_round_trip():
    rng = np.random.default_rng(5)
    w = rng.standard_normal((8, 128)).astype(np.float32)
    packed, scales = H.mxfp4_quantize(w)
    assert packed.shape == (8, 16) and scales.shape == (8, 4) and scales.dtype == np.uint8
    back = H.mxfp4_dequantize(packed, scales)
    amax = np.abs(w.reshape(8, 4, 32)).max(-1, keepdims=True)
    assert np.all(np.abs(back.reshape(8, 4, 32) - w.reshape(8, 4, 32)) <= 0.26 * amax + 1e-6)
    exact = np.array([[0.5, -1.0, 1.5, 2.0, -3.0, 4.0, 6.0, 0.0] * 4], dtype=np.float32)
    p, s = H.mxfp4_quantize(exact)
    assert np.array_equal(H.mxfp4_dequantize(p, s), exact)


def test_quantize_checkpoint_tool_round_trip(tmp_path):
    """quantize_checkpoint writes MLX-LM packed tensors + both config keys; the packed directory loads and runs, its
    dense reading equals the host dequantiser, already-packed sources are refused."""
    import dataclasses
    import json

    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.formats.quantize import eligible, quantize_checkpoint
    from eredu_b200.lib import _eredu_host as H
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import random_state

    cfg = dataclasses.replace(C.tiny_llama(), vocab_size=512, intermediate_size=704)
    sd = random_state(cfg, seed=0, std=0.05)
    ck.save_safetensors_checkpoint(tmp_path / "src", cfg, sd, torch.float32)
    rep = quantize_checkpoint(tmp_path / "src", tmp_path / "q4", bits=4, group_size=64)
    assert rep["quantized"] == cfg.num_hidden_layers * 7 and rep["bytes_after"] < rep["bytes_before"]
    qcfg = json.loads((tmp_path / "q4" / "config.json").read_text())
    assert qcfg["quantization"] == qcfg["quantization_config"] == {"group_size": 64, "bits": 4, "mode": "affine"}
    src = ck.open_checkpoint(tmp_path / "q4")
    name = "model.layers.0.mlp.down_proj.weight"
    packed, scales, biases, bits, group = src.to_affine(name)
    assert packed.shape == (cfg.hidden_size, cfg.intermediate_size * 4 // 32) and (bits, group) == (4, 64)
    hp, hs, hb = H.affine_quantize(sd[name].numpy(), 4, 64, "f16")
    assert np.array_equal(packed.numpy().view(np.uint32), hp)
    dense = src.get(name)
    assert float((dense - sd[name]).abs().max()) < float(sd[name].abs().max()) / 7       # within one 4-bit step
    assert torch.equal(src.get("model.norm.weight"), sd["model.norm.weight"])              # norms stay dense
    assert not eligible("model.embed_tokens.weight", (512, 256), "F32", 64) and not eligible("x.weight", (8, 48), "F32", 64)
    lm = LoadedModel.load(tmp_path / "q4", ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    assert len(lm.generate([list(range(10))], None, 5)[0]) == 5
    with pytest.raises(ValueError):
        quantize_checkpoint(tmp_path / "q4", tmp_path / "again")
