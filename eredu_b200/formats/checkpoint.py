"""Checkpoint I/O: Hugging Face-style SafeTensors directories and (sharded) GGUF files.

Tensor names, GGUF <-> HF name translation and metadata keys follow eredu-architectures/src/llama/
checkpoint.rs:19-123,236-343 and llama/config.rs:206-312; Qwen3-MoE GGUF names follow
eredu/src/backend/mlx/architectures/qwen/dense.rs:3203-3267.

GGUF Llama files store Q/K projection rows in llama.cpp's permuted order (pairs interleaved for its RoPE).
The reference keeps that order and switches to interleaved RoPE (llama/config.rs:295); here the rows are put
back into Hugging Face order when the tensor is read, so both checkpoint kinds run the *same* arithmetic and
give bit-identical logits.
"""
from __future__ import annotations

import json
import os
import re
from pathlib import Path
from typing import Callable, Optional

import numpy as np
import torch

from ..lib import _eredu_host as H
from ..models.config import ModelConfig

GGML = {"F32": 0, "F16": 1, "Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q8_0": 8, "Q2_K": 10, "Q3_K": 11, "Q4_K": 12,
        "Q5_K": 13, "Q6_K": 14, "BF16": 30, "MXFP4": 39}
GGML_NAME = {v: k for k, v in GGML.items()}

_ST_DTYPES = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.int32: "I32",
              torch.int64: "I64", torch.uint8: "U8", torch.int8: "I8", torch.bool: "BOOL", torch.float64: "F64",
              torch.int16: "I16", torch.float8_e4m3fn: "F8_E4M3"}
_ST_TO_TORCH = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I32": torch.int32,
                "I64": torch.int64, "U8": torch.uint8, "I8": torch.int8, "BOOL": torch.bool, "F64": torch.float64,
                "I16": torch.int16, "U32": torch.int32, "U16": torch.int16, "F8_E4M3": torch.float8_e4m3fn,
                "F8_E5M2": torch.float8_e5m2, "F8_E8M0": torch.uint8, "F4": torch.uint8}

# ---------------------------------------------------------------------------------------------- names
_LAYER_MAP = {
    "input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm",
    "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v",
    "self_attn.o_proj": "attn_output", "self_attn.q_norm": "attn_q_norm", "self_attn.k_norm": "attn_k_norm",
    "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down", "mlp.gate": "ffn_gate_inp",
}
_LAYER_MAP_INV = {v: k for k, v in _LAYER_MAP.items()}


def hf_to_gguf_name(name: str) -> Optional[str]:
    if name == "model.embed_tokens.weight":
        return "token_embd.weight"
    if name == "model.norm.weight":
        return "output_norm.weight"
    if name == "lm_head.weight":
        return "output.weight"
    m = re.match(r"model\.layers\.(\d+)\.(.+)\.(weight|bias)$", name)
    if not m:
        return None
    li, mid, kind = m.groups()
    if mid in _LAYER_MAP:
        return f"blk.{li}.{_LAYER_MAP[mid]}.{kind}"
    return None


def gguf_to_hf_name(name: str) -> Optional[str]:
    if name == "token_embd.weight":
        return "model.embed_tokens.weight"
    if name == "output_norm.weight":
        return "model.norm.weight"
    if name == "output.weight":
        return "lm_head.weight"
    m = re.match(r"blk\.(\d+)\.(.+)\.(weight|bias)$", name)
    if not m:
        return None
    li, mid, kind = m.groups()
    if mid in _LAYER_MAP_INV:
        return f"model.layers.{li}.{_LAYER_MAP_INV[mid]}.{kind}"
    return None


def permute_qk_to_ggml(w: torch.Tensor, n_head: int) -> torch.Tensor:
    """HF (split-half) row order -> llama.cpp (interleaved) row order."""
    rows = w.shape[0]
    rest = w.shape[1:]
    return w.reshape(n_head, 2, rows // n_head // 2, *rest).transpose(1, 2).reshape(rows, *rest)


def permute_qk_from_ggml(w: torch.Tensor, n_head: int) -> torch.Tensor:
    rows = w.shape[0]
    rest = w.shape[1:]
    return w.reshape(n_head, rows // n_head // 2, 2, *rest).transpose(1, 2).reshape(rows, *rest)


def _qk_row_index(rows: int, n_head: int) -> torch.Tensor:
    """Row gather index that undoes the llama.cpp permutation (usable on any per-row payload)."""
    return permute_qk_from_ggml(torch.arange(rows), n_head)


# ---------------------------------------------------------------------------------------------- writers
def _np(t: torch.Tensor):
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def save_safetensors_checkpoint(path: str | Path, cfg: ModelConfig, state: dict, dtype=torch.float32,
                                shard_bytes: Optional[int] = None, extra_files: Optional[dict] = None) -> None:
    """Write ``config.json`` + ``model.safetensors`` (or an indexed shard set when ``shard_bytes`` is given)."""
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    d = cfg.to_hf_dict()
    d["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16", torch.float16: "float16"}[dtype]
    (path / "config.json").write_text(json.dumps(d, indent=1))
    items = []
    for name, t in state.items():
        if (t.is_floating_point() and t.dtype not in (dtype, torch.float8_e4m3fn)
                and not name.endswith((".scales", ".biases", ".weight_scale_inv", ".weight_scale"))):
            t = t.to(dtype)
        items.append((name, _ST_DTYPES[t.dtype], list(t.shape), _np(t)))
    if shard_bytes is None:
        H.write_safetensors(str(path / "model.safetensors"), items, {"format": "pt"})
    else:
        shards, cur, cur_b = [], [], 0
        for it in items:
            nb = it[3].nbytes
            if cur and cur_b + nb > shard_bytes:
                shards.append(cur)
                cur, cur_b = [], 0
            cur.append(it)
            cur_b += nb
        if cur:
            shards.append(cur)
        weight_map = {}
        for i, sh in enumerate(shards):
            fname = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
            H.write_safetensors(str(path / fname), sh, {"format": "pt"})
            for it in sh:
                weight_map[it[0]] = fname
        (path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    for name, content in (extra_files or {}).items():
        (path / name).write_text(content)


def save_gguf_checkpoint(path: str | Path, cfg: ModelConfig, state: dict, default_type: str = "F32",
                         type_for: Optional[Callable[[str], str]] = None, tokens: Optional[list] = None) -> None:
    """Write a GGUF v3 file of an HF-named state dict. Matrices are encoded as ``type_for(gguf_name)`` (or
    ``default_type``), vectors (norms, biases) stay F32. Q/K rows go out in llama.cpp's permuted order."""
    arch = {"llama": "llama", "mistral": "llama", "qwen2": "qwen2", "qwen3": "qwen3", "qwen3_moe": "qwen3moe"}[
        cfg.model_type]
    w = H.GgufWriter(32)
    w.add_metadata("general.architecture", arch)
    w.add_metadata("general.name", "eredu-b200-synthetic")
    w.add_metadata("general.alignment", 32)
    w.add_metadata(f"{arch}.block_count", cfg.num_hidden_layers)
    w.add_metadata(f"{arch}.context_length", cfg.max_position_embeddings)
    w.add_metadata(f"{arch}.embedding_length", cfg.hidden_size)
    w.add_metadata(f"{arch}.feed_forward_length", cfg.intermediate_size)
    w.add_metadata(f"{arch}.attention.head_count", cfg.num_attention_heads)
    w.add_metadata(f"{arch}.attention.head_count_kv", cfg.num_key_value_heads)
    w.add_metadata(f"{arch}.attention.key_length", cfg.head_dim)
    w.add_metadata(f"{arch}.attention.value_length", cfg.head_dim)
    w.add_metadata(f"{arch}.attention.layer_norm_rms_epsilon", float(cfg.rms_norm_eps))
    w.add_metadata(f"{arch}.rope.freq_base", float(cfg.rope_theta))
    w.add_metadata(f"{arch}.vocab_size", cfg.vocab_size)
    if cfg.is_moe:
        w.add_metadata(f"{arch}.expert_count", cfg.num_experts)
        w.add_metadata(f"{arch}.expert_used_count", cfg.num_experts_per_tok)
        w.add_metadata(f"{arch}.expert_feed_forward_length", cfg.moe_intermediate_size)
    if tokens is not None:
        w.add_metadata("tokenizer.ggml.model", "llama")
        w.add_metadata("tokenizer.ggml.tokens", list(tokens))
    permute = arch == "llama"

    def add(gname: str, t: torch.Tensor):
        t = t.detach().float().cpu().contiguous()
        typ = "F32"
        if t.dim() >= 2:
            typ = (type_for(gname) if type_for else None) or default_type
            elems, _ = H.ggml_block_geometry(GGML[typ])
            if t.shape[-1] % elems != 0:
                typ = "F32"
        w.add_tensor(gname, list(t.shape), GGML[typ], np.frombuffer(H.ggml_quantize(GGML[typ], t.numpy()),
                                                                     dtype=np.uint8))

    moe_acc: dict = {}
    for name, t in state.items():
        m = re.match(r"model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(gate|up|down)_proj\.weight$", name)
        if m:
            li, e, kind = int(m.group(1)), int(m.group(2)), m.group(3)
            moe_acc.setdefault((li, kind), {})[e] = t
            continue
        g = hf_to_gguf_name(name)
        if g is None:
            raise KeyError(f"no GGUF name for {name}")
        if permute and ".attn_q." in g:
            t = permute_qk_to_ggml(t, cfg.num_attention_heads)
        elif permute and ".attn_k." in g:
            t = permute_qk_to_ggml(t, cfg.num_key_value_heads)
        add(g, t)
    for (li, kind), experts in sorted(moe_acc.items()):
        stacked = torch.stack([experts[e] for e in range(len(experts))], 0)
        add(f"blk.{li}.ffn_{kind}_exps.weight", stacked)
    w.write(str(path))


# ---------------------------------------------------------------------------------------------- readers
class TensorSource:
    """Uniform, lazy view of a checkpoint: ``get(hf_name)`` -> CPU tensor, ``has(hf_name)``, ``raw(hf_name)`` for
    block-quantised GGUF payloads. Reads are zero-copy views of the memory-mapped file until converted."""

    def __init__(self, cfg: ModelConfig):
        self.cfg = cfg

    def has(self, name: str) -> bool:
        raise NotImplementedError

    def get(self, name: str) -> torch.Tensor:
        raise NotImplementedError

    def quant_info(self, name: str):
        """None for dense tensors, else a dict describing the stored quantised form."""
        return None


class SafetensorsSource(TensorSource):
    def __init__(self, path: str | Path, mapped_shards: int = 4):
        path = Path(path)
        super().__init__(ModelConfig.from_pretrained(path))
        self.path = path
        self.store = H.SafetensorsStore(str(path), mapped_shards)
        self._keys = set(self.store.keys())
        self._packed_experts = any(k.endswith("mlp.experts.gate_up_proj") for k in self._keys)

    def has(self, name: str) -> bool:
        return name in self._keys

    def keys(self):
        return sorted(self._keys)

    def _wrap(self, arr: np.ndarray, dtype: str) -> torch.Tensor:
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only; tensors built on it are never written
            t = torch.from_numpy(arr)
        want = _ST_TO_TORCH[dtype]
        if t.dtype != want:
            t = t.view(want)
        return t

    def fp8_scale_name(self, name: str) -> Optional[str]:
        """Name of the block-scale tensor that goes with an E4M3 weight (HF ``quant_method: fp8`` checkpoints:
        ``<base>.weight`` F8_E4M3 + ``<base>.weight_scale_inv`` [ceil(N/128), ceil(K/128)]), else None."""
        if not name.endswith(".weight"):
            return None
        # ``<base>.scale`` is the sibling form of checkpoints that keep the inference layout (DeepSeek-V4)
        for sname in (name + "_scale_inv", name + "_scale", name[:-len("weight")] + "scale"):
            if sname in self._keys and self.store.info(name)["dtype"] == "F8_E4M3":
                return sname
        return None

    def mxfp4_scale_name(self, name: str) -> Optional[str]:
        """Name of the block-exponent tensor of a microscaling FP4 weight: ``<base>.weight`` holds two E2M1 codes per byte
        ([N, K / 2], stored as F4 or as plain bytes), ``<base>.scale`` one E8M0 exponent per 32 weights ([N, K / 32]) - the
        expert banks of DeepSeek-V4 (``expert_dtype: fp4``; eredu/src/backend/mlx/architectures/deepseek_v4/
        layerwise.rs:2207-2222 views the same bytes as 32-bit code words of a group-32 MXFP4 matrix). Else None."""
        if not name.endswith(".weight"):
            return None
        sname = name[:-len("weight")] + "scale"
        if sname not in self._keys:
            return None
        w, sc = self.store.info(name), self.store.info(sname)
        if w["dtype"] not in ("F4", "I8", "U8") or sc["dtype"] not in ("F8_E8M0", "U8"):
            return None
        ws, ss = list(w["shape"]), list(sc["shape"])
        if len(ws) != 2 or len(ss) != 2 or ws[0] != ss[0] or ws[1] * 2 != ss[1] * 32:
            return None
        return sname

    def to_fp8(self, name: str):
        """(E4M3 bytes as uint8 [N, K], fp32 block scales [ceil(N/128), ceil(K/128)]) of a block-scaled weight.
        Scales stored as E8M0 exponent bytes are decoded to 2^(e-127) (eredu/src/backend/mlx/nn/fp8.rs:74-92)."""
        sname = self.fp8_scale_name(name)
        if sname is None:
            raise RuntimeError(f"{name} is not a block-scaled FP8 tensor")
        w = self._wrap(self.store.tensor(name), "U8")
        sinfo = self.store.info(sname)
        sc = self._wrap(self.store.tensor(sname), sinfo["dtype"])
        if sinfo["dtype"] in ("U8", "F8_E8M0"):
            sc = torch.pow(2.0, sc.to(torch.float32) - 127.0)
        return w, sc.to(torch.float32)

    def get(self, name: str) -> torch.Tensor:
        if self.fp8_scale_name(name) is not None:
            w, sc = self.to_fp8(name)
            N, K = w.shape
            full = sc.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
            return w.view(torch.float8_e4m3fn).to(torch.float32) * full
        sname = self.mxfp4_scale_name(name)
        if sname is not None:
            # two E2M1 codes per byte (low nibble first), one power-of-two scale per 32 weights -> dense fp32
            codes = np.ascontiguousarray(self._wrap(self.store.tensor(name), "U8").numpy())
            exps = np.ascontiguousarray(self._wrap(self.store.tensor(sname), "U8").numpy())
            return torch.from_numpy(np.asarray(H.mxfp4_dequantize(codes.view(np.uint32), exps)))
        qi = self.quant_info(name)
        if qi is not None and qi["kind"] == "affine":
            # MLX-LM packed tensor: uint32 code words + per-group scales / biases -> dense fp32 (w = scale * q + bias)
            packed, scales, biases, bits, group = self.to_affine(name)
            dense = H.affine_dequantize(packed.numpy().view(np.uint32), scales.float().numpy(), biases.float().numpy(),
                                        bits, group)
            return torch.from_numpy(np.asarray(dense))
        info = self.store.info(name)
        return self._wrap(self.store.tensor(name), info["dtype"])

    def to_affine(self, name: str):
        """(packed int32 [N, K*bits/32], scales, biases, bits, group) of a packed tensor, as stored."""
        qi = self.quant_info(name)
        if qi is None or qi["biases"] is None:
            raise RuntimeError(f"{name} is not an affine-packed tensor")
        raw = lambda k: self._wrap(self.store.tensor(k), self.store.info(k)["dtype"])   # noqa: E731
        return raw(name).view(torch.int32), raw(qi["scales"]), raw(qi["biases"]), qi["bits"], qi["group_size"]

    def get_rows(self, name: str, start: int, stop: int) -> torch.Tensor:
        """Rank-selective read: only rows [start, stop) are touched (and paged in)."""
        info = self.store.info(name)
        return self._wrap(self.store.rows(name, start, stop), info["dtype"])

    def quant_info(self, name: str):
        q = self.cfg.quantization
        if not q or not name.endswith(".weight"):
            return None
        base = name[: -len(".weight")]
        if base + ".scales" in self._keys:
            mode = q.get("mode", "affine")
            return {"kind": mode, "bits": int(q.get("bits", 4)), "group_size": int(q.get("group_size", 64)),
                    "scales": base + ".scales", "biases": base + ".biases" if base + ".biases" in self._keys else None}
        return None


class GgufSource(TensorSource):
    def __init__(self, path: str | Path):
        self.reader = H.GgufReader(str(path))
        md = self.reader.metadata
        self.infos = {t["name"]: t for t in self.reader.tensors()}
        super().__init__(ModelConfig.from_gguf_metadata(md, "output.weight" in self.infos))
        self.cfg.rope_traditional = False  # rows are un-permuted on read (see module docstring)
        self.metadata = md
        self.arch = md.get("general.architecture", "llama")
        self._permute = self.arch == "llama"

    def _gname(self, name: str) -> Optional[str]:
        m = re.match(r"model\.layers\.(\d+)\.mlp\.experts\.(gate|up|down)_exps\.weight$", name)
        if m:
            return f"blk.{m.group(1)}.ffn_{m.group(2)}_exps.weight"
        return hf_to_gguf_name(name)

    def has(self, name: str) -> bool:
        g = self._gname(name)
        return g is not None and g in self.infos

    def _row_perm(self, gname: str, rows: int):
        if not self._permute:
            return None
        if ".attn_q." in gname:
            return _qk_row_index(rows, self.cfg.num_attention_heads)
        if ".attn_k." in gname:
            return _qk_row_index(rows, self.cfg.num_key_value_heads)
        return None

    def get(self, name: str) -> torch.Tensor:
        g = self._gname(name)
        t = torch.from_numpy(self.reader.dequantize(g))
        perm = self._row_perm(g, t.shape[0])
        if perm is not None:
            t = t[perm]
        return t

    def quant_info(self, name: str):
        g = self._gname(name)
        if g is None or g not in self.infos:
            return None
        tn = self.infos[g]["type_name"]
        if tn in ("F32", "F16", "BF16", "F64"):
            return None
        return {"kind": "ggml", "type": tn, "type_code": self.infos[g]["type"], "shape": self.infos[g]["shape"]}

    def raw_blocks(self, name: str) -> torch.Tensor:
        """Raw GGML block bytes as a uint8 tensor [rows, row_bytes] (rows un-permuted for Q/K)."""
        g = self._gname(name)
        info = self.infos[g]
        shape = info["shape"]
        rows = int(np.prod(shape[:-1]))
        raw = torch.from_numpy(np.array(self.reader.raw(g), copy=False)).view(rows, -1)
        perm = self._row_perm(g, rows) if len(shape) == 2 else None
        if perm is not None:
            raw = raw[perm]
        return raw

    def to_affine(self, name: str):
        g = self._gname(name)
        packed, scales, biases, bits, group = self.reader.to_affine(g)
        packed, scales, biases = (torch.from_numpy(a.copy()) for a in (packed, scales, biases))
        perm = self._row_perm(g, packed.shape[0])
        if perm is not None:
            packed, scales, biases = packed[perm], scales[perm], biases[perm]
        return packed.view(torch.int32), scales.view(torch.float16), biases.view(torch.float16), bits, group


def open_checkpoint(path: str | Path, mapped_shards: int = 4) -> TensorSource:
    path = Path(path)
    if path.is_dir():
        ggufs = sorted(path.glob("*.gguf"))
        if (path / "config.json").exists():
            return SafetensorsSource(path, mapped_shards)
        if ggufs:
            return GgufSource(ggufs[0])
        raise FileNotFoundError(f"{path}: neither config.json nor *.gguf")
    if path.suffix == ".gguf":
        return GgufSource(path)
    raise ValueError(f"unsupported checkpoint path {path}")
