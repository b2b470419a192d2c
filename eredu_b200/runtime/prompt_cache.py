"""Reusable prompt (prefix) caches on disk: a JSON manifest plus SafeTensors shards per rank.

Counterpart of eredu-core/src/cache/prompt.rs:16,281-379 (schema version 7: identity fingerprints, owned layer
range, block catalogue with SHA-256 of every payload, SHA-256 over the little-endian prefix token ids, rank-local
topology) and of the save / open / load entry points of eredu/src/backend/mlx/runtime/cache/residency.rs. A cache
written by one topology or checkpoint is refused by another: every mismatch is an error, never a silent miss.

Layout of a cache directory::

    manifest.json                         (rank 0 of a single-rank run)   or
    rank-pp{P}-tp{T}-ep{E}/manifest.json  (one directory per rank of a distributed run)
        layer-0000.safetensors ...        arrays  "k.{start}" / "v.{start}"  of shape [n_kv_local, tokens, head_dim]
        state.safetensors                 hybrid models: "layer.{i}.convolution" / "layer.{i}.recurrent", the fixed-size
                                          states after the last cached token (catalogued in ``state_tensors``)
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Optional

import numpy as np
import torch

from .kv_cache import PAGE

PROMPT_CACHE_SCHEMA_VERSION = 7


class PromptCacheError(Exception):
    pass


class UnsupportedSchema(PromptCacheError):
    pass


class Incompatible(PromptCacheError):
    pass


class Malformed(PromptCacheError):
    pass


class Corrupt(PromptCacheError):
    pass


def sha256_tokens(tokens) -> str:
    """SHA-256 over the token ids as little-endian u32."""
    return hashlib.sha256(struct.pack(f"<{len(tokens)}I", *[int(t) for t in tokens])).hexdigest()


def _is_sha256_hex(s: str) -> bool:
    return isinstance(s, str) and len(s) == 64 and all(c in "0123456789abcdef" for c in s)


@dataclass
class PromptCacheTopology:
    pipeline: Optional[tuple] = None          # (size, rank)
    tensor_parallel: Optional[tuple] = None
    expert_parallel: Optional[tuple] = None
    expert_parallel_cache_replicated: bool = True

    def validate(self):
        for name in ("pipeline", "tensor_parallel", "expert_parallel"):
            ax = getattr(self, name)
            if ax is not None and (ax[0] == 0 or ax[1] >= ax[0]):
                raise Malformed(f"invalid {name} topology")

    @classmethod
    def of(cls, par) -> "PromptCacheTopology":
        if par is None:
            return cls()
        return cls((par.pp_size, par.pp_rank) if par.pp_size > 1 else None,
                   (par.tp_size, par.tp_rank) if par.tp_size > 1 else None,
                   (par.ep_size, par.ep_rank) if par.ep_size > 1 else None, True)

    def rank_dir(self) -> str:
        if self.pipeline is None and self.tensor_parallel is None and self.expert_parallel is None:
            return ""
        g = lambda ax: ax[1] if ax else 0  # noqa: E731
        return f"rank-pp{g(self.pipeline)}-tp{g(self.tensor_parallel)}-ep{g(self.expert_parallel)}"


@dataclass
class PromptCacheBlock:
    global_layer: int
    representation: str          # "key_value"
    start: int
    end: int
    rank: Optional[dict]
    shard: str
    first_array: str
    second_array: str
    first_shape: list
    second_shape: list
    first_dtype: str
    second_dtype: str
    logical_bytes: int
    payload_sha256: str


@dataclass
class PromptCacheManifest:
    schema_version: int
    model_family: str
    effective_model_type: str
    checkpoint_fingerprint: str
    prefix_content_fingerprint: str
    architecture_fingerprint: str
    layer_count: int
    global_layer_start: int
    global_layer_end: int
    block_size_tokens: int
    batch_size: int
    total_prefix_tokens: int
    prefix_sha256: str
    layer_layout: list
    layer_prefix_offsets: list
    sink_tokens: int
    topology: PromptCacheTopology
    application_namespace: Optional[str] = None
    blocks: list = field(default_factory=list)
    state_tensors: list = field(default_factory=list)

    def validate(self):
        if self.schema_version != PROMPT_CACHE_SCHEMA_VERSION:
            raise UnsupportedSchema(f"prompt-cache schema {self.schema_version} (supported: {PROMPT_CACHE_SCHEMA_VERSION})")
        owned = self.global_layer_end - self.global_layer_start
        if (not self.prefix_content_fingerprint or self.block_size_tokens <= 0 or self.layer_count == 0
                or self.global_layer_start >= self.global_layer_end or self.global_layer_end > self.layer_count
                or owned != len(self.layer_layout) or owned != len(self.layer_prefix_offsets) or self.batch_size <= 0
                or self.total_prefix_tokens == 0 or not _is_sha256_hex(self.prefix_sha256)
                or any(o > 0 for o in self.layer_prefix_offsets)):
            raise Malformed("invalid global cache dimensions")
        self.topology.validate()
        # coverage: per layer the blocks tile [0, total_prefix_tokens) without gap or overlap
        per_layer: dict[int, list] = {}
        for b in self.blocks:
            if not (self.global_layer_start <= b.global_layer < self.global_layer_end):
                raise Malformed(f"block of layer {b.global_layer} outside the owned range")
            if b.start < 0 or b.end <= b.start or not _is_sha256_hex(b.payload_sha256):
                raise Malformed("invalid block geometry")
            if os.path.isabs(b.shard) or ".." in Path(b.shard).parts:
                raise Malformed(f"unsafe shard path {b.shard!r}")
            per_layer.setdefault(b.global_layer, []).append(b)
        self._validate_state_tensors()
        for li in range(self.global_layer_start, self.global_layer_end):
            if self.layer_layout[li - self.global_layer_start].get("kind") != "key_value":
                if per_layer.get(li):
                    raise Malformed(f"layer {li} keeps no K/V but has K/V blocks")
                continue
            pos = 0
            for b in sorted(per_layer.get(li, []), key=lambda x: x.start):
                if b.start != pos:
                    raise Malformed(f"layer {li}: blocks leave a gap or overlap at token {pos}")
                pos = b.end
            if pos != self.total_prefix_tokens:
                raise Malformed(f"layer {li}: blocks cover {pos} of {self.total_prefix_tokens} tokens")

    def _validate_state_tensors(self):
        """Fixed-size recurrent states: exactly one entry per (layer, role) the layout declares, taken at the end of the
        prefix, with a safe shard path and a payload hash."""
        expected = set()
        for i, layer in enumerate(self.layer_layout):
            for role in layer.get("fixed_state", []):
                expected.add((self.global_layer_start + i, role))
        seen = set()
        for e in self.state_tensors:
            key = (e.get("layer"), e.get("role"))
            if key in seen:
                raise Malformed("fixed-state tensors contain duplicate owner/role entries")
            seen.add(key)
            if os.path.isabs(e.get("shard", "/")) or ".." in Path(e["shard"]).parts or not _is_sha256_hex(e.get("sha256")):
                raise Malformed("invalid fixed-state tensor entry")
            if e.get("tokens") != self.total_prefix_tokens:
                raise Malformed("fixed-state tensor was not taken at the end of the prefix")
        if seen != expected:
            raise Malformed(f"fixed-state tensor count {len(seen)} does not match layout count {len(expected)}")

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=1)

    @classmethod
    def from_json(cls, text: str) -> "PromptCacheManifest":
        try:
            d = json.loads(text)
            if d.get("schema_version") != PROMPT_CACHE_SCHEMA_VERSION:
                raise UnsupportedSchema(f"prompt-cache schema {d.get('schema_version')} (supported: {PROMPT_CACHE_SCHEMA_VERSION})")
            t = d["topology"]
            topo = PromptCacheTopology(*(tuple(t[k]) if t.get(k) is not None else None
                                         for k in ("pipeline", "tensor_parallel", "expert_parallel")),
                                       bool(t.get("expert_parallel_cache_replicated", True)))
            blocks = [PromptCacheBlock(**b) for b in d.get("blocks", [])]
            d = dict(d, topology=topo, blocks=blocks)
            return cls(**d)
        except PromptCacheError:
            raise
        except Exception as e:  # missing keys, wrong types
            raise Malformed(f"unreadable manifest: {e}") from e


# ---------------------------------------------------------------------------------------------------------------
def architecture_fingerprint(cfg) -> str:
    """Everything that changes the meaning of cached K/V: head geometry, positional encoding, norms."""
    keys = ("model_type", "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
            "rope_theta", "rope_scaling", "rms_norm_eps", "qk_norm", "sliding_window", "attention_bias",
            # hybrid families: which layers keep what state, and the state geometry
            "layer_types", "conv_l_cache", "linear_conv_kernel_dim", "linear_num_key_heads", "linear_num_value_heads",
            "linear_key_head_dim", "linear_value_head_dim", "mamba_num_heads", "mamba_head_dim", "ssm_state_size",
            "mamba_conv_kernel", "kv_lora_rank", "qk_rope_head_dim")
    blob = json.dumps({k: getattr(cfg, k, None) for k in keys}, sort_keys=True, default=str)
    return hashlib.sha256(blob.encode()).hexdigest()


def model_identity(engine, checkpoint_fingerprint: str) -> dict:
    model = engine.model
    cfg = model.cfg
    first = model.first_layer
    n_local = model.num_local_layers()
    window = getattr(cfg, "sliding_window", None)
    layout = []
    for li in range(first, first + n_local):
        if cfg.layer_has_kv(li):
            layout.append({"kind": "key_value", "attention": ({"sliding": int(window)} if window else "full"),
                           "num_key_value_heads": int(model.n_kv_local), "head_dim": int(cfg.head_dim)})
        elif cfg.layer_is_conv(li):
            layout.append({"kind": "recurrent", "fixed_state": ["convolution"]})
        elif cfg.layer_has_recurrent_state(li):
            layout.append({"kind": "recurrent", "fixed_state": ["convolution", "recurrent"]})
        else:
            layout.append({"kind": "stateless"})
    return dict(model_family=cfg.model_type.split("_")[0], effective_model_type=cfg.model_type,
                checkpoint_fingerprint=checkpoint_fingerprint, architecture_fingerprint=architecture_fingerprint(cfg),
                layer_count=cfg.num_hidden_layers, global_layer_start=first, global_layer_end=first + n_local,
                layer_layout=layout, layer_prefix_offsets=[0] * n_local, sink_tokens=0,
                topology=PromptCacheTopology.of(getattr(model, "par", None)))


_DT = {torch.bfloat16: "BF16", torch.float16: "F16", torch.float32: "F32"}
_DT_INV = {v: k for k, v in _DT.items()}


def _bytes_of(t: torch.Tensor) -> bytes:
    t = t.contiguous().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    return t.numpy().tobytes()


def save_prompt_cache(engine, seq, directory, checkpoint_fingerprint: str, prefix_tokens: Optional[int] = None,
                      block_tokens: int = 256, namespace: Optional[str] = None, replace_existing: bool = False) -> Path:
    """Persist the K/V of the first ``prefix_tokens`` cached tokens of ``seq`` (default: all cached tokens).
    Every rank of a distributed run calls this with the same arguments and writes its own directory."""
    from ..formats.checkpoint import _np
    from ..lib import _eredu_host as H

    ident = model_identity(engine, checkpoint_fingerprint)
    topo: PromptCacheTopology = ident["topology"]
    n = seq.kv_len if prefix_tokens is None else int(prefix_tokens)
    if n <= 0 or n > seq.kv_len:
        raise PromptCacheError(f"cannot save {n} tokens of a sequence with {seq.kv_len} cached tokens")
    if engine.kv.has_recurrent_state() and n != seq.kv_len:
        # the convolution histories and recurrent matrices exist for the current length only
        raise PromptCacheError(f"a hybrid model's cache is saved at the sequence's current length ({seq.kv_len}), not at {n}")
    if block_tokens % PAGE != 0:
        raise PromptCacheError(f"block size must be a multiple of the {PAGE}-token page")
    tokens = (seq.prompt + seq.output)[:n]
    final = Path(directory) / topo.rank_dir() if topo.rank_dir() else Path(directory)
    tmp = final.with_name(final.name + ".partial")
    if (final / "manifest.json").exists() and not replace_existing:
        raise PromptCacheError(f"{final} already holds a prompt cache")
    if tmp.exists():
        import shutil

        shutil.rmtree(tmp)
    tmp.mkdir(parents=True)
    pages = torch.as_tensor(seq.pages[:(n + PAGE - 1) // PAGE], dtype=torch.long, device=engine.device)
    rank_id = None
    if topo.rank_dir():
        rank_id = {"pipeline_rank": topo.pipeline[1] if topo.pipeline else None,
                   "tensor_parallel_rank": topo.tensor_parallel[1] if topo.tensor_parallel else None,
                   "expert_parallel_rank": topo.expert_parallel[1] if topo.expert_parallel else None}
    blocks = []
    state_entries = []
    state_items = []
    snap = engine.snapshot_state(seq)
    if snap is not None:
        conv, la = snap
        per_layer_states = {}
        if conv is not None:
            for li, i in engine.kv._conv_index.items():
                per_layer_states.setdefault(li, {})["convolution"] = conv[i]
        if la is not None:
            for li, i in engine.kv._la_index.items():
                per_layer_states.setdefault(li, {})["convolution"] = la[0][i]
                per_layer_states[li]["recurrent"] = la[1][i]
        for li in sorted(per_layer_states):
            for role, t in sorted(per_layer_states[li].items()):
                t = t.contiguous().cpu()
                name = f"layer.{li}.{role}"
                state_items.append((name, _DT[t.dtype], list(t.shape), _np(t)))
                state_entries.append({"layer": li, "role": role, "shard": "state.safetensors", "array": name,
                                      "shape": list(t.shape), "dtype": _DT[t.dtype], "tokens": n,
                                      "logical_bytes": t.numel() * t.element_size(),
                                      "sha256": hashlib.sha256(_bytes_of(t)).hexdigest()})
        H.write_safetensors(str(tmp / "state.safetensors"), state_items, {"format": "eredu-prompt-cache"})
    for li in range(ident["global_layer_start"], ident["global_layer_end"]):
        if not engine.cfg.layer_has_kv(li):
            continue
        k_pool, v_pool = engine.kv.layer(li)
        # [pages, n_kv, PAGE, D] -> [n_kv, pages * PAGE, D]
        k = k_pool[pages].permute(1, 0, 2, 3).reshape(k_pool.shape[1], -1, k_pool.shape[3])[:, :n]
        v = v_pool[pages].permute(1, 0, 2, 3).reshape(v_pool.shape[1], -1, v_pool.shape[3])[:, :n]
        shard = f"layer-{li:04d}.safetensors"
        items = []
        for start in range(0, n, block_tokens):
            end = min(n, start + block_tokens)
            kb, vb = k[:, start:end].contiguous().cpu(), v[:, start:end].contiguous().cpu()
            digest = hashlib.sha256(_bytes_of(kb) + _bytes_of(vb)).hexdigest()
            items.append((f"k.{start}", _DT[kb.dtype], list(kb.shape), _np(kb)))
            items.append((f"v.{start}", _DT[vb.dtype], list(vb.shape), _np(vb)))
            blocks.append(PromptCacheBlock(li, "key_value", start, end, rank_id, shard, f"k.{start}", f"v.{start}",
                                           list(kb.shape), list(vb.shape), _DT[kb.dtype], _DT[vb.dtype],
                                           kb.numel() * kb.element_size() + vb.numel() * vb.element_size(), digest))
        H.write_safetensors(str(tmp / shard), items, {"format": "eredu-prompt-cache"})
    content = hashlib.sha256((sha256_tokens(tokens) + ident["checkpoint_fingerprint"]).encode()).hexdigest()
    man = PromptCacheManifest(schema_version=PROMPT_CACHE_SCHEMA_VERSION, prefix_content_fingerprint=content,
                              block_size_tokens=block_tokens, batch_size=1, total_prefix_tokens=n,
                              prefix_sha256=sha256_tokens(tokens), application_namespace=namespace, blocks=blocks,
                              state_tensors=state_entries, **ident)
    man.validate()
    (tmp / "manifest.json").write_text(man.to_json())
    # publish atomically: readers either see the old cache or the complete new one
    if (final / "manifest.json").exists():
        import shutil

        shutil.rmtree(final)
    elif final.is_dir():
        if any(final.iterdir()):
            raise PromptCacheError(f"{final} exists and is not a prompt cache")
        final.rmdir()
    os.replace(tmp, final)
    return final


def open_prompt_cache(directory, topology: Optional[PromptCacheTopology] = None) -> PromptCacheManifest:
    """Read and validate the manifest of this rank (no tensor payload is touched)."""
    topo = topology or PromptCacheTopology()
    path = Path(directory) / topo.rank_dir() / "manifest.json"
    if not path.exists():
        raise PromptCacheError(f"no prompt cache at {path}")
    man = PromptCacheManifest.from_json(path.read_text())
    man.validate()
    return man


def load_prompt_cache(engine, directory, tokens, checkpoint_fingerprint: str, sampling=None, max_new_tokens: int = 256,
                      eos_ids=(), verify_payload: bool = True):
    """Create a sequence for ``tokens`` whose leading K/V come from the cache. The cached prefix must be a prefix
    of ``tokens`` (checked by hash); at least the last token is left to prefill so that logits exist."""
    from ..lib import _eredu_host as H

    ident = model_identity(engine, checkpoint_fingerprint)
    man = open_prompt_cache(directory, ident["topology"])
    for key in ("model_family", "effective_model_type", "checkpoint_fingerprint", "architecture_fingerprint", "layer_count",
                "global_layer_start", "global_layer_end", "sink_tokens", "layer_layout", "layer_prefix_offsets"):
        if getattr(man, key) != ident[key]:
            raise Incompatible(f"prompt cache {key} does not match the loaded model")
    if man.topology != ident["topology"]:
        raise Incompatible("prompt cache was written by a different parallel topology")
    n = man.total_prefix_tokens
    tokens = [int(t) for t in tokens]
    if n > len(tokens) or sha256_tokens(tokens[:n]) != man.prefix_sha256:
        raise Incompatible("the cached prefix is not a prefix of the request")
    if man.state_tensors and len(tokens) <= n:
        # recurrent states exist for exactly n tokens: the request must bring at least one more so that logits can be made
        raise Incompatible("a hybrid model's cached prefix must be a strict prefix of the request")
    seq = engine.new_sequence(tokens, sampling, max_new_tokens, eos_ids)
    try:
        usable = min(n, len(tokens) - 1)
        root = Path(directory) / man.topology.rank_dir()
        stores: dict[str, object] = {}
        for b in sorted(man.blocks, key=lambda x: (x.global_layer, x.start)):
            if b.start >= usable:
                continue
            st = stores.get(b.shard)
            if st is None:
                st = stores[b.shard] = H.SafetensorsStore(str(root / b.shard), 4)
            kb = np.asarray(st.tensor(b.first_array))
            vb = np.asarray(st.tensor(b.second_array))
            if verify_payload and hashlib.sha256(kb.tobytes() + vb.tobytes()).hexdigest() != b.payload_sha256:
                raise Corrupt(f"payload hash mismatch in {b.shard}:{b.first_array}")
            dt = _DT_INV[b.first_dtype]
            kt = _to_tensor(kb, dt, b.first_shape).to(engine.device)
            vt = _to_tensor(vb, dt, b.second_shape).to(engine.device)
            end = min(b.end, usable)
            pos = torch.arange(b.start, end, device=engine.device)
            page_ids = torch.as_tensor(seq.pages, dtype=torch.long, device=engine.device)[pos // PAGE]
            k_pool, v_pool = engine.kv.layer(b.global_layer)
            # pool[page, head, offset, :] = block[head, token, :]
            k_pool[page_ids, :, pos % PAGE] = kt[:, :end - b.start].transpose(0, 1).to(k_pool.dtype)
            v_pool[page_ids, :, pos % PAGE] = vt[:, :end - b.start].transpose(0, 1).to(v_pool.dtype)
        if man.state_tensors:
            st = H.SafetensorsStore(str(root / "state.safetensors"), 4)
            first_page = seq.pages[0]
            slot = engine.kv._slot_of_page.get(int(first_page)) if engine.kv.page_to_slot is not None else None
            for e in man.state_tensors:
                raw = np.asarray(st.tensor(e["array"]))
                if verify_payload and hashlib.sha256(raw.tobytes()).hexdigest() != e["sha256"]:
                    raise Corrupt(f"payload hash mismatch in state.safetensors:{e['array']}")
                t = _to_tensor(raw, _DT_INV[e["dtype"]], e["shape"]).to(engine.device)
                li = e["layer"]
                if li in engine.kv._conv_index:
                    dst = engine.kv.conv_state[engine.kv._conv_index[li], int(first_page)]
                elif e["role"] == "convolution":
                    dst = engine.kv.la_conv_state[engine.kv._la_index[li], slot]
                else:
                    dst = engine.kv.la_rec_state[engine.kv._la_index[li], slot]
                if tuple(dst.shape) != tuple(t.shape):
                    raise Incompatible(f"fixed-state tensor {e['array']} has shape {tuple(t.shape)}, the model keeps {tuple(dst.shape)}")
                dst.copy_(t.to(dst.dtype))
        seq.kv_len = usable
    except Exception:
        engine.release(seq)
        raise
    return seq


def _to_tensor(arr: np.ndarray, dtype, shape) -> torch.Tensor:
    raw = np.ascontiguousarray(arr)
    if dtype == torch.bfloat16:
        return torch.from_numpy(raw.view(np.int16).copy()).view(torch.bfloat16).reshape(shape)
    return torch.from_numpy(raw.copy()).view(dtype).reshape(shape)
