"""``quantize_checkpoint``: rewrite a SafeTensors checkpoint directory with MLX-LM-style affine-packed weights.

Counterpart of eredu/src/backend/mlx/runtime/checkpoint/quantization.rs:137-232,262-... (example
eredu/examples/quantize_checkpoint.rs): every eligible tensor ``X.weight`` becomes ``X.weight`` (uint32 code words,
little-endian bit stream, [out, in * bits / 32]) + ``X.scales`` + ``X.biases`` ([out, in / group]), and ``config.json``
gains both ``quantization`` and ``quantization_config`` {group_size, bits, mode}. Eligibility (quantization.rs:24-38,
105-115): the name ends in ``.weight``, rank 2, floating point, ``in % group == 0`` and ``in % 32 == 0``; norms,
routers, embeddings and the output head stay dense. Already-packed checkpoints are refused (no transcoding).

    python -m eredu_b200.formats.quantize SRC_DIR DST_DIR --bits 4 --group-size 64
"""
from __future__ import annotations

import argparse
import json
import shutil
from pathlib import Path

import numpy as np
import torch

from ..lib import _eredu_host as H
from .checkpoint import _ST_DTYPES, _np, SafetensorsSource

DENSE_SUFFIXES = ("norm.weight", "layernorm.weight", "embed_tokens.weight", "lm_head.weight", "mlp.gate.weight",
                  "router.weight", "q_norm.weight", "k_norm.weight")


def eligible(name: str, shape, dtype, group: int) -> bool:
    if not name.endswith(".weight") or name.endswith(DENSE_SUFFIXES) or len(shape) != 2:
        return False
    if dtype not in ("F32", "F16", "BF16"):
        return False
    cols = int(shape[1])
    return cols % group == 0 and cols % 32 == 0


def quantize_checkpoint(src_dir, dst_dir, bits: int = 4, group_size: int = 64, mode: str = "affine",
                        shard_bytes: int = 4 << 30, mapped_shards: int = 4) -> dict:
    """Returns a report: tensors quantised / kept, bytes before / after."""
    if mode != "affine":
        raise NotImplementedError("quantize_checkpoint writes the affine format")
    if bits not in (2, 3, 4, 5, 6, 8):
        raise ValueError("bits must be one of 2, 3, 4, 5, 6, 8")
    if group_size != 16 and group_size % 32 != 0:
        raise ValueError("group size must be 16 or a multiple of 32")
    src_dir, dst_dir = Path(src_dir), Path(dst_dir)
    src = SafetensorsSource(src_dir, mapped_shards)
    if src.cfg.quantization:
        raise ValueError("the source checkpoint is already quantised: packed checkpoints are not transcoded")
    dst_dir.mkdir(parents=True, exist_ok=True)
    report = {"quantized": 0, "kept": 0, "bytes_before": 0, "bytes_after": 0}
    shards, cur, cur_bytes = [], [], 0

    def emit(name, dtype, shape, arr):
        nonlocal cur, cur_bytes
        nb = arr.nbytes
        if cur and cur_bytes + nb > shard_bytes:
            shards.append(cur)
            cur, cur_bytes = [], 0
        cur.append((name, dtype, list(shape), arr))
        cur_bytes += nb
        report["bytes_after"] += nb

    for name in src.keys():
        info = src.store.info(name)
        t = src.get(name)
        report["bytes_before"] += t.numel() * t.element_size()
        if eligible(name, info["shape"], info["dtype"], group_size):
            packed, scales, biases = H.affine_quantize(np.ascontiguousarray(t.float().numpy()), bits, group_size, "f16")
            base = name[: -len(".weight")]
            emit(name, "U32", packed.shape, np.ascontiguousarray(packed))
            emit(base + ".scales", "F16", scales.shape, np.asarray(scales, dtype=np.float32).astype(np.float16))
            emit(base + ".biases", "F16", biases.shape, np.asarray(biases, dtype=np.float32).astype(np.float16))
            report["quantized"] += 1
        else:
            emit(name, _ST_DTYPES[t.dtype], t.shape, _np(t))
            report["kept"] += 1
    if cur:
        shards.append(cur)
    if len(shards) == 1:
        H.write_safetensors(str(dst_dir / "model.safetensors"), shards[0], {"format": "mlx"})
    else:
        weight_map = {}
        for i, sh in enumerate(shards):
            fname = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
            H.write_safetensors(str(dst_dir / fname), sh, {"format": "mlx"})
            for it in sh:
                weight_map[it[0]] = fname
        (dst_dir / "model.safetensors.index.json").write_text(json.dumps(
            {"metadata": {"total_size": report["bytes_after"]}, "weight_map": weight_map}, indent=1))
    cfg = json.loads((src_dir / "config.json").read_text())
    q = {"group_size": group_size, "bits": bits, "mode": mode}
    cfg["quantization"] = dict(q)
    cfg["quantization_config"] = dict(q)
    (dst_dir / "config.json").write_text(json.dumps(cfg, indent=1))
    for extra in ("tokenizer.json", "tokenizer_config.json", "generation_config.json", "special_tokens_map.json",
                  "chat_template.jinja", "chat_template.json"):
        if (src_dir / extra).exists():
            shutil.copy2(src_dir / extra, dst_dir / extra)
    return report


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="eredu-quantize")
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--group-size", type=int, default=64)
    a = ap.parse_args(argv)
    print(json.dumps(quantize_checkpoint(a.src, a.dst, a.bits, a.group_size)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
