"""``python -m eredu_b200.validation --model PATH [--profile NAME] [--device cuda] [--report out.json]``"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    import torch

    from ..api import LoadedModel, ModelLoadOptions
    from .compare import profile_for
    from . import PROFILES, compare_probes, default_token_ids, probe_checkpoint, probe_reference

    ap = argparse.ArgumentParser(prog="eredu-validate")
    ap.add_argument("--model", required=True, help="SafeTensors checkpoint directory (also loadable by Transformers)")
    ap.add_argument("--profile", default="auto", choices=["auto"] + sorted(PROFILES))
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--prompt", default=None, help="text to tokenize (default: deterministic token ids)")
    ap.add_argument("--length", type=int, default=48)
    ap.add_argument("--decode-steps", type=int, default=16)
    ap.add_argument("--reference-dtype", default=None, choices=[None, "float32", "bfloat16"])
    ap.add_argument("--report", default=None)
    a = ap.parse_args(argv)

    import transformers

    lm = LoadedModel.load(a.model, ModelLoadOptions(device=a.device, max_batch=1, max_seq_len=max(256, a.length + 64)))
    if a.prompt and lm.tokenizer is not None:
        ids = lm.encode(a.prompt)
        while len(ids) < a.decode_steps + 8:
            ids = ids + ids
    else:
        ids = default_token_ids(lm.config.vocab_size, a.length)
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16, None: torch.float32 if a.device == "cpu" else torch.bfloat16}[a.reference_dtype]
    ref_model = transformers.AutoModelForCausalLM.from_pretrained(a.model, torch_dtype=dtype).to(a.device).eval()
    ours = probe_checkpoint(lm, ids, decode_steps=a.decode_steps)
    ref = probe_reference(ref_model, ids, decode_steps=a.decode_steps)
    if a.profile == "auto":
        a.profile = profile_for(lm.config.model_type, a.device)
    verdict = compare_probes(ours, ref, PROFILES[a.profile])
    worst = max((r for r in verdict["rows"] if "cosine" in r), key=lambda r: r["relative_l2"])
    print(f"{'validated' if verdict['passed'] else 'FAILED'}: {len(verdict['rows'])} rows, worst relative L2 "
          f"{worst['relative_l2']:.4g} (cos {worst['cosine']:.6f}) at {worst['row']}")
    for f in verdict["failures"]:
        print("  " + f)
    if a.report:
        with open(a.report, "w") as fh:
            json.dump({"model": a.model, "profile": a.profile, "device": a.device, **verdict}, fh, indent=1)
    return 0 if verdict["passed"] else 1


if __name__ == "__main__":
    sys.exit(main())
