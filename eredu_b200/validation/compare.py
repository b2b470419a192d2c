"""Gates that turn two probe records into a verdict."""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class CorrectnessProfile:
    relative_l2_max: float = 0.02
    cosine_similarity_min: float = 0.999
    top_k: int = 5
    top_k_overlap_min: int = 4
    require_unambiguous_argmax_match: bool = True
    argmax_margin_min: float = 0.0        # the reference's top-1 / top-2 logit gap below which an argmax flip is not an error
    require_cached_vs_full_recompute: bool = True
    cached_relative_l2_max: float = 0.02


# Tolerances per numeric regime: bf16 compute against a bf16 reference; families whose recurrences amplify rounding;
# checkpoint-native low-precision weights (MXFP4, block FP8).
PROFILES = {
    "fp32_exact": CorrectnessProfile(1e-4, 0.999999, 5, 5, True, 0.0, True, 1e-4),
    "bf16_reference": CorrectnessProfile(),
    "lfm2_bf16_reference": CorrectnessProfile(relative_l2_max=0.06, cosine_similarity_min=0.9985),
    "nemotron_h_bf16_reference": CorrectnessProfile(relative_l2_max=0.025, argmax_margin_min=0.25),
    "native_mxfp4_reference": CorrectnessProfile(0.05, 0.995, 5, 3),
    "native_block_fp8_reference": CorrectnessProfile(0.05, 0.995, 5, 3),
}


# Default profile per checkpoint family (``model_type``) and weight format; anything else is ``bf16_reference``.
FAMILY_PROFILES = {"lfm2": "lfm2_bf16_reference", "lfm2_moe": "lfm2_bf16_reference", "nemotron_h": "nemotron_h_bf16_reference",
                   "gpt_oss": "native_mxfp4_reference", "deepseek_v3": "native_block_fp8_reference"}


def profile_for(model_type: str, device: str = "cuda") -> str:
    if device == "cpu":
        return "fp32_exact"
    return FAMILY_PROFILES.get(model_type, "bf16_reference")


def _row_metrics(ours: torch.Tensor, ref: torch.Tensor, prof: CorrectnessProfile) -> dict:
    a, b = ours.double(), ref.double()
    rel = float((a - b).norm() / b.norm().clamp_min(1e-30))
    cos = float(torch.nn.functional.cosine_similarity(a, b, dim=0))
    ta, tb = torch.topk(a, prof.top_k).indices.tolist(), torch.topk(b, prof.top_k).indices.tolist()
    top2 = torch.topk(b, 2).values
    margin = float(top2[0] - top2[1])
    return {"relative_l2": rel, "cosine": cos, "top_k_overlap": len(set(ta) & set(tb)), "argmax_ours": ta[0],
            "argmax_reference": tb[0], "reference_margin": margin, "finite": bool(torch.isfinite(a).all())}


def compare_probes(ours: dict, reference: dict, profile: CorrectnessProfile) -> dict:
    """Both probes: {"token_ids", "prefill": {position: logits}, "decode": [logits per teacher-forced step],
    "recompute": {position: logits}}. Returns {"passed", "failures": [...], "rows": [...]}"""
    if ours["token_ids"] != reference["token_ids"]:
        raise ValueError("the two probes were taken on different token ids")
    rows, failures = [], []

    def gate(label, a, b):
        m = dict(_row_metrics(a, b, profile), row=label)
        rows.append(m)
        if not m["finite"]:
            failures.append(f"{label}: non-finite logits")
        if m["relative_l2"] > profile.relative_l2_max:
            failures.append(f"{label}: relative L2 {m['relative_l2']:.4g} > {profile.relative_l2_max}")
        if m["cosine"] < profile.cosine_similarity_min:
            failures.append(f"{label}: cosine {m['cosine']:.6f} < {profile.cosine_similarity_min}")
        if m["top_k_overlap"] < profile.top_k_overlap_min:
            failures.append(f"{label}: top-{profile.top_k} overlap {m['top_k_overlap']} < {profile.top_k_overlap_min}")
        if (profile.require_unambiguous_argmax_match and m["argmax_ours"] != m["argmax_reference"]
                and m["reference_margin"] > profile.argmax_margin_min):
            failures.append(f"{label}: argmax {m['argmax_ours']} != {m['argmax_reference']} at reference margin "
                            f"{m['reference_margin']:.3g}")

    for pos, ref_logits in reference["prefill"].items():
        gate(f"prefill[{pos}]", ours["prefill"][pos], ref_logits)
    for i, ref_logits in enumerate(reference["decode"]):
        gate(f"decode[{i}]", ours["decode"][i], ref_logits)
    if profile.require_cached_vs_full_recompute:
        for pos, full in ours.get("recompute", {}).items():
            inc = ours["decode"][pos] if isinstance(pos, int) and pos < len(ours["decode"]) else None
            if inc is None:
                continue
            rel = float((inc.double() - full.double()).norm() / full.double().norm().clamp_min(1e-30))
            rows.append({"row": f"cached_vs_recompute[{pos}]", "relative_l2": rel})
            if rel > profile.cached_relative_l2_max:
                failures.append(f"cached_vs_recompute[{pos}]: relative L2 {rel:.4g} > {profile.cached_relative_l2_max}")
    return {"passed": not failures, "failures": failures, "rows": rows}
