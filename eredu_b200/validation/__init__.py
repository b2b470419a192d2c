"""Real-checkpoint validation: this runtime's logits against Hugging Face Transformers on the same token ids.

Counterpart of the reference's ``validation/`` harness (``checkpoint_probe`` -> ``reference_runner.py`` ->
``compare_checkpoints.py`` with the tolerance profiles of ``models.yaml``): sampled prefill positions, a teacher-forced
run of decode steps, cached-versus-recompute agreement, and gates on relative L2 error, cosine similarity, top-k overlap
and the argmax (only where the reference's own margin makes it unambiguous).

    python -m eredu_b200.validation --model /models/Qwen3-8B --profile bf16_reference --device cuda
"""
from .compare import CorrectnessProfile, PROFILES, compare_probes
from .probe import probe_checkpoint, probe_reference, default_token_ids

__all__ = ["CorrectnessProfile", "PROFILES", "compare_probes", "probe_checkpoint", "probe_reference", "default_token_ids"]
