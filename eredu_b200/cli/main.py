"""``eredu`` command line: load a local model (SafeTensors directory or GGUF file) and generate.

Flag set, defaults and output conventions follow eredu-cli/src/main.rs:209-484 (stdout = generated text, stderr =
diagnostics, ``--telemetry-json PATH`` for the structured report, ``--timing`` for load / TTFT / decode rate as defined
at :667-711). Flags that steer subsystems this runtime plans differently (MLX cache limit, MTP devices, dense disk
streaming ...) are accepted, validated and recorded in the telemetry so that existing invocations keep working.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
import time


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="eredu", description="Blackwell-native local LLM inference")
    p.add_argument("-m", "--model", required=True, metavar="PATH_OR_ID[:QUANT]")
    p.add_argument("prompt", nargs="?", default=None, help="prompt text (stdin when absent)")
    p.add_argument("--auto", choices=["plan", "quick", "benchmark"], default="quick")
    p.add_argument("--no-auto", action="store_true")
    p.add_argument("--auto-cache", default=None)
    p.add_argument("--auto-feedback", action="append", default=[])
    p.add_argument("--auto-benchmark-tokens", type=int, default=32)
    p.add_argument("--auto-benchmark-runs", type=int, default=1)
    p.add_argument("--auto-benchmark-timeout-seconds", type=int, default=300)
    p.add_argument("--auto-trial-plan", default=None, help=argparse.SUPPRESS)   # set by --auto benchmark for its child runs
    p.add_argument("--draft-model", default=None)
    p.add_argument("--device", default="gpu:0", help="cpu | gpu:N")
    p.add_argument("--mlx-cache-limit-bytes", type=int, default=None)
    p.add_argument("--mtp-draft-tokens", type=int, default=3)
    p.add_argument("--disable-mtp-lookahead", action="store_true")
    p.add_argument("--disable-mtp-adaptive-lookahead", action="store_true")
    p.add_argument("--mtp-draft-device", default="target")
    p.add_argument("--revision", default=None)
    p.add_argument("--allow-mixed-revisions", action="store_true")
    p.add_argument("--require-same-revision", action="store_true")
    p.add_argument("-n", "--max-tokens", type=int, default=256)
    p.add_argument("-t", "--temperature", type=float, default=None)
    p.add_argument("--top-k", type=int, default=None)
    p.add_argument("--top-p", type=float, default=None)
    p.add_argument("--min-p", type=float, default=None)
    p.add_argument("--mirostat-v2", action="store_true")
    p.add_argument("--mirostat-tau", type=float, default=5.0)
    p.add_argument("--mirostat-eta", type=float, default=0.1)
    p.add_argument("--repeat-penalty", type=float, default=1.0)
    p.add_argument("--repeat-last-n", type=int, default=64)
    p.add_argument("--frequency-penalty", type=float, default=0.0)
    p.add_argument("--presence-penalty", type=float, default=0.0)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--quantize", type=int, default=None, metavar="BITS")
    p.add_argument("--quantization-mode", choices=["affine", "mxfp4", "fp8"], default="affine")
    p.add_argument("--quantization-group-size", type=int, default=64)
    p.add_argument("--layerwise-host", action="store_true")
    p.add_argument("--dense-disk-stream", action="store_true")
    p.add_argument("--dense-host-lookahead", type=int, default=2)
    p.add_argument("--dense-background-queue", type=int, default=2)
    p.add_argument("--expert-cache", action="store_true")
    p.add_argument("--device-layer-window", type=int, default=1)
    p.add_argument("--device-budget-bytes", type=int, default=None)
    p.add_argument("--host-budget-bytes", type=int, default=None)
    p.add_argument("--expert-cache-device-budget-bytes", type=int, default=None)
    p.add_argument("--expert-cache-host-budget-bytes", type=int, default=None)
    p.add_argument("--expert-cache-scratch-bytes", type=int, default=1 << 30)
    p.add_argument("--expert-cache-prefill-bank-bytes", type=int, default=1 << 30)
    p.add_argument("--expert-cache-eviction", choices=["lru", "lfu"], default="lru")
    p.add_argument("--expert-cache-benchmark", action="store_true")
    p.add_argument("--mapped-shards", type=int, default=4)
    p.add_argument("--raw", action="store_true", help="no chat template: the prompt is fed verbatim")
    p.add_argument("--image", action="append", default=[], metavar="PATH", help="image part of the prompt (vision-language models)")
    p.add_argument("--tools", default=None, metavar="PATH")
    p.add_argument("--json-schema", default=None, metavar="PATH", help="constrain the reply to this JSON schema")
    p.add_argument("--grammar", default=None, metavar="PATH", help="constrain the reply to this Lark grammar")
    p.add_argument("--regex", default=None, help="constrain the reply to this regular expression")
    p.add_argument("--tool-choice", choices=["none", "auto", "required"], default="auto")
    p.add_argument("--max-parallel-tool-calls", type=int, default=None)
    p.add_argument("--stop", action="append", default=[], metavar="TEXT")
    p.add_argument("--thinking", choices=["auto", "on", "off"], default="auto")
    p.add_argument("--allow-unparsed-reasoning", action="store_true")
    p.add_argument("-v", "--verbose", action="store_true")
    p.add_argument("--timing", action="store_true")
    p.add_argument("--telemetry-json", default=None, metavar="PATH")
    p.add_argument("--profile-components", action="store_true")
    return p


def validate_args(a) -> None:
    if a.max_tokens <= 0:
        raise SystemExit("--max-tokens must be positive")
    if a.dense_disk_stream and a.layerwise_host:
        raise SystemExit("--dense-disk-stream conflicts with --layerwise-host")
    if a.dense_disk_stream and (a.dense_host_lookahead < 1 or a.dense_background_queue < 1):
        raise SystemExit("--dense-host-lookahead and --dense-background-queue must be at least 1")
    if a.quantization_mode == "fp8" and a.quantize not in (None, 8):
        raise SystemExit("--quantization-mode fp8 stores 8-bit E4M3 codes: use --quantize 8")
    if a.quantize is not None and a.quantize not in (2, 3, 4, 5, 6, 8):
        raise SystemExit("--quantize must be one of 2, 3, 4, 5, 6, 8")
    if a.quantization_group_size != 16 and a.quantization_group_size % 32 != 0:
        raise SystemExit("--quantization-group-size must be 16 or a multiple of 32")
    if a.allow_mixed_revisions and a.require_same_revision:
        raise SystemExit("--allow-mixed-revisions conflicts with --require-same-revision")
    if not (a.device == "cpu" or a.device.startswith("gpu:")):
        raise SystemExit("--device must be cpu or gpu:N")
    # flags of the reference's front end that have no counterpart in this runtime are refused, not silently recorded
    if a.mtp_draft_device != "target":
        raise SystemExit("--mtp-draft-device: not supported on this runtime (the prediction head runs on the target's GPU; "
                         "only 'target' is accepted)")
    if a.mlx_cache_limit_bytes is not None and a.mlx_cache_limit_bytes <= 0:
        raise SystemExit("--mlx-cache-limit-bytes must be positive")
    for flag, val in (("--expert-cache-scratch-bytes", a.expert_cache_scratch_bytes),
                      ("--expert-cache-prefill-bank-bytes", a.expert_cache_prefill_bank_bytes)):
        if val <= 0:
            raise SystemExit(f"{flag} must be positive")


def resolve_revision(model_path: str, revision, allow_mixed: bool, require_same: bool) -> str:
    """``--revision`` for models named by a Hugging Face cache entry (``.../models--org--name``: ``refs/<name>`` holds a
    commit id, ``snapshots/<commit>`` the files). Nothing is downloaded (eredu-cli/src/main.rs:3139-3230 resolves local
    cache entries the same way). A plain directory or a GGUF file has no revisions: asking for one is an error, and
    ``--require-same-revision`` then has nothing to check."""
    import os

    snaps = os.path.join(model_path, "snapshots")
    if not os.path.isdir(snaps):
        if revision is not None:
            raise SystemExit(f"--revision {revision}: {model_path} is not a Hugging Face cache entry (no snapshots/ directory)")
        return model_path
    commits = sorted(os.listdir(snaps))
    if not commits:
        raise SystemExit(f"{model_path}: the cache entry has no snapshot")
    want = revision
    if want is None:
        ref = os.path.join(model_path, "refs", "main")
        want = open(ref).read().strip() if os.path.isfile(ref) else None
    else:
        ref = os.path.join(model_path, "refs", want)
        if os.path.isfile(ref):
            want = open(ref).read().strip()
    if want is None:
        if len(commits) > 1 and not allow_mixed:
            raise SystemExit(f"{model_path}: several snapshots and no refs/main; pass --revision (or --allow-mixed-revisions "
                             f"to take the newest)")
        want = max(commits, key=lambda c: os.path.getmtime(os.path.join(snaps, c)))
    match = [c for c in commits if c == want or c.startswith(want)]
    if len(match) != 1:
        raise SystemExit(f"--revision {revision or want}: no unique snapshot among {commits}")
    return os.path.join(snaps, match[0])


def resolve_sampling(a, generation_config: dict):
    """Merge checkpoint defaults with explicit flags (eredu-core/src/generation.rs:706-800): greedy unless sampling
    is requested; with a checkpoint config top-k 50 / top-p 1.0 / min-p 0, without one 40 / 0.95 / 0.05."""
    from ..ops.sampling import SamplingParams

    has_cfg = bool(generation_config)
    do_sample = bool(generation_config.get("do_sample", False))
    temp = a.temperature if a.temperature is not None else (float(generation_config.get("temperature", 1.0)) if do_sample else 0.0)
    return SamplingParams(
        temperature=temp,
        top_k=a.top_k if a.top_k is not None else int(generation_config.get("top_k", 50 if has_cfg else 40)),
        top_p=a.top_p if a.top_p is not None else float(generation_config.get("top_p", 1.0 if has_cfg else 0.95)),
        min_p=a.min_p if a.min_p is not None else float(generation_config.get("min_p", 0.0 if has_cfg else 0.05)),
        repeat_penalty=a.repeat_penalty, repeat_last_n=a.repeat_last_n, frequency_penalty=a.frequency_penalty,
        presence_penalty=a.presence_penalty, seed=a.seed)


AUTO_BENCHMARK_PROMPT = "Write a short paragraph about the history of the telescope."


def read_feedback(paths) -> list:
    """Telemetry records of earlier runs (eredu-cli/src/main.rs:1383-1408): each file holds one record or an array."""
    out = []
    for path in paths:
        try:
            val = json.load(open(path))
        except OSError as e:
            raise SystemExit(f"failed to read automatic feedback {path}: {e}")
        except ValueError as e:
            raise SystemExit(f"failed to parse automatic feedback {path}: {e}")
        out.extend(val if isinstance(val, list) else [val])
    for t in out:
        if not isinstance(t, dict):
            raise SystemExit("automatic feedback must be telemetry objects")
    return out


def write_plan_cache(path, key, plan, rate) -> None:
    try:
        book = json.load(open(path))
    except (OSError, ValueError):
        book = {}
    book[key] = {"plan": json.loads(plan.to_json()), "benchmark_token_rate": rate}
    json.dump(book, open(path, "w"), indent=1)


def benchmark_candidates(model_path: str, a, candidates: list, prompt: str) -> dict:
    """Times every candidate plan in a fresh process (eredu-cli/src/main.rs:1516-1745): the child gets the serialized
    plan through ``--auto-trial-plan`` and reports through ``--telemetry-json``; the selection metric is the median
    decode rate over ``--auto-benchmark-runs`` runs. A candidate whose runs all fail (or time out) is kept in the report
    with its error and is not eligible."""
    import subprocess
    import tempfile

    from ..runtime.plan import _median

    rows, best = [], None
    with tempfile.TemporaryDirectory(prefix="eredu-auto-") as tmp:
        for ci, plan in enumerate(candidates):
            print(f"[eredu] automatic benchmark: candidate {ci + 1}/{len(candidates)} ({plan.residency.get('mode')}"
                  f"{', expert cache' if plan.expert_cache else ''})", file=sys.stderr)
            trials, rates = [], []
            for run in range(a.auto_benchmark_runs):
                plan_path, tel_path = f"{tmp}/plan-{ci}-{run}.json", f"{tmp}/tel-{ci}-{run}.json"
                open(plan_path, "w").write(plan.to_json())
                cmd = [sys.executable, "-m", "eredu_b200.cli", "--model", model_path, "--device", a.device, "--auto-trial-plan",
                       plan_path, "--telemetry-json", tel_path, "--max-tokens", str(a.auto_benchmark_tokens), "--raw",
                       "--mapped-shards", str(a.mapped_shards), prompt]
                trial = {"run": run}
                try:
                    r = subprocess.run(cmd, stdin=subprocess.DEVNULL, stdout=subprocess.DEVNULL, stderr=subprocess.PIPE,
                                       timeout=a.auto_benchmark_timeout_seconds)
                    if r.returncode != 0:
                        trial["error"] = f"exit {r.returncode}: " + r.stderr.decode(errors="replace").strip()[-400:]
                    else:
                        t = json.load(open(tel_path))
                        timing = t.get("timing", {})
                        rate = timing.get("decode_token_rate") or timing.get("token_rate") or 0.0
                        trial.update(token_rate=rate, generated_tokens=t.get("generated_tokens"),
                                     load_time=timing.get("load_time"), time_to_first_token=timing.get("time_to_first_token"))
                        if rate > 0:
                            rates.append(rate)
                except subprocess.TimeoutExpired:
                    trial["error"] = f"timed out after {a.auto_benchmark_timeout_seconds}s"
                except (OSError, ValueError) as e:
                    trial["error"] = str(e)
                trials.append(trial)
            med = _median(rates) if rates else None
            rows.append({"plan": json.loads(plan.to_json()), "trials": trials, "median_token_rate": med})
            if med is not None and (best is None or med > rows[best]["median_token_rate"]):
                best = ci
    if best is None:
        raise SystemExit("every isolated automatic benchmark candidate failed:\n" +
                         "\n".join(t.get("error", "") for r in rows for t in r["trials"]))
    return {"schema_version": 2, "generated_tokens_per_trial": a.auto_benchmark_tokens, "runs_per_candidate": a.auto_benchmark_runs,
            "timeout_seconds": a.auto_benchmark_timeout_seconds, "selection_metric": "median_decode_token_rate",
            "selected": rows[best]["plan"], "selected_index": best, "selected_median_token_rate": rows[best]["median_token_rate"],
            "candidates": rows, "_selected_plan": candidates[best]}


def _draft_model_type(path) -> str:
    cfg = os.path.join(path, "config.json")
    if not os.path.isfile(cfg):
        return ""
    with open(cfg) as f:
        return str(json.load(f).get("model_type", ""))


def _is_gemma4_assistant(path) -> bool:
    """A draft directory whose config.json names the Gemma 4 assistant drafter."""
    return _draft_model_type(path).startswith("gemma4_assistant")


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    validate_args(a)
    prompt = a.prompt if a.prompt is not None else sys.stdin.read()
    from ..api import LoadedModel, ModelLoadOptions, QuantizationOptions
    from ..runtime.telemetry import ExecutionTelemetry, hardware_profile

    model_path, _, quant_suffix = a.model.partition(":")
    model_path = resolve_revision(model_path, a.revision, a.allow_mixed_revisions, a.require_same_revision)
    if a.draft_model and a.require_same_revision:
        # draft and target must come from the same commit when both are cache entries
        import os

        d = resolve_revision(a.draft_model, a.revision, a.allow_mixed_revisions, True)
        if os.path.basename(d) != os.path.basename(model_path) and os.path.isdir(os.path.join(a.draft_model, "snapshots")):
            raise SystemExit("--require-same-revision: draft and target snapshots differ")
        a.draft_model = d
    device = "cpu" if a.device == "cpu" else "cuda:" + a.device.split(":", 1)[1]
    if a.mlx_cache_limit_bytes is not None and device != "cpu":
        # the tensor engine's caching allocator here is PyTorch's: the limit becomes its per-process cap
        import torch

        idx = int(device.split(":")[1])
        total = torch.cuda.get_device_properties(idx).total_memory
        torch.cuda.set_per_process_memory_fraction(min(1.0, a.mlx_cache_limit_bytes / total), idx)
    quant = None
    bits = a.quantize or (int(quant_suffix) if quant_suffix.isdigit() else None)
    if bits:
        quant = QuantizationOptions(bits=bits, group_size=a.quantization_group_size, mode=a.quantization_mode)
    # ---- automatic planning (--auto plan|quick|benchmark; --no-auto keeps exactly what the flags say)
    plan = None
    report = None
    layerwise, window = a.layerwise_host, a.device_layer_window
    if a.auto_trial_plan:
        # a benchmark trial: the parent's serialized candidate is applied as is, nothing is replanned
        from ..runtime.plan import ExecutionPlan

        plan = ExecutionPlan.from_json(open(a.auto_trial_plan).read())
    elif not a.no_auto:
        from ..runtime.plan import (AutomaticPlanner, ExecutionPlan, HardwareProfile, candidate_plans, estimate_runtime_state,
                                    inspect_artifact, select_from_feedback)

        report = inspect_artifact(model_path)
        if not report.is_loadable:
            for issue in report.issues:
                print(f"[eredu] {issue.severity}: {issue.code}: {issue.message}", file=sys.stderr)
            raise SystemExit(2)
        context = max(4096, a.max_tokens + 2048)
        hw = HardwareProfile.discover() if device != "cpu" else HardwareProfile(device_count=1, device_memory_bytes=1 << 62, name="cpu")
        hw.device_count = 1     # the command-line front end drives one device; multi-GPU runs use the library API
        prof = estimate_runtime_state(report.config, report.tensor_bytes)
        feedback = read_feedback(a.auto_feedback)
        cache_path = a.auto_cache
        key = f"{report.model_type}:{report.tensor_bytes}:{device}:{a.max_tokens}"
        cached = None
        if cache_path and a.auto != "benchmark":
            try:
                cached = json.load(open(cache_path)).get(key)
            except (OSError, ValueError):
                cached = None
        picked = select_from_feedback(feedback, report.model_type, report.tensor_bytes, device) if feedback else None
        if picked is not None:
            plan = picked[0]
            plan.rationale = list(plan.rationale) + [f"selected using {picked[1]} matching runtime sample(s), median "
                                                     f"{picked[2]:.2f} tok/s"]
        elif cached:
            plan = ExecutionPlan.from_json(json.dumps(cached.get("plan", cached)))
        else:
            plan = AutomaticPlanner(hw).plan(report.config, prof, context=context, batch=1,
                                             draft_model=a.draft_model, allow_quantization=quant is None)
        bench_rate = None
        if a.auto == "benchmark":
            cands = candidate_plans(plan, report.config, prof, hw, context=context)
            bench = benchmark_candidates(model_path, a, cands, prompt if a.prompt is not None else AUTO_BENCHMARK_PROMPT)
            plan, bench_rate = bench.pop("_selected_plan"), bench["selected_median_token_rate"]
            if cache_path:
                write_plan_cache(cache_path, key, plan, bench_rate)
            json.dump(bench, sys.stdout, indent=1)
            sys.stdout.write("\n")
            return 0
        if cache_path and not cached and picked is None:
            write_plan_cache(cache_path, key, plan, None)
        if a.auto == "plan":
            json.dump({"schema_version": 2, "model": {"path": model_path, "model_type": report.model_type,
                                                      "tensor_bytes": report.tensor_bytes},
                       "hardware": dataclasses.asdict(hw), "plan": json.loads(plan.to_json()),
                       "explanation": {"summary": "; ".join(plan.rationale), "entries": list(plan.rationale)}}, sys.stdout, indent=1)
            sys.stdout.write("\n")
            return 0
        print("[eredu] automatic plan: " + "; ".join(plan.rationale), file=sys.stderr)
    dense_disk = a.dense_disk_stream
    expert_cache, ec_budget, ec_eviction = a.expert_cache, a.expert_cache_device_budget_bytes, a.expert_cache_eviction
    if plan is not None:
        # explicit flags win over the plan: the plan only fills what the command line left at its default
        wt = plan.weight_transformation
        if quant is None and wt.get("mode") in ("affine", "mxfp4") and device != "cpu":
            quant = QuantizationOptions(bits=wt.get("bits", 4), group_size=wt.get("group_size", 64), mode=wt["mode"])
        mode = plan.residency.get("mode")
        if mode == "layerwise_host" and not (layerwise or dense_disk):
            layerwise, window = True, int(plan.residency.get("device_layer_window", 1))
        elif mode == "dense_disk_stream" and not (layerwise or dense_disk):
            dense_disk = True
            a.dense_host_lookahead = max(1, int(plan.residency.get("host_lookahead") or a.dense_host_lookahead))
            a.dense_background_queue = max(1, int(plan.residency.get("background_queue") or a.dense_background_queue))
        if plan.drafting.get("mode") == "disabled" and a.auto_trial_plan:
            a.mtp_draft_tokens = 0                       # a trial measures exactly its plan
        elif plan.drafting.get("mode") == "embedded" and a.auto_trial_plan:
            a.mtp_draft_tokens = int(plan.drafting.get("max_draft_tokens", a.mtp_draft_tokens))
        if plan.expert_cache and not expert_cache:
            expert_cache = True
            ec_budget = ec_budget or plan.expert_cache.get("device_budget_bytes")
            ec_eviction = plan.expert_cache.get("eviction", ec_eviction)
    t0 = time.perf_counter()
    lm = LoadedModel.load(model_path, ModelLoadOptions(device=device, quantization=quant, mapped_shards=a.mapped_shards,
                                                       max_batch=1, max_seq_len=max(4096, a.max_tokens + 2048),
                                                       weight_residency=("dense_disk_stream" if dense_disk else
                                                                         "layerwise_host" if layerwise else "device"),
                                                       dense_host_lookahead=a.dense_host_lookahead,
                                                       dense_background_queue=a.dense_background_queue,
                                                       host_budget_bytes=a.host_budget_bytes,
                                                       device_layer_window=window,
                                                       embedded_mtp=a.mtp_draft_tokens > 0 and not a.draft_model,
                                                       expert_cache=expert_cache,
                                                       expert_cache_device_budget_bytes=ec_budget,
                                                       expert_cache_eviction=ec_eviction,
                                                       expert_cache_scratch_bytes=a.expert_cache_scratch_bytes,
                                                       expert_cache_prefill_bank_bytes=a.expert_cache_prefill_bank_bytes))
    load_time = time.perf_counter() - t0
    gen_cfg = lm.tokenizer.generation_config if lm.tokenizer else {}
    sp = resolve_sampling(a, gen_cfg)
    if a.verbose:
        print(f"[eredu] loaded {model_path} ({lm.config.model_type}, {lm.model.weight_bytes() / 2**30:.2f} GiB) in "
              f"{load_time:.2f}s on {device}", file=sys.stderr)

    def on_event(ev):
        if ev.kind == "text":
            sys.stdout.write(ev.text)
            sys.stdout.flush()
        elif ev.kind == "reasoning" and a.verbose:
            sys.stderr.write(ev.text)
        elif ev.kind == "tool_call_end":
            sys.stdout.write(json.dumps({"tool_call": {"name": ev.tool_name, "arguments": ev.arguments}}) + "\n")

    if a.image:
        # vision-language prompt: the images come first in the user turn, generation is host-driven
        from ..media import load_image

        images = [load_image(p_) for p_ in a.image]
        content = [{"type": "image"} for _ in images] + [{"type": "text", "text": prompt}]
        segments = lm.chat_segments([{"role": "user", "content": content}], images, thinking=a.thinking) \
            if (lm.tokenizer is not None and lm.tokenizer.chat_template and not a.raw) else images + [prompt]
        from ..text.tokenizer import TextDecoder

        dec = TextDecoder(lm.tokenizer)
        t_gen = time.perf_counter()

        def show(tok):
            sys.stdout.write(dec.push(tok))
            sys.stdout.flush()

        toks = lm.generate_multimodal(segments, sp, a.max_tokens, on_token=show)
        sys.stdout.write(dec.flush() + "\n")
        if a.timing or a.verbose:
            dt = time.perf_counter() - t_gen
            print(f"[eredu] load {load_time:.3f}s  generation {dt:.3f}s  {len(toks) / max(dt, 1e-9):.2f} tok/s  images {len(images)}",
                  file=sys.stderr)
        return 0
    if a.raw or lm.tokenizer is None or not lm.tokenizer.chat_template:
        from ..text.chat import ParserPlan, PreparedChat

        prepared = PreparedChat(prompt=prompt, plan=ParserPlan(), stop=list(a.stop))
    else:
        from ..text.chat import ToolChoice

        tools = json.load(open(a.tools)) if a.tools else None
        prepared = lm.prepare_chat([{"role": "user", "content": prompt}], tools=tools,
                                   tool_choice=ToolChoice(a.tool_choice, a.max_parallel_tool_calls), thinking=a.thinking,
                                   stop=a.stop, allow_unparsed_reasoning=a.allow_unparsed_reasoning)
    mirostat = None
    if a.mirostat_v2:
        from ..ops.controlled import MirostatV2

        if sp.temperature <= 0:
            raise SystemExit("--mirostat-v2 requires an effective temperature greater than zero")
        mirostat = MirostatV2(a.mirostat_tau, a.mirostat_eta, sp.temperature, sp.seed, sp.repeat_penalty, sp.repeat_last_n,
                              sp.frequency_penalty, sp.presence_penalty)
    constraint = None
    given = [(k, v) for k, v in (("json_schema", a.json_schema), ("lark", a.grammar), ("regex", a.regex)) if v]
    if len(given) > 1:
        raise SystemExit("give at most one of --json-schema, --grammar, --regex")
    if given:
        kind, val = given[0]
        constraint = lm.constraint_for(kind, val if kind == "regex" else open(val).read())
    draft = None
    if a.draft_model:
        if mirostat is not None:
            raise SystemExit("--draft-model cannot be combined with --mirostat-v2")
        if _is_gemma4_assistant(a.draft_model):
            lm.attach_assistant(a.draft_model)              # no cache of its own: it reads the target's keys and values
        elif _draft_model_type(a.draft_model) == "muse_glimmer_assistant":
            lm.attach_dflash(a.draft_model)                 # block drafter conditioned on the target's layer outputs
        else:
            draft = LoadedModel.load(a.draft_model, ModelLoadOptions(device=device, max_batch=1,
                                                                      max_seq_len=max(4096, a.max_tokens + 2048)))
            if draft.config.vocab_size != lm.config.vocab_size:
                raise SystemExit("--draft-model must share the target's vocabulary")
    # speculative requests run through the fair scheduler; the two switches shape its lookahead
    from ..runtime.mtp_scheduler import MtpSchedulerOptions

    mtp_options = MtpSchedulerOptions(adaptive_lookahead=not a.disable_mtp_adaptive_lookahead).with_lookahead(
        not a.disable_mtp_lookahead)
    res = lm.generate_prepared_chat(prepared, sp, a.max_tokens, on_event=on_event, raw=a.raw, mirostat=mirostat,
                                    constraint=constraint, draft=draft, draft_tokens=a.mtp_draft_tokens,
                                    embedded_mtp=a.mtp_draft_tokens > 0, mtp_options=mtp_options)
    sys.stdout.write("\n")
    timing = dict(res["timing"], load_time=load_time)
    if a.timing or a.verbose:
        print(f"[eredu] load {load_time:.3f}s  generation {timing['generation_time']:.3f}s  TTFT "
              f"{timing['time_to_first_token']:.3f}s  decode {timing['decode_token_rate']:.2f} tok/s  total "
              f"{timing['token_rate']:.2f} tok/s  stop={res['finish_reason']}", file=sys.stderr)
    components = None
    if a.profile_components:
        from ..runtime.inspection import ComponentProfiler, observed

        prof = ComponentProfiler(lm.model.device)
        ids = lm.tokenizer.encode(prepared.prompt) if lm.tokenizer is not None else [0]
        with observed(lm.model, prof):
            prof.start()
            lm.prefill_logits(ids)
            prof.finish()
        components = prof.summary()
        print("[eredu] prefill components (eager pass over the prompt):", file=sys.stderr)
        for st in components["stages"]:
            print(f"[eredu]   {st['name']:<28} {st['seconds'] * 1e3:9.3f} ms  {st['share'] * 100:5.1f} %", file=sys.stderr)
    if a.telemetry_json:
        tel = ExecutionTelemetry(plan={"device": device, "auto": None if a.no_auto else a.auto, "model_type": lm.config.model_type,
                                       "tensor_bytes": report.tensor_bytes if report is not None else None, "quantization": vars(quant) if quant else None,
                                       "execution_plan": json.loads(plan.to_json()) if plan is not None else None,
                                       "flags": {k: v for k, v in vars(a).items() if k not in ("prompt",)}},
                                 hardware=hardware_profile(device), prompt_tokens=res["prompt_tokens"],
                                 generated_tokens=len(res["tokens"]), stop_reason=res["finish_reason"], timing=timing,
                                 weights_bytes=lm.model.weight_bytes(), kv_bytes=lm.engine.kv.bytes())
        from ..runtime.telemetry import allocator_metrics

        tel.counters["memory"] = allocator_metrics(device)
        store = getattr(lm.source, "store", None)
        if store is not None and hasattr(store, "diagnostics"):
            tel.counters["weight_store"] = dict(store.diagnostics())
        if components is not None:
            tel.counters["components"] = components
        if getattr(lm, "last_speculative_stats", None) is not None:
            tel.plan["speculative"] = lm.last_speculative_stats
        if a.expert_cache_benchmark or a.expert_cache:
            tel.plan["expert_cache"] = [lw.moe.expert_cache.report() for lw in lm.model.layers
                                        if lw.moe is not None and getattr(lw.moe, "expert_cache", None) is not None]
        if lm.model.residency is not None:
            tel.plan["weight_residency"] = lm.model.residency.report()
        tel.write(a.telemetry_json)
    return 0


if __name__ == "__main__":
    sys.exit(main())
