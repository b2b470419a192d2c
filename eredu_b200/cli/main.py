"""``eredu`` command line: load a local model (SafeTensors directory or GGUF file) and generate.

Flag set, defaults and output conventions follow eredu-cli/src/main.rs:209-484 (stdout = generated text, stderr =
diagnostics, ``--telemetry-json PATH`` for the structured report, ``--timing`` for load / TTFT / decode rate as defined
at :667-711). Flags that steer subsystems this runtime plans differently (MLX cache limit, MTP devices, dense disk
streaming ...) are accepted, validated and recorded in the telemetry so that existing invocations keep working.
"""
from __future__ import annotations

import argparse
import json
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


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    validate_args(a)
    prompt = a.prompt if a.prompt is not None else sys.stdin.read()
    from ..api import LoadedModel, ModelLoadOptions, QuantizationOptions
    from ..runtime.telemetry import ExecutionTelemetry, hardware_profile

    model_path, _, quant_suffix = a.model.partition(":")
    device = "cpu" if a.device == "cpu" else "cuda:" + a.device.split(":", 1)[1]
    quant = None
    bits = a.quantize or (int(quant_suffix) if quant_suffix.isdigit() else None)
    if bits:
        quant = QuantizationOptions(bits=bits, group_size=a.quantization_group_size, mode=a.quantization_mode)
    # ---- automatic planning (--auto plan|quick|benchmark; --no-auto keeps exactly what the flags say)
    plan = None
    layerwise, window = a.layerwise_host, a.device_layer_window
    if not a.no_auto:
        from ..runtime.plan import AutomaticPlanner, ExecutionPlan, HardwareProfile, estimate_runtime_state, inspect_artifact

        report = inspect_artifact(model_path)
        if not report.is_loadable:
            for issue in report.issues:
                print(f"[eredu] {issue.severity}: {issue.code}: {issue.message}", file=sys.stderr)
            raise SystemExit(2)
        cache_path = a.auto_cache
        key = f"{report.model_type}:{report.tensor_bytes}:{device}:{a.max_tokens}"
        cached = None
        if cache_path:
            try:
                cached = json.load(open(cache_path)).get(key)
            except (OSError, ValueError):
                cached = None
        if cached:
            plan = ExecutionPlan.from_json(json.dumps(cached))
        else:
            hw = HardwareProfile.discover() if device != "cpu" else HardwareProfile(device_count=1, device_memory_bytes=1 << 62, name="cpu")
            hw.device_count = 1     # the command-line front end drives one device; multi-GPU runs use the library API
            prof = estimate_runtime_state(report.config, report.tensor_bytes)
            plan = AutomaticPlanner(hw).plan(report.config, prof, context=max(4096, a.max_tokens + 2048), batch=1,
                                             draft_model=a.draft_model, allow_quantization=quant is None)
            if cache_path:
                try:
                    book = json.load(open(cache_path))
                except (OSError, ValueError):
                    book = {}
                book[key] = json.loads(plan.to_json())
                json.dump(book, open(cache_path, "w"), indent=1)
        if quant is None and plan.weight_transformation.get("mode") == "affine" and device != "cpu":
            quant = QuantizationOptions(bits=plan.weight_transformation["bits"], group_size=plan.weight_transformation["group_size"])
        if plan.residency.get("mode") == "layerwise_host" and not layerwise:
            layerwise, window = True, int(plan.residency.get("device_layer_window", 1))
        if a.verbose or a.auto == "plan":
            print("[eredu] plan: " + "; ".join(plan.rationale), file=sys.stderr)
    t0 = time.perf_counter()
    lm = LoadedModel.load(model_path, ModelLoadOptions(device=device, quantization=quant, mapped_shards=a.mapped_shards,
                                                       max_batch=1, max_seq_len=max(4096, a.max_tokens + 2048),
                                                       weight_residency=("dense_disk_stream" if a.dense_disk_stream else
                                                                         "layerwise_host" if layerwise else "device"),
                                                       dense_host_lookahead=a.dense_host_lookahead,
                                                       dense_background_queue=a.dense_background_queue,
                                                       host_budget_bytes=a.host_budget_bytes,
                                                       device_layer_window=window,
                                                       expert_cache=a.expert_cache,
                                                       expert_cache_device_budget_bytes=a.expert_cache_device_budget_bytes,
                                                       expert_cache_eviction=a.expert_cache_eviction))
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
        if mirostat is not None or constraint is not None:
            raise SystemExit("--draft-model cannot be combined with --mirostat-v2 or a grammar constraint")
        draft = LoadedModel.load(a.draft_model, ModelLoadOptions(device=device, max_batch=1,
                                                                  max_seq_len=max(4096, a.max_tokens + 2048)))
        if draft.config.vocab_size != lm.config.vocab_size:
            raise SystemExit("--draft-model must share the target's vocabulary")
    res = lm.generate_prepared_chat(prepared, sp, a.max_tokens, on_event=on_event, raw=a.raw, mirostat=mirostat,
                                    constraint=constraint, draft=draft, draft_tokens=a.mtp_draft_tokens)
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
        tel = ExecutionTelemetry(plan={"device": device, "auto": None if a.no_auto else a.auto, "quantization": vars(quant) if quant else None,
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
        if draft is not None:
            tel.plan["speculative"] = getattr(lm, "last_speculative_stats", None)
        if a.expert_cache_benchmark or a.expert_cache:
            tel.plan["expert_cache"] = [lw.moe.expert_cache.report() for lw in lm.model.layers
                                        if lw.moe is not None and getattr(lw.moe, "expert_cache", None) is not None]
        if lm.model.residency is not None:
            tel.plan["weight_residency"] = lm.model.residency.report()
        tel.write(a.telemetry_json)
    return 0


if __name__ == "__main__":
    sys.exit(main())
