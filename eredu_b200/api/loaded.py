"""``LoadedModel``: the user-facing entry point (load -> generate / chat / stream).

Counterpart of ``LoadedModel::{load, generate_tokens, prepare_chat, generate_prepared_chat}``
(eredu/src/api/loaded.rs:154-612, api/portable.rs:138-250) and ``ModelLoadOptions``
(eredu/src/backend/mlx/config.rs:13-49).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Iterator, Optional

import torch

from ..formats.checkpoint import GgufSource, SafetensorsSource, TensorSource, open_checkpoint
from ..models.llama import CausalLM, build_from_tensors
from ..ops.sampling import SamplingParams
from ..runtime.engine import Engine


@dataclass
class QuantizationOptions:
    """Load-time weight quantisation (``--quantize BITS --quantization-mode affine|mxfp4 --quantization-group-size``)."""
    bits: int = 4
    group_size: int = 64
    mode: str = "affine"


@dataclass
class ModelLoadOptions:
    device: str = "cuda" if torch.cuda.is_available() else "cpu"
    dtype: Optional[torch.dtype] = None          # None: bf16 on CUDA, fp32 on CPU
    quantization: Optional[QuantizationOptions] = None
    parallel: object = None                      # ParallelContext
    mapped_shards: int = 4
    max_batch: int = 8
    max_seq_len: int = 4096
    kv_pages: Optional[int] = None
    prefix_cache: bool = False           # later requests lease the published KV pages of an equal prompt prefix
    kv_host_tier_bytes: int = 0          # with prefix_cache: evicted published pages are kept in pinned host memory ...
    kv_disk_tier_dir: Optional[str] = None   # ... and spilled to files in this directory when the host tier is full
    kv_disk_tier_bytes: int = 0
    native_gguf: bool = True                     # keep Q4_K/Q6_K/... blocks and run the native kernels
    use_cuda_graph: Optional[bool] = None
    weight_residency: str = "device"             # "device" | "layerwise_host" | "dense_disk_stream"
    device_layer_window: int = 1                 # layers resident on the device at a time in layerwise_host mode
    dense_host_lookahead: int = 2                # dense_disk_stream: imminent layers kept materialised on the host
    dense_background_queue: int = 2              # dense_disk_stream: pending background disk reads
    dense_spill_dir: Optional[str] = None        # dense_disk_stream: where the prepared layers are written (default: temp)
    host_budget_bytes: Optional[int] = None      # dense_disk_stream: byte cap of the host copies
    expert_cache: bool = False                   # routed experts in host memory behind a bounded device bank
    expert_cache_device_budget_bytes: Optional[int] = None   # per sparse layer; None: a quarter of the experts
    expert_cache_eviction: str = "lru"
    expert_cache_scratch_bytes: int = 1 << 30        # permuted activations of one expert-cache pass (longer inputs are sliced)
    expert_cache_prefill_bank_bytes: int = 1 << 30   # transient expert bank of prompt-sized calls
    embedded_mtp: bool = True                    # bind the checkpoint's own prediction layer (when it has one) as a drafter


class LoadedModel:
    def __init__(self, model: CausalLM, engine: Engine, source: TensorSource, tokenizer=None, path=None):
        self.model = model
        self.engine = engine
        self.source = source
        self.tokenizer = tokenizer
        self.path = path
        self.config = model.cfg

    # ------------------------------------------------------------------------------------------ load
    @classmethod
    def load_execution_plan(cls, path: str | Path, plan, options: Optional[ModelLoadOptions] = None) -> "LoadedModel":
        """Load a checkpoint the way an :class:`runtime.plan.ExecutionPlan` says (``load_execution_plan``,
        eredu/src/api/loaded.rs): weight transformation, residency form, expert cache and drafting come from the plan;
        everything the plan does not name (device, batch, context, ...) comes from ``options``. A plan over several
        ranks needs ``options.parallel`` bound to a topology of the same shape (one process per GPU); a mismatch is an
        error, not a silent single-rank load."""
        import dataclasses

        plan.validate()
        opt = dataclasses.replace(options) if options is not None else ModelLoadOptions()
        topo = plan.topology
        world = int(topo.get("pipeline", 1)) * int(topo.get("tensor", 1)) * (
            1 if topo.get("expert_over_tensor") else int(topo.get("expert", 1)))
        if int(topo.get("data", 1)) != 1:
            raise ValueError("execution plan asks for data parallelism, which is declared but unsupported")
        if world > 1:
            par = opt.parallel
            have = None if par is None else (par.topology.pipeline, par.topology.tensor, par.topology.expert,
                                             bool(par.topology.expert_over_tensor))
            want = (int(topo.get("pipeline", 1)), int(topo.get("tensor", 1)), int(topo.get("expert", 1)),
                    bool(topo.get("expert_over_tensor")))
            if have != want:
                raise ValueError(f"execution plan needs the topology (pipeline, tensor, expert, shared) = {want}; "
                                 f"options.parallel is bound to {have}")
        wt = plan.weight_transformation
        if wt.get("mode") in ("affine", "mxfp4") and opt.quantization is None and torch.device(opt.device).type == "cuda":
            opt.quantization = QuantizationOptions(bits=int(wt.get("bits", 4)), group_size=int(wt.get("group_size", 64)),
                                                   mode=wt["mode"])
        mode = plan.residency.get("mode")
        if mode == "layerwise_host":
            opt.weight_residency = "layerwise_host"
            opt.device_layer_window = int(plan.residency.get("device_layer_window", 1))
        elif mode == "dense_disk_stream":
            opt.weight_residency = "dense_disk_stream"
            opt.dense_host_lookahead = max(1, int(plan.residency.get("host_lookahead") or opt.dense_host_lookahead))
            opt.dense_background_queue = max(1, int(plan.residency.get("background_queue") or opt.dense_background_queue))
        if plan.residency.get("host_budget_bytes"):
            opt.host_budget_bytes = int(plan.residency["host_budget_bytes"])
        if plan.expert_cache:
            opt.expert_cache = True
            opt.expert_cache_device_budget_bytes = plan.expert_cache.get("device_budget_bytes") or opt.expert_cache_device_budget_bytes
            opt.expert_cache_eviction = plan.expert_cache.get("eviction", opt.expert_cache_eviction)
        opt.mapped_shards = int(plan.max_mapped_shards)
        opt.embedded_mtp = plan.drafting.get("mode") == "embedded"
        lm = cls.load(path, opt)
        lm.execution_plan = plan
        return lm

    @classmethod
    def plan_and_load(cls, path: str | Path, options: Optional[ModelLoadOptions] = None, hardware=None, context: int = 4096,
                      batch: int = 1, allow_quantization: bool = True) -> "LoadedModel":
        """Inspect the checkpoint header, let the automatic planner choose topology, transformation and residency for
        this node, and load accordingly (``plan_and_load``, eredu/src/api/loaded.rs). Single-process callers get the
        single-device plan; a process that is one rank of a group passes ``options.parallel`` and gets the plan of that
        topology. The chosen plan is kept as ``execution_plan`` on the result."""
        from ..runtime.plan import AutomaticPlanner, HardwareProfile, estimate_runtime_state, inspect_artifact

        opt = options or ModelLoadOptions()
        report = inspect_artifact(str(path))
        if not report.is_loadable:
            raise ValueError("checkpoint is not loadable: " + "; ".join(f"{i.code}: {i.message}" for i in report.issues))
        on_cpu = torch.device(opt.device).type != "cuda"
        hw = hardware or (HardwareProfile(device_count=1, device_memory_bytes=1 << 62, name="cpu") if on_cpu
                          else HardwareProfile.discover())
        par = opt.parallel
        ranks = 1 if par is None else par.topology.tensor
        hw.device_count = max(1, ranks)                  # this process drives one device of `ranks`
        prof = estimate_runtime_state(report.config, report.tensor_bytes)
        plan = AutomaticPlanner(hw).plan(report.config, prof, context=context, batch=batch,
                                         allow_quantization=allow_quantization and opt.quantization is None and not on_cpu,
                                         prefer_devices=ranks if ranks > 1 else None)
        if par is not None and ranks > 1:
            plan.topology.update({"pipeline": par.topology.pipeline, "expert": par.topology.expert,
                                  "expert_over_tensor": bool(par.topology.expert_over_tensor)})
        return cls.load_execution_plan(path, plan, opt)

    @classmethod
    def load(cls, path: str | Path, options: Optional[ModelLoadOptions] = None) -> "LoadedModel":
        opt = options or ModelLoadOptions()
        src = open_checkpoint(path, opt.mapped_shards)
        device = torch.device(opt.device)
        dtype = opt.dtype or (torch.bfloat16 if device.type == "cuda" else torch.float32)
        moe_factory = None
        if src.cfg.model_type in ("deepseek_v4", "inkling_mm_model"):
            return cls._load_unpaged(path, src, opt, device, dtype)
        if src.cfg.is_moe:
            from ..models.moe import make_moe_factory

            moe_factory = make_moe_factory(src)
        quantizer = None
        if device.type == "cuda":
            from ..ops.quant import make_quantizer

            quantizer = make_quantizer(src, opt)
        residency = None
        on_layer = None
        if opt.weight_residency == "layerwise_host":
            from ..runtime.weight_residency import LayerwiseHostResidency

            def on_layer(m, li, lw):
                nonlocal residency
                if residency is None:
                    residency = LayerwiseHostResidency(m, opt.device_layer_window, defer=True)
                residency.adopt_layer(lw)
        elif opt.weight_residency == "dense_disk_stream":
            from ..runtime.weight_residency import DiskStreamResidency

            def on_layer(m, li, lw):
                nonlocal residency
                if residency is None:
                    residency = DiskStreamResidency(m, opt.dense_host_lookahead, opt.dense_background_queue,
                                                    opt.dense_spill_dir, opt.host_budget_bytes, defer=True)
                residency.adopt_layer(lw)
        elif opt.weight_residency != "device":
            raise ValueError(f"unknown weight residency {opt.weight_residency!r}")
        get, has = src.get, src.has
        if has("model.language_model.embed_tokens.weight") and not has("model.embed_tokens.weight"):
            # vision-language checkpoint used as a text model: the decoder sits under model.language_model.*, the towers
            # are not loaded (requests with image / audio / video parts are refused by media.prepare_for_text_model)
            base_get, base_has = get, has

            def _lm(name):
                return "model.language_model." + name[len("model."):] if name.startswith("model.") else name

            get = lambda name: base_get(_lm(name)) if base_has(_lm(name)) else base_get(name)      # noqa: E731
            has = lambda name: base_has(_lm(name)) or base_has(name)                                # noqa: E731
        if src.cfg.model_type in ("lfm2", "lfm2_moe"):
            from ..models.lfm2 import canonical_access

            get, has = canonical_access(get, has)
        elif src.cfg.model_type == "kimi_linear":
            from ..models.kimi_linear import canonical_access

            get, has = canonical_access(get, has)
        elif src.cfg.model_type == "nemotron_h":
            from ..models.nemotron_h import canonical_access

            get, has = canonical_access(get, has)
        model = build_from_tensors(src.cfg, get, has, device, dtype, opt.parallel, moe_factory, quantizer,
                                   on_layer=on_layer)
        if residency is not None:
            residency.finalize()
        if opt.expert_cache and src.cfg.is_moe:
            from ..runtime.expert_cache import attach_expert_cache

            sizing = dict(eviction=opt.expert_cache_eviction, scratch_bytes=opt.expert_cache_scratch_bytes,
                          prefill_bank_bytes=opt.expert_cache_prefill_bank_bytes)
            if opt.expert_cache_device_budget_bytes:
                attach_expert_cache(model, device_budget_bytes=opt.expert_cache_device_budget_bytes, **sizing)
            else:
                attach_expert_cache(model, slots=max(1, src.cfg.num_experts // 4), **sizing)
        if opt.parallel is not None and opt.parallel.tp_size > 1:
            from ..parallel import tp

            tp.attach(model, opt.parallel)
        engine = Engine(model, max_batch=opt.max_batch, max_seq_len=opt.max_seq_len, num_pages=opt.kv_pages,
                        use_cuda_graph=opt.use_cuda_graph, prefix_cache=opt.prefix_cache,
                        kv_host_tier_bytes=opt.kv_host_tier_bytes, kv_disk_tier_dir=opt.kv_disk_tier_dir,
                        kv_disk_tier_bytes=opt.kv_disk_tier_bytes)
        tokenizer = None
        try:
            from ..text.tokenizer import load_tokenizer

            tokenizer = load_tokenizer(path, src)
        except Exception:
            tokenizer = None
        lm = cls(model, engine, src, tokenizer, Path(path))
        lm.mtp, lm.mtp_error = None, None
        if src.cfg.mtp_layers > 0 and opt.embedded_mtp and (opt.parallel is None or opt.parallel.tp_size * opt.parallel.pp_size * opt.parallel.ep_size == 1) \
                and residency is None:
            from ..models.mtp import build_embedded_mtp

            try:
                lm.mtp = build_embedded_mtp(src.cfg, get, has, model, device, dtype, moe_factory, quantizer)
            except (RuntimeError, KeyError, ValueError) as e:
                lm.mtp_error = f"embedded prediction layer not loaded: {e}"     # the model itself is unaffected
        vis = src.cfg.extra.get("vision")
        if vis and src.cfg.model_type == "gemma4" and src.has("model.vision_tower.patch_embedder.input_proj.weight") \
                and (opt.parallel is None or opt.parallel.owns_embedding()):
            from ..models.gemma4_vision import Gemma4VisionConfig, Gemma4VisionTower

            try:
                lm.vision = Gemma4VisionTower(Gemma4VisionConfig.from_dict(vis["vision_config"]), src.get, src.has, device,
                                              torch.float32 if device.type == "cpu" else dtype)
                lm.vision_tokens = {k: vis.get(k) for k in ("image_token_id", "video_token_id", "boi_token_id", "eoi_token_id")}
            except (RuntimeError, KeyError, ValueError) as e:
                lm.vision, lm.vision_error = None, f"vision tower not loaded: {e}"
        if vis and vis.get("audio_config") and src.cfg.model_type == "gemma4" \
                and src.has("model.audio_tower.subsample_conv_projection.input_proj_linear.weight") \
                and (opt.parallel is None or opt.parallel.owns_embedding()):
            from ..models.gemma4_audio import Gemma4AudioConfig, Gemma4AudioTower

            try:
                lm.audio = Gemma4AudioTower(Gemma4AudioConfig.from_dict(vis["audio_config"]), src.get, src.has, device,
                                            torch.float32 if device.type == "cpu" else dtype)
                lm.audio_tokens = {"audio_token_id": vis.get("audio_token_id"), "boa_token_id": vis.get("boa_token_id"),
                                   "eoa_token_id": vis.get("eoa_token_id", vis.get("eoa_token_index"))}
            except (RuntimeError, KeyError, ValueError) as e:
                lm.audio, lm.audio_error = None, f"audio tower not loaded: {e}"
        if vis and src.cfg.model_type == "muse_glimmer" and src.has("model.vision_tower.patch_embedder.patch_embedding.weight") \
                and (opt.parallel is None or opt.parallel.owns_embedding()):
            from ..models.muse_glimmer_vision import load_muse_glimmer_vision, load_processor

            try:
                lm.vision = load_muse_glimmer_vision(vis, src.cfg.hidden_size, src.get, src.has, device,
                                                     torch.float32 if device.type == "cpu" else dtype)
                lm.vision_tokens = {k: vis.get(k) for k in ("image_token_id", "video_token_id")}
                lm.vision_processor = load_processor(path)
            except (RuntimeError, KeyError, ValueError) as e:
                lm.vision, lm.vision_error = None, f"vision tower not loaded: {e}"
        if lm.vision is not None:
            pass
        elif vis and src.has("model.visual.patch_embed.proj.weight") and (opt.parallel is None or opt.parallel.owns_embedding()):
            from ..models.qwen_vl import VisionConfig, VisionTower

            try:
                lm.vision = VisionTower(VisionConfig.from_dict(vis["vision_config"]), src.get, device, torch.float32
                                        if device.type == "cpu" else dtype)
                lm.vision_tokens = {k: vis.get(k) for k in ("image_token_id", "video_token_id", "vision_start_token_id",
                                                            "vision_end_token_id")}
            except (RuntimeError, KeyError, ValueError) as e:
                # a tower this loader cannot bind (other family, truncated export): the model stays usable for text
                # and image parts are refused with this reason
                lm.vision, lm.vision_error = None, f"vision tower not loaded: {e}"
        return lm

    # ------------------------------------------------------------------------------------------ tokens
    def encode(self, text: str) -> list[int]:
        if self.tokenizer is None:
            raise RuntimeError("this checkpoint has no tokenizer")
        return self.tokenizer.encode(text)

    def decode(self, ids) -> str:
        if self.tokenizer is None:
            raise RuntimeError("this checkpoint has no tokenizer")
        return self.tokenizer.decode(list(ids))

    def eos_ids(self) -> tuple:
        e = self.config.eos_token_id
        if e is None:
            return ()
        return tuple(e) if isinstance(e, (list, tuple)) else (int(e),)

    def generate_tokens(self, prompt_ids, sampling: Optional[SamplingParams] = None, max_new_tokens: int = 256,
                        stop_on_eos: bool = True) -> Iterator[int]:
        """Raw token iterator (``generate_tokens``, api/portable.rs:224): yields ids as they are committed."""
        out: list[int] = []
        self.engine.generate([list(prompt_ids)], sampling or SamplingParams(), max_new_tokens,
                             eos_ids=self.eos_ids() if stop_on_eos else (), on_token=lambda i, t: out.append(t))
        yield from out

    def generate(self, prompts, sampling: Optional[SamplingParams] = None, max_new_tokens: int = 256):
        return self.engine.generate([list(p) for p in prompts], sampling or SamplingParams(), max_new_tokens,
                                    eos_ids=self.eos_ids())

    @torch.no_grad()
    def prefill_logits(self, prompt_ids) -> torch.Tensor:
        """Logits of the last prompt position (fp32, [V]) - the probe the parity harness compares."""
        import numpy as np

        from ..models.llama import ForwardBatch
        from ..runtime.kv_cache import PAGE

        eng = self.engine
        seq = eng.new_sequence(list(prompt_ids), max_new_tokens=1)
        if not getattr(eng, "paged", True):
            try:
                return eng.prefill_logits([seq])[0].float().cpu()
            finally:
                eng.release(seq)
        try:
            n = len(seq.prompt)
            p = np.arange(n)
            pages = np.asarray(seq.pages, dtype=np.int64)
            batch = ForwardBatch(
                token_ids=eng._t(np.asarray(seq.prompt, dtype=np.int32), torch.int32),
                positions=eng._t(p.astype(np.int32), torch.int32),
                slots=eng._t(pages[p // PAGE] * PAGE + (p % PAGE), torch.int64),
                block_table=eng._block_table([seq]), seq_lens=eng._t(np.asarray([n], dtype=np.int32), torch.int32),
                is_prefill=True, cu_q=eng._t(np.asarray([0, n], dtype=np.int32), torch.int32), max_q_len=n,
                logit_rows=eng._t(np.asarray([n - 1], dtype=np.int64), torch.int64))
            return self.model.forward(batch, eng.kv)[0].float().cpu()
        finally:
            eng.release(seq)

    # ------------------------------------------------------------------------------------------ multimodal
    vision = None          # models.qwen_vl.VisionTower when the checkpoint carries an image tower
    audio = None           # models.gemma4_audio.Gemma4AudioTower when the checkpoint carries an audio tower
    audio_tokens: dict = {}
    audio_error: str = ""
    vision_tokens: dict = {}
    vision_error: str = ""

    def multimodal_inputs(self, segments: list, min_pixels: int = 64 * 32 * 32, max_pixels: int = 16384 * 32 * 32,
                          wrap: bool = True, video_limits: Optional[dict] = None, image_limits: Optional[dict] = None):
        """Token ids and tower features of a prompt made of text segments (``str`` or lists of token ids) and
        ``media.RgbImage`` / ``media.Video`` parts (``video_limits``: keyword arguments of ``video_to_patches``; a video
        becomes one timestamped, framed placeholder run per temporal group): every image becomes ``<vision_start> <image> x n <vision_end>`` and its merged patch
        features replace the placeholder embeddings (``wrap=False``: the surrounding text, e.g. a rendered chat template,
        already carries the start / end markers and only the placeholder run is inserted).
        Returns (token_ids, multimodal dict for ``Engine.feed_logits``)."""
        from ..media import MultimodalPreparationError, RgbImage
        from ..media.request import Video
        from ..models.qwen_vl import image_to_patches, mrope_positions, video_to_patches

        if self.config.model_type == "inkling_mm_model":
            return self._inkling_inputs(segments)
        if self.config.model_type == "muse_glimmer" and self.vision is not None:
            return self._muse_glimmer_inputs(segments, wrap, (video_limits or {}).get("frame_count"))
        if self.config.model_type == "gemma4" and (self.vision is not None or self.audio is not None):
            return self._gemma4_inputs(segments, wrap, **(image_limits or {}))
        if self.vision is None:
            kinds = sorted({"image" if isinstance(s, RgbImage) else "video" for s in segments if isinstance(s, (RgbImage, Video))})
            if kinds:
                raise MultimodalPreparationError(f"this model accepts text only; the request carries {kinds}"
                                                 + (f" ({self.vision_error})" if self.vision_error else ""))
            ids = [t for s in segments for t in (self.encode(s) if isinstance(s, str) else list(s))]
            return ids, None
        if self.config.model_type == "gemma4":
            return self._gemma4_inputs(segments, wrap, **(image_limits or {}))
        vt, cfg = self.vision_tokens, self.vision.cfg
        ids, patches, grids = [], [], []          # grids: what the tower sees; lm_grids: one entry per placeholder run
        lm_grids = []
        for seg in segments:
            if isinstance(seg, Video):
                # every temporal group is announced by its time and framed like an image of its own
                if vt.get("video_token_id") is None:
                    raise MultimodalPreparationError("this checkpoint declares no video placeholder token")
                p, g, stamps = video_to_patches(seg, cfg, **(video_limits or {}))
                per = (g[1] // cfg.spatial_merge_size) * (g[2] // cfg.spatial_merge_size)
                for stamp in stamps:
                    if self.tokenizer is not None:
                        ids.extend(self.encode(f"<{stamp:.1f} seconds>"))
                    if vt.get("vision_start_token_id") is not None:
                        ids.append(int(vt["vision_start_token_id"]))
                    ids.extend([int(vt["video_token_id"])] * per)
                    if vt.get("vision_end_token_id") is not None:
                        ids.append(int(vt["vision_end_token_id"]))
                    lm_grids.append((1, g[1], g[2]))
                patches.append(p)
                grids.append(g)
            elif isinstance(seg, RgbImage):
                p, g = image_to_patches(seg, cfg, min_pixels, max_pixels)
                n = g[0] * (g[1] // cfg.spatial_merge_size) * (g[2] // cfg.spatial_merge_size)
                if wrap and vt.get("vision_start_token_id") is not None:
                    ids.append(int(vt["vision_start_token_id"]))
                ids.extend([int(vt["image_token_id"])] * n)
                if wrap and vt.get("vision_end_token_id") is not None:
                    ids.append(int(vt["vision_end_token_id"]))
                patches.append(p)
                grids.append(g)
                lm_grids.append(g)
            else:
                ids.extend(self.encode(seg) if isinstance(seg, str) else [int(t) for t in seg])
        if not grids:
            return ids, None
        feats, deep = self.vision.forward(torch.cat(patches, 0), grids)
        marks = {int(vt[k]) for k in ("image_token_id", "video_token_id") if vt.get(k) is not None}
        pos, delta = mrope_positions(ids, marks, lm_grids, cfg.spatial_merge_size)
        rows = [i for i, t in enumerate(ids) if t in marks]
        return ids, {"rows": rows, "values": feats, "deepstack": deep, "rope_positions": pos, "rope_delta": delta}

    def _gemma4_inputs(self, segments: list, wrap: bool, max_soft_tokens: int = 280):
        """Gemma 4: an image is ``<boi> <image> x n <eoi>``; the placeholders are embedded as the padding token (also for the
        per-layer inputs), their rows take the tower's soft tokens, and the soft tokens of one image form a
        bidirectional-attention group."""
        from ..media import MultimodalPreparationError, RgbImage
        from ..media.audio import AudioWaveform, LogMelConfig, LogMelFeatures, extract_log_mel
        from ..models.gemma4_vision import image_to_patches

        vt = self.vision_tokens
        pad = int((self.config.extra.get("gemma4") or {}).get("pad_token_id") or 0)
        ids, rows, groups, feats = [], [], [], []
        for seg in segments:
            if isinstance(seg, (AudioWaveform, LogMelFeatures)) or (isinstance(seg, torch.Tensor) and seg.dim() == 2):
                # an audio clip is <boa> <audio> x n <eoa>: log-mel frames -> tower -> embedder; its soft tokens attend
                # causally like text (only vision tokens form bidirectional groups)
                if self.audio is None:
                    raise MultimodalPreparationError("this checkpoint has no audio tower"
                                                     + (f" ({self.audio_error})" if self.audio_error else ""))
                if isinstance(seg, AudioWaveform):
                    seg = extract_log_mel(seg, LogMelConfig())
                mel = torch.as_tensor(seg.values[seg.mask] if isinstance(seg, LogMelFeatures) else seg, dtype=torch.float32)
                soft = self.audio.forward(mel).to(self.model.dtype)
                at = self.audio_tokens
                if wrap and at.get("boa_token_id") is not None:
                    ids.append(int(at["boa_token_id"]))
                    groups.append(-1)
                rows.extend(range(len(ids), len(ids) + soft.shape[0]))
                ids.extend([pad] * soft.shape[0])
                groups.extend([-1] * soft.shape[0])
                feats.append(soft)
                if wrap and at.get("eoa_token_id") is not None:
                    ids.append(int(at["eoa_token_id"]))
                    groups.append(-1)
                continue
            if isinstance(seg, RgbImage):
                if self.vision is None:
                    raise MultimodalPreparationError("this checkpoint has no vision tower"
                                                     + (f" ({self.vision_error})" if self.vision_error else ""))
                patches, pos, n = image_to_patches(seg, self.vision.cfg, max_soft_tokens)
                soft = self.vision.forward(patches, pos)
                if wrap and vt.get("boi_token_id") is not None:
                    ids.append(int(vt["boi_token_id"]))
                    groups.append(-1)
                rows.extend(range(len(ids), len(ids) + n))
                ids.extend([pad] * n)
                groups.extend([len(feats)] * n)
                feats.append(soft)
                if wrap and vt.get("eoi_token_id") is not None:
                    ids.append(int(vt["eoi_token_id"]))
                    groups.append(-1)
            elif isinstance(seg, (str, list, tuple)):
                new = self.encode(seg) if isinstance(seg, str) else [int(t) for t in seg]
                ids.extend(new)
                groups.extend([-1] * len(new))
            else:
                raise MultimodalPreparationError(f"this model accepts text and images; the request carries {type(seg).__name__}")
        if not feats:
            return ids, None
        bidir = groups if ((self.config.extra.get("gemma4") or {}).get("use_bidirectional_attention") == "vision"
                           and any(g >= 0 for g in groups)) else None
        placeholder = vt.get("image_token_id") if vt else None
        if placeholder is None:
            placeholder = self.audio_tokens.get("audio_token_id")
        return ids, {"rows": rows, "values": torch.cat([f.to(feats[0].dtype) for f in feats], 0), "deepstack": None,
                     "rope_positions": None, "rope_delta": 0, "bidir_groups": bidir, "placeholder_id": int(placeholder)}

    def _muse_glimmer_inputs(self, segments: list, wrap: bool, frame_count=None):
        """Muse-Glimmer prompt parts (``prepare_input``, eredu/src/backend/mlx/architectures/muse_glimmer/processor.rs:
        190-310): an image becomes ``<|image_start|>``, one placeholder per merged patch, ``<|image_end|>``; a video
        becomes ``<|vid_start|>`` and, per temporal group, ``Time: x.xs``, its placeholders and a frame separator (the
        last group closes with ``<|vid_end|>``). ``wrap=False`` leaves the marker text to the caller's template."""
        from ..media import MultimodalPreparationError, RgbImage
        from ..media.request import Video
        from ..models.muse_glimmer_vision import image_to_patches, video_to_groups

        image_cfg, video_cfg = self.vision_processor
        vt, m = self.vision_tokens, self.vision.cfg.merge_size
        ids, rows, patches, grids = [], [], [], []
        mark = (lambda text: ids.extend(self.encode(text))) if wrap else (lambda text: None)

        def media(token, p, grid):
            if token is None:
                raise MultimodalPreparationError("this checkpoint declares no placeholder token for that medium")
            n = grid[0] * (grid[1] // m) * (grid[2] // m)
            rows.extend(range(len(ids), len(ids) + n))
            ids.extend([int(token)] * n)
            patches.append(p)
            grids.append(grid)

        for seg in segments:
            if isinstance(seg, str):
                ids.extend(self.encode(seg))
            elif isinstance(seg, RgbImage):
                mark("<|image_start|>")
                media(vt.get("image_token_id"), *image_to_patches(seg, image_cfg))
                mark("<|image_end|>")
            elif isinstance(seg, Video):
                groups = video_to_groups(seg, video_cfg, frame_count)
                mark("<|vid_start|>")
                for gi, (seconds, p, grid) in enumerate(groups):
                    mark(f"Time: {seconds:.1f}s")
                    media(vt.get("video_token_id"), p, grid)
                    mark("<|vid_end|>" if gi + 1 == len(groups) else "<|vid_frame_separator|>")
            elif isinstance(seg, (list, tuple)):
                ids.extend(int(t) for t in seg)
            else:
                raise MultimodalPreparationError(f"Muse-Glimmer processor does not support parts of type {type(seg).__name__}")
        if not rows:
            return ids, None
        values = self.vision(torch.cat(patches), grids)
        return ids, {"rows": torch.tensor(rows, dtype=torch.int64), "values": values, "deepstack": None,
                     "rope_positions": None, "rope_delta": 0}

    def _inkling_inputs(self, segments: list):
        """Typed prompt parts of the Inkling family (``prepare_typed_input``, eredu/src/backend/mlx/architectures/inkling/
        layerwise.rs:2680-2760): text (``str`` or token ids), ``media.RgbImage`` (one placeholder per 40 x 40 patch, the
        hMLP tower's soft tokens), ``{"audio_ids": [frames, codebooks]}`` with an optional ``"valid_frames"`` (summed
        codebook embeddings) and ready ``{"image_embeds": ...}`` / ``{"audio_embeds": ...}`` rows of the decoder's width.
        Returns (token_ids, (rows, values)) for ``UnpagedEngine.feed_logits``."""
        from ..media import MultimodalPreparationError, RgbImage
        import numpy as np

        from ..models.inkling import image_patches

        extra = {**self.config.extra["inkling"], **self.config.extra.get("vision", {})}   # nested configs keep them outside
        image_id, audio_id = int(extra.get("image_token_id", 200054)), int(extra.get("audio_token_id", 200053))
        hidden = int(self.engine.model.cfg.hidden_size)
        ids, rows, vals = [], [], []

        def soft(token, emb):
            if emb.dim() != 2 or emb.shape[1] != hidden:
                raise MultimodalPreparationError(f"media embeddings must be [tokens, {hidden}], got {tuple(emb.shape)}")
            rows.extend(range(len(ids), len(ids) + emb.shape[0]))
            ids.extend([token] * emb.shape[0])
            vals.append(emb.to(self.engine.device, self.engine.model.dtype))

        for seg in segments:
            if isinstance(seg, str):
                ids.extend(self.encode(seg))
            elif isinstance(seg, RgbImage):
                if self.vision is None:
                    raise MultimodalPreparationError("Inkling image input requires vision_config and vision weights")
                soft(image_id, self.vision(image_patches(torch.from_numpy(np.ascontiguousarray(seg.pixels)))))
            elif isinstance(seg, dict) and "audio_ids" in seg:
                if self.audio is None:
                    raise MultimodalPreparationError("Inkling audio input requires audio_config and audio weights")
                soft(audio_id, self.audio(torch.as_tensor(seg["audio_ids"]), seg.get("valid_frames")))
            elif isinstance(seg, dict) and ("image_embeds" in seg or "audio_embeds" in seg):
                kind = "image_embeds" if "image_embeds" in seg else "audio_embeds"
                soft(image_id if kind == "image_embeds" else audio_id, torch.as_tensor(seg[kind]))
            elif isinstance(seg, (list, tuple)):
                ids.extend(int(t) for t in seg)
            else:
                raise MultimodalPreparationError(f"Inkling input does not support parts of type {type(seg).__name__}")
        if not rows:
            return ids, None
        return ids, (torch.tensor(rows, dtype=torch.int64), torch.cat(vals))

    def chat_segments(self, messages: list, images: list, placeholder: str = "<|image_pad|>", **template_kwargs) -> list:
        """Render a conversation whose user content lists contain ``{"type": "image"}`` items with the chat template and
        cut the prompt at the template's image placeholders: text pieces interleaved with ``images`` in order (for
        :meth:`multimodal_inputs` with ``wrap=False``)."""
        prepared = self.prepare_chat(messages, **template_kwargs)
        pieces = prepared.prompt.split(placeholder)
        if len(pieces) - 1 != len(images):
            raise ValueError(f"the rendered prompt has {len(pieces) - 1} image placeholders for {len(images)} images")
        segments = []
        for i, piece in enumerate(pieces):
            if piece:
                segments.append(piece)
            if i < len(images):
                segments.append(images[i])
        return segments

    def generate_multimodal(self, segments: list, sampling: Optional[SamplingParams] = None, max_new_tokens: int = 128,
                            on_token=None, **image_limits) -> list[int]:
        """Greedy / sampled continuation of a prompt with images (host-driven: one eager step per token)."""
        from ..ops.sampling import sample_ref

        ids, mm = self.multimodal_inputs(segments, **image_limits)
        sp = sampling or SamplingParams(temperature=0.0)
        eos = set(self.eos_ids()) | (set(self.tokenizer.eos_ids) if self.tokenizer else set())
        seq = self.engine.new_sequence(ids, sp, max_new_tokens, tuple(eos))
        out: list[int] = []
        try:
            logits = self.engine.feed_logits(seq, ids, mm)
            for step in range(max_new_tokens):
                tok, _ = sample_ref(logits.float().cpu(), sp, len(ids) + step, history=out, stream=seq.seq_id)
                if tok in eos:
                    break
                out.append(tok)
                if on_token is not None and on_token(tok):
                    break
                if step + 1 < max_new_tokens:
                    logits = self.engine.step_logits(seq, tok)
        finally:
            self.engine.release(seq)
        return out

    # ------------------------------------------------------------------------------------------ chat
    def prepare_chat(self, messages, tools=None, tool_choice=None, thinking: str = "auto", stop=None,
                     allow_unparsed_reasoning: bool = False, **template_kwargs):
        """Render a conversation with the checkpoint's chat template (``prepare_chat``, api/loaded.rs:426)."""
        from ..text.chat import prepare_chat

        tb = self.tokenizer
        return prepare_chat(messages, template=tb.chat_template if tb else None, bos_token=tb.bos_token if tb else "",
                            eos_token=tb.eos_token if tb else "", tools=tools, tool_choice=tool_choice,
                            thinking=thinking, stop=stop, allow_unparsed_reasoning=allow_unparsed_reasoning,
                            **template_kwargs)

    def constraint_for(self, kind: str, spec):
        """Grammar constraint over this model's tokenizer: ``kind`` is "json_schema", "lark" or "regex"
        (response_format / structured tool arguments; eredu/src/backend/mlx/runtime/chat/constraints.rs)."""
        from ..ops.controlled import GrammarConstraint

        if self.tokenizer is None:
            raise RuntimeError("this checkpoint has no tokenizer")
        return GrammarConstraint(self.tokenizer, kind, spec)

    @classmethod
    def _load_unpaged(cls, path, src, opt, device, dtype):
        """Families whose cache is not a paged K / V pool run on ``runtime.unpaged.UnpagedEngine`` (text generation, chat,
        logits; no batching, parallelism, residency tiers, prefix reuse or speculation)."""
        from ..runtime.unpaged import UnpagedEngine

        par = opt.parallel
        if par is not None and par.tp_size * par.pp_size * par.ep_size > 1:
            raise NotImplementedError(f"{src.cfg.model_type}: tensor / pipeline / expert parallelism is not built for this family")
        if opt.weight_residency != "device" or opt.expert_cache or opt.prefix_cache:
            raise NotImplementedError(f"{src.cfg.model_type}: weight residency tiers, expert caches and prefix reuse are not built for this family")
        if src.cfg.model_type == "inkling_mm_model":
            from ..models.inkling import InklingConfig, InklingModel

            model = InklingModel(InklingConfig.from_dict(src.cfg.extra["inkling"]), src.get, src.has, device, dtype)
        else:
            from ..models.deepseek_v4 import DeepseekV4Config, DeepseekV4Model

            model = DeepseekV4Model(DeepseekV4Config.from_dict(src.cfg.extra["deepseek_v4"]), src.get, src.has, device, dtype)
        model.par = None
        engine = UnpagedEngine(model, max_batch=1, max_seq_len=opt.max_seq_len)
        engine.cfg = src.cfg
        tokenizer = None
        try:
            from ..text.tokenizer import load_tokenizer

            tokenizer = load_tokenizer(path, src)
        except Exception:
            tokenizer = None
        lm = cls(model, engine, src, tokenizer, Path(path))
        lm.config = src.cfg
        lm.mtp, lm.mtp_error = None, None
        lm.vision = lm.audio = None
        if src.cfg.model_type == "inkling_mm_model":
            from ..models.inkling import InklingAudio, InklingVision

            raw = {**src.cfg.extra["inkling"], **src.cfg.extra.get("vision", {})}
            hidden = int(model.cfg.hidden_size)
            if raw.get("vision_config") and (src.has("visual.final_norm.weight") or src.has("model.visual.final_norm.weight")):
                lm.vision = InklingVision({"text_hidden_size": hidden, **raw["vision_config"]}, src.get, src.has, device, dtype)
            if raw.get("audio_config") and (src.has("audio.encoder.weight") or src.has("model.audio.encoder.weight")):
                lm.audio = InklingAudio(raw["audio_config"], src.get, src.has, device, dtype)
        return lm

    def attach_dflash(self, path) -> None:
        """Load a DFlash block drafter (the assistant released with Muse-Glimmer) next to this model."""
        from ..models.dflash import load_dflash

        self.dflash = load_dflash(path, self.engine.device, self.engine.model.dtype)

    def attach_assistant(self, path) -> None:
        """Load a Gemma 4 assistant drafter (its own directory) next to this model: speculative generation then drafts
        with it (``load_gemma4_assistant_model``, eredu/src/backend/mlx/architectures/gemma4/assistant.rs:499)."""
        from ..models.gemma4_assistant import load_gemma4_assistant

        if "gemma4" not in self.engine.cfg.extra:
            raise ValueError("an assistant drafter attaches to a Gemma 4 target")
        self.assistant = load_gemma4_assistant(path, self.engine.model)

    def _mtp_decoder(self, draft, draft_tokens: int, embedded_mtp: bool = True):
        """The speculative decoder this model can run: an external draft model, else its own prediction layer."""
        from ..runtime.speculative import EmbeddedMtpDecoder, SpeculativeDecoder

        if draft_tokens <= 0:
            return None
        if not getattr(self.engine, "paged", True):
            # the request scheduler drives paged lanes; an unpaged target drafts through UnpagedSpeculativeDecoder
            # (generate_prepared_chat without scheduler options)
            if draft is not None:
                raise NotImplementedError("the speculative request scheduler needs the paged engine; pass the draft without "
                                          "scheduler options to run this family's draft-and-verify decoder")
            return None
        if draft is not None:
            return SpeculativeDecoder(self.engine, draft.engine, k=draft_tokens)
        if getattr(self, "assistant", None) is not None:
            from ..runtime.speculative import Gemma4AssistantDecoder

            return Gemma4AssistantDecoder(self.engine, self.assistant, k=draft_tokens)
        if getattr(self, "dflash", None) is not None:
            from ..runtime.speculative import DFlashDecoder

            return DFlashDecoder(self.engine, self.dflash, k=draft_tokens)
        if embedded_mtp and getattr(self, "mtp", None) is not None:
            return EmbeddedMtpDecoder(self.engine, self.mtp, k=draft_tokens)
        return None

    def generate_prepared_chat_mtp_batch(self, prepared: list, sampling: Optional[SamplingParams] = None,
                                         max_new_tokens: int = 256, on_event=None, draft: Optional["LoadedModel"] = None,
                                         draft_tokens: int = 3, mtp_options=None, cancellations=None) -> dict:
        """Several prepared chats as independently progressing speculative lanes over the shared weights
        (``generate_prepared_chat_mtp_batch``, eredu/src/api/loaded.rs:285): one scheduler request per chat, each with
        its own cache, sampler stream, semantic parser and statistics. ``on_event(lane, event)``. Returns
        ``{"results": [per-lane dict as generate_prepared_chat], "scheduler": aggregate scheduler counters}``."""
        import time

        from ..runtime.mtp_scheduler import MtpScheduler, MtpSchedulerOptions
        from ..runtime.streaming import FinishReason
        from ..text.dialects import pipeline_for
        from ..text.tokenizer import TextDecoder

        if self.tokenizer is None:
            raise RuntimeError("this checkpoint has no tokenizer")
        spec = self._mtp_decoder(draft, draft_tokens)
        if spec is None:
            raise ValueError("speculative batch generation needs a draft model or a checkpoint with a prediction layer")
        eos = set(self.eos_ids()) | set(self.tokenizer.eos_ids)
        sched = MtpScheduler(spec, mtp_options or MtpSchedulerOptions())
        lanes = []
        t0 = time.perf_counter()
        for i, prep in enumerate(prepared):
            plan = prep.plan
            show_special = bool(plan is not None and plan.render_special_tokens)
            cb = (lambda ev, i=i: on_event(i, ev)) if on_event is not None else None
            pipe = pipeline_for(plan)(TextDecoder(self.tokenizer, skip_special_tokens=not show_special), plan, prep.stop, cb,
                                      prep.tool_choice.max_parallel_calls)
            pipe.tools = prep.tools
            lane = {"pipe": pipe, "tokens": [], "first": None, "prompt": self.tokenizer.encode(prep.prompt)}

            def on_token(tok, lane=lane):
                if lane["first"] is None:
                    lane["first"] = time.perf_counter()
                if tok in eos:
                    return FinishReason.EOS
                lane["tokens"].append(tok)
                lane["pipe"].push(tok)
                return lane["pipe"].finished or None

            cancel = cancellations[i].is_cancelled if cancellations is not None and cancellations[i] is not None else None
            sched.submit(lane["prompt"], sampling or SamplingParams(), max_new_tokens, (), on_token, cancel)
            lanes.append(lane)
        done = sched.finish()
        t1 = time.perf_counter()
        results = []
        for lane, req in zip(lanes, done.requests):
            pipe = lane["pipe"]
            pipe.finish(req.finish_reason or FinishReason.MAX_TOKENS)
            n = len(lane["tokens"])
            results.append({"text": "".join(pipe.text_out), "reasoning": "".join(pipe.reasoning_out),
                            "tool_calls": pipe.tool_calls, "finish_reason": pipe.finished, "tokens": lane["tokens"],
                            "prompt_tokens": len(lane["prompt"]), "stats": vars(req.stats),
                            "timing": {"generation_time": req.stats.elapsed,
                                       "time_to_first_token": (lane["first"] or t1) - t0,
                                       "token_rate": n / max(1e-9, req.stats.elapsed)}})
        self.last_speculative_stats = dict(spec.stats.summary(), scheduler=vars(done.scheduler))
        return {"results": results, "scheduler": vars(done.scheduler)}

    def generate_prepared_chat(self, prepared, sampling: Optional[SamplingParams] = None, max_new_tokens: int = 256,
                               on_event=None, cancellation=None, raw: bool = False, mirostat=None, constraint=None,
                               draft: Optional["LoadedModel"] = None, draft_tokens: int = 3, embedded_mtp: bool = True,
                               mtp_options=None):
        """Generate a reply for a :class:`PreparedChat`, streaming semantic events (reasoning, text, tool-call
        start / arguments / end, finished) to ``on_event`` (``generate_prepared_chat``, api/loaded.rs:154-227).
        ``draft`` (another loaded model with the same vocabulary) turns on speculative decoding with ``draft_tokens``
        proposals per round (``generate_prepared_chat_mtp``, api/loaded.rs:238; the committed tokens are exactly those
        plain decoding would emit). Without a draft model, a checkpoint that carries its own prediction layer
        (``self.mtp``) drafts for itself unless ``embedded_mtp`` is false or ``draft_tokens`` is 0. ``mirostat`` (an :class:`ops.controlled.MirostatV2`) and ``constraint`` (a :class:`GrammarConstraint`, e.g.
        from :meth:`constraint_for`) switch to the host-driven controlled sampler. ``mtp_options`` (a
        :class:`runtime.mtp_scheduler.MtpSchedulerOptions`) runs the speculative request through the fair scheduler:
        verification submitted asynchronously, optimistic lookahead behind it, adaptive switch-off.
        Returns a dict with text, reasoning, tool_calls, finish_reason, token ids and timing."""
        import time

        from ..runtime.streaming import CommittedTokenPipeline, FinishReason
        from ..text.tokenizer import TextDecoder

        if self.tokenizer is None:
            raise RuntimeError("this checkpoint has no tokenizer")
        prompt_ids = self.tokenizer.encode(prepared.prompt)
        eos = set(self.eos_ids()) | set(self.tokenizer.eos_ids)
        from ..text.dialects import pipeline_for

        plan = None if raw else prepared.plan
        show_special = bool(plan is not None and plan.render_special_tokens)
        pipe = pipeline_for(plan)(TextDecoder(self.tokenizer, skip_special_tokens=not show_special), plan, prepared.stop,
                                  on_event, prepared.tool_choice.max_parallel_calls)
        pipe.tools = prepared.tools           # parameter types of tagged-syntax calls come from the declarations
        t0 = time.perf_counter()
        first_token_at = [None]
        tokens: list[int] = []

        def on_token(i, tok):
            if first_token_at[0] is None:
                first_token_at[0] = time.perf_counter()
            if tok in eos:
                return FinishReason.EOS
            tokens.append(tok)
            pipe.push(tok)
            if pipe.finished:
                return pipe.finished
            if cancellation is not None and cancellation.is_cancelled():
                return FinishReason.CANCELLED
            return None

        if (constraint is None and not raw and prepared.tools and plan is not None and plan.dialect == "generic"
                and plan.tool_open and prepared.tool_choice.mode in ("auto", "required")):
            # declared tools: calls are grammar-constrained to a declared name and its parameter schema
            from ..text.tool_constraints import constraint_for_tools

            constraint = constraint_for_tools(self.tokenizer, prepared.tools, prepared.tool_choice.mode,
                                              prepared.tool_choice.max_parallel_calls, plan.tool_open, plan.tool_close)
        if constraint is not None and mirostat is None and draft is not None:
            # speculation under a grammar: proposals run the grammar ahead, rejected ones are rolled back
            from ..runtime.speculative import SpeculativeDecoder

            spec = SpeculativeDecoder(self.engine, draft.engine, k=draft_tokens)
            _, why = spec.generate_constrained(prompt_ids, constraint, sampling, max_new_tokens, tuple(eos),
                                               on_token=lambda tok: on_token(0, tok))
            reason = {"eos": FinishReason.EOS, "max_tokens": FinishReason.MAX_TOKENS,
                      "grammar_complete": FinishReason.GRAMMAR_COMPLETE}.get(why, why)
            self.last_speculative_stats = dict(spec.stats.summary(), constrained=True)
            if first_token_at[0] is None:
                first_token_at[0] = time.perf_counter()
        elif mirostat is not None or constraint is not None:
            from ..ops.controlled import controlled_generate

            _, why = controlled_generate(self.engine, prompt_ids, sampling, max_new_tokens, tuple(eos), constraint,
                                         mirostat, on_token=lambda tok: on_token(0, tok))
            reason = {"eos": FinishReason.EOS, "max_tokens": FinishReason.MAX_TOKENS,
                      "grammar_complete": FinishReason.GRAMMAR_COMPLETE}.get(why, why)
            if first_token_at[0] is None:
                first_token_at[0] = time.perf_counter()
        elif mtp_options is not None and self._mtp_decoder(draft, draft_tokens, embedded_mtp) is not None:
            from ..runtime.mtp_scheduler import MtpScheduler

            spec = self._mtp_decoder(draft, draft_tokens, embedded_mtp)
            sched = MtpScheduler(spec, mtp_options)
            sched.submit(prompt_ids, sampling or SamplingParams(), max_new_tokens, (), lambda tok: on_token(0, tok))
            done = sched.finish()
            reason = done.requests[0].finish_reason or FinishReason.MAX_TOKENS
            self.last_speculative_stats = dict(spec.stats.summary(), scheduler=vars(done.scheduler),
                                               request=vars(done.requests[0].stats),
                                               drafter="external" if draft is not None else
                                               "assistant" if getattr(self, "assistant", None) is not None else
                                               "dflash" if getattr(self, "dflash", None) is not None else "embedded")
        elif draft is not None:
            from ..runtime.speculative import SpeculativeDecoder
            from ..runtime.unpaged import UnpagedSpeculativeDecoder

            spec = (SpeculativeDecoder if getattr(self.engine, "paged", True) else UnpagedSpeculativeDecoder)(
                self.engine, draft.engine, k=draft_tokens)
            spec.generate([prompt_ids], sampling or SamplingParams(), max_new_tokens, eos_ids=(), on_token=on_token)
            reason = spec.last_finish_reasons[0] or FinishReason.MAX_TOKENS
            self.last_speculative_stats = spec.stats.summary()
        elif embedded_mtp and draft_tokens > 0 and getattr(self, "mtp", None) is not None:
            from ..runtime.speculative import EmbeddedMtpDecoder

            spec = EmbeddedMtpDecoder(self.engine, self.mtp, k=draft_tokens)
            spec.generate([prompt_ids], sampling or SamplingParams(), max_new_tokens, eos_ids=(), on_token=on_token)
            reason = spec.last_finish_reasons[0] or FinishReason.MAX_TOKENS
            self.last_speculative_stats = dict(spec.stats.summary(), drafter="embedded")
        else:
            self.engine.generate([prompt_ids], sampling or SamplingParams(), max_new_tokens, eos_ids=(), on_token=on_token)
            reason = self.engine.last_finish_reasons[0] or FinishReason.MAX_TOKENS
        pipe.finish(reason)
        t1 = time.perf_counter()
        ttft = (first_token_at[0] or t1) - t0
        n = len(tokens)
        return {"text": "".join(pipe.text_out), "reasoning": "".join(pipe.reasoning_out), "tool_calls": pipe.tool_calls,
                "finish_reason": pipe.finished, "tokens": tokens, "prompt_tokens": len(prompt_ids),
                "timing": {"generation_time": t1 - t0, "time_to_first_token": ttft,
                           "decode_token_rate": (n - 1) / max(1e-9, (t1 - t0) - ttft) if n > 1 else 0.0,
                           "token_rate": n / max(1e-9, t1 - t0)}}
