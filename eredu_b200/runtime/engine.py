"""Batch execution engine: chunked prefill, CUDA-graph decode, device-side sampling and bookkeeping.

The reference submits one lazy graph per token and blocks on a host read of the sampled id
(eredu-core/src/backend.rs:834-912, eredu/src/backend/mlx/session.rs:816-1019). Here a decode step is a
captured CUDA graph: model forward -> fused sampler -> ``decode_advance`` (token feedback, positions, KV
slot, RNG position, penalty history — all on the device), so replaying step n+1 needs nothing from the
host. The host only *observes* tokens through an asynchronous copy into pinned memory.

Under tensor parallelism every rank runs this engine in lock-step on identical inputs; logits are
identical on all ranks after the gather, the sampler is deterministic, so every rank commits the same
token without a broadcast (the reference uses two all-sums and a host sync per step for this:
eredu/src/backend/mlx/runtime/distributed/parallel.rs:46-105).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from .. import ops
from ..models.llama import CausalLM, ForwardBatch
from ..ops.sampling import ROW_DTYPE, SamplingParams, pack_rows
from ..utils import nvtx
from .kv_cache import PAGE, PagedKVCache


@dataclass
class Sequence:
    seq_id: int
    prompt: list[int]
    sampling: SamplingParams = field(default_factory=SamplingParams)
    max_new_tokens: int = 256
    eos_ids: tuple = ()
    output: list[int] = field(default_factory=list)
    pages: list[int] = field(default_factory=list)
    kv_len: int = 0            # tokens whose K/V are in the cache
    finished: bool = False
    finish_reason: Optional[str] = None
    slot: int = -1             # row in the decode batch
    cached_tokens: int = 0     # prompt tokens whose K/V came from published pages of earlier requests

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.output)


class Engine:
    def __init__(self, model: CausalLM, max_batch: int = 32, max_seq_len: int = 4096, num_pages: Optional[int] = None,
                 use_cuda_graph: Optional[bool] = None, prefill_chunk: int = 8192, hist_cap: int = 1024,
                 prefix_cache: bool = False, kv_host_tier_bytes: int = 0, kv_disk_tier_dir=None, kv_disk_tier_bytes: int = 0):
        self.model = model
        self.cfg = model.cfg
        self.device = model.device
        self.max_batch = max_batch
        self.max_seq_len = max_seq_len
        self.max_pages = PagedKVCache.pages_for(max_seq_len)
        if num_pages is None:
            num_pages = max_batch * self.max_pages + 1
        local = range(model.first_layer, model.last_layer)
        conv_layers = [li for li in local if self.cfg.layer_is_conv(li)]
        kv_layers = [li for li in local if self.cfg.layer_has_kv(li)]
        _, key_dim, value_dim = self.cfg.kv_cache_dims
        self.kv = PagedKVCache(model.num_local_layers(), model.n_kv_local, key_dim, num_pages, model.dtype,
                               self.device, first_layer=model.first_layer, value_dim=value_dim,
                               attention_layers=kv_layers,
                               conv_layers=conv_layers,
                               conv_channels=self.cfg.hidden_size // model.par.tp_size if conv_layers else 0,
                               conv_hist=self.cfg.conv_l_cache - 1)
        mamba_layers = [li for li in local if self.cfg.layer_is_mamba(li)]
        if mamba_layers:
            from ..models.nemotron_h import mamba_dims

            heads, _, _, conv_dim = mamba_dims(self.cfg, model.par.tp_size)
            self.kv.enable_linear_attention_state(mamba_layers, slots=max(2 * max_batch, 8),
                                                  conv_hist=self.cfg.mamba_conv_kernel - 1, conv_channels=conv_dim, heads=heads,
                                                  dk=self.cfg.mamba_head_dim, dv=self.cfg.ssm_state_size)
        kda_layers = [li for li in local if self.cfg.layer_is_kda(li)]
        if kda_layers:
            c = self.cfg
            kh = c.linear_num_value_heads // model.par.tp_size
            self.kv.enable_linear_attention_state(kda_layers, slots=max(2 * max_batch, 8), conv_hist=c.linear_conv_kernel_dim - 1,
                                                  conv_channels=3 * kh * c.linear_value_head_dim,
                                                  heads=kh, dk=c.linear_value_head_dim,
                                                  dv=c.linear_value_head_dim)
        la_layers = [li for li in local if self.cfg.layer_is_linear_attention(li)]
        if la_layers:
            c = self.cfg
            tp = model.par.tp_size
            self.kv.enable_linear_attention_state(
                la_layers, slots=max(2 * max_batch, 8), conv_hist=c.linear_conv_kernel_dim - 1,
                conv_channels=(2 * c.linear_num_key_heads * c.linear_key_head_dim
                               + c.linear_num_value_heads * c.linear_value_head_dim) // tp,
                heads=c.linear_num_value_heads // tp, dk=c.linear_key_head_dim, dv=c.linear_value_head_dim)
        self.cuda = self.device.type == "cuda"
        self.use_graph = self.cuda if use_cuda_graph is None else (use_cuda_graph and self.cuda)
        self.prefill_chunk = prefill_chunk
        self.hist_cap = hist_cap
        # Prefix reuse over sealed pages (eredu/src/backend/mlx/runtime/cache/kv.rs:2018-2128: immutable sealed blocks
        # shared by lease): full 16-token pages are published under the chained hash of their tokens when a prompt has
        # been prefilled and again when the sequence is released; a new request leases the longest published prefix of
        # its prompt and prefills only the rest. Unreferenced published pages stay cached until the pool needs them
        # (LRU / LFU eviction inside the block manager). Models with recurrent state cannot resume from pages alone.
        self.prefix_cache = bool(prefix_cache and hasattr(self.kv.allocator, "match_prefix")
                                 and not self.kv.has_recurrent_state())
        self.prefix_stats = {"lookups": 0, "hits": 0, "hit_tokens": 0, "prompt_tokens": 0, "sealed_pages": 0}
        # Lower tiers for published pages: evicted pages are demoted to pinned host memory and on to files, and promoted
        # back when a prompt continues through them (runtime/block_tiers.py).
        self.block_tiers = None
        if self.prefix_cache and (kv_host_tier_bytes or (kv_disk_tier_dir and kv_disk_tier_bytes)) \
                and hasattr(self.kv.allocator, "take_evicted"):
            from .block_tiers import BlockTierStore

            self.block_tiers = BlockTierStore(self.kv, kv_host_tier_bytes, kv_disk_tier_dir, kv_disk_tier_bytes)
            self.kv.block_tiers = self.block_tiers      # every allocation path demotes what it evicts (kv.alloc)
        self._next_id = 0
        self._graphs: dict = {}
        self._decode_state = None
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count if self.cuda else 1
        # Pipeline parallelism: ``forward`` returns None on stages without the output head and ``token_sync``
        # distributes the tokens sampled on the last stage (set by parallel.pipeline.PipelineRunner).
        self.token_sync = None

    # ------------------------------------------------------------------------------------------ requests
    def new_sequence(self, prompt, sampling=None, max_new_tokens=256, eos_ids=()) -> Sequence:
        seq = Sequence(self._next_id, list(prompt), sampling or SamplingParams(), max_new_tokens, tuple(eos_ids))
        self._next_id += 1
        if len(seq.prompt) + max_new_tokens > self.max_seq_len:
            raise ValueError(f"prompt ({len(seq.prompt)}) + max_new_tokens ({max_new_tokens}) exceeds "
                             f"max_seq_len {self.max_seq_len}")
        # Reserve every page the request can need up front: the block table is then static for the
        # whole decode and the captured graph never needs a host update.
        need = PagedKVCache.pages_for(len(seq.prompt) + max_new_tokens)
        if self.prefix_cache:
            # at least one prompt token is always prefilled: its logits choose the first output token
            usable = (len(seq.prompt) - 1) // PAGE * PAGE
            if self.block_tiers is not None:
                leased = self._lease_prefix_through_tiers(seq.prompt[:usable], need)
            else:
                leased = list(self.kv.allocator.match_prefix(seq.prompt[:usable])) if usable else []
            try:
                seq.pages = leased + self.kv.alloc(need - len(leased))
            except RuntimeError:
                if leased:
                    self.kv.allocator.release(leased)
                raise
            seq.kv_len = seq.cached_tokens = len(leased) * PAGE
            st = self.prefix_stats
            st["lookups"] += 1
            st["hits"] += 1 if leased else 0
            st["hit_tokens"] += seq.cached_tokens
            st["prompt_tokens"] += len(seq.prompt)
            return seq
        seq.pages = self.kv.alloc(need)
        if self.kv.page_to_slot is not None:
            try:
                self.kv.bind_state(seq.pages[0])
            except RuntimeError:
                self.kv.allocator.release(seq.pages)
                seq.pages = []
                raise
        return seq

    def _lease_prefix_through_tiers(self, tokens, need: int) -> list:
        """The longest prefix of ``tokens`` (whole pages) that is published on the device or held in a lower tier: device
        pages are leased as they are, tier blocks get a fresh device page, are copied into it and published again."""
        al, tiers = self.kv.allocator, self.block_tiers
        plan, h = [], 0
        for i in range(0, len(tokens) // PAGE * PAGE, PAGE):
            h = al.chain_hash(h, [int(t) for t in tokens[i:i + PAGE]])
            page = al.lookup(h)
            if page >= 0:
                al.retain([page])                     # leased now, so that the allocations below cannot evict it
                plan.append((h, page, None))
            elif tiers.where(h) is not None:
                plan.append((h, -1, tiers.where(h)))
            else:
                break
        pages, promote = [], []
        try:
            for h, page, tier in plan:
                if tier is not None:
                    if al.free_pages() <= need - len(plan):     # the pool cannot take promoted blocks and the rest of the request
                        break
                    page = self.kv.alloc(1)[0]
                    promote.append((h, page))
                pages.append(page)
        finally:
            tail = [p for _, p, t in plan[len(pages):] if t is None]
            if tail:
                al.release(tail)                      # device hits behind a block that could not be promoted
        tiers.promote(promote)                        # evicted pages were copied out as they were allocated (kv.alloc)
        for h, page in promote:
            al.seal(page, h)
        return pages

    def publish_pages(self, seq: Sequence) -> None:
        """Publish the full pages below ``kv_len`` (prompt and committed output) for reuse by later requests."""
        if self.prefix_cache and seq.pages and seq.kv_len >= PAGE:
            tokens = (seq.prompt + seq.output)[:seq.kv_len // PAGE * PAGE]
            self.prefix_stats["sealed_pages"] += int(self.kv.allocator.seal_prefix(seq.pages, tokens))

    def release(self, seq: Sequence) -> None:
        if seq.pages:
            self.publish_pages(seq)
            self.kv.unbind_state(seq.pages[0])
            self.kv.allocator.release(seq.pages)
            seq.pages = []

    def snapshot_state(self, seq: Sequence):
        """Recurrent state of a hybrid model's sequence at its current length (None when there is none to keep)."""
        return self.kv.snapshot_state(seq.pages[0]) if seq.pages else None

    def restore_state(self, seq: Sequence, snap) -> None:
        if seq.pages:
            self.kv.restore_state(seq.pages[0], snap)

    # ------------------------------------------------------------------------------------------ helpers
    def _t(self, data, dtype):
        t = torch.as_tensor(data, dtype=dtype)
        if self.cuda:
            t = t.pin_memory().to(self.device, non_blocking=True)
        return t

    def _block_table(self, seqs) -> torch.Tensor:
        bt = np.zeros((len(seqs), self.max_pages), dtype=np.int32)
        for i, s in enumerate(seqs):
            bt[i, :len(s.pages)] = s.pages
        return self._t(bt, torch.int32)

    def _sample(self, logits, seqs, positions, history=None):
        """Sample one token per row. CUDA: fused kernel; CPU: the oracle chain."""
        if self.cuda:
            rows = pack_rows([s.sampling for s in seqs], positions,
                             hist_lens=[min(len(s.output), self.hist_cap) for s in seqs],
                             stream_ids=[s.seq_id for s in seqs])
            hist = None
            if any(s.sampling.repeat_penalty != 1.0 or s.sampling.frequency_penalty != 0.0
                   or s.sampling.presence_penalty != 0.0 for s in seqs):
                h = np.zeros((len(seqs), self.hist_cap), dtype=np.int32)
                for i, s in enumerate(seqs):
                    tail = s.output[-self.hist_cap:]
                    h[i, :len(tail)] = tail
                hist = self._t(h, torch.int32)
            rows_t = self._t(rows.view(np.uint8).reshape(len(seqs), ROW_DTYPE.itemsize), torch.uint8)
            return ops.sample(logits.contiguous(), rows_t, history=hist,
                              all_greedy=all(s.sampling.greedy for s in seqs))
        toks = []
        for i, s in enumerate(seqs):
            tok, _ = ops.sample_ref(logits[i], s.sampling, positions[i], history=s.output, stream=s.seq_id)
            toks.append(tok)
        return torch.tensor(toks, dtype=torch.int32)

    # ------------------------------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, seqs: list[Sequence], limits: Optional[list[int]] = None) -> torch.Tensor:
        """Run the prompts through the model (chunked), sample the first token of each. Returns [B] int32.
        ``limits[i]`` caps the number of prompt tokens processed for sequence i in this call (chunked prefill driven
        by a scheduler); the token sampled for a sequence whose prompt is not finished yet is meaningless."""
        self._limits = {s.seq_id: int(n) for s, n in zip(seqs, limits)} if limits is not None else None
        groups, cur, cur_tokens = [], [], 0
        for s in seqs:
            n = len(s.prompt) - s.kv_len
            if self._limits is not None:
                n = min(n, self._limits[s.seq_id])
            if cur and cur_tokens + n > self.prefill_chunk:
                groups.append(cur)
                cur, cur_tokens = [], 0
            cur.append(s)
            cur_tokens += n
        if cur:
            groups.append(cur)
        outs = []
        try:
            for g in groups:
                outs.append(self._prefill_group(g))
        finally:
            self._limits = None
        if any(o is None for o in outs):
            return None
        return torch.cat(outs)

    def _prefill_group(self, seqs):
        toks, pos, slots, cu, lens = [], [], [], [0], []
        max_q = 0
        for s in seqs:
            new = s.prompt[s.kv_len:]
            if getattr(self, "_limits", None) is not None:
                new = new[:self._limits[s.seq_id]]
            n = len(new)
            p = np.arange(s.kv_len, s.kv_len + n)
            pages = np.asarray(s.pages, dtype=np.int64)
            toks.extend(new)
            pos.append(p)
            slots.append(pages[p // PAGE] * PAGE + (p % PAGE))
            cu.append(cu[-1] + n)
            lens.append(s.kv_len + n)
            max_q = max(max_q, n)
        batch = ForwardBatch(
            token_ids=self._t(np.asarray(toks, dtype=np.int32), torch.int32),
            positions=self._t(np.concatenate(pos).astype(np.int32), torch.int32),
            slots=self._t(np.concatenate(slots), torch.int64),
            block_table=self._block_table(seqs),
            seq_lens=self._t(np.asarray(lens, dtype=np.int32), torch.int32),
            is_prefill=True,
            cu_q=self._t(np.asarray(cu, dtype=np.int32), torch.int32),
            max_q_len=max_q,
            logit_rows=self._t(np.asarray(cu[1:], dtype=np.int64) - 1, torch.int64),
        )
        with nvtx.annotate(f"prefill[{len(seqs)}x{max_q}]"):
            logits = self.model.forward(batch, self.kv)
        for s, n in zip(seqs, lens):
            s.kv_len = n
            if self.prefix_cache and n == len(s.prompt):
                self.publish_pages(s)           # concurrent requests with the same system prompt hit from here on
        tokens = None
        if logits is not None:
            tokens = self._sample(logits, seqs, [len(s.prompt) for s in seqs])
        if self.token_sync is not None:
            tokens = self.token_sync(tokens, len(seqs))
        return tokens

    # ------------------------------------------------------------------------------------------ decode
    def start_decode(self, seqs: list[Sequence], first_tokens: torch.Tensor) -> None:
        """Load the decode state of a batch into the static device buffers (one H2D per buffer)."""
        B = len(seqs)
        assert B <= self.max_batch
        dev = self.device
        pos = np.asarray([s.kv_len for s in seqs], dtype=np.int32)
        pages = [np.asarray(s.pages, dtype=np.int64) for s in seqs]
        slots = np.asarray([pg[p // PAGE] * PAGE + (p % PAGE) for pg, p in zip(pages, pos)], dtype=np.int64)
        rows = pack_rows([s.sampling for s in seqs], [int(p) + 1 for p in pos],
                         hist_lens=[min(len(s.output), self.hist_cap) for s in seqs],
                         stream_ids=[s.seq_id for s in seqs])
        need_hist = any(s.sampling.repeat_penalty != 1.0 or s.sampling.frequency_penalty != 0.0
                        or s.sampling.presence_penalty != 0.0 for s in seqs)
        hist = None
        if need_hist:
            h = np.zeros((B, self.hist_cap), dtype=np.int32)
            for i, s in enumerate(seqs):
                tail = s.output[-self.hist_cap:]
                h[i, :len(tail)] = tail
            hist = self._t(h, torch.int32)
        max_len = int(pos.max()) + 1 + max(s.max_new_tokens for s in seqs)
        splits = ops.decode_splits(B, self.model.n_kv_local, max_len, self.sm_count) if self.cuda else 1
        st = {
            "B": B,
            "seqs": list(seqs),
            "token_ids": first_tokens.to(dev, torch.int32).clone(),
            "positions": self._t(pos, torch.int32),
            "seq_lens": self._t(pos + 1, torch.int32),
            "slots": self._t(slots, torch.int64),
            "block_table": self._block_table(seqs),
            "active": self._t(np.ones(B, dtype=np.int32), torch.int32),
            "rows": self._t(rows.view(np.uint8).reshape(B, ROW_DTYPE.itemsize), torch.uint8),
            "history": hist,
            "sampled": torch.zeros(B, dtype=torch.int32, device=dev),
            "splits": splits,
            "all_greedy": all(s.sampling.greedy for s in seqs),
            "scratch": ops.decode_scratch(B, 1, self.model.n_q_local, self.cfg.head_dim, splits, dev)
            if (self.cuda and splits > 1) else None,
            "graph": None,
            "host_tokens": torch.zeros(B, dtype=torch.int32).pin_memory() if self.cuda else None,
            "host_in": torch.zeros(B, dtype=torch.int32).pin_memory() if self.cuda else None,
        }
        self._decode_state = st
        for i, s in enumerate(seqs):
            s.slot = i

    # ------------------------------------------------------------------------------------------ host-driven steps
    @torch.no_grad()
    def feed_logits(self, seq: Sequence, tokens: list[int], multimodal=None) -> torch.Tensor:
        """Append ``tokens`` to the sequence's cache and return the logits after the last one ([V], on the model's
        device). For samplers that must see every distribution on the host (grammar masks, Mirostat).

        ``multimodal``: dict with ``rows`` (indices into ``tokens`` whose embeddings are replaced), ``values`` [n, H],
        optional ``deepstack`` (list of [n, H]), ``rope_positions`` [3, len(tokens)] and ``bidir_groups`` (one group id per
        token, -1 for text: tokens of a group attend to each other in both directions) for prompts with images; it sets
        ``seq.rope_delta`` so that later text tokens continue after the largest position the images used."""
        n = len(tokens)
        p = np.arange(seq.kv_len, seq.kv_len + n)
        pages = np.asarray(seq.pages, dtype=np.int64)
        extra = {}
        delta = getattr(seq, "rope_delta", 0)
        if multimodal is not None:
            dev = self.device
            extra = dict(embed_rows=torch.as_tensor(multimodal["rows"], dtype=torch.int64, device=dev),
                         embed_values=multimodal["values"].to(dev),
                         deepstack=[d.to(dev) for d in multimodal.get("deepstack") or []] or None)
            if multimodal.get("rope_positions") is not None:
                extra["rope_positions"] = multimodal["rope_positions"].to(dev)
            if multimodal.get("bidir_groups") is not None:
                # group ids of the fed tokens; earlier positions of the sequence belong to no group
                grp = torch.full((seq.kv_len + n,), -1, dtype=torch.int64, device=dev)
                grp[seq.kv_len:] = torch.as_tensor(multimodal["bidir_groups"], dtype=torch.int64, device=dev)
                extra["bidir_groups"] = [grp]
            seq.rope_delta = int(multimodal.get("rope_delta", 0))
        elif delta:
            extra = dict(rope_positions=self._t((p + delta).astype(np.int32), torch.int32))
        batch = ForwardBatch(**extra, 
            token_ids=self._t(np.asarray(tokens, dtype=np.int32), torch.int32),
            positions=self._t(p.astype(np.int32), torch.int32),
            slots=self._t(pages[p // PAGE] * PAGE + (p % PAGE), torch.int64),
            block_table=self._block_table([seq]), seq_lens=self._t(np.asarray([seq.kv_len + n], dtype=np.int32), torch.int32),
            is_prefill=True, cu_q=self._t(np.asarray([0, n], dtype=np.int32), torch.int32), max_q_len=n,
            logit_rows=self._t(np.asarray([n - 1], dtype=np.int64), torch.int64))
        logits = self.model.forward(batch, self.kv)
        seq.kv_len += n
        return logits[0]

    def prefill_logits(self, seqs: list[Sequence]) -> list[torch.Tensor]:
        return [self.feed_logits(s, s.prompt[s.kv_len:]) for s in seqs]

    def step_logits(self, seq: Sequence, token: int) -> torch.Tensor:
        seq.output.append(int(token))
        return self.feed_logits(seq, [int(token)])

    # ------------------------------------------------------------------------------------------ slot-based decode
    def open_decode(self, penalties: bool = False, max_context: Optional[int] = None) -> None:
        """Create a decode state with ``max_batch`` slots, all free. Sequences :meth:`join` and :meth:`leave`
        between steps by small copies into the static device buffers, so a captured graph stays valid while the
        batch membership changes (continuous batching)."""
        B = self.max_batch
        dev = self.device
        rows = pack_rows([SamplingParams(temperature=0.0)] * B, [1] * B, hist_lens=[0] * B, stream_ids=[0] * B)
        max_len = max_context or self.max_seq_len
        splits = ops.decode_splits(B, self.model.n_kv_local, max_len, self.sm_count) if self.cuda else 1
        st = {
            "B": B, "seqs": [None] * B, "slotted": True,
            "token_ids": torch.zeros(B, dtype=torch.int32, device=dev),
            "positions": torch.zeros(B, dtype=torch.int32, device=dev),
            "seq_lens": torch.ones(B, dtype=torch.int32, device=dev),
            "slots": torch.full((B,), -1, dtype=torch.int64, device=dev),
            "block_table": torch.zeros((B, self.max_pages), dtype=torch.int32, device=dev),
            "active": torch.zeros(B, dtype=torch.int32, device=dev),
            "rows": self._t(rows.view(np.uint8).reshape(B, ROW_DTYPE.itemsize), torch.uint8),
            "history": torch.zeros((B, self.hist_cap), dtype=torch.int32, device=dev) if penalties else None,
            "sampled": torch.zeros(B, dtype=torch.int32, device=dev),
            "splits": splits, "all_greedy": True,
            "scratch": ops.decode_scratch(B, 1, self.model.n_q_local, self.cfg.head_dim, splits, dev)
            if (self.cuda and splits > 1) else None,
            "graph": None, "graphs": {},
            "host_tokens": torch.zeros(B, dtype=torch.int32).pin_memory() if self.cuda else None,
            "host_in": torch.zeros(B, dtype=torch.int32).pin_memory() if self.cuda else None,
        }
        self._decode_state = st

    def free_slots(self) -> list[int]:
        return [i for i, s in enumerate(self._decode_state["seqs"]) if s is None]

    def join(self, seq: Sequence, first_token: int) -> int:
        """Put a prefilled sequence into a free slot; ``first_token`` is its next input token."""
        st = self._decode_state
        free = self.free_slots()
        if not free:
            raise RuntimeError("no free decode slot")
        i = free[0]
        pos = seq.kv_len
        pages = np.asarray(seq.pages, dtype=np.int64)
        bt = np.zeros(self.max_pages, dtype=np.int32)
        bt[:len(seq.pages)] = seq.pages
        row = pack_rows([seq.sampling], [pos + 1], hist_lens=[min(len(seq.output), self.hist_cap)], stream_ids=[seq.seq_id])
        st["token_ids"][i] = int(first_token)
        st["positions"][i] = pos
        st["seq_lens"][i] = pos + 1
        st["slots"][i] = int(pages[pos // PAGE] * PAGE + pos % PAGE)
        st["block_table"][i].copy_(self._t(bt, torch.int32))
        st["rows"][i].copy_(self._t(row.view(np.uint8).reshape(ROW_DTYPE.itemsize), torch.uint8))
        st["active"][i] = 1
        if st["history"] is not None:
            h = np.zeros(self.hist_cap, dtype=np.int32)
            tail = seq.output[-self.hist_cap:]
            h[:len(tail)] = tail
            st["history"][i].copy_(self._t(h, torch.int32))
        needs_hist = (seq.sampling.repeat_penalty != 1.0 or seq.sampling.frequency_penalty != 0.0
                      or seq.sampling.presence_penalty != 0.0)
        if needs_hist and st["history"] is None:
            raise RuntimeError("this decode state was opened without penalty history (open_decode(penalties=True))")
        st["seqs"][i] = seq
        seq.slot = i
        self._refresh_mode(st)
        return i

    def leave(self, seq: Sequence) -> None:
        st = self._decode_state
        i = seq.slot
        if i < 0 or st["seqs"][i] is not seq:
            return
        st["seqs"][i] = None
        seq.slot = -1
        st["active"][i] = 0
        st["slots"][i] = -1
        st["seq_lens"][i] = 1
        st["positions"][i] = 0
        st["block_table"][i].zero_()
        self._refresh_mode(st)

    def set_step_mask(self, stepping: list[bool]) -> None:
        """Which occupied slots take part in the next step (a scheduler may hold a request back for one step)."""
        st = self._decode_state
        act = np.asarray([1 if (s is not None and not s.finished and on) else 0 for s, on in zip(st["seqs"], stepping)],
                         dtype=np.int32)
        if self.cuda:
            st["active"].copy_(self._t(act, torch.int32))
        else:
            st["active"] = torch.as_tensor(act)

    def _refresh_mode(self, st) -> None:
        greedy = all(s is None or s.sampling.greedy for s in st["seqs"])
        if greedy != st["all_greedy"]:
            st["all_greedy"] = greedy
            st["graph"] = st["graphs"].get(greedy)  # graphs are captured per sampler path

    def _decode_body(self, st):
        batch = ForwardBatch(token_ids=st["token_ids"], positions=st["positions"], slots=st["slots"],
                             block_table=st["block_table"], seq_lens=st["seq_lens"], is_prefill=False, q_per_seq=1,
                             splits=st["splits"], scratch=st["scratch"])
        logits = self.model.forward(batch, self.kv)
        if logits is not None:
            ops.sample(logits, st["rows"], history=st["history"], out=st["sampled"], all_greedy=st["all_greedy"])
        if self.token_sync is not None:
            self._in_decode_body = True          # a pipeline runner may hand the ids over with kernels here (graph-safe)
            try:
                st["sampled"].copy_(self.token_sync(st["sampled"] if logits is not None else None, st["B"]))
            finally:
                self._in_decode_body = False
        hist = st["history"]
        code = ops.native.lib().eredu_decode_advance(
            st["sampled"].data_ptr(), st["token_ids"].data_ptr(), st["positions"].data_ptr(),
            st["seq_lens"].data_ptr(), st["slots"].data_ptr(), st["block_table"].data_ptr(),
            st["block_table"].stride(0), st["active"].data_ptr(), st["rows"].data_ptr(), ROW_DTYPE.itemsize // 4,
            None if hist is None else hist.data_ptr(), 0 if hist is None else hist.stride(0), st["B"],
            ops.native.stream_ptr(self.device))
        ops.native.check(code, "eredu_decode_advance")

    @torch.no_grad()
    def _host_driven(self) -> bool:
        """True when a forward pass needs the host between kernels (layerwise host residency, expert cache)."""
        m = self.model
        if self.cfg.head_dim not in (64, 128) or self.cfg.is_mla or self.cfg.model_type == "gemma4":
            return True    # no attention kernel for this head size: the tensor-operation path reads lengths on the host
        if getattr(m, "residency", None) is not None or getattr(getattr(m, "inner", m), "observer", None) is not None:
            return True
        if int((self.cfg.extra.get("muse_glimmer") or {}).get("num_experts") or 0) > 0:
            return True    # the routed experts of this family are grouped on the host
        if getattr(m, "eager_collectives", False):
            return True    # a collective of the step reads counts on the host (the torch.distributed all-to-all baseline)
        return any(getattr(getattr(lw, "moe", None), "expert_cache", None) is not None for lw in getattr(m, "layers", []))

    def decode_step(self, host_tokens: Optional[torch.Tensor] = None, sync: bool = True) -> Optional[torch.Tensor]:
        """One decode step for the batch loaded by :meth:`start_decode`.

        ``host_tokens`` (pinned int32 [B]) overrides the device-side token feedback: the step then includes
        the host->device copy of its inputs. With ``sync`` the sampled ids are copied back and returned.
        """
        st = self._decode_state
        if not self.cuda:
            with nvtx.annotate("decode_step"):
                return self._decode_step_cpu(st)
        nvtx.mark("decode_step")
        if host_tokens is not None:
            st["token_ids"].copy_(host_tokens, non_blocking=True)
        if self.use_graph:
            eager = st.get("eager")
            if eager is None:
                eager = st["eager"] = self._host_driven()
            if eager:
                # host-resident layers stream through device slots on a copy stream, and an expert cache reads the
                # routed ids on the host: such steps cannot be captured and run eagerly
                self._decode_body(st)
            elif st["graph"] is None:
                # warm-up run outside capture (lazy kernel attribute setup), then restore the state it advanced
                saved = {k: st[k].clone() for k in ("token_ids", "positions", "seq_lens", "slots", "rows")}
                saved_h = st["history"].clone() if st["history"] is not None else None
                saved_rec = [(t, t.clone()) for t in self.kv.recurrent_tensors()]   # hybrid layers: not idempotent
                s = torch.cuda.Stream(device=self.device)
                s.wait_stream(torch.cuda.current_stream(self.device))
                with torch.cuda.stream(s):
                    self._decode_body(st)
                torch.cuda.current_stream(self.device).wait_stream(s)
                torch.cuda.synchronize(self.device)
                for k, v in saved.items():
                    st[k].copy_(v)
                if saved_h is not None:
                    st["history"].copy_(saved_h)
                for t, copy in saved_rec:
                    t.copy_(copy)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._decode_body(st)
                # capture does not execute: state is still the pre-step state
                st["graph"] = g
                if "graphs" in st:
                    st["graphs"][st["all_greedy"]] = g
            if not eager:
                st["graph"].replay()
        else:
            self._decode_body(st)
        if not sync:
            return None
        st["host_tokens"].copy_(st["sampled"], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return st["host_tokens"]

    def _decode_step_cpu(self, st):
        idle = Sequence(0, [0], SamplingParams(temperature=0.0))
        seqs = [s if s is not None else idle for s in st["seqs"]]
        batch = ForwardBatch(token_ids=st["token_ids"], positions=st["positions"], slots=st["slots"],
                             block_table=st["block_table"], seq_lens=st["seq_lens"], is_prefill=False, q_per_seq=1)
        logits = self.model.forward(batch, self.kv)
        pos = st["positions"].tolist()
        toks = None
        if logits is not None:
            toks = self._sample(logits, seqs, [p + 1 for p in pos])
        if self.token_sync is not None:
            toks = self.token_sync(toks, len(seqs))
        active = st["active"].bool()
        st["sampled"] = toks
        newpos = st["positions"] + 1
        bt = st["block_table"].long()
        page = bt.gather(1, (newpos.long() // PAGE)[:, None]).squeeze(1)
        st["token_ids"] = torch.where(active, toks, st["token_ids"])
        st["positions"] = torch.where(active, newpos, st["positions"])
        st["seq_lens"] = torch.where(active, newpos + 1, st["seq_lens"])
        st["slots"] = torch.where(active, page * PAGE + (newpos.long() % PAGE), torch.full_like(page, -1))
        return toks

    def commit(self, tokens) -> list[bool]:
        """Record one sampled token per running sequence (host side); returns per-sequence 'just finished'."""
        st = self._decode_state
        done = []
        changed = False
        stepped = st.get("stepped")
        for i, s in enumerate(st["seqs"]):
            if s is None or s.finished or (stepped is not None and not stepped[i]):
                done.append(False)
                continue
            tok = int(tokens[i])
            s.output.append(tok)
            s.kv_len += 1
            fin = False
            if tok in s.eos_ids:
                s.finished, s.finish_reason, fin = True, "eos", True
            elif len(s.output) >= s.max_new_tokens:
                s.finished, s.finish_reason, fin = True, "max_tokens", True
            if fin:
                changed = True
            done.append(fin)
        if changed:
            act = np.asarray([0 if (s is None or s.finished) else 1 for s in st["seqs"]], dtype=np.int32)
            if self.cuda:
                st["active"].copy_(self._t(act, torch.int32))
            else:
                st["active"] = torch.as_tensor(act)
        return done

    # ------------------------------------------------------------------------------------------ generate
    @torch.no_grad()
    def generate(self, prompts: list[list[int]], sampling: Optional[SamplingParams] = None, max_new_tokens: int = 64,
                 eos_ids=(), on_token=None) -> list[list[int]]:
        """Greedy / stochastic generation for a batch of token-id prompts. ``on_token(seq_index, token)`` is called
        as tokens are committed; a truthy return value ends that sequence with the value as its finish reason.
        ``self.last_finish_reasons`` holds the per-sequence reasons afterwards."""
        seqs = [self.new_sequence(p, sampling, max_new_tokens, eos_ids) for p in prompts]
        try:
            first = self.prefill(seqs)
            first_host = first.tolist()
            for i, (s, t) in enumerate(zip(seqs, first_host)):
                s.output.append(int(t))
                if on_token:
                    why = on_token(i, int(t))
                    if why:
                        s.finished, s.finish_reason = True, str(why)
                        continue
                if int(t) in s.eos_ids:
                    s.finished, s.finish_reason = True, "eos"
                elif len(s.output) >= s.max_new_tokens:
                    s.finished, s.finish_reason = True, "max_tokens"
            if not all(s.finished for s in seqs):
                self.start_decode(seqs, first)
                if any(s.finished for s in seqs):
                    act = np.asarray([0 if s.finished else 1 for s in seqs], dtype=np.int32)
                    self._decode_state["active"] = self._t(act, torch.int32)
                while not all(s.finished for s in seqs):
                    toks = self.decode_step()
                    was = [s.finished for s in seqs]
                    self.commit(toks.tolist())
                    if on_token:
                        stopped = False
                        for i, s in enumerate(seqs):
                            if not was[i]:
                                why = on_token(i, s.output[-1])
                                if why and not s.finished:  # stop sequence, cancellation, grammar complete
                                    s.finished, s.finish_reason, stopped = True, str(why), True
                        if stopped:
                            act = np.asarray([0 if s.finished else 1 for s in seqs], dtype=np.int32)
                            if self.cuda:
                                self._decode_state["active"].copy_(self._t(act, torch.int32))
                            else:
                                self._decode_state["active"] = torch.as_tensor(act)
            if self.cuda:
                ops.native.check_status(self.device)
            self.last_finish_reasons = [s.finish_reason for s in seqs]
            return [list(s.output) for s in seqs]
        finally:
            for s in seqs:
                self.release(s)
            self._decode_state = None
