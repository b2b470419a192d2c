"""Pipeline parallelism: contiguous layer ranges per stage, activations handed stage to stage with NCCL p2p.

Semantics follow eredu/src/backend/mlx/architectures/distributed/pipeline.rs:5665-5714,6357-6510: the first
stage embeds, every stage runs its contiguous layers, the last stage applies the final norm and the head;
``[tokens, hidden]`` activations travel ``send``/``recv`` between neighbouring stages; sampling happens on the
last stage and the chosen ids are distributed to the other stages. There is no micro-batch schedule inside one
forward; different requests can occupy different stages through the scheduler.

Two transports. ``nccl``: NCCL p2p (gloo on CPU ranks) with a checked frame header; on CUDA it is issued on a side
stream and ordered with events so that the copy engine overlaps the next kernels of the sending stage. It needs the
host at every hop, so decode runs eagerly. ``peer`` (CUDA, one node): decode steps hand activations and sampled ids
over with kernels that store into the neighbour's staging memory and wait on flags (``parallel.comm.PeerP2P``) - no
host in the loop, so a stage's whole decode step (its layers, the hand-off, the token feedback) is one CUDA graph.
Shapes of such steps are fixed by the decode state; prompts still travel over the framed transport.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..runtime.engine import Engine

WIRE_MAGIC = 0x45524455  # frames carry [magic, rows, cols] so a desynchronised peer is detected, not trusted


class _StageModel:
    """Wraps a model shard so that ``forward`` receives from the previous stage and sends to the next one."""

    def __init__(self, model, par, p2p=None):
        self.inner = model
        self.p2p = p2p                # PeerP2P over the pipeline group, or None: every hop goes through torch.distributed
        self.par = par
        self.cfg = model.cfg
        self.device = model.device
        self.dtype = model.dtype
        self.n_kv_local = model.n_kv_local
        self.n_q_local = model.n_q_local
        self.first_layer = model.first_layer
        self.last_layer = model.last_layer
        topo = par.topology
        self.prev = topo.pipeline_predecessor(par.rank)
        self.next = topo.pipeline_successor(par.rank)
        self.side = torch.cuda.Stream(device=model.device) if model.device.type == "cuda" else None
        self.stats = {"sent": 0, "received": 0, "bytes": 0}

    def num_local_layers(self):
        return self.inner.num_local_layers()

    def _header(self, rows, cols):
        return torch.tensor([WIRE_MAGIC, rows, cols], dtype=torch.int64, device=self.device)

    def forward(self, batch, kv):
        M = batch.token_ids.shape[0]
        H = self.cfg.hidden_size
        if self.p2p is not None and not batch.is_prefill:
            return self._forward_peer(batch, kv, M, H)
        if self.prev is not None:
            hdr = torch.empty(3, dtype=torch.int64, device=self.device)
            dist.recv(hdr, src=self.prev)
            magic, rows, cols = (int(v) for v in hdr.tolist())
            if magic != WIRE_MAGIC or rows != M or cols != H:
                raise RuntimeError(f"pipeline frame mismatch: got ({magic:#x}, {rows}, {cols}), expected ({M}, {H})")
            h = torch.empty((M, H), dtype=self.dtype, device=self.device)
            dist.recv(h, src=self.prev)
            batch.hidden_in = h
            self.stats["received"] += 1
        out = self.inner.forward(batch, kv)
        if self.next is None:
            return out
        out = out.contiguous()
        if self.side is not None:
            self.side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.side):
                dist.send(self._header(M, H), dst=self.next)
                dist.send(out, dst=self.next)
            out.record_stream(self.side)
        else:
            dist.send(self._header(M, H), dst=self.next)
            dist.send(out, dst=self.next)
        self.stats["sent"] += 1
        self.stats["bytes"] += out.numel() * out.element_size()
        return None


    def _forward_peer(self, batch, kv, M, H):
        """Decode hop over peer memory: no header, no host. The decode state fixes (M, H) for the life of the graph."""
        stage = self.par.pp_rank
        if self.prev is not None:
            if self._h_in is None or self._h_in.shape[0] != M:
                self._h_in = torch.empty((M, H), dtype=self.dtype, device=self.device)
            self.p2p.recv(stage - 1, self._h_in, channel=0)
            batch.hidden_in = self._h_in
            self.stats["received"] += 1
        out = self.inner.forward(batch, kv)
        if self.next is None:
            return out
        self.p2p.send(stage + 1, out.contiguous(), channel=0)
        self.stats["sent"] += 1
        self.stats["bytes"] += out.numel() * out.element_size()
        return None


class PipelineRunner:
    def __init__(self, model, par, max_batch=8, max_seq_len=4096, num_pages=None, transport: str = "nccl"):
        self.par = par
        p2p = None
        if transport == "peer":
            if model.device.type != "cuda" or par.pp_size < 2:
                raise ValueError("the peer-memory transport needs CUDA ranks of one node and at least two stages")
            from .comm import PeerP2P

            p2p = PeerP2P(par.pp_group, model.device, max_batch * model.cfg.hidden_size * 2)
        elif transport != "nccl":
            raise ValueError(f"unknown pipeline transport {transport!r}")
        self.p2p = p2p
        # the placed execution DAG is the authority on who owns what: this stage's layers, embedding and head must be
        # exactly what the plan gives its pipeline coordinate (placement.rs validates before any weight is read; here
        # the model is already sharded, so a disagreement is a construction error)
        from .placement import decoder_placement

        self.placement = decoder_placement(model.cfg.num_hidden_layers, par.pp_size, sparse=getattr(model.cfg, "is_moe", False))
        dec = self.placement.group("decoder")
        want = dec.local_units(par.pp_rank)
        have = (model.first_layer, model.last_layer)
        if want is not None and tuple(want) != have:
            raise RuntimeError(f"pipeline stage {par.pp_rank} holds layers {have}, the placement assigns {tuple(want)}")
        if (self.placement.static_owner("embedding") == par.pp_rank) != par.owns_embedding() or \
                (self.placement.static_owner("output_head") == par.pp_rank) != par.owns_output_head():
            raise RuntimeError("embedding / output head ownership differs from the placement")
        self.stage = _StageModel(model, par, p2p)
        self.stage._h_in = None
        self.engine = Engine(self.stage, max_batch=max_batch, max_seq_len=max_seq_len, num_pages=num_pages,
                             use_cuda_graph=p2p is not None)
        self.engine.token_sync = self._sync_tokens
        topo = par.topology
        members = topo.axis_members(par.rank, "pipeline")
        self.last_rank = members[-1]
        self.pp_group = par.pp_group
        self._tok_pad = None

    def _sync_tokens_peer(self, tokens, n):
        """Sampled ids from the last stage to every other stage as a 16-byte aligned int32 message on channel 1."""
        dev = self.stage.device
        words = (n + 3) // 4 * 4
        if self._tok_pad is None or self._tok_pad.numel() != words:
            self._tok_pad = torch.zeros(words, dtype=torch.int32, device=dev)
        last = self.par.pp_size - 1
        if self.par.pp_rank == last:
            self._tok_pad[:n].copy_(tokens)
            for s in range(last):
                self.p2p.send(s, self._tok_pad, channel=1)
        else:
            self.p2p.recv(last, self._tok_pad, channel=1)
        return self._tok_pad[:n]

    def _sync_tokens(self, tokens, n):
        dev = self.stage.device
        if self.p2p is not None and self.engine._decode_state is not None and self._in_decode():
            return self._sync_tokens_peer(tokens, n)
        if tokens is None:
            tokens = torch.empty(n, dtype=torch.int32, device=dev)
        else:
            tokens = tokens.to(dev, torch.int32).contiguous()
        if self.par.pp_size > 1:
            dist.broadcast(tokens, src=self.last_rank, group=self.pp_group)
        return tokens

    def generate(self, prompts, sampling=None, max_new_tokens=64, eos_ids=()):
        return self.engine.generate(prompts, sampling, max_new_tokens, eos_ids)

    def _in_decode(self) -> bool:
        return getattr(self.engine, "_in_decode_body", False)
