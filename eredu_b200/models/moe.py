"""Sparse mixture-of-experts block (Qwen3-MoE / Mixtral / GPT-OSS style routed SwiGLU experts).

Router: dense ``[E, H]`` projection -> scores -> top-k -> optional renormalisation
(eredu/src/backend/mlx/nn/moe.rs:433-507,652-656; config architectures/qwen/dense.rs:934-951). Expert bank layout:
``gate_up [E, 2I, H]`` (gate rows then up rows per expert) and ``down [E, H, I]``
(runtime/checkpoint/load.rs:1109-1150; split HF keys ``mlp.experts.{e}.{gate,up,down}_proj.weight`` :1073-1104).

Expert parallelism: every rank of the expert group owns a contiguous range of experts. With replicated
activations (attention ran tensor-parallel on the same ranks) each rank routes all tokens identically, runs its
own experts and the partial outputs are summed over the group (the reference's production path,
runtime/distributed/expert.rs:703-766) - here through the peer-memory all-reduce with the residual folded in.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import moe as moe_ops


class MoEBlock:
    def __init__(self, cfg, router_w, w_gate_up, w_down, e0: int, n_experts: int, ep_ops=None, ep_size: int = 1,
                 shared=None, router_bias=None, router_linear_bias=None, gu_bias=None, down_bias=None, act="swiglu",
                 shared_gate_w=None):
        self.cfg = cfg
        self.router_w = router_w          # [E, H]
        self.w_gate_up = w_gate_up        # [E_local, 2I, H]
        self.w_down = w_down              # [E_local, H, I]
        self.e0 = e0
        self.n_experts = n_experts
        self.ep_ops = ep_ops
        self.ep_size = ep_size
        self.shared = shared              # optional (w_gate_up [2Is, H], w_down [H, Is]) dense shared expert
        self.shared_gate_w = shared_gate_w  # optional [1, H]: the shared expert's output is scaled by sigmoid(x . w)
        self.router_bias = router_bias                # selection-only bias (added to the scores used for top-k)
        self.router_linear_bias = router_linear_bias  # bias of the router projection itself (GPT-OSS)
        self.gu_bias = gu_bias                        # [E_local, 2I] per-expert bias, gate part then up part
        self.down_bias = down_bias                    # [E_local, H]
        self.act = act
        self.stats = {"calls": 0}
        # benchmark knob: (period, boost [E] fp32 on the device) - every period-th token gets `boost` added to its router
        # logits (a skewed-router load: 1 / period of the tokens crowd onto the boosted experts)
        self.skew = None

    def tensors(self):
        out = [self.router_w, self.w_gate_up, self.w_down]
        out.extend(t for t in (self.router_bias, self.router_linear_bias, self.gu_bias, self.down_bias, self.shared_gate_w)
                   if t is not None)
        if self.shared is not None:
            out.extend(self.shared)
        return out

    def _shared_out(self, x):
        """Dense shared expert (None without one), scaled by its sigmoid gate when the family has it."""
        if self.shared is None:
            return None
        sgu, sd = self.shared
        if self.act in moe_ops.UNGATED:
            y = ops.linear(torch.relu(ops.linear(x, sgu)).square_(), sd)
        else:
            y = ops.linear(ops.gated_linear(x, sgu, sgu.shape[0] // 2), sd)
        if self.shared_gate_w is not None:
            y = (y.float() * torch.sigmoid(x.float() @ self.shared_gate_w.float().t())).to(y.dtype)
        return y

    def router_logits(self, x, row0: int = 0):
        """fp32 router logits of the rows of x; ``row0`` is the global token index of row 0 (token-sharded callers)."""
        logits = ops.linear(x, self.router_w, bias=self.router_linear_bias, out_dtype=torch.float32)
        if self.skew is not None:
            period, boost = self.skew
            rows = torch.arange(row0, row0 + x.shape[0], device=x.device)
            pick = ((rows % period) == 0).to(logits.dtype)[:, None]
            logits = logits + pick * boost[None, :]
        return logits

    def route(self, x):
        cfg = self.cfg
        logits = self.router_logits(x)
        return moe_ops.route(logits.contiguous(), cfg.num_experts_per_tok, cfg.router_scoring, cfg.norm_topk_prob,
                             cfg.routed_scaling_factor, self.router_bias, cfg.n_group, cfg.topk_group)

    def observed_call(self, x, residual, observer):
        """Unfused pass that materialises what an activation observer is shown (routing ids, scores, weights, routed /
        shared / combined outputs); numerically the same block."""
        from ..runtime.inspection import MoeRoutingObservation

        cfg = self.cfg
        logits = ops.linear(x, self.router_w, bias=self.router_linear_bias, out_dtype=torch.float32)
        ids, w = moe_ops.route(logits.contiguous(), cfg.num_experts_per_tok, cfg.router_scoring, cfg.norm_topk_prob,
                               cfg.routed_scaling_factor, self.router_bias, cfg.n_group, cfg.topk_group)
        _, raw = moe_ops.route_ref(logits, cfg.num_experts_per_tok, cfg.router_scoring, False, 1.0, self.router_bias)
        shared = self._shared_out(x)
        cache = getattr(self, "expert_cache", None)
        if cache is not None:
            local = cache.forward(x, ids, w, limit=cfg.swiglu_limit, act=self.act)
        else:
            local = moe_ops.experts_forward(x, ids, w, self.w_gate_up, self.w_down, self.e0, limit=cfg.swiglu_limit,
                                            gu_bias=self.gu_bias, down_bias=self.down_bias, act=self.act)
        reduced = self.ep_ops.all_reduce(local.clone()) if self.ep_size > 1 else None
        routed = reduced if reduced is not None else local
        combined = routed.float() + (shared.float() if shared is not None else 0.0)
        prefix = f"model.layers.{getattr(self, 'layer_index', '?')}.mlp"
        observer.observe_moe_routing(MoeRoutingObservation(
            prefix=prefix, selected_experts=ids, selected_scores=raw, routing_weights=w, routed_output=routed,
            num_experts=self.n_experts, local_routed_output=local if reduced is not None else None,
            reduced_routed_output=reduced, shared_output=shared, combined_output=combined.to(x.dtype)))
        out = combined + (residual.float() if residual is not None else 0.0)
        return out.to(x.dtype)

    def __call__(self, x, residual=None):
        """x: normalised hidden states [T, H]; returns residual + MoE(x)."""
        self.stats["calls"] += 1
        a2a = getattr(self, "ep_a2a", None)
        if a2a is not None and self.ep_size > 1:
            # token-sharded expert parallelism: routes travel to their expert's owner and back (parallel/ep_a2a.py)
            return a2a.forward(self, x, residual)
        cache = getattr(self, "expert_cache", None)
        if cache is not None:
            # experts live in host memory behind a bounded device bank: route, then let the cache run the experts
            ids, w = self.route(x)
            extra = self._shared_out(x)
            if self.ep_size == 1:
                return cache.forward(x, ids, w, residual=residual, extra=extra, limit=self.cfg.swiglu_limit, act=self.act)
            partial = cache.forward(x, ids, w, extra=extra if self.e0 == 0 else None, limit=self.cfg.swiglu_limit,
                                    act=self.act)
            return self.ep_ops.all_reduce(partial, residual=residual)
        plan = xp = None
        if x.is_cuda and x.shape[0] <= 64 and self.cfg.n_group <= 1:
            # decode-sized: routing, expert plan and row gather in one kernel
            cfg = self.cfg
            logits = self.router_logits(x)
            ids, w, plan, xp = moe_ops.route_plan_gather(logits.contiguous(), x, cfg.num_experts_per_tok, cfg.router_scoring,
                                                         cfg.norm_topk_prob, cfg.routed_scaling_factor, self.router_bias,
                                                         self.e0,
                                                         self.w_gate_up.shape[0])
        else:
            ids, w = self.route(x)
        extra = self._shared_out(x)
        if self.ep_size == 1:
            return moe_ops.experts_forward(x, ids, w, self.w_gate_up, self.w_down, self.e0, residual=residual,
                                           extra=extra, limit=self.cfg.swiglu_limit, plan=plan, xp=xp, gu_bias=self.gu_bias,
                                           down_bias=self.down_bias, act=self.act)
        # shared experts are replicated: add them on one rank only so that the group sum counts them once
        own_extra = extra if self.e0 == 0 else None
        comm = getattr(self.ep_ops, "fused_comm", lambda tokens, hidden: None)(x.shape[0], x.shape[1]) if x.is_cuda else None
        if comm is not None:  # decode-sized step: combine and all-reduce are one kernel over peer memory
            return moe_ops.experts_forward(x, ids, w, self.w_gate_up, self.w_down, self.e0, residual=residual,
                                           extra=own_extra, limit=self.cfg.swiglu_limit, comm=comm, plan=plan, xp=xp,
                                           gu_bias=self.gu_bias, down_bias=self.down_bias, act=self.act)
        partial = moe_ops.experts_forward(x, ids, w, self.w_gate_up, self.w_down, self.e0, residual=None,
                                          extra=own_extra, limit=self.cfg.swiglu_limit, plan=plan, xp=xp, gu_bias=self.gu_bias,
                                           down_bias=self.down_bias, act=self.act)
        return self.ep_ops.all_reduce(partial, residual=residual)


def make_moe_factory(src=None, router_std_scale: bool = False):
    """Factory ``(model, layer, get, has) -> MoEBlock`` used by ``build_from_tensors``. Only the experts owned by
    this rank are read and uploaded."""

    def factory(model, li, get, has):
        cfg = model.cfg
        par = model.par
        p = f"model.layers.{li}.mlp."
        dev, dt = model.device, model.dtype
        e0, e1 = par.expert_range(cfg.num_experts) if par.ep_size > 1 else (0, cfg.num_experts)
        # execution id -> checkpoint id (identity unless the experts are dealt round-robin or by an explicit table)
        order = par.expert_order(cfg.num_experts) if par.ep_size > 1 else None
        mine = list(range(e0, e1)) if order is None else order[e0:e1]
        rows = None if order is None else torch.tensor(order, dtype=torch.long)

        def renamed(t):            # a per-expert tensor (router rows, score biases) in execution order
            return t if rows is None else t.index_select(0, rows.to(t.device))

        def bank(t):               # this rank's slice of a stacked expert bank
            return t[e0:e1] if rows is None else t.index_select(0, rows[e0:e1].to(t.device))

        mx = f"model.layers.{li}.block_sparse_moe."   # Mixtral naming: w1 = gate, w3 = up, w2 = down
        if has(mx + "gate.weight") and not has(p + "gate.weight"):
            router = renamed(get(mx + "gate.weight")).to(device=dev, dtype=dt).contiguous()
            gu = torch.stack([torch.cat((get(mx + f"experts.{e}.w1.weight"), get(mx + f"experts.{e}.w3.weight")), 0)
                              for e in mine], 0).to(device=dev, dtype=dt).contiguous()
            dn = torch.stack([get(mx + f"experts.{e}.w2.weight") for e in mine], 0).to(device=dev, dtype=dt).contiguous()
            block = MoEBlock(cfg, router, gu, dn, e0, cfg.num_experts, ep_size=par.ep_size)
            block._model = model
            block.layer_index = li
            return block
        nm = f"model.layers.{li}.mixer."
        if has(p + "router.weight") or has(nm + "gate.weight"):
            if order is not None:
                raise NotImplementedError("GPT-OSS and Nemotron-H sparse blocks take the balanced expert assignment only")
            return _gpt_oss_block(model, li, get, has, e0, e1) if has(p + "router.weight") else _nemotron_block(model, li, get, has, e0, e1)
        router = renamed(get(p + "gate.weight")).to(device=dev, dtype=dt).contiguous()
        if has(p + "experts.gate_up_proj"):
            gu = bank(get(p + "experts.gate_up_proj"))
            dn = bank(get(p + "experts.down_proj"))
        elif has(p + "experts.gate_exps.weight"):  # GGUF stacked banks
            g = bank(get(p + "experts.gate_exps.weight"))
            u = bank(get(p + "experts.up_exps.weight"))
            gu = torch.cat((g, u), dim=1)
            dn = bank(get(p + "experts.down_exps.weight"))
        else:
            gu = torch.stack([torch.cat((get(p + f"experts.{e}.gate_proj.weight"), get(p + f"experts.{e}.up_proj.weight")), 0)
                              for e in mine], 0)
            dn = torch.stack([get(p + f"experts.{e}.down_proj.weight") for e in mine], 0)
        gu = gu.to(device=dev, dtype=dt).contiguous()
        dn = dn.to(device=dev, dtype=dt).contiguous()
        shared = None
        for sh in ("shared_expert", "shared_experts"):      # Qwen / DeepSeek spellings
            if has(p + f"{sh}.gate_proj.weight"):
                sgu = torch.cat((get(p + f"{sh}.gate_proj.weight"), get(p + f"{sh}.up_proj.weight")), 0)
                shared = (sgu.to(device=dev, dtype=dt).contiguous(),
                          get(p + f"{sh}.down_proj.weight").to(device=dev, dtype=dt).contiguous())
        sel_bias = None
        for name in ("expert_bias", "gate.e_score_correction_bias"):   # LFM2-MoE / DeepSeek: selection-only score bias
            if has(p + name):
                sel_bias = renamed(get(p + name)).to(device=dev, dtype=torch.float32).contiguous()
        shared_gate = None
        if has(p + "shared_expert_gate.weight"):
            shared_gate = get(p + "shared_expert_gate.weight").to(device=dev, dtype=dt).contiguous()
        block = MoEBlock(cfg, router, gu, dn, e0, cfg.num_experts, ep_size=par.ep_size, shared=shared, router_bias=sel_bias,
                         shared_gate_w=shared_gate)
        block._model = model
        block.layer_index = li
        return block

    return factory


def _gpt_oss_block(model, li, get, has, e0, e1):
    """GPT-OSS sparse block: router with a linear bias, experts with biases and the clamped (u + 1) * g * sigmoid(1.702 g)
    gate. Checkpoint layout (eredu/src/backend/mlx/architectures/gpt_oss/checkpoint.rs): ``mlp.router.{weight,bias}``;
    ``mlp.experts.gate_up_proj`` [E, H, 2I] with gate and up INTERLEAVED on the last axis (+ ``_bias`` [E, 2I]),
    ``mlp.experts.down_proj`` [E, I, H] (+ ``_bias`` [E, H]); or the MXFP4 form ``*_blocks`` u8 [E, rows, K/32, 16] with
    ``*_scales`` u8 [E, rows, K/32] (E8M0), which is decoded to the compute dtype at load."""
    import numpy as np

    from ..lib import _eredu_host as H

    cfg, dev, dt = model.cfg, model.device, model.dtype
    p = f"model.layers.{li}.mlp."

    def bank(name):
        """[E_local, rows, K] in the compute dtype, rows = output features."""
        if has(p + f"experts.{name}_blocks"):
            blocks = get(p + f"experts.{name}_blocks")[e0:e1]
            scales = get(p + f"experts.{name}_scales")[e0:e1]
            E, rows = blocks.shape[0], blocks.shape[1]
            packed = np.ascontiguousarray(blocks.cpu().numpy()).reshape(E * rows, -1).view(np.uint32)
            sc = np.ascontiguousarray(scales.cpu().numpy()).reshape(E * rows, -1)
            w = torch.from_numpy(np.asarray(H.mxfp4_dequantize(packed, sc))).reshape(E, rows, -1)
            return w
        return get(p + f"experts.{name}")[e0:e1].transpose(1, 2)     # stored input-major: [E, K, rows]

    gu = bank("gate_up_proj").float()                                # [E, 2I, H], rows interleaved gate / up
    gu = torch.cat((gu[:, 0::2], gu[:, 1::2]), dim=1)                # -> gate rows then up rows
    dn = bank("down_proj")
    gub = get(p + "experts.gate_up_proj_bias")[e0:e1].float()
    gub = torch.cat((gub[:, 0::2], gub[:, 1::2]), dim=1)
    dnb = get(p + "experts.down_proj_bias")[e0:e1]
    up = lambda t: t.to(device=dev, dtype=dt).contiguous()           # noqa: E731
    block = MoEBlock(cfg, up(get(p + "router.weight")), up(gu), up(dn), e0, cfg.num_experts, ep_size=model.par.ep_size,
                     router_linear_bias=up(get(p + "router.bias")), gu_bias=up(gub), down_bias=up(dnb), act="oss_glu")
    block._model = model
    block.layer_index = li
    return block


def _nemotron_block(model, li, get, has, e0, e1):
    """Nemotron-H sparse mixer: sigmoid router with a score-correction bias (selection only), experts with a single up
    projection and relu^2, an ungated relu^2 shared expert (architectures/nemotron_h/model.rs:1038-1290)."""
    cfg, dev, dt = model.cfg, model.device, model.dtype
    p = f"model.layers.{li}.mixer."
    up = lambda t: t.to(device=dev, dtype=dt).contiguous()                         # noqa: E731
    if has(p + "experts.up_proj"):        # packed banks [E, I, H] / [E, H, I]
        w_up, w_dn = get(p + "experts.up_proj")[e0:e1], get(p + "experts.down_proj")[e0:e1]
    else:
        w_up = torch.stack([get(p + f"experts.{e}.up_proj.weight") for e in range(e0, e1)], 0)
        w_dn = torch.stack([get(p + f"experts.{e}.down_proj.weight") for e in range(e0, e1)], 0)
    sel = get(p + "gate.e_score_correction_bias").to(device=dev, dtype=torch.float32).contiguous() \
        if has(p + "gate.e_score_correction_bias") else None
    shared = None
    if has(p + "shared_experts.up_proj.weight"):
        shared = (up(get(p + "shared_experts.up_proj.weight")), up(get(p + "shared_experts.down_proj.weight")))
    block = MoEBlock(cfg, up(get(p + "gate.weight")), up(w_up), up(w_dn), e0, cfg.num_experts, ep_size=model.par.ep_size,
                     shared=shared, router_bias=sel, act="relu2")
    block._model = model
    block.layer_index = li
    return block


def attach_ep(model, ep_ops) -> None:
    """Give every MoE block of a model shard the collective used to sum partial expert outputs."""
    for lw in model.layers:
        if lw.moe is not None:
            lw.moe.ep_ops = ep_ops
