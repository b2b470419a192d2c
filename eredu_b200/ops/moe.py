"""Mixture-of-experts operators: routing, permute, grouped expert GEMMs, weighted combine.

CUDA tensors run the kernels of ``csrc/kernels/moe.cu`` and the grouped mode of the tcgen05 GEMM; CPU tensors
run the PyTorch reference with the same semantics (eredu/src/backend/mlx/nn/moe.rs:433-507,652-738,1061-1163).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import native
from .core import _sm_count, linear
from .native import I, P, check, lib, ptr, status_word, stream_ptr

native.register("eredu_moe_route", I, [P, P, P, P, I, I, I, I, I, native.F, P])
native.register("eredu_moe_plan", I, [P, I, I, I, I, I, P, P, P, P, I, P, P])
native.register("eredu_moe_gather", I, [P, P, P, P, I, I, P])
native.register("eredu_moe_combine", I, [P, P, P, P, P, P, I, I, I, P])
native.register("eredu_moe_route_plan_gather", I, [P, P, P, P, I, I, I, I, I, native.F, I, I, I, P, P, P, P, I, P, P, P, I, P])
native.register("eredu_moe_combine_ar", I, [P, P, P, P, P, P, I, I, I, P, P, P])
native.register("eredu_gemm_bf16_grouped", I, [P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, I, P, P, I, I, native.F, P])

SCORING = {"softmax": 0, "sigmoid": 1, "sqrt_softplus": 2, "topk_softmax": 3}


def route_ref(logits, k, scoring="softmax", renorm=True, scale=1.0, sel_bias=None, n_group=1, topk_group=1,
              norm_eps=0.0, routing_indices=None):
    """Reference router (eredu/src/backend/mlx/nn/moe.rs:433-507,652-702). Scores -> (+ selection bias) -> top-k, with the
    group-limited form when ``n_group > 1`` (experts in n_group equal groups, a group's score is the sum of its two best
    experts, only the topk_group best groups stay eligible) -> weights gathered from the UNBIASED scores -> optional
    renormalisation (``norm_eps`` added to the sum) -> scale. ``routing_indices`` [T, k] replaces the selection
    (hash routing: a table chooses the experts, the router only weights them)."""
    x = logits.float()
    if scoring == "softmax":
        score = torch.softmax(x, -1)
    elif scoring == "sigmoid":
        score = torch.sigmoid(x)
    elif scoring == "sqrt_softplus":
        score = torch.sqrt(F.softplus(x))
    else:
        score = x
    if routing_indices is not None:
        ids = routing_indices.long()
    else:
        select = score + (sel_bias.float() if sel_bias is not None else 0.0)
        if n_group > 1 or topk_group > 1:
            T, E = select.shape
            if n_group <= 0 or topk_group <= 0 or topk_group > n_group or E % n_group != 0:
                raise ValueError("invalid grouped MoE router configuration")
            per = E // n_group
            grouped = select.view(T, n_group, per)
            group_scores = torch.topk(grouped, min(2, per), dim=-1).values.sum(-1)
            keep = torch.topk(group_scores, topk_group, dim=-1).indices
            mask = torch.zeros((T, n_group), dtype=torch.bool, device=select.device).scatter_(1, keep, True)
            select = torch.where(mask[:, :, None].expand(T, n_group, per).reshape(T, E), select,
                                 torch.full_like(select, float("-inf")))
        ids = torch.topk(select, k, dim=-1).indices
    w = score.gather(-1, ids)
    if scoring == "topk_softmax":
        w = torch.softmax(w, -1)
    elif renorm:
        w = w / (w.sum(-1, keepdim=True) + norm_eps).clamp(min=1e-20)
    return ids.to(torch.int32), (w * scale).float()


def route(logits, k, scoring="softmax", renorm=True, scale=1.0, sel_bias=None, n_group=1, topk_group=1, norm_eps=0.0,
          routing_indices=None):
    """Router logits [T, E] fp32 -> (ids [T, k] int32, weights [T, k] fp32). Group-limited selection, a renormalisation
    epsilon and table-driven (hash) routing run as tensor operations; the plain forms use the routing kernel."""
    if not logits.is_cuda or n_group > 1 or topk_group > 1 or norm_eps != 0.0 or routing_indices is not None:
        return route_ref(logits, k, scoring, renorm, scale, sel_bias, n_group, topk_group, norm_eps, routing_indices)
    T, E = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    code = lib().eredu_moe_route(ptr(logits), ptr(sel_bias), ptr(ids), ptr(w), T, E, k, SCORING[scoring],
                                 1 if renorm else 0, scale, stream_ptr(logits.device))
    check(code, "eredu_moe_route")
    return ids, w


ACTS = {"swiglu": 0, "oss_glu": 1}
UNGATED = ("relu2",)   # activations of experts with a single up projection: w_gate_up is then [E, I, H]


def gated_act_ref(g, u, act="swiglu", limit=0.0):
    """silu(g) * u, or the GPT-OSS gate g * sigmoid(1.702 g) * (u + 1); with ``limit`` the gate is clamped from above
    and the linear branch to [-limit, limit] first."""
    if limit > 0:
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    if act == "oss_glu":
        return g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return F.silu(g) * u


def experts_ref(x, ids, weights, w_gate_up, w_down, e0=0, limit=0.0, gu_bias=None, down_bias=None, act="swiglu"):
    """Reference expert computation for local experts [e0, e0 + E_local): sum_k w * down_e(act(gate_e x, up_e x)).
    ``gu_bias`` [E_local, 2I] (gate part then up part) and ``down_bias`` [E_local, H] are per-expert biases."""
    T, H = x.shape
    E_local, two_i, _ = w_gate_up.shape
    inter = two_i if act in UNGATED else two_i // 2
    out = torch.zeros((T, H), dtype=torch.float32, device=x.device)
    xf = x.float()
    for slot in range(ids.shape[1]):
        for e in range(E_local):
            sel = (ids[:, slot].long() == e + e0).nonzero().squeeze(1)
            if sel.numel() == 0:
                continue
            y = xf[sel] @ w_gate_up[e].float().t()
            if gu_bias is not None:
                y = y + gu_bias[e].float()
            if act in UNGATED:
                a = torch.relu(y).square().to(x.dtype).float()
            else:
                g, u = y[:, :inter], y[:, inter:]
                a = gated_act_ref(g, u, act, limit).to(x.dtype).float()
            o = a @ w_down[e].float().t()
            if down_bias is not None:
                o = o + down_bias[e].float()
            o = o.to(x.dtype).float()
            out[sel] += weights[sel, slot, None] * o
    return out


class ExpertPlan:
    """Device-side routing plan for the local experts of one MoE layer invocation."""

    def __init__(self, ids, k, e0, e1, tile, rows_cap, device=None, routes=None, run=True):
        dev = ids.device if ids is not None else device
        routes = ids.numel() if ids is not None else routes
        n_local = e1 - e0
        self.tile = tile
        self.rows_cap = rows_cap
        self.n_work = (rows_cap + tile - 1) // tile + n_local
        self.seg = torch.empty(n_local + 1, dtype=torch.int32, device=dev)
        self.route_pos = torch.empty(routes, dtype=torch.int32, device=dev)
        self.row_token = torch.empty(max(rows_cap, 1), dtype=torch.int32, device=dev)
        self.work = torch.empty((self.n_work, 4), dtype=torch.int32, device=dev)
        self.counts = torch.empty(2, dtype=torch.int32, device=dev)
        if not run:
            return
        code = lib().eredu_moe_plan(ptr(ids), routes, k, e0, e1, tile, ptr(self.seg), ptr(self.route_pos),
                                    ptr(self.row_token), ptr(self.work), self.n_work, ptr(self.counts),
                                    stream_ptr(dev))
        check(code, "eredu_moe_plan")


def pick_tile(expected_rows_per_expert: float) -> int:
    for t in (16, 32, 64, 128):
        if expected_rows_per_expert <= t:
            return t
    return 128


def route_plan_gather(logits, x, k, scoring, renorm, scale, sel_bias, e0, n_local):
    """Decode-sized steps (<= 64 tokens): routing, the local experts' plan and the row gather in one kernel.
    Returns (ids, weights, plan, xp) for :func:`experts_forward`."""
    T, E = logits.shape
    H = x.shape[1]
    routes = T * k
    tile = pick_tile(routes / max(1, n_local))
    dev = x.device
    ids = torch.empty((T, k), dtype=torch.int32, device=dev)
    w = torch.empty((T, k), dtype=torch.float32, device=dev)
    plan = ExpertPlan(None, k, e0, e0 + n_local, tile, routes, device=dev, routes=routes, run=False)
    xp = torch.empty((routes, H), dtype=x.dtype, device=dev)
    # one CTA copies the rows itself only when there are few of them (expected local routes <= 64)
    inline_gather = routes * n_local <= 64 * E
    code = lib().eredu_moe_route_plan_gather(ptr(logits), ptr(sel_bias), ptr(ids), ptr(w), T, E, k, SCORING[scoring],
                                             1 if renorm else 0, scale, e0, e0 + n_local, tile, ptr(plan.seg),
                                             ptr(plan.route_pos), ptr(plan.row_token), ptr(plan.work), plan.n_work,
                                             ptr(plan.counts), ptr(x), ptr(xp) if inline_gather else None, H, stream_ptr(dev))
    check(code, "eredu_moe_route_plan_gather")
    if not inline_gather:
        check(lib().eredu_moe_gather(ptr(x), ptr(plan.row_token), ptr(plan.counts), ptr(xp), routes, H, stream_ptr(dev)),
              "eredu_moe_gather")
    return ids, w, plan, xp


def experts_forward(x, ids, weights, w_gate_up, w_down, e0=0, residual=None, extra=None, limit=0.0, rows_cap=None,
                    comm=None, plan=None, xp=None, gu_bias=None, down_bias=None, act="swiglu", rows_only=False):
    """Local-expert MoE computation. x: [T, H] bf16; ids / weights: [T, k]; w_gate_up: [E_local, 2I, H];
    w_down: [E_local, H, I]. Returns residual + extra + sum over local routes (bf16 [T, H]). With ``comm`` (a peer
    communication context of the expert group) the combine kernel also sums the partial outputs of all ranks:
    ``extra`` is then counted once per rank that passes it, ``residual`` once in total. ``rows_only`` (CUDA, with a
    ``plan`` and permuted rows ``xp``): stop after the two grouped GEMMs and return the rows in plan order."""
    if not x.is_cuda:
        out = experts_ref(x, ids, weights, w_gate_up, w_down, e0, limit, gu_bias, down_bias, act)
        if residual is not None:
            out = out + residual.float()
        if extra is not None:
            out = out + extra.float()
        return out.to(x.dtype)
    T, H = x.shape
    k = ids.shape[1] if ids is not None else 1
    E_local, two_i, _ = w_gate_up.shape
    ungated = act in UNGATED
    inter = two_i if ungated else two_i // 2
    routes = T * k
    rows_cap = rows_cap or routes
    dev = x.device
    if plan is None:
        tile = pick_tile(routes / max(1, E_local))
        plan = ExpertPlan(ids, k, e0, e0 + E_local, tile, rows_cap)
        xp = torch.empty((rows_cap, H), dtype=x.dtype, device=dev)
        check(lib().eredu_moe_gather(ptr(x), ptr(plan.row_token), ptr(plan.counts), ptr(xp), rows_cap, H, stream_ptr(dev)),
              "eredu_moe_gather")
    tile = plan.tile
    gated = torch.empty((rows_cap, inter), dtype=x.dtype, device=dev)
    st = status_word(dev)
    sm = _sm_count(dev)
    wgu = w_gate_up.view(E_local * two_i, H)
    code = lib().eredu_gemm_bf16_grouped(ptr(xp), ptr(wgu), ptr(gated), ptr(plan.work), plan.n_work, tile, rows_cap, inter,
                                         H, H, H, inter, E_local * two_i, two_i, 0 if ungated else 1, 0, sm, ptr(st),
                                         ptr(gu_bias), two_i if gu_bias is not None else 0, 0 if ungated else ACTS[act],
                                         float(limit), stream_ptr(dev))
    check(code, "eredu_gemm_bf16_grouped(gate_up)")
    if ungated:
        gated = torch.relu(gated).square_()      # relu^2 between the two grouped GEMMs (rows past the plan are unused)
    y = torch.empty((rows_cap, H), dtype=x.dtype, device=dev)
    wd = w_down.view(E_local * H, inter)
    code = lib().eredu_gemm_bf16_grouped(ptr(gated), ptr(wd), ptr(y), ptr(plan.work), plan.n_work, tile, rows_cap, H,
                                         inter, inter, inter, H, E_local * H, H, 0, 0, sm, ptr(st), ptr(down_bias),
                                         H if down_bias is not None else 0, 0, 0.0, stream_ptr(dev))
    check(code, "eredu_gemm_bf16_grouped(down)")
    if rows_only:      # expert-contiguous output rows (row order of the plan); the caller combines them
        return y
    out = torch.empty((T, H), dtype=x.dtype, device=dev)
    if comm is not None:
        code = lib().eredu_moe_combine_ar(ptr(y), ptr(plan.route_pos), ptr(weights), ptr(residual), ptr(extra), ptr(out),
                                          T, k, H, comm, ptr(st), stream_ptr(dev))
        check(code, "eredu_moe_combine_ar")
        return out
    code = lib().eredu_moe_combine(ptr(y), ptr(plan.route_pos), ptr(weights), ptr(residual), ptr(extra), ptr(out), T, k,
                                   H, stream_ptr(dev))
    check(code, "eredu_moe_combine")
    return out
