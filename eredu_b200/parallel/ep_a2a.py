"""Token-sharded expert parallelism: all-to-all dispatch of routes to their expert owners and the matching combine.

The reference's ``dispatch_sharded`` (eredu/src/backend/mlx/runtime/distributed/expert.rs:1054-1222) exchanges a count
vector (all-gather + host sync, :781-842), then four forward ``all_to_all_v`` messages (hidden rows, expert ids, route
indices, weights) and two reverse ones, and sums the returned rows per token (``segment_sum``). Two implementations of
that data flow behind one interface:

* :class:`PeerA2A` - four kernels over NVLink peer memory (``csrc/kernels/moe.cu``): the routing permute is the peer
  store, counts never leave the device, the owner returns rows into the source's ``[token, k]`` slots and the source's
  weighted sum in slot order is fused with the all-gather that restores replicated activations. CUDA-graph safe.
* :class:`CollectiveA2A` - the same exchanges through ``torch.distributed`` (``all_to_all_single`` with split sizes,
  count exchange read on the host like the reference): the library baseline on NCCL, and the CPU path on gloo.

Activations are replicated across the ranks (attention ran tensor-parallel on the same GPUs); rank r is the *source* of
tokens ``[r * ceil(T / n), (r + 1) * ceil(T / n))``. Each route is computed once, by the rank that owns its expert.
"""
from __future__ import annotations

import ctypes

import torch

from .. import ops
from ..ops import moe as moe_ops
from ..ops import native
from ..ops.native import I, L, P

native.register("eredu_moe_a2a_dispatch", I, [P, P, P, P, I, P, P, P])
native.register("eredu_moe_a2a_recv_plan", I, [P, P, I, I, I, P, P, P, P, P, I, P, P, P])
native.register("eredu_moe_a2a_return", I, [P, P, P, P, P, P])
native.register("eredu_moe_a2a_combine", I, [P, P, P, P, P, I, I, P, P])


def _slice_of(T: int, n: int, rank: int):
    per = (T + n - 1) // n
    t0 = min(T, rank * per)
    return per, t0, min(T, t0 + per) - t0


def _route_own(block, x_own, t0=0):
    cfg = block.cfg
    logits = block.router_logits(x_own, t0)
    return moe_ops.route(logits.contiguous(), cfg.num_experts_per_tok, cfg.router_scoring, cfg.norm_topk_prob,
                         cfg.routed_scaling_factor, block.router_bias, cfg.n_group, cfg.topk_group)


class CollectiveA2A:
    """The six-exchange data flow on ``torch.distributed`` collectives (NCCL on GPUs, gloo on CPU ranks)."""

    def __init__(self, group, rank: int, size: int):
        self.group, self.rank, self.size = group, rank, size
        self.stats = {"calls": 0, "routes_sent": 0, "routes_remote": 0}

    def _exchange(self, rows, send_counts, recv_counts):
        import torch.distributed as dist

        out = rows.new_empty((int(sum(recv_counts)),) + tuple(rows.shape[1:]))
        try:
            dist.all_to_all_single(out, rows.contiguous(), recv_counts, send_counts, group=self.group)
        except (RuntimeError, NotImplementedError):     # a backend without the fused form: pairwise messages
            outs = list(out.split(recv_counts))
            ins = list(rows.contiguous().split(send_counts))
            reqs = []
            for peer in range(self.size):
                if peer == self.rank:
                    outs[peer].copy_(ins[peer])
                    continue
                reqs.append(dist.isend(ins[peer], dist.get_global_rank(self.group, peer), group=self.group))
                reqs.append(dist.irecv(outs[peer], dist.get_global_rank(self.group, peer), group=self.group))
            for r in reqs:
                r.wait()
        return out

    def forward(self, block, x, residual=None):
        import torch.distributed as dist

        cfg = block.cfg
        T, H = x.shape
        k = cfg.num_experts_per_tok
        n = self.size
        per, t0, n_own = _slice_of(T, n, self.rank)
        e_local = block.w_gate_up.shape[0]
        x_own = x[t0:t0 + n_own]
        if n_own > 0:
            ids, w = _route_own(block, x_own, t0)
        else:
            ids = torch.empty((0, k), dtype=torch.int32, device=x.device)
            w = torch.empty((0, k), dtype=torch.float32, device=x.device)
        flat_ids = ids.reshape(-1).long()
        owner = flat_ids // e_local
        order = torch.argsort(owner, stable=True)                      # routes grouped by owner, route order inside
        send_counts = torch.bincount(owner, minlength=n).to(torch.int64)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group) if x.is_cuda else \
            recv_counts.copy_(self._exchange(send_counts, [1] * n, [1] * n))
        sc, rc = send_counts.tolist(), recv_counts.tolist()            # the host reads the counts, as the reference does
        rows = x_own.index_select(0, order // k) if n_own > 0 else x_own.new_empty((0, H))
        got_rows = self._exchange(rows, sc, rc)
        got_ids = self._exchange(flat_ids[order].to(torch.int32), sc, rc)
        R = got_rows.shape[0]
        if R > 0:
            ones = torch.ones((R, 1), dtype=torch.float32, device=x.device)
            y = moe_ops.experts_forward(got_rows, got_ids.view(R, 1), ones, block.w_gate_up, block.w_down, block.e0,
                                        limit=cfg.swiglu_limit, gu_bias=block.gu_bias, down_bias=block.down_bias, act=block.act)
        else:
            y = got_rows
        back = self._exchange(y, rc, sc)                               # reverse plan: rows return in the order they left
        ret = torch.empty((n_own * k, H), dtype=x.dtype, device=x.device)
        if n_own > 0:
            ret[order] = back
        out_own = (ret.view(n_own, k, H).float() * w[:, :, None]).sum(1)       # slot order
        if residual is not None:
            out_own = out_own + residual[t0:t0 + n_own].float()
        extra = block._shared_out(x_own) if n_own > 0 else None
        if extra is not None:
            out_own = out_own + extra.float()
        padded = torch.zeros((per, H), dtype=x.dtype, device=x.device)
        padded[:n_own] = out_own.to(x.dtype)
        full = torch.empty((per * n, H), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(full, padded, group=self.group)
        self.stats["calls"] += 1
        self.stats["routes_sent"] += int(n_own * k)
        self.stats["routes_remote"] += int(n_own * k - sc[self.rank])
        return full[:T]


class PeerA2A:
    """Dispatch / combine as kernels over peer memory (symmetric buffer of its own, sized for ``max_tokens`` per call)."""

    def __init__(self, group, device, hidden: int, k: int, e_local: int, max_tokens: int = 8192):
        import torch.distributed as dist

        from .comm import PeerGroup

        self.device = torch.device(device)
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        n = self.size
        self.H, self.k, self.e_local, self.max_tokens = hidden, k, e_local, max_tokens
        self.per_max = (max_tokens + n - 1) // n
        cap = self.per_max * k
        r256 = lambda b: (b + 255) // 256 * 256                                          # noqa: E731
        self.recv_bytes = r256(n * cap * hidden * 2)
        self.meta_bytes = r256(n * cap * 8)
        self.cnt_bytes = 256
        self.ret_bytes = r256(cap * hidden * 2)
        self.out_half = r256(self.per_max * n * hidden * 2)
        total = self.recv_bytes + self.meta_bytes + self.cnt_bytes + self.ret_bytes + 2 * self.out_half
        self.pg = PeerGroup(group, self.device, 256, total)
        o = self.pg.out_off
        self.off = {"recv": o, "meta": o + self.recv_bytes, "cnt": o + self.recv_bytes + self.meta_bytes}
        self.off["ret"] = self.off["cnt"] + self.cnt_bytes
        self.off["out"] = self.off["ret"] + self.ret_bytes
        self.cursor = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.calls = 0
        self.lib = native.lib()
        self.stats = {"calls": 0}

    def _view(self, T, per, cap, parity):
        vals = [self.off["recv"], self.off["meta"], self.off["cnt"], self.off["ret"], self.off["out"], self.out_half,
                T, per, self.k, self.H, self.e_local, cap, parity]
        return (ctypes.c_longlong * len(vals))(*vals)

    def forward(self, block, x, residual=None):
        T, H = x.shape
        if T > self.max_tokens:       # longer inputs go through in slices of the buffer size
            parts = [self.forward(block, x[a:a + self.max_tokens], None if residual is None else residual[a:a + self.max_tokens]).clone()
                     for a in range(0, T, self.max_tokens)]
            return torch.cat(parts, 0)
        cfg = block.cfg
        k, n, dev = self.k, self.size, self.device
        per, t0, n_own = _slice_of(T, n, self.rank)
        cap = per * k
        parity = self.calls & 1
        self.calls += 1
        view = self._view(T, per, cap, parity)
        st = native.status_word(dev)
        stream = native.stream_ptr(dev)
        x_own = x[t0:t0 + n_own]
        if n_own > 0:
            ids, w = _route_own(block, x_own, t0)
        else:
            ids = torch.zeros((1, k), dtype=torch.int32, device=dev)
            w = torch.zeros((1, k), dtype=torch.float32, device=dev)
        native.check(self.lib.eredu_moe_a2a_dispatch(self.pg.comm, view, native.ptr(x_own) if n_own > 0 else None, native.ptr(ids),
                                                     n_own, native.ptr(self.cursor), native.ptr(st), stream), "eredu_moe_a2a_dispatch")
        rows_cap = n * cap
        tile = moe_ops.pick_tile(T * k / max(1, cfg.num_experts))
        plan = moe_ops.ExpertPlan(None, 1, block.e0, block.e0 + self.e_local, tile, rows_cap, device=dev, routes=rows_cap, run=False)
        ids_flat = torch.empty(rows_cap, dtype=torch.int32, device=dev)
        native.check(self.lib.eredu_moe_a2a_recv_plan(self.pg.comm, view, block.e0, block.e0 + self.e_local, tile, native.ptr(ids_flat),
                                                      native.ptr(plan.seg), native.ptr(plan.route_pos), native.ptr(plan.row_token),
                                                      native.ptr(plan.work), plan.n_work, native.ptr(plan.counts), native.ptr(st),
                                                      stream), "eredu_moe_a2a_recv_plan")
        recv = self.pg.out_view((rows_cap, H), torch.bfloat16)       # the receive area sits first in the region
        xp = torch.empty((rows_cap, H), dtype=x.dtype, device=dev)
        native.check(self.lib.eredu_moe_gather(native.ptr(recv), native.ptr(plan.row_token), native.ptr(plan.counts), native.ptr(xp),
                                               rows_cap, H, stream), "eredu_moe_gather")
        y = moe_ops.experts_forward(xp, None, None, block.w_gate_up, block.w_down, block.e0, limit=cfg.swiglu_limit,
                                    rows_cap=rows_cap, plan=plan, xp=xp, gu_bias=block.gu_bias, down_bias=block.down_bias,
                                    act=block.act, rows_only=True)
        native.check(self.lib.eredu_moe_a2a_return(self.pg.comm, view, native.ptr(y), native.ptr(plan.route_pos), native.ptr(st),
                                                   stream), "eredu_moe_a2a_return")
        extra = block._shared_out(x_own) if n_own > 0 else None
        res_own = residual[t0:t0 + n_own] if (residual is not None and n_own > 0) else None
        native.check(self.lib.eredu_moe_a2a_combine(self.pg.comm, view, native.ptr(w), native.ptr(res_own), native.ptr(extra), n_own,
                                                    t0, native.ptr(st), stream), "eredu_moe_a2a_combine")
        self.stats["calls"] += 1
        from .comm import view_raw

        base = self.pg.own + self.off["out"] + parity * self.out_half
        return view_raw(base, (T, H), torch.bfloat16, dev)


def attach_ep_a2a(model, par, backend: str = "peer", max_tokens: int = 8192) -> None:
    """Route every sparse block of a model shard through the token-sharded all-to-all form of expert parallelism.
    ``backend``: "peer" (kernels over NVLink peer memory, CUDA only) or "collective" (torch.distributed)."""
    import torch.distributed as dist

    if par.ep_size <= 1:
        return
    group = par.ep_group
    impl = None
    for lw in model.layers:
        if lw.moe is None:
            continue
        if impl is None:
            if backend == "peer" and model.device.type == "cuda":
                impl = PeerA2A(group, model.device, model.cfg.hidden_size, model.cfg.num_experts_per_tok,
                               lw.moe.w_gate_up.shape[0], max_tokens)
            else:
                impl = CollectiveA2A(group, dist.get_rank(group), dist.get_world_size(group))
                model.eager_collectives = True      # split sizes are read on the host: such steps cannot be captured
        lw.moe.ep_a2a = impl
    model.ep_a2a = impl
