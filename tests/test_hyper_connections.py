"""Hyper-connection residual mixing: the Sinkhorn split is doubly stochastic for any leading shape, collapse / expand agree
with explicit per-token loops, parameters are validated."""
import pytest
import torch

from eredu_b200.ops.hyper_connections import HyperConnection, HyperHead, expand, split_sinkhorn


def test_split_keeps_leading_dimensions_and_normalises_rows_and_columns():
    n = 4
    g = torch.Generator().manual_seed(0)
    mixes = torch.randn(2, 3, (2 + n) * n, generator=g) * 2
    scale, base = torch.tensor([0.7, 1.3, 2.0]), torch.randn((2 + n) * n, generator=g) * 0.3
    pre, post, comb = split_sinkhorn(mixes, scale, base, n, 20, 1e-6)
    assert pre.shape == post.shape == (2, 3, n) and comb.shape == (2, 3, n, n)
    assert torch.allclose(comb.sum(-2), torch.ones(2, 3, n), atol=1e-4)
    row_err = float((comb.sum(-1) - 1).abs().max())
    assert (pre > 0).all() and (pre <= 1.0 + 2e-6).all() and (post >= 0).all() and (post <= 2).all() and (comb > 0).all()
    # one iteration normalises columns only
    _, _, once = split_sinkhorn(mixes, scale, base, n, 1, 1e-6)
    assert torch.allclose(once.sum(-2), torch.ones(2, 3, n), atol=5e-3)      # a nearly empty column feels the epsilon
    assert row_err < 0.05 and row_err < 0.2 * float((once.sum(-1) - 1).abs().max())      # the iterations pull the rows to one as well
    # zero logits: uniform mixing, pre = 0.5 + eps, post = 1
    p0, q0, c0 = split_sinkhorn(torch.zeros(5, 8), torch.ones(3), torch.zeros(8), 2, 20, 1e-6)
    assert torch.allclose(p0, torch.full((5, 2), 0.5 + 1e-6)) and torch.allclose(q0, torch.ones(5, 2)) and torch.allclose(c0, torch.full((5, 2, 2), 0.5), atol=1e-5)
    for bad in (dict(streams=0), dict(iterations=0), dict(eps=0.0), dict(eps=float("inf"))):
        kw = dict(streams=2, iterations=3, eps=1e-6)
        kw.update(bad)
        with pytest.raises(ValueError):
            split_sinkhorn(torch.zeros(5, 8), torch.ones(3), torch.zeros(8), kw["streams"], kw["iterations"], kw["eps"])
    with pytest.raises(ValueError):
        split_sinkhorn(torch.zeros(5, 7), torch.ones(3), torch.zeros(8), 2, 3, 1e-6)
    with pytest.raises(ValueError):
        split_sinkhorn(torch.zeros(5, 8), torch.ones(2), torch.zeros(8), 2, 3, 1e-6)


def test_collapse_and_expand_match_token_by_token_arithmetic():
    n, H, T = 3, 8, 5
    g = torch.Generator().manual_seed(1)
    width = (2 + n) * n
    hc = HyperConnection(torch.randn(width, n * H, generator=g) * 0.2, torch.randn(width, generator=g) * 0.1,
                         torch.tensor([1.0, 0.5, 1.5]), n, H, iterations=7, eps=1e-6)
    R = torch.randn(T, n, H, generator=g)
    x, post, comb = hc.collapse(R, 1e-5)
    assert x.shape == (T, H) and post.shape == (T, n) and comb.shape == (T, n, n)
    for t in range(T):
        flat = R[t].reshape(-1)
        mixes = (flat * torch.rsqrt(flat.square().mean() + 1e-5)) @ hc.function.t()
        pre, po, co = split_sinkhorn(mixes, hc.scale, hc.base, n, 7, 1e-6)
        assert torch.allclose(x[t], sum(pre[i] * R[t, i] for i in range(n)), atol=1e-6)
        assert torch.allclose(post[t], po) and torch.allclose(comb[t], co)
    y = torch.randn(T, H, generator=g)
    out = expand(y, R, post, comb)
    for t in range(T):
        for i in range(n):
            want = post[t, i] * y[t] + sum(comb[t, j, i] * R[t, j] for j in range(n))
            assert torch.allclose(out[t, i], want, atol=1e-6)
    # batched layout [batch, tokens, n, H] gives the same numbers as the flat one
    xb, pb, cb = hc.collapse(R.reshape(1, T, n, H), 1e-5)
    assert torch.allclose(xb[0], x) and torch.allclose(expand(y[None], R[None], pb, cb)[0], out)
    # bf16 streams: arithmetic in fp32, results in the input dtype
    xh, ph, ch = hc.collapse(R.bfloat16(), 1e-5)
    assert xh.dtype == torch.bfloat16 and ph.dtype == torch.float32 and expand(y.bfloat16(), R.bfloat16(), ph, ch).dtype == torch.bfloat16
    head = HyperHead(torch.randn(n, n * H, generator=g) * 0.2, torch.randn(n, generator=g) * 0.1, torch.tensor([1.2]), n, H, 1e-5)
    h = head(R)
    flat = R[2].reshape(-1)
    pre = torch.sigmoid(((flat * torch.rsqrt(flat.square().mean() + 1e-5)) @ head.function.t()) * 1.2 + head.base) + 1e-6
    assert h.shape == (T, H) and torch.allclose(h[2], sum(pre[i] * R[2, i] for i in range(n)), atol=1e-6)
    with pytest.raises(ValueError):
        HyperConnection(torch.zeros(width, n * H + 1), torch.zeros(width), torch.ones(3), n, H)
    with pytest.raises(ValueError):
        hc.collapse(torch.zeros(T, n + 1, H), 1e-5)
    with pytest.raises(ValueError):
        HyperHead(torch.zeros(n, n * H), torch.zeros(n + 1), torch.ones(1), n, H, 1e-5)
