"""Gated delta-rule scan: hand-checked step, scalar vs per-channel decay, chunked == one scan, CUDA kernel vs reference."""
import pytest
import torch

from eredu_b200.ops import gated_delta_scan, gated_delta_scan_ref


def test_single_step_by_hand():
    q = torch.tensor([0.5, -0.25]).view(1, 1, 1, 2)
    k = torch.tensor([0.3, 0.4]).view(1, 1, 1, 2)
    v = torch.tensor([1.0, -0.5, 2.0]).view(1, 1, 1, 3)
    g = torch.tensor([-0.2]).view(1, 1, 1)
    beta = torch.tensor([0.8]).view(1, 1, 1)
    S0 = torch.arange(6, dtype=torch.float32).view(1, 1, 2, 3) * 0.1
    S, out = gated_delta_scan_ref(q, k, v, g, beta, S0)
    Sd = S0[0, 0] * torch.exp(torch.tensor(-0.2))
    mem = Sd.t() @ k.view(2)
    want = Sd + torch.outer(k.view(2), 0.8 * (v.view(3) - mem))
    assert torch.allclose(S[0, 0], want, atol=1e-6) and torch.allclose(out.view(3), want.t() @ q.view(2), atol=1e-6)


def test_vector_decay_chunks_and_validation():
    torch.manual_seed(0)
    B, T, H, Dk, Dv = 2, 9, 3, 8, 5
    q, k, v = torch.randn(B, T, H, Dk), torch.randn(B, T, H, Dk) * 0.3, torch.randn(B, T, H, Dv)
    g = -torch.rand(B, T, H)
    beta = torch.rand(B, T, H)
    S1, o1 = gated_delta_scan_ref(q, k, v, g, beta)
    S2, o2 = gated_delta_scan_ref(q, k, v, g[..., None].expand(B, T, H, Dk).contiguous(), beta)
    assert torch.allclose(o1, o2, atol=1e-6) and torch.allclose(S1, S2, atol=1e-6)
    st, outs = None, []
    for a, b in ((0, 4), (4, 5), (5, 9)):                       # prefill chunk, one decode token, another chunk
        st, o = gated_delta_scan_ref(q[:, a:b], k[:, a:b], v[:, a:b], g[:, a:b], beta[:, a:b], st)
        outs.append(o)
    assert torch.allclose(torch.cat(outs, 1), o1, atol=1e-5) and torch.allclose(st, S1, atol=1e-5)
    for bad in (lambda: gated_delta_scan_ref(q[0], k, v, g, beta), lambda: gated_delta_scan_ref(q, k, v, g[:, :2], beta),
                lambda: gated_delta_scan_ref(q, k, v, g, beta[..., None]),
                lambda: gated_delta_scan_ref(q, k, v, g, beta, torch.zeros(B, H, Dk, Dv + 1))):
        with pytest.raises(ValueError):
            bad()
    assert gated_delta_scan(q, k, v, g, beta)[1].shape == (B, T, H, Dv)      # CPU tensors take the reference


@pytest.mark.gpu
@pytest.mark.parametrize("Dk,Dv,vector", [(128, 128, False), (64, 96, True), (128, 40, True)])
def test_gated_delta_kernel_matches_reference(Dk, Dv, vector):
    torch.manual_seed(Dk + Dv)
    dev = "cuda"
    B, T, H = 2, 33, 4
    q = (torch.randn(B, T, H, Dk, device=dev) * 0.3).bfloat16()
    k = torch.nn.functional.normalize(torch.randn(B, T, H, Dk, device=dev), dim=-1).bfloat16()
    v = torch.randn(B, T, H, Dv, device=dev).bfloat16()
    g = -torch.rand((B, T, H, Dk) if vector else (B, T, H), device=dev) * 0.5
    beta = torch.rand(B, T, H, device=dev)
    S0 = torch.randn(B, H, Dk, Dv, device=dev) * 0.1
    S_ref, o_ref = gated_delta_scan_ref(q, k, v, g, beta, S0)
    S, o = gated_delta_scan(q, k, v, g, beta, S0)
    assert float((o.float() - o_ref.float()).abs().max()) <= 0.02 * float(o_ref.float().abs().max()) + 1e-3
    assert torch.allclose(S, S_ref, atol=2e-3, rtol=1e-3)
    # chunked through the kernel: a decode token after a prefill chunk continues the same recurrence
    Sa, oa = gated_delta_scan(q[:, :32], k[:, :32], v[:, :32], g[:, :32], beta[:, :32], S0)
    Sb, ob = gated_delta_scan(q[:, 32:], k[:, 32:], v[:, 32:], g[:, 32:], beta[:, 32:], Sa)
    assert torch.allclose(Sb, S, atol=1e-4) and torch.equal(torch.cat((oa, ob), 1), o)


def test_mamba2_reference_groups_and_chunks():
    from eredu_b200.ops.recurrent import mamba2_scan, mamba2_scan_ref

    torch.manual_seed(3)
    Bt, T, H, G, P, N = 2, 9, 4, 2, 8, 16
    x, dt = torch.randn(Bt, T, H, P), torch.rand(Bt, T, H) * 0.5 + 0.01
    Bm, Cm = torch.randn(Bt, T, G, N), torch.randn(Bt, T, G, N)
    A, D = -torch.rand(H) - 0.1, torch.randn(H)
    S, y = mamba2_scan_ref(x, Bm, Cm, dt, A, D)
    Se, ye = mamba2_scan_ref(x, Bm.repeat_interleave(2, 2), Cm.repeat_interleave(2, 2), dt, A, D)
    assert torch.equal(S, Se) and torch.equal(y, ye)                     # grouped B / C == expanded to heads
    # one step by hand for head 3 (group 1)
    s1 = x[0, 0, 3][:, None] * (dt[0, 0, 3] * Bm[0, 0, 1])[None, :]
    y1 = s1 @ Cm[0, 0, 1] + D[3] * x[0, 0, 3]
    assert torch.allclose(mamba2_scan_ref(x[:1, :1], Bm[:1, :1], Cm[:1, :1], dt[:1, :1], A, D)[1][0, 0, 3], y1, atol=1e-6)
    Sa, ya = mamba2_scan(x[:, :5], Bm[:, :5], Cm[:, :5], dt[:, :5], A, D)           # CPU tensors take the reference
    Sb, yb = mamba2_scan(x[:, 5:], Bm[:, 5:], Cm[:, 5:], dt[:, 5:], A, D, Sa)
    assert torch.allclose(Sb, S, atol=1e-6) and torch.allclose(torch.cat((ya, yb), 1), y, atol=1e-6)
    with pytest.raises(ValueError):
        mamba2_scan_ref(x, Bm[:, :, :1].expand(-1, -1, 3, -1), Cm[:, :, :1].expand(-1, -1, 3, -1), dt, A, D)


@pytest.mark.gpu
@pytest.mark.parametrize("H,G,P,N", [(8, 2, 64, 128), (4, 4, 40, 64), (4, 1, 64, 256)])
def test_mamba2_kernel_matches_reference(H, G, P, N):
    from eredu_b200.ops.recurrent import mamba2_scan, mamba2_scan_ref

    torch.manual_seed(H + P + N)
    dev = "cuda"
    Bt, T = 2, 33
    x = torch.randn(Bt, T, H, P, device=dev).bfloat16()
    Bm, Cm = (torch.randn(Bt, T, G, N, device=dev) * 0.3).bfloat16(), (torch.randn(Bt, T, G, N, device=dev) * 0.3).bfloat16()
    dt = torch.rand(Bt, T, H, device=dev) * 0.3 + 0.01
    A, D = -torch.rand(H, device=dev) - 0.1, torch.randn(H, device=dev)
    S0 = torch.randn(Bt, H, P, N, device=dev) * 0.1
    S_ref, y_ref = mamba2_scan_ref(x, Bm, Cm, dt, A, D, S0)
    S, y = mamba2_scan(x, Bm, Cm, dt, A, D, S0)
    assert float((y.float() - y_ref.float()).abs().max()) <= 0.02 * float(y_ref.float().abs().max()) + 1e-3
    assert torch.allclose(S, S_ref, atol=2e-3, rtol=1e-3)
    Sa, ya = mamba2_scan(x[:, :32], Bm[:, :32], Cm[:, :32], dt[:, :32], A, D, S0)
    Sb, yb = mamba2_scan(x[:, 32:], Bm[:, 32:], Cm[:, 32:], dt[:, 32:], A, D, Sa)
    assert torch.allclose(Sb, S, atol=1e-4) and torch.equal(torch.cat((ya, yb), 1), y)


@pytest.mark.parametrize("T,chunk,groups", [(130, 64, 2), (64, 64, 4), (37, 16, 1), (5, 8, 2)])
def test_mamba2_chunk_parallel_form_equals_the_recurrence(T, chunk, groups):
    from eredu_b200.ops.recurrent import mamba2_scan_chunked, mamba2_scan_ref

    g = torch.Generator().manual_seed(T)
    Bt, H, P, N = 2, 4, 8, 16
    x = torch.randn(Bt, T, H, P, generator=g)
    Bm, Cm = torch.randn(Bt, T, groups, N, generator=g), torch.randn(Bt, T, groups, N, generator=g)
    dt = torch.nn.functional.softplus(torch.randn(Bt, T, H, generator=g)) + 0.01
    A = -torch.rand(H, generator=g) * 2 - 0.1
    D = torch.randn(H, generator=g)
    S0 = torch.randn(Bt, H, P, N, generator=g)
    S_ref, y_ref = mamba2_scan_ref(x, Bm, Cm, dt, A, D, S0)
    S, y = mamba2_scan_chunked(x, Bm, Cm, dt, A, D, S0, chunk=chunk)
    assert torch.allclose(y, y_ref, atol=2e-4, rtol=1e-4) and torch.allclose(S, S_ref, atol=2e-4, rtol=1e-4)
    # two calls that cut the sequence anywhere give the same outputs and state as one
    cut = T // 3 + 1
    Sa, ya = mamba2_scan_chunked(x[:, :cut], Bm[:, :cut], Cm[:, :cut], dt[:, :cut], A, D, S0, chunk=chunk)
    Sb, yb = mamba2_scan_chunked(x[:, cut:], Bm[:, cut:], Cm[:, cut:], dt[:, cut:], A, D, Sa, chunk=chunk)
    assert torch.allclose(torch.cat((ya, yb), 1), y_ref, atol=2e-4, rtol=1e-4) and torch.allclose(Sb, S_ref, atol=2e-4, rtol=1e-4)


@pytest.mark.gpu
def test_mamba2_long_prefill_takes_the_chunk_parallel_form_on_the_gpu():
    from eredu_b200.ops import recurrent as R

    g = torch.Generator().manual_seed(1)
    Bt, T, H, G, P, N = 1, 2100, 8, 2, 64, 128
    x = (torch.randn(Bt, T, H, P, generator=g) * 0.5).cuda().bfloat16()
    Bm, Cm = (torch.randn(Bt, T, G, N, generator=g) * 0.3).cuda().bfloat16(), (torch.randn(Bt, T, G, N, generator=g) * 0.3).cuda().bfloat16()
    dt = (torch.nn.functional.softplus(torch.randn(Bt, T, H, generator=g)) * 0.1 + 0.001).cuda()
    A, D = (-torch.rand(H, generator=g) * 4 - 0.5).cuda(), torch.randn(H, generator=g).cuda()
    S_ref, y_ref = R.mamba2_scan_ref(x.float(), Bm.float(), Cm.float(), dt, A, D)
    assert T >= R.CHUNKED_SCAN_MIN_TOKENS
    S, y = R.mamba2_scan(x, Bm, Cm, dt, A, D)
    assert float((y.float() - y_ref).norm() / y_ref.norm()) < 2e-2
    assert float((S - S_ref).norm() / S_ref.norm()) < 2e-2
    # and agrees with the token-by-token kernel on a call short enough for it
    Sk, yk = R.mamba2_scan(x[:, :100], Bm[:, :100], Cm[:, :100], dt[:, :100], A, D)
    Sc, yc = R.mamba2_scan_chunked(x[:, :100], Bm[:, :100], Cm[:, :100], dt[:, :100], A, D)
    assert float((yk.float() - yc.float()).norm() / yc.float().norm()) < 2e-2


@pytest.mark.parametrize("T,chunk", [(130, 64), (64, 32), (37, 16), (3, 8)])
def test_gated_delta_chunk_parallel_form_equals_the_recurrence(T, chunk):
    from eredu_b200.ops.recurrent import gated_delta_scan_chunked, gated_delta_scan_ref

    g = torch.Generator().manual_seed(T + 1)
    B, H, Dk, Dv = 2, 3, 16, 24
    q = torch.randn(B, T, H, Dk, generator=g) * 0.5
    k = torch.nn.functional.normalize(torch.randn(B, T, H, Dk, generator=g), dim=-1)
    v = torch.randn(B, T, H, Dv, generator=g)
    log_decay = -torch.rand(B, T, H, generator=g) * 0.3
    beta = torch.rand(B, T, H, generator=g)
    S0 = torch.randn(B, H, Dk, Dv, generator=g) * 0.3
    S_ref, o_ref = gated_delta_scan_ref(q, k, v, log_decay, beta, S0)
    S, o = gated_delta_scan_chunked(q, k, v, log_decay, beta, S0, chunk=chunk)
    assert torch.allclose(o, o_ref, atol=3e-4, rtol=1e-4) and torch.allclose(S, S_ref, atol=3e-4, rtol=1e-4)
    cut = T // 2 + 1
    Sa, oa = gated_delta_scan_chunked(q[:, :cut], k[:, :cut], v[:, :cut], log_decay[:, :cut], beta[:, :cut], S0, chunk=chunk)
    Sb, ob = gated_delta_scan_chunked(q[:, cut:], k[:, cut:], v[:, cut:], log_decay[:, cut:], beta[:, cut:], Sa, chunk=chunk)
    assert torch.allclose(torch.cat((oa, ob), 1), o_ref, atol=3e-4, rtol=1e-4) and torch.allclose(Sb, S_ref, atol=3e-4, rtol=1e-4)
    with pytest.raises(ValueError, match="one decay per head"):
        gated_delta_scan_chunked(q, k, v, log_decay[..., None].expand(-1, -1, -1, Dk), beta)


@pytest.mark.gpu
def test_gated_delta_chunk_parallel_form_on_the_gpu():
    from eredu_b200.ops import recurrent as R

    g = torch.Generator().manual_seed(2)
    B, T, H, Dk, Dv = 2, 600, 4, 128, 128
    q = (torch.randn(B, T, H, Dk, generator=g) * 0.3).cuda().bfloat16()
    k = torch.nn.functional.normalize(torch.randn(B, T, H, Dk, generator=g), dim=-1).cuda().bfloat16()
    v = torch.randn(B, T, H, Dv, generator=g).cuda().bfloat16()
    log_decay = (-torch.rand(B, T, H, generator=g) * 0.2).cuda()
    beta = torch.rand(B, T, H, generator=g).cuda()
    S_ref, o_ref = R.gated_delta_scan_ref(q.float(), k.float(), v.float(), log_decay, beta)
    S, o = R.gated_delta_scan_chunked(q, k, v, log_decay, beta)
    assert float((o.float() - o_ref).norm() / o_ref.norm()) < 3e-2
    assert float((S - S_ref).norm() / S_ref.norm()) < 3e-2
