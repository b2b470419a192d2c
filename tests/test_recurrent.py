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
