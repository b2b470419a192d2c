"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

from eredu_b200 import ops
from eredu_b200.ops import native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_l2(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def check_status():
    native.check_status(torch.device("cuda", torch.cuda.current_device()))


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (1, 4096, 4096), (7, 384, 512), (16, 6144, 4096), (32, 4096, 14336),
                                   (33, 1024, 1024), (64, 512, 192), (100, 640, 320), (128, 256, 256),
                                   (300, 1152, 1024), (2048, 1024, 512)])
def test_gemm(M, N, K):
    torch.manual_seed(M * 7 + N)
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    y = ops.linear(x, w)
    ref = ops.linear_ref(x, w, out_dtype=torch.float32)
    check_status()
    assert rel_l2(y, ref) < 1e-2


@pytest.mark.parametrize("split", [1, 2, 4, 8])
@pytest.mark.parametrize("M", [1, 5, 32, 48])
def test_gemm_split_k_cluster(M, split):
    torch.manual_seed(split)
    K, N = 2048, 640
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    r = torch.randn(M, N, device=DEV).bfloat16()
    b = torch.randn(N, device=DEV).bfloat16()
    y = ops.linear(x, w, bias=b, residual=r, force_split=split)
    ref = ops.linear_ref(x, w, bias=b, residual=r, out_dtype=torch.float32)
    check_status()
    assert rel_l2(y, ref) < 1e-2
    # bitwise determinism of the cluster reduction
    y2 = ops.linear(x, w, bias=b, residual=r, force_split=split)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("M", [1, 16, 40, 130, 700])
def test_gemm_fp32_out_and_strided(M):
    K, N = 512, 1000  # N not a multiple of 128
    big = (torch.randn(M, K + 64, device=DEV) * 0.5).bfloat16()
    x = big[:, 32:32 + K]  # row stride K+64, 64-byte offset (16-byte aligned)
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    y = ops.linear(x, w, out_dtype=torch.float32)
    ref = ops.linear_ref(x, w, out_dtype=torch.float32)
    check_status()
    assert y.dtype == torch.float32 and rel_l2(y, ref) < 1e-2


@pytest.mark.parametrize("M,N,K", [(100, 1024, 512), (129, 1000, 320), (300, 1096, 1024), (777, 4096, 512), (1500, 640, 2048),
                                   (4100, 2048, 1088)])
def test_gemm_fused_epilogue_large_m(M, N, K):
    """Prefill-sized GEMMs (staged / persistent kernels): RMSNorm row scale in, bias, residual, sums of squares out."""
    torch.manual_seed(M + N)
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    b = torch.randn(N, device=DEV).bfloat16()
    r = torch.randn(M, N, device=DEV).bfloat16()
    parts = 3
    ssq = (x.float().pow(2).sum(-1, keepdim=True) / parts).repeat(1, parts).contiguous()
    y, ssq_out = ops.linear(x, w, bias=b, residual=r, row_ssq=ssq, norm_eps=1e-5, want_ssq=True)
    check_status()
    scale = torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)
    ref = (x.float() @ w.float().t()) * scale + b.float() + r.float()
    assert rel_l2(y, ref) < 1e-2
    want = y.float().pow(2).sum(-1)
    assert torch.allclose(ssq_out.sum(-1), want, rtol=2e-3, atol=1e-3)
    y2 = ops.linear(x, w)  # plain path, same kernels
    assert rel_l2(y2, x.float() @ w.float().t()) < 1e-2
    check_status()


@pytest.mark.parametrize("M,K,I", [(300, 1024, 1408), (1000, 512, 832), (2300, 2048, 1472)])
def test_gated_gemm_large_m(M, K, I):
    torch.manual_seed(M)
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV) * 0.05).bfloat16()
    b = (torch.randn(2 * I, device=DEV) * 0.1).bfloat16()
    ssq = x.float().pow(2).sum(-1, keepdim=True).contiguous()
    y = ops.gated_linear(x, w, I, bias=b, row_ssq=ssq, norm_eps=1e-6)
    check_status()
    xs = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    z = xs @ w.float().t() + b.float()
    ref = torch.nn.functional.silu(z[:, :I]) * z[:, I:]
    assert rel_l2(y, ref) < 1.5e-2


@pytest.mark.parametrize("M,split", [(1, 0), (8, 1), (8, 2), (32, 4), (64, 0), (100, 0), (300, 0)])
def test_gated_gemm(M, split):
    K, I = 1024, 1408
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV) * 0.05).bfloat16()
    y = ops.gated_linear(x, w, I, force_split=split)
    ref = ops.gated_linear_ref(x, w, I, out_dtype=torch.float32)
    check_status()
    assert rel_l2(y, ref) < 1.5e-2


@pytest.mark.parametrize("M,H", [(1, 256), (3, 2048), (17, 4096), (5, 8192)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(M, H, with_res):
    x = torch.randn(M, H, device=DEV).bfloat16()
    r = torch.randn(M, H, device=DEV).bfloat16() if with_res else None
    w = torch.rand(H, device=DEV) + 0.5
    y, h = ops.rmsnorm(x, w, 1e-5, residual=r)
    yr, hr = ops.rmsnorm_ref(x, w, 1e-5, residual=r)
    assert rel_l2(y, yr) < 5e-3
    if with_res:
        assert torch.equal(h, hr)


def _mk_cache(n_pages, n_kv, D):
    k = torch.zeros(n_pages, n_kv, 16, D, device=DEV, dtype=torch.bfloat16)
    return k, torch.zeros_like(k)


@pytest.mark.parametrize("D,interleaved,qknorm,rot", [(128, False, False, None), (64, True, False, None),
                                                      (128, False, True, None), (128, False, False, 64)])
def test_rope_kv(D, interleaved, qknorm, rot):
    M, n_q, n_kv = 37, 8, 2
    qkv = torch.randn(M, (n_q + 2 * n_kv) * D, device=DEV).bfloat16()
    pos = torch.randint(0, 5000, (M,), device=DEV, dtype=torch.int32)
    perm = torch.randperm(20 * 16, device=DEV)[:M].long() + 16
    perm[3] = -1
    inv = (1.0 / (10000.0 ** (torch.arange(0, rot or D, 2, device=DEV).float() / (rot or D))))
    qn = (torch.rand(D, device=DEV) + 0.5) if qknorm else None
    kn = (torch.rand(D, device=DEV) + 0.5) if qknorm else None
    kc, vc = _mk_cache(24, n_kv, D)
    kr, vr = _mk_cache(24, n_kv, D)
    q = ops.rope_kv(qkv, pos, perm, inv, kc, vc, n_q, n_kv, D, rot=rot, interleaved=interleaved, q_norm_w=qn,
                    k_norm_w=kn)
    qr = ops.rope_kv_ref(qkv, pos, perm, inv, kr, vr, n_q, n_kv, D, rot=rot, interleaved=interleaved, q_norm_w=qn,
                         k_norm_w=kn)
    assert rel_l2(q, qr) < 1e-2
    assert rel_l2(kc, kr) < 1e-2
    assert torch.equal(vc, vr)


def _paged_setup(B, kv_lens, n_kv, D, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    max_pages = max((l + 15) // 16 for l in kv_lens) + 1
    n_pages = B * max_pages + 1
    kc = (torch.randn(n_pages, n_kv, 16, D, device=DEV, generator=g)).bfloat16()
    vc = (torch.randn(n_pages, n_kv, 16, D, device=DEV, generator=g)).bfloat16()
    ids = torch.randperm(n_pages - 1, device=DEV, generator=g)[: B * max_pages].int() + 1
    bt = ids.view(B, max_pages).contiguous()
    return kc, vc, bt


@pytest.mark.parametrize("D,n_q,n_kv", [(128, 8, 2), (64, 4, 2), (128, 4, 4)])
@pytest.mark.parametrize("window", [0, 100])
def test_attention_prefill(D, n_q, n_kv, window):
    q_lens = [200, 64, 1, 77]
    kv_lens = [200, 300, 50, 77]
    B = len(q_lens)
    kc, vc, bt = _paged_setup(B, kv_lens, n_kv, D)
    total = sum(q_lens)
    q = torch.randn(total, n_q, D, device=DEV).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device=DEV, dtype=torch.int32)
    sl = torch.tensor(kv_lens, device=DEV, dtype=torch.int32)
    scale = 1 / math.sqrt(D)
    out = ops.attention_prefill(q, kc, vc, bt, sl, cu, max(q_lens), scale, window=window)
    ref = ops.attention_ref(q, kc, vc, bt, sl, q_lens, scale, window=window)
    assert rel_l2(out, ref) < 1.5e-2


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("window,with_sinks", [(0, True), (100, False), (128, True), (700, False), (1, False)])
def test_attention_prefill_on_tcgen05_with_windows_sinks_and_head_size_64(D, window, with_sinks):
    """The same kernel with a sliding window (key tiles before the window are skipped, windows that start inside a tile
    are masked), sink logits in the normaliser, and head size 64."""
    from eredu_b200.ops import core, native

    q_lens, kv_lens = [300, 129, 5, 700], [900, 129, 260, 700]
    n_q, n_kv = 8, 2
    kc, vc, bt = _paged_setup(len(q_lens), kv_lens, n_kv, D, seed=5)
    q = torch.randn(sum(q_lens), n_q, D, device=DEV).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device=DEV, dtype=torch.int32)
    sl = torch.tensor(kv_lens, device=DEV, dtype=torch.int32)
    sinks = torch.randn(n_q, device=DEV) if with_sinks else None
    scale = 1 / math.sqrt(D)
    before = native.launch_count()
    assert core.TC_PREFILL
    out = ops.attention_prefill(q, kc, vc, bt, sl, cu, max(q_lens), scale, window=window, sinks=sinks)
    assert native.launch_count() == before + 1
    native.check_status(torch.device(DEV))
    ref = ops.attention_ref(q, kc, vc, bt, sl, q_lens, scale, window=window, sinks=sinks)
    assert rel_l2(out, ref) < 1.5e-2


@pytest.mark.parametrize("q_lens,kv_lens", [([200, 64, 1, 77], [200, 300, 50, 77]), ([2048], [2048]), ([129, 128, 127], [1000, 128, 513]),
                                            ([300], [4396])])
@pytest.mark.parametrize("n_q,n_kv", [(8, 2), (4, 4)])
def test_attention_prefill_on_tcgen05_matches_reference_and_the_mma_kernel(q_lens, kv_lens, n_q, n_kv, monkeypatch):
    """The tensor-memory kernel (head size 128, causal, cached prefixes, ragged batches, key tiles that end inside a page
    table) against the fp32 reference, and against the mma.sync kernel it replaced as a second opinion."""
    from eredu_b200.ops import core, native

    D = 128
    B = len(q_lens)
    kc, vc, bt = _paged_setup(B, kv_lens, n_kv, D, seed=3)
    q = torch.randn(sum(q_lens), n_q, D, device=DEV).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device=DEV, dtype=torch.int32)
    sl = torch.tensor(kv_lens, device=DEV, dtype=torch.int32)
    scale = 1 / math.sqrt(D)
    before = native.launch_count()
    assert core.TC_PREFILL
    out = ops.attention_prefill(q, kc, vc, bt, sl, cu, max(q_lens), scale)
    assert native.launch_count() == before + 1
    native.check_status(torch.device(DEV))
    ref = ops.attention_ref(q, kc, vc, bt, sl, q_lens, scale)
    assert rel_l2(out, ref) < 1.5e-2
    monkeypatch.setattr(core, "TC_PREFILL", False)
    old = ops.attention_prefill(q, kc, vc, bt, sl, cu, max(q_lens), scale)
    assert rel_l2(out, old) < 1.5e-2


@pytest.mark.parametrize("D,n_q,n_kv,qps", [(128, 32, 8, 1), (128, 32, 8, 5), (64, 4, 2, 1), (128, 64, 8, 1),
                                            (128, 64, 8, 3), (128, 4, 4, 2)])
@pytest.mark.parametrize("splits", [1, 3, 8])
def test_attention_decode(D, n_q, n_kv, qps, splits):
    kv_lens = [517, 33, 2048, 16, 5]
    B = len(kv_lens)
    kc, vc, bt = _paged_setup(B, kv_lens, n_kv, D, seed=1)
    q = torch.randn(B * qps, n_q, D, device=DEV).bfloat16()
    sl = torch.tensor(kv_lens, device=DEV, dtype=torch.int32)
    scale = 1 / math.sqrt(D)
    out = ops.attention_decode(q, kc, vc, bt, sl, qps, scale, splits=splits)
    ref = ops.attention_ref(q, kc, vc, bt, sl, [qps] * B, scale)
    assert rel_l2(out, ref) < 1.5e-2


def test_attention_sinks():
    D, n_q, n_kv = 64, 4, 2
    kv_lens = [100, 40]
    kc, vc, bt = _paged_setup(2, kv_lens, n_kv, D, seed=2)
    sinks = torch.randn(n_q, device=DEV)
    sl = torch.tensor(kv_lens, device=DEV, dtype=torch.int32)
    q = torch.randn(2, n_q, D, device=DEV).bfloat16()
    out = ops.attention_decode(q, kc, vc, bt, sl, 1, 0.125, splits=2, sinks=sinks)
    ref = ops.attention_ref(q, kc, vc, bt, sl, [1, 1], 0.125, sinks=sinks)
    assert rel_l2(out, ref) < 1.5e-2
    qp = torch.randn(140, n_q, D, device=DEV).bfloat16()
    cu = torch.tensor([0, 100, 140], device=DEV, dtype=torch.int32)
    outp = ops.attention_prefill(qp, kc, vc, bt, sl, cu, 100, 0.125, sinks=sinks)
    refp = ops.attention_ref(qp, kc, vc, bt, sl, [100, 40], 0.125, sinks=sinks)
    assert rel_l2(outp, refp) < 1.5e-2


def test_embedding_and_silu():
    table = torch.randn(1000, 256, device=DEV).bfloat16()
    ids = torch.tensor([0, 5, 999, 400, 1200], device=DEV, dtype=torch.int32)
    out = ops.embedding(ids, table[400:800].contiguous(), vocab_start=400)
    assert torch.equal(out[3], table[400]) and out[0].abs().sum() == 0 and out[4].abs().sum() == 0
    x = torch.randn(9, 512, device=DEV).bfloat16()
    y = ops.silu_mul(x, 256)
    ref = torch.nn.functional.silu(x[:, :256].float()) * x[:, 256:].float()
    assert rel_l2(y, ref) < 1e-2


SP = ops.SamplingParams


@pytest.mark.parametrize("sp", [SP(temperature=0.0), SP(temperature=0.8, top_k=40, top_p=0.95, min_p=0.05, seed=7),
                                SP(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, seed=3),
                                SP(temperature=0.7, top_k=0, top_p=1.0, min_p=0.1, seed=4),
                                SP(temperature=1.3, top_k=5, top_p=1.0, min_p=0.0, seed=5),
                                SP(temperature=0.9, top_k=0, top_p=0.9, min_p=0.0, seed=6),
                                SP(temperature=0.8, top_k=50, top_p=0.9, min_p=0.02, repeat_penalty=1.3,
                                   frequency_penalty=0.2, presence_penalty=0.1, seed=8)])
def test_sampler_matches_reference_chain(sp):
    V, R = 32000, 6
    torch.manual_seed(11)
    logits = torch.randn(R, V, device=DEV) * 3.0
    history = torch.randint(0, V, (R, 64), device=DEV, dtype=torch.int32)
    hist_lens = [0, 3, 64, 10, 64, 1]
    rows = ops.pack_rows([sp] * R, positions=list(range(100, 100 + R)), hist_lens=hist_lens,
                         stream_ids=list(range(R)))
    probs = torch.empty(R, V, device=DEV)
    work = logits.clone()
    toks = ops.sample(work, ops.rows_to_tensor(rows, DEV), history=history, probs=probs)
    for r in range(R):
        tok_ref, p_ref = ops.sample_ref(logits[r].cpu(), sp, 100 + r, history=history[r, :hist_lens[r]].tolist(),
                                        stream=r)
        p = probs[r].cpu()
        assert abs(float(p.sum()) - 1.0) < 1e-3
        assert float((p - p_ref).abs().max()) < 2e-3, f"row {r}"
        if sp.temperature == 0.0:
            assert int(toks[r]) == tok_ref
        else:
            assert p_ref[int(toks[r])] > 0


def test_sampler_distribution_and_determinism():
    V = 1000
    logits = torch.log_softmax(torch.randn(V, device=DEV) * 2, 0)
    sp = SP(temperature=1.0, top_k=8, top_p=1.0, min_p=0.0, seed=1)
    R = 4000
    rows = ops.pack_rows([sp] * R, positions=list(range(R)))
    rows_t = ops.rows_to_tensor(rows, DEV)
    a = ops.sample(logits.repeat(R, 1).contiguous(), rows_t)
    b = ops.sample(logits.repeat(R, 1).contiguous(), rows_t)
    assert torch.equal(a, b)
    p_ref = ops.process_logits_ref(logits.cpu(), sp)
    counts = torch.bincount(a.cpu().long(), minlength=V).float() / R
    assert float((counts - p_ref).abs().max()) < 0.04


def test_token_filter_mask():
    V = 5000
    logits = torch.randn(2, V, device=DEV)
    allowed = torch.zeros(V, dtype=torch.bool, device=DEV)
    allowed[[17, 4000, 4999]] = True
    mask = ops.pack_allow_mask(allowed[None])
    rows = ops.pack_rows([SP(temperature=0.0), SP(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0)], [0, 1])
    toks = ops.sample(logits.clone(), ops.rows_to_tensor(rows, DEV), allow=mask)
    assert int(toks[0]) in (17, 4000, 4999) and int(toks[1]) in (17, 4000, 4999)
    assert int(toks[0]) == [17, 4000, 4999][int(torch.argmax(logits[0, [17, 4000, 4999]]))]


@pytest.mark.parametrize("temp", [0.0, 0.8])
def test_spec_verify(temp):
    V, B, k = 2000, 5, 4
    torch.manual_seed(3)
    sp = SP(temperature=temp, top_k=20, top_p=0.95, min_p=0.0, seed=9)
    lt = torch.randn(B * (k + 1), V, device=DEV) * 2
    ld = lt[: B * k].clone() + torch.randn(B * k, V, device=DEV) * 0.7
    rows_t = ops.rows_to_tensor(ops.pack_rows([sp] * (B * (k + 1)), list(range(B * (k + 1)))), DEV)
    p_t = torch.empty(B * (k + 1), V, device=DEV)
    p_d = torch.empty(B * k, V, device=DEV)
    ops.sample(lt.clone(), rows_t, probs=p_t)
    drafted = ops.sample(ld.clone(), rows_t[: B * k].contiguous(), probs=p_d)
    p_t = p_t.view(B, k + 1, V)
    p_d3 = torch.empty(B, k, V, device=DEV)
    dr = torch.empty(B, k, device=DEV, dtype=torch.int32)
    for b in range(B):  # rows were laid out position-major above; regroup per sequence
        p_d3[b] = p_d[b * k:(b + 1) * k]
        dr[b] = drafted[b * k:(b + 1) * k]
    p_t3 = torch.stack([lt.new_empty(0)] * 0) if False else p_t
    seq_rows = ops.pack_rows([sp] * B, positions=[50 + 10 * b for b in range(B)], stream_ids=list(range(B)))
    out = ops.spec_verify(p_t3.contiguous(), p_d3.contiguous(), dr.contiguous(), ops.rows_to_tensor(seq_rows, DEV))
    for b in range(B):
        acc, nxt = ops.verify_ref(p_t3[b].cpu(), p_d3[b].cpu(), dr[b].tolist(), sp.seed, b, 50 + 10 * b)
        assert int(out[b, 0]) == acc
        if temp == 0.0:
            assert int(out[b, 1]) == nxt
        else:
            resid_ok = p_t3[b, acc].cpu()[int(out[b, 1])] > 0
            assert resid_ok


@pytest.mark.parametrize("D,n_q,n_kv,qps,qknorm,interleaved,rot,splits", [
    (128, 32, 8, 1, False, False, None, 1), (128, 32, 8, 1, False, False, None, 5), (128, 4, 1, 1, False, False, None, 4),
    (128, 32, 8, 5, True, False, None, 3), (64, 4, 2, 1, True, True, None, 2), (128, 8, 2, 3, False, False, 64, 2),
    (128, 64, 8, 3, False, False, None, 2), (128, 64, 8, 5, False, False, None, 4), (128, 32, 8, 1, False, False, None, 12),
    (128, 32, 8, 4, True, False, None, 8)])
def test_decode_attention_with_fused_rope_and_append(D, n_q, n_kv, qps, qknorm, interleaved, rot, splits):
    """The decode kernel that takes the qkv projection output (q/k norm, RoPE and the KV append inside the kernel)
    against the separate RoPE + append kernel followed by fp32 reference attention; the caches must end up equal."""
    torch.manual_seed(D + n_q + qps + splits)
    kv_lens = [517, 33, 2050, 16, 5, 700][: 6 if qps == 1 else 5]
    kv_lens = [max(l, qps) for l in kv_lens]
    B = len(kv_lens)
    max_pages = max((l + 15) // 16 for l in kv_lens) + 1
    n_pages = B * max_pages + 1
    kc = torch.randn(n_pages, n_kv, 16, D, device=DEV).bfloat16()
    vc = torch.randn(n_pages, n_kv, 16, D, device=DEV).bfloat16()
    bt = (torch.randperm(n_pages - 1, device=DEV)[: B * max_pages].int() + 1).view(B, max_pages).contiguous()
    sl = torch.tensor(kv_lens, device=DEV, dtype=torch.int32)
    width = (n_q + 2 * n_kv) * D
    qkv = torch.randn(B * qps, width + 64, device=DEV).bfloat16()[:, :width]       # row stride != width
    pos = torch.cat([torch.arange(l - qps, l) for l in kv_lens]).to(DEV, torch.int32)
    slots = torch.cat([bt[b, (torch.arange(l - qps, l) // 16).to(DEV)].long() * 16 + (torch.arange(l - qps, l) % 16).to(DEV)
                       for b, l in enumerate(kv_lens)])
    if B > 2 and qps == 1:
        slots[2] = -1       # an inactive row: nothing is stored for it
    inv = (1.0 / (10000.0 ** (torch.arange(0, (rot or D) // 2, device=DEV).float() / ((rot or D) // 2)))).contiguous()
    qw = (torch.rand(D, device=DEV) + 0.5) if qknorm else None
    kw = (torch.rand(D, device=DEV) + 0.5) if qknorm else None
    scale = 1 / math.sqrt(D)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    q_ref = ops.rope_kv(qkv, pos, slots, inv, kc_ref, vc_ref, n_q, n_kv, D, rot=rot, interleaved=interleaved,
                        attn_factor=1.1, q_norm_w=qw, k_norm_w=kw, norm_eps=1e-6)
    want = ops.attention_ref(q_ref, kc_ref, vc_ref, bt, sl, [qps] * B, scale)
    got = ops.attention_decode_rope(qkv, kc, vc, bt, sl, qps, scale, pos, slots, inv, n_q, n_kv, D, rot=rot,
                                    interleaved=interleaved, attn_factor=1.1, q_norm_w=qw, k_norm_w=kw, norm_eps=1e-6,
                                    splits=splits)
    torch.cuda.synchronize()
    # same arithmetic in two kernels: at most a last-place bf16 difference where the compiler contracted differently
    assert torch.equal(vc, vc_ref) and torch.allclose(kc.float(), kc_ref.float(), atol=0.04, rtol=0.01)
    keep = (slots >= 0).view(B, qps).all(1).repeat_interleave(qps)
    rel = float((got[keep].float() - want[keep].float()).norm() / want[keep].float().norm())
    assert rel < 1.5e-2, rel
