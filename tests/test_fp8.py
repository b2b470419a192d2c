"""Block-scaled FP8 (E4M3, 128 x 128 blocks) weights: quantiser, checkpoint form, and the tcgen05 dequant-GEMM."""
import dataclasses

import pytest
import torch

from eredu_b200.ops.quant import Fp8Linear


def _fp8_state(sd):
    """Turn every 2-D projection of a dense state dict into (E4M3 weight, weight_scale_inv) like an HF FP8 export."""
    out = {}
    for name, t in sd.items():
        if name.endswith("_proj.weight") and t.shape[1] % 128 == 0:
            q = Fp8Linear.from_dense(t.float())
            N, K = t.shape
            out[name] = q.wq.view(torch.float8_e4m3fn)
            # row-expanded table [K/128, N] -> block table [ceil(N/128), K/128]
            out[name + "_scale_inv"] = q.scales_t.t()[::128].contiguous()
        else:
            out[name] = t
    return out


def test_fp8_quantiser_error_bound_and_slicing():
    torch.manual_seed(0)
    w = torch.randn(320, 512) * 0.05
    q = Fp8Linear.from_dense(w)
    deq = q.dequantize()
    # E4M3 keeps 3 mantissa bits: relative error per element at most 2^-4 of the block maximum's binade
    assert float((deq - w).abs().max()) <= float(w.abs().max()) * 2 ** -4
    assert float((deq - w).norm() / w.norm()) < 0.04
    assert q.scales_t.shape == (4, 320) and q.nbytes() == 320 * 512 + 4 * 320 * 4
    a, b = q.slice_rows(0, 200), q.slice_rows(200, 320)
    assert torch.equal(Fp8Linear.concat_rows([a, b]).dequantize(), deq)
    assert torch.equal(q.slice_cols(128, 384).dequantize(), deq[:, 128:384])
    x = torch.randn(5, 512)
    assert torch.allclose(q(x), x @ deq.t(), atol=1e-4)


def test_fp8_checkpoint_reads_as_dequantised_weights_on_cpu(tmp_path):
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import random_state

    cfg = dataclasses.replace(C.tiny_llama(), hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                              intermediate_size=384, vocab_size=512, num_hidden_layers=2)
    sd = random_state(cfg, seed=1, std=0.05)
    fp8 = _fp8_state(sd)
    ck.save_safetensors_checkpoint(tmp_path / "fp8", cfg, fp8, torch.float32)
    src = ck.open_checkpoint(tmp_path / "fp8")
    name = "model.layers.0.self_attn.q_proj.weight"
    assert src.fp8_scale_name(name) == name + "_scale_inv"
    w8, sc = src.to_fp8(name)
    assert w8.dtype == torch.uint8 and sc.shape == (2, 2)
    ref = Fp8Linear(w8, sc, "cpu").dequantize()
    assert torch.equal(src.get(name), ref)
    # the whole model loads (dense fp32 from the dequantised weights) and agrees with the same weights saved dense
    deq = {k: (src.get(k) if k in fp8 and fp8[k].dtype == torch.float8_e4m3fn else v) for k, v in sd.items()}
    ck.save_safetensors_checkpoint(tmp_path / "dense", cfg, deq, torch.float32)
    a = LoadedModel.load(tmp_path / "fp8", ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    b = LoadedModel.load(tmp_path / "dense", ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=64))
    prompt = list(range(3, 20))
    assert torch.allclose(a.prefill_logits(prompt), b.prefill_logits(prompt), atol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 7, 32, 50, 128, 300])
@pytest.mark.parametrize("N,K", [(640, 1024), (200, 512), (1284, 256)])
def test_fp8_gemm_matches_dequantised_matmul(M, N, K, monkeypatch):
    monkeypatch.setattr(Fp8Linear, "TENSOR_CORE_FP8", False)        # bf16 activations on every path of this test
    torch.manual_seed(M * 7 + N)
    w = (torch.randn(N, K, device="cuda") * 0.05)
    q = Fp8Linear.from_dense(w)
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    y = q(x, bias=bias, residual=res)
    ref = x.float() @ q.dequantize().t() + bias.float() + res.float()
    rel = float((y.float() - ref).norm() / ref.norm())
    assert rel < 1e-2, rel
    y32 = q(x, out_dtype=torch.float32)
    ref32 = x.float() @ q.dequantize().t()
    assert float((y32 - ref32).norm() / ref32.norm()) < 5e-3
    from eredu_b200.ops import native
    native.check_status(torch.device("cuda", torch.cuda.current_device()))


def _quantise_rows_ref(x):
    """1 x 128 dynamic activation quantisation in tensor operations: scale = max(|x|, 1e-4) / 448, E4M3 round to nearest."""
    M, K = x.shape
    b = x.float().view(M, K // 128, 128)
    scale = b.abs().amax(-1).clamp_min(1e-4) / 448.0
    codes = (b / scale[..., None]).to(torch.float8_e4m3fn)
    return codes.view(M, K), scale


@pytest.mark.gpu
@pytest.mark.parametrize("M", [257, 512, 1000])
@pytest.mark.parametrize("N,K", [(640, 1024), (128, 128), (1280, 3072)])
def test_fp8_tensor_core_gemm_against_the_oracles(M, N, K):
    """The FP8 tensor-core path: exact against the same quantised operands multiplied in fp32, and inside the native-FP8
    gates (rel-L2 <= 0.05, cosine >= 0.995) against the unquantised activations."""
    from eredu_b200.ops import native

    torch.manual_seed(M + N + K)
    w = torch.randn(N, K, device="cuda") * 0.05
    w[: N // 2] *= 8.0                                                  # blocks with very different scales
    q = Fp8Linear.from_dense(w)
    assert q.block_scales is not None and q.block_scales.shape == (K // 128, N // 128)
    x = (torch.randn(M, K, device="cuda") * torch.rand(M, 1, device="cuda") * 3).bfloat16()
    x[:, K // 2:] *= 0.01                                               # and columns blocks of very different magnitude
    res = torch.randn(M, N, device="cuda").bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    y = q.tensor_core(x, bias=bias, residual=res, out_dtype=torch.float32)
    codes, scale = _quantise_rows_ref(x)
    xd = (codes.float().view(M, K // 128, 128) * scale[..., None]).view(M, K)
    same = xd @ q.dequantize().t() + bias.float() + res.float()
    assert float((y - same).norm() / same.norm()) < 5e-3       # a few codes differ by one step (reciprocal-multiply against divide)
    y16 = q(x)                                                          # the dispatching call takes this path above 256 tokens
    full = x.float() @ q.dequantize().t()
    rel = float((y16.float() - full).norm() / full.norm())
    cos = float(torch.nn.functional.cosine_similarity(y16.float().flatten(), full.flatten(), dim=0))
    assert rel <= 0.05 and cos >= 0.995, (rel, cos)
    native.check_status(torch.device("cuda", torch.cuda.current_device()))


@pytest.mark.gpu
def test_fp8_activation_quantiser_matches_the_rule():
    from eredu_b200.ops import native
    from eredu_b200.ops.native import lib, ptr, stream_ptr

    torch.manual_seed(3)
    M, K = 77, 512
    big = (torch.randn(M, K + 128, device="cuda") * 2).bfloat16()
    x = big[:, :K]                                                      # a strided view: the row stride is passed
    x[5] = 0                                                            # an all-zero row takes the floor of the scale
    xq = torch.empty((M, K), dtype=torch.uint8, device="cuda")
    sx = torch.empty((K // 128, 128), dtype=torch.float32, device="cuda")
    assert lib().eredu_fp8_quant_act(ptr(x), x.stride(0), ptr(xq), ptr(sx), 128, M, K, stream_ptr(x.device)) == 0
    codes, scale = _quantise_rows_ref(x)
    assert torch.allclose(sx[:, :M].t(), scale, rtol=1e-6)
    got = xq.view(torch.float8_e4m3fn).float()
    want = codes.float()
    assert float((got != want).float().mean()) < 2e-3                   # reciprocal-multiply against divide: rare one-step ties
    assert float((got - want).abs().max()) <= 32.0
    native.check_status(torch.device("cuda", torch.cuda.current_device()))


@pytest.mark.gpu
def test_fp8_checkpoint_runs_on_native_codes(tmp_path):
    from eredu_b200.api import LoadedModel, ModelLoadOptions
    from eredu_b200.formats import checkpoint as ck
    from eredu_b200.models import config as C
    from eredu_b200.models.llama import random_state

    cfg = dataclasses.replace(C.tiny_llama(), hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
                              intermediate_size=1024, vocab_size=1024, num_hidden_layers=2, tie_word_embeddings=False)
    sd = random_state(cfg, seed=0, std=0.05)
    ck.save_safetensors_checkpoint(tmp_path / "fp8", cfg, _fp8_state(sd), torch.bfloat16)
    lm = LoadedModel.load(tmp_path / "fp8", ModelLoadOptions(device="cuda", max_batch=1, max_seq_len=128))
    l0 = lm.model.layers[0]
    assert isinstance(l0.qlin["qkv"], Fp8Linear) and isinstance(l0.qlin["down"], Fp8Linear) and l0.wqkv is None
    cpu = LoadedModel.load(tmp_path / "fp8", ModelLoadOptions(device="cpu", max_batch=1, max_seq_len=128))
    prompt = list(range(3, 40))
    a, b = lm.prefill_logits(prompt), cpu.prefill_logits(prompt)
    assert float((a - b).norm() / b.norm()) < 0.03
    # load-time FP8 of a dense checkpoint
    from eredu_b200.api.loaded import QuantizationOptions

    ck.save_safetensors_checkpoint(tmp_path / "dense", cfg, sd, torch.bfloat16)
    q = LoadedModel.load(tmp_path / "dense", ModelLoadOptions(device="cuda", max_batch=1, max_seq_len=128,
                                                              quantization=QuantizationOptions(bits=8, mode="fp8")))
    assert isinstance(q.model.layers[1].qlin["gate_up"], Fp8Linear)
    c = q.prefill_logits(prompt)
    d = LoadedModel.load(tmp_path / "dense", ModelLoadOptions(device="cuda", max_batch=1, max_seq_len=128)).prefill_logits(prompt)
    assert torch.nn.functional.cosine_similarity(c, d, dim=0) > 0.99
