"""The Python <-> C ABI of the CUDA library, checked without a GPU.

1. Every ``extern "C"`` entry point declared in the CUDA sources has a ctypes registration with the same number
   and kinds of parameters (pointer / int / float / long long), and every registration names an exported symbol.
2. The CUDA branches of the operator wrappers run on CPU tensors against a recording stub of the library
   (tensors report ``is_cuda``, launches are no-ops): argument counts and kinds of every call are checked and
   Python-level mistakes in code that otherwise only runs on a GPU surface here.
"""
import ctypes
import re
from pathlib import Path

import pytest
import torch

import eredu_b200
from eredu_b200 import ops
from eredu_b200.ops import native

CSRC = Path(eredu_b200.__file__).resolve().parent / "csrc"


def _import_all_registrations():
    import eredu_b200.ops.conv  # noqa: F401
    import eredu_b200.ops.moe  # noqa: F401
    import eredu_b200.ops.quant  # noqa: F401
    import eredu_b200.ops.recurrent  # noqa: F401
    import eredu_b200.ops.sampling  # noqa: F401
    try:
        import eredu_b200.parallel.comm  # noqa: F401
        import eredu_b200.parallel.tp  # noqa: F401
        import eredu_b200.utils.trace  # noqa: F401
    except Exception:
        pass


def _kind(ctype_decl: str) -> str:
    t = ctype_decl.strip()
    if "*" in t or "cudaStream_t" in t or "PeerComm" in t and "*" in t:
        return "P"
    base = re.sub(r"\b(const|unsigned|signed)\b", "", t).split()
    if not base:
        return "?"
    base = " ".join(base[:-1]) if len(base) > 1 else base[0]
    return {"int": "I", "float": "F", "long long": "L", "uint32_t": "I", "int64_t": "L", "size_t": "L",
            "unsigned": "I", "bool": "I", "double": "D", "uint64_t": "L", "int32_t": "I"}.get(base.strip(), "?")


def c_declarations():
    out = {}
    pat = re.compile(r'extern\s+"C"\s+([\w\s\*]+?)\s+(eredu_\w+)\s*\(([^)]*)\)\s*\{', re.S)
    for src in sorted(CSRC.rglob("*.cu")):
        text = re.sub(r"//[^\n]*", "", src.read_text())
        for ret, name, args in pat.findall(text):
            args = " ".join(args.split())
            kinds = [] if args in ("", "void") else [_kind(a) for a in args.split(",")]
            out[name] = (ret.strip(), kinds, src.name)
    return out


_CT = {ctypes.c_void_p: "P", ctypes.c_int: "I", ctypes.c_float: "F", ctypes.c_longlong: "L"}


def _reg_kind(t) -> str:
    if t in _CT:
        return _CT[t]
    if isinstance(t, type) and issubclass(t, ctypes._Pointer):
        return "P"
    return "?"


def test_registered_signatures_match_the_c_declarations():
    _import_all_registrations()
    decls = c_declarations()
    assert len(decls) > 30
    problems = []
    for name, (res, argtypes) in native._SIGNATURES.items():
        if name not in decls:
            problems.append(f"{name}: registered but not declared extern \"C\" in any CUDA source")
            continue
        _, kinds, src = decls[name]
        reg = [_reg_kind(t) for t in argtypes]
        if len(reg) != len(kinds):
            problems.append(f"{name} ({src}): {len(kinds)} C parameters, {len(reg)} registered")
        elif any(a != b for a, b in zip(reg, kinds) if "?" not in (a, b)):
            problems.append(f"{name} ({src}): C kinds {''.join(kinds)} vs registered {''.join(reg)}")
    assert not problems, "\n".join(problems)


class _StubLib:
    """Stands in for the loaded library: checks each call against its registration and launches nothing."""

    def __init__(self):
        self.calls = []

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        if name not in native._SIGNATURES:
            raise AssertionError(f"{name} is called but was never registered")
        res, argtypes = native._SIGNATURES[name]

        def call(*args):
            assert len(args) == len(argtypes), f"{name}: {len(args)} arguments for {len(argtypes)} parameters"
            for i, (a, t) in enumerate(zip(args, argtypes)):
                k = _reg_kind(t)
                if k == "P":
                    assert a is None or isinstance(a, int) or hasattr(a, "_obj") or isinstance(a, ctypes._Pointer), \
                        f"{name} argument {i}: {type(a).__name__} given for a pointer"
                elif k in ("I", "L"):
                    assert isinstance(a, int) and not isinstance(a, float), f"{name} argument {i}: {a!r} given for an integer"
                elif k == "F":
                    assert isinstance(a, (int, float)), f"{name} argument {i}: {a!r} given for a float"
            self.calls.append(name)
            if name == "eredu_sampler_row_bytes":
                return 64
            if name == "eredu_gemm_pick_split":
                return 1
            return 0 if res is not None else None

        return call


@pytest.fixture
def dry_cuda(monkeypatch):
    """CPU tensors claim to be CUDA tensors and the library is a stub: the wrappers' GPU branches execute."""
    _import_all_registrations()
    stub = _StubLib()
    status = torch.zeros(1, dtype=torch.int32)
    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True), raising=False)
    import eredu_b200.ops.conv as conv_mod
    import eredu_b200.ops.core as core_mod
    import eredu_b200.ops.moe as moe_mod
    import eredu_b200.ops.quant as quant_mod
    import eredu_b200.ops.recurrent as rec_mod
    import eredu_b200.ops.sampling as samp_mod

    for mod in (native, conv_mod, core_mod, moe_mod, quant_mod, rec_mod, samp_mod):
        for attr, val in (("lib", lambda: stub), ("stream_ptr", lambda device=None: 0),
                          ("status_word", lambda device=None: status), ("_sm_count", lambda device=None: 148),
                          ("check_status", lambda device=None: None)):
            if hasattr(mod, attr):
                monkeypatch.setattr(mod, attr, val)
    return stub


def test_dense_and_quantised_wrappers_dry_run(dry_cuda):
    from eredu_b200.ops.quant import Fp8Linear, QuantLinear

    bf = torch.bfloat16
    x = torch.randn(8, 256).to(bf)
    w = torch.randn(384, 256).to(bf)
    ops.linear(x, w, bias=torch.zeros(384, dtype=bf), residual=torch.zeros(8, 384, dtype=bf))
    ops.linear(x, w, out_dtype=torch.float32)
    ops.gated_linear(x, w, 192)
    ops.silu_mul(torch.randn(8, 384).to(bf), 192, 7.0)
    ops.rmsnorm(x, torch.ones(256), 1e-5)
    assert {"eredu_gemm_bf16", "eredu_silu_mul", "eredu_rmsnorm"} <= set(dry_cuda.calls)
    for bits, group in ((4, 64), (8, 32)):
        q = QuantLinear.from_dense(w.float(), bits, group)
        q(x, bias=torch.zeros(384, dtype=bf), residual=torch.zeros(8, 384, dtype=bf))
        q(torch.randn(300, 256).to(bf))                      # whole-matrix dequant + dense GEMM
    f8 = Fp8Linear.from_dense(w.float())
    f8(x, residual=torch.zeros(8, 384, dtype=bf))
    f8(torch.randn(300, 256).to(bf), out_dtype=torch.float32)        # 256 < tokens <= 1024: the FP8 tensor-core kernel
    f8(torch.randn(1100, 256).to(bf))                                # beyond: decode the weight once, bf16 GEMM
    assert {"eredu_qgemm", "eredu_dequant_affine", "eredu_qgemm_fp8", "eredu_dequant_fp8", "eredu_fp8_quant_act",
            "eredu_gemm_fp8_tc"} <= set(dry_cuda.calls)


def test_moe_and_conv_wrappers_dry_run(dry_cuda):
    from eredu_b200.ops import moe as M

    bf = torch.bfloat16
    T, H, E, I_, k = 6, 128, 8, 64, 2
    x = torch.randn(T, H).to(bf)
    logits = torch.randn(T, E)
    gu = torch.randn(E, 2 * I_, H).to(bf)
    dn = torch.randn(E, H, I_).to(bf)
    ids, w = M.route(logits, k, "softmax", True, 1.0, None)
    M.experts_forward(x, ids, w, gu, dn, 0, residual=x)
    M.experts_forward(x, ids, w, gu, dn, 0, gu_bias=torch.zeros(E, 2 * I_, dtype=bf), down_bias=torch.zeros(E, H, dtype=bf),
                      act="oss_glu", limit=7.0)
    ids2, w2, plan, xp = M.route_plan_gather(logits, x, k, "sigmoid", True, 1.5, torch.zeros(E), 0, E)
    M.experts_forward(x, ids2, w2, gu, dn, 0, plan=plan, xp=xp)
    assert {"eredu_moe_route", "eredu_moe_plan", "eredu_moe_gather", "eredu_gemm_bf16_grouped", "eredu_moe_combine",
            "eredu_moe_route_plan_gather"} <= set(dry_cuda.calls)
    C_, L = 64, 3
    ops.short_conv(torch.randn(5, 3 * C_).to(bf), torch.randn(C_, L), None, torch.zeros(4, L - 1, C_, dtype=bf),
                   torch.zeros(1, 2, dtype=torch.int32), torch.tensor([0, 5], dtype=torch.int32), 1,
                   torch.arange(5, dtype=torch.int32), torch.zeros(5, dtype=torch.int64), max_q_len=5)
    assert "eredu_short_conv" in dry_cuda.calls


def test_moe_block_and_expert_cache_dry_run(dry_cuda):
    import dataclasses

    from eredu_b200.models import config as C
    from eredu_b200.models.moe import MoEBlock
    from eredu_b200.runtime.expert_cache import ExpertCache

    bf = torch.bfloat16
    cfg = dataclasses.replace(C.tiny_llama(), model_type="qwen3_moe", num_experts=8, num_experts_per_tok=2,
                              moe_intermediate_size=64, hidden_size=128)
    H, E, I_ = 128, 8, 64
    blk = MoEBlock(cfg, torch.randn(E, H).to(bf), torch.randn(E, 2 * I_, H).to(bf), torch.randn(E, H, I_).to(bf), 0, E)
    for T in (4, 100):                       # decode-sized (fused route + plan + gather) and prefill-sized steps
        x = torch.randn(T, H).to(bf)
        y = blk(x, residual=x)
        assert y.shape == (T, H)
    oss = MoEBlock(cfg, torch.randn(E, H).to(bf), torch.randn(E, 2 * I_, H).to(bf), torch.randn(E, H, I_).to(bf), 0, E,
                   router_linear_bias=torch.zeros(E, dtype=bf), gu_bias=torch.zeros(E, 2 * I_, dtype=bf),
                   down_bias=torch.zeros(E, H, dtype=bf), act="oss_glu")
    oss(torch.randn(4, H).to(bf), residual=torch.randn(4, H).to(bf))
    # expert cache: the ids the stub leaves behind are arbitrary, the bookkeeping must cope with any of them
    blk.expert_cache = ExpertCache(blk.w_gate_up, blk.w_down, 3, "lru", 0)
    x = torch.randn(4, H).to(bf)
    assert blk(x, residual=x).shape == (4, H)


@pytest.mark.parametrize("family", ["llama", "qwen3_moe", "gpt_oss", "lfm2", "qwen3_next", "nemotron_h", "deepseek_v3", "kimi_linear"])
def test_whole_model_forward_dry_run(dry_cuda, family):
    """Prefill and decode passes of every family through the CUDA branches of the operator wrappers (stub library,
    CPU tensors): argument kinds, shapes the wrappers assert on, and the Python glue between kernels."""
    import dataclasses
    import sys

    from eredu_b200.models import config as C
    from eredu_b200.models.llama import build_from_tensors, random_state
    from eredu_b200.models.moe import make_moe_factory
    from eredu_b200.runtime.engine import Engine

    sys.path.insert(0, str(Path(__file__).parent))
    bf = torch.bfloat16
    kw = {}
    if family == "llama":
        cfg = dataclasses.replace(C.tiny_llama(), hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                                  intermediate_size=512, vocab_size=512, num_hidden_layers=2)
        sd = random_state(cfg, seed=0)
    elif family == "qwen3_moe":
        cfg = dataclasses.replace(C.tiny_llama(), model_type="qwen3_moe", qk_norm=True, hidden_size=256, num_attention_heads=4,
                                  num_key_value_heads=2, head_dim=64, vocab_size=512, num_hidden_layers=2, num_experts=8,
                                  num_experts_per_tok=2, moe_intermediate_size=64, tie_word_embeddings=False)
        sd = random_state(cfg, seed=0)
        kw["moe_factory"] = make_moe_factory()
    elif family == "gpt_oss":
        from test_gpt_oss import oss_cfg, oss_state

        cfg = oss_cfg()
        sd = oss_state(cfg)
        kw["moe_factory"] = make_moe_factory()
    elif family == "lfm2":
        from test_lfm2 import lfm2_cfg

        cfg = lfm2_cfg(hidden_size=256, intermediate_size=512, num_attention_heads=4, num_key_value_heads=2, vocab_size=512)
        sd = random_state(cfg, seed=0)
    elif family == "deepseek_v3":
        from test_deepseek import ds_cfg, state_for as ds_state

        cfg = ds_cfg(hidden_size=256, vocab_size=512, kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                     q_lora_rank=64)
        sd = ds_state(cfg)
        kw["moe_factory"] = make_moe_factory()
    elif family == "kimi_linear":
        from test_kimi_linear import kimi_cfg, state_for as kimi_state

        cfg = kimi_cfg(hidden_size=256, vocab_size=512, kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                       linear_attn_config={"kda_layers": [1, 2, 3], "full_attn_layers": [4], "num_heads": 4, "head_dim": 64,
                                           "short_conv_kernel_size": 4})
        sd = kimi_state(cfg)
        kw["moe_factory"] = make_moe_factory()
    elif family == "nemotron_h":
        from test_nemotron_h import nh_cfg, state_for as nh_state

        cfg = nh_cfg(hidden_size=256, head_dim=64, vocab_size=512, intermediate_size=256, ssm_state_size=64)
        sd = nh_state(cfg)
        kw["moe_factory"] = make_moe_factory()
    else:
        from test_qwen_next import next_cfg, state_for

        cfg = next_cfg(hidden_size=256, head_dim=64, linear_key_head_dim=64, linear_value_head_dim=64, vocab_size=512)
        sd = state_for(cfg)
        kw["moe_factory"] = make_moe_factory()
    model = build_from_tensors(cfg, lambda n: sd[n], sd.__contains__, "cpu", bf, **kw)
    eng = Engine(model, max_batch=2, max_seq_len=64)
    seqs = [eng.new_sequence(list(range(3, 3 + n)), max_new_tokens=4) for n in (5, 9)]
    dry_cuda.calls.clear()
    logits = eng.prefill_logits(seqs)
    assert len(logits) == 2 and logits[0].shape[-1] == cfg.vocab_size
    for sq in seqs:
        eng.release(sq)
    from eredu_b200.ops import SamplingParams

    outs = eng.generate([list(range(3, 9)), list(range(4, 15))], SamplingParams(temperature=0.0), 3)   # decode-shaped passes
    assert [len(o) for o in outs] == [3, 3]
    calls = set(dry_cuda.calls)
    assert {"eredu_gemm_bf16", "eredu_rmsnorm"} <= calls
    if family not in ("deepseek_v3", "kimi_linear"):     # latent attention has no kernel: tensor operations around the GEMMs
        assert "eredu_rope_kv" in calls
        assert calls & {"eredu_attn_prefill", "eredu_attn_prefill_tc"}     # the second is the tcgen05 kernel (16-token pages)
        assert calls & {"eredu_attn_decode", "eredu_attn_decode_rope"}      # the second fuses the rotation into the decode kernel
    if family in ("qwen3_moe", "gpt_oss", "qwen3_next", "nemotron_h", "deepseek_v3", "kimi_linear"):
        assert "eredu_gemm_bf16_grouped" in calls
    if family in ("lfm2", "nemotron_h"):
        assert "eredu_short_conv" in calls
    if family == "nemotron_h":
        assert "eredu_mamba2_scan" in calls
    if family in ("qwen3_next", "kimi_linear"):
        assert {"eredu_short_conv", "eredu_gated_delta_scan"} <= calls
