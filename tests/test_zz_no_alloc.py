"""The allocation-free decode-attention entry point, called through its exported C symbol.

It serves embedders that must not allocate device memory after start-up (fixed-budget serving loops, plug-ins that
only receive raw pointers): the split-KV scratch lives in a fixed array inside the library. The file name sorts
after every other test file, so a failure here cannot hide another test's result under ``-x``; the test also passes
when run alone in a fresh process."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, q, kc, vc, out, bt, sl, B, qps, n_q, n_kv, D, splits, scale):
    fn = lib.eredu_attn_decode_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 8 + [ctypes.c_float, ctypes.c_void_p]
    return fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), bt.data_ptr(), sl.data_ptr(), None, B, qps,
              bt.stride(0), n_q, n_kv, D, splits, 0, scale, torch.cuda.current_stream().cuda_stream)


def test_static_scratch_entry_matches_the_allocating_one_twice_in_a_row():
    from eredu_b200 import ops
    from eredu_b200.ops import native

    lib = native.lib()
    dev = "cuda"
    D, n_q, n_kv, qps, splits = 128, 32, 8, 1, 12   # more splits than a cluster combines: both entries use scratch
    kv_lens = [517, 33, 2048, 700]
    B = len(kv_lens)
    g = torch.Generator(device=dev).manual_seed(5)
    max_pages = max((l + 15) // 16 for l in kv_lens) + 1
    n_pages = B * max_pages + 1
    kc = torch.randn(n_pages, n_kv, 16, D, device=dev, generator=g).bfloat16()
    vc = torch.randn(n_pages, n_kv, 16, D, device=dev, generator=g).bfloat16()
    bt = (torch.randperm(n_pages - 1, device=dev, generator=g)[: B * max_pages].int() + 1).view(B, max_pages).contiguous()
    sl = torch.tensor(kv_lens, device=dev, dtype=torch.int32)
    scale = 1 / math.sqrt(D)
    for trial in range(2):  # the second call finds the array as the first one left it
        q = torch.randn(B * qps, n_q, D, device=dev, generator=g).bfloat16()
        want = ops.attention_decode(q, kc, vc, bt, sl, qps, scale, splits=splits)
        got = torch.empty_like(q)
        code = _call_static(lib, q, kc, vc, got, bt, sl, B, qps, n_q, n_kv, D, splits, scale)
        assert code == 0, code
        torch.cuda.synchronize()
        assert torch.equal(got, want), trial          # same kernel, same splits: the bits must agree
        ref = ops.attention_ref(q, kc, vc, bt, sl, [qps] * B, scale)
        rel = float((got.float() - ref.float()).norm() / ref.float().norm())
        assert rel < 1.5e-2, (trial, rel)
    # sizes beyond the built-in scratch are refused with a clear code, nothing is launched
    big = torch.empty(300 * 64, n_q, D, device=dev, dtype=torch.bfloat16)
    assert _call_static(lib, big, kc, vc, big, bt, sl, 300, 64, n_q, n_kv, D, 8, scale) == -2
