"""Operators of the runtime: sm_100a kernels for CUDA tensors, PyTorch references for CPU tensors."""
from .core import (KERNEL_HEAD_DIMS, PAGE, attention_decode, attention_decode_rope, attention_prefill, attention_ref, decode_scratch, decode_splits, embedding,
                   gated_linear, gated_linear_ref, linear, linear_ref, rmsnorm, rmsnorm_ref, rope_kv, rope_kv_ref,
                   silu_mul)
from .sampling import (SamplingParams, pack_allow_mask, pack_rows, philox_uniform, process_logits_ref, rows_to_tensor,
                       sample, sample_ref, spec_verify, verify_ref)
from .conv import short_conv, short_conv_ref
from .recurrent import gated_delta_scan, gated_delta_scan_ref, mamba2_scan, mamba2_scan_ref
from . import native
