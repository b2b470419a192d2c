// Split-KV paged decode attention for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference runtime; it exists for embedders of this library.
//
// Who needs it: a serving loop that fixed its memory budget at start-up and must not call cudaMalloc (or the
// PyTorch caching allocator) afterwards - an allocation there can synchronise the device, take the allocator
// lock another thread holds, or simply fail under a full pool; a plug-in that receives raw device pointers and
// owns no allocator at all; a latency-critical thread that may only enqueue work. eredu_attn_decode() needs
// three scratch buffers from its caller for the split-KV partial results. eredu_attn_decode_static() takes the
// same inputs and outputs and no scratch: the partials live in a fixed array inside the library image.
//
// Limits (checked, -2 is returned beyond them):
//   batch * q_per_seq * n_q_heads * splits <= EREDU_NOALLOC_MAX_ROW_SPLITS (8192)
//   batch * n_kv_heads                     <= EREDU_NOALLOC_MAX_GROUPS     (4096)
//   head_dim 64 or 128
// The array costs about 4.1 MB of device memory on every GPU that loads the library, until the process exits.
//
// First call on a device: the library looks up the device address of its array (cudaGetSymbolAddress, with that
// device current) and caches it. Make that first call outside any stream capture. A process that drives several
// GPUs gets one array, one cached address and one kernel configuration per device; call with the device of the
// pointers current.
//
// All calls share the one array and it keeps whatever the previous call left in it. The arrival counters are
// cleared on the stream at the start of every call; the partials are fully rewritten before they are read.
// Two calls whose kernels can overlap on the GPU (different streams without an ordering between them, or two
// host threads) would use the same scratch at the same time and race: serialise them.
//
// The function calls no cudaMalloc, cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define EREDU_NOALLOC_MAX_ROW_SPLITS 8192
#define EREDU_NOALLOC_MAX_GROUPS 4096

#ifdef __cplusplus
extern "C" {
#endif

// Same contract as eredu_attn_decode (q: [batch * q_per_seq, n_q_heads, head_dim] bf16, paged K/V caches
// [pages, n_kv_heads, 16, head_dim], block_table [batch, max_pages] int32, seq_lens [batch] int32, optional
// sinks [n_q_heads] fp32, out like q) minus the scratch arguments. Returns 0, a cudaError_t, -1 for an
// unsupported shape, -2 when the sizes exceed the limits above.
int eredu_attn_decode_static(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                             const int* seq_lens, const float* sinks, int batch, int q_per_seq, int max_pages,
                             int n_q_heads, int n_kv_heads, int head_dim, int splits, int window, float scale,
                             cudaStream_t stream);

#ifdef __cplusplus
}
#endif
