// Gated causal short convolution of the LFM2 family, fused with its recurrent state:
//   proj = in_proj(x) = [B | C | X]  (three blocks of `C` channels per token)
//   bx   = B * X
//   y[t] = sum_j w[c, j] * bx[t - (L-1) + j]        depthwise, causal, kernel width L (2..4)
//   out  = C * (y + bias)
// (eredu/src/backend/mlx/architectures/lfm2/model.rs:899-914). The L-1 newest bx rows of every sequence live in a
// state pool indexed by the sequence's first KV page, so the same launch serves chunked prefill (values before the
// chunk come from the state), decode (one token per sequence, graph-replayable: every index is read on the device)
// and batches that mix sequences of different lengths.
//
// Grid (channel blocks, sequences, token segments): a thread owns two adjacent channels and walks its segment of the
// sequence's chunk with the window in registers; segment 0 is the only one that reads the old state (before the
// chunk's first token) and the only one that writes the new one (after it has read), so no other block races it.
#include "../common/launch.h"
#include "../common/launch_count.h"
#include "../common/ptx.cuh"

namespace eredu {

struct ShortConvParams {
  const __nv_bfloat16* proj;  // [M, 3C], row stride ldp
  const float* w;             // [C, L]
  const float* bias;          // [C] or null
  __nv_bfloat16* state;       // [pages, L-1, C]
  const int* block_table;     // [B, ld_bt]: column 0 = the page that names the sequence's state
  const int* cu_q;            // [B+1] token offsets (prefill) or null: q_per_seq tokens per sequence
  const int* positions;       // [M]
  const long long* slots;     // [M] KV slot of every token; negative = inactive row
  __nv_bfloat16* out;         // [M, C]
  int ldp, ld_bt, q_per_seq, C, B;
  int mode;   // 0: gated (LFM2): input B * X, output C * y.  1: plain: input proj[:, x_off + c], output silu(y)
  int x_off;
};

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16(v)); }

template <int L>
__global__ void __launch_bounds__(128) short_conv_kernel(ShortConvParams p) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.y;
  const int r0 = p.cu_q != nullptr ? p.cu_q[b] : b * p.q_per_seq;
  const int r1 = p.cu_q != nullptr ? p.cu_q[b + 1] : (b + 1) * p.q_per_seq;
  const int n = r1 - r0;
  if (n <= 0 || p.slots[r0] < 0) return;
  const int nseg = gridDim.z, seg = blockIdx.z;
  const int seglen = max(16, (n + nseg - 1) / nseg);  // >= L-1: only segment 0 reaches back before the chunk
  const int t0 = seg * seglen, t1 = min(n, t0 + seglen);
  if (t0 >= t1) return;
  const int c = (blockIdx.x * 128 + threadIdx.x) * 2;
  if (c >= p.C) return;
  const int C = p.C;
  const int pos0 = p.positions[r0];
  __nv_bfloat16* st = p.state + static_cast<size_t>(p.block_table[static_cast<size_t>(b) * p.ld_bt]) * (L - 1) * C + c;

  float w0[L], w1[L];
#pragma unroll
  for (int j = 0; j < L; ++j) {
    w0[j] = p.w[static_cast<size_t>(c) * L + j];
    w1[j] = p.w[static_cast<size_t>(c + 1) * L + j];
  }
  const float bias0 = p.bias != nullptr ? p.bias[c] : 0.f, bias1 = p.bias != nullptr ? p.bias[c + 1] : 0.f;

  auto bx_of = [&](int t, float& v0, float& v1) {  // B * X of chunk row t, rounded like the stored state
    const __nv_bfloat16* row = p.proj + static_cast<size_t>(r0 + t) * p.ldp + c;
    if (p.mode == 1) {
      const uint32_t xx = *reinterpret_cast<const uint32_t*>(row + p.x_off);
      v0 = bf16_lo(xx);
      v1 = bf16_hi(xx);
      return;
    }
    const uint32_t bb = *reinterpret_cast<const uint32_t*>(row);
    const uint32_t xx = *reinterpret_cast<const uint32_t*>(row + 2 * C);
    v0 = round_bf16(bf16_lo(bb) * bf16_lo(xx));
    v1 = round_bf16(bf16_hi(bb) * bf16_hi(xx));
  };

  // window: bx at chunk rows t0-(L-1) .. t0-1; rows before the chunk come from the state (zero before the sequence)
  float win0[L - 1], win1[L - 1], hist0[L - 1], hist1[L - 1];
#pragma unroll
  for (int j = 0; j < L - 1; ++j) {
    hist0[j] = hist1[j] = 0.f;
    if (t0 == 0) {  // segment 0: state row j holds bx of position pos0 - (L-1) + j
      if (pos0 - (L - 1) + j >= 0) {
        const uint32_t s = *reinterpret_cast<const uint32_t*>(st + static_cast<size_t>(j) * C);
        hist0[j] = bf16_lo(s);
        hist1[j] = bf16_hi(s);
      }
      win0[j] = hist0[j];
      win1[j] = hist1[j];
    } else {        // later segments start at least L-1 rows into the chunk
      bx_of(t0 - (L - 1) + j, win0[j], win1[j]);
    }
  }

  for (int t = t0; t < t1; ++t) {
    float cur0, cur1;
    bx_of(t, cur0, cur1);
    float y0 = w0[L - 1] * cur0 + bias0, y1 = w1[L - 1] * cur1 + bias1;
#pragma unroll
    for (int j = 0; j < L - 1; ++j) {
      y0 += w0[j] * win0[j];
      y1 += w1[j] * win1[j];
    }
    uint32_t packed;
    if (p.mode == 1) {
      packed = pack_bf16x2(y0 / (1.f + __expf(-y0)), y1 / (1.f + __expf(-y1)));
    } else {
      const uint32_t cc = *reinterpret_cast<const uint32_t*>(p.proj + static_cast<size_t>(r0 + t) * p.ldp + C + c);
      packed = pack_bf16x2(bf16_lo(cc) * y0, bf16_hi(cc) * y1);
    }
    *reinterpret_cast<uint32_t*>(p.out + static_cast<size_t>(r0 + t) * C + c) = packed;
#pragma unroll
    for (int j = 0; j + 1 < L - 1; ++j) {
      win0[j] = win0[j + 1];
      win1[j] = win1[j + 1];
    }
    win0[L - 2] = cur0;
    win1[L - 2] = cur1;
  }

  if (seg == 0) {
    // new state: bx at chunk rows n-(L-1) .. n-1; rows before the chunk are the old state shifted
    float ns0[L - 1], ns1[L - 1];
#pragma unroll
    for (int j = 0; j < L - 1; ++j) {
      const int idx = n - (L - 1) + j;
      if (idx >= 0) {
        bx_of(idx, ns0[j], ns1[j]);
      } else {  // chunk shorter than the window: old state row n + j moves up
        ns0[j] = ns1[j] = 0.f;
#pragma unroll
        for (int k = 0; k < L - 1; ++k)
          if (k == n + j) {
            ns0[j] = hist0[k];
            ns1[j] = hist1[k];
          }
      }
    }
#pragma unroll
    for (int j = 0; j < L - 1; ++j)
      *reinterpret_cast<uint32_t*>(st + static_cast<size_t>(j) * C) = pack_bf16x2(ns0[j], ns1[j]);
  }
}

}  // namespace eredu

using namespace eredu;

// out[M, C] = gated short convolution of proj[M, 3C] (mode 0) or silu(conv(proj[:, x_off : x_off + C])) (mode 1: the
// causal depthwise convolution in front of a gated-delta layer); state [pages, L-1, C] bf16 is read and updated in place.
// cu_q null: B sequences of q_per_seq tokens each (decode); else B sequences with token offsets cu_q (prefill chunks,
// at most max_q_len tokens each). C even, L in 2..4.
extern "C" int eredu_short_conv(const void* proj, int ldp, const float* w, const float* bias, void* state,
                                const int* block_table, int ld_bt, const int* cu_q, int q_per_seq, const int* positions,
                                const long long* slots, void* out, int C, int L, int B, int max_q_len, int mode, int x_off,
                                cudaStream_t stream) {
  if (B <= 0 || C <= 0) return 0;
  if (C % 2 != 0 || ldp % 2 != 0 || L < 2 || L > 4 || x_off % 2 != 0 || (mode != 0 && mode != 1)) return -1;
  ShortConvParams p = {};
  p.proj = static_cast<const __nv_bfloat16*>(proj);
  p.w = w;
  p.bias = bias;
  p.state = static_cast<__nv_bfloat16*>(state);
  p.block_table = block_table;
  p.cu_q = cu_q;
  p.positions = positions;
  p.slots = slots;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldp = ldp;
  p.ld_bt = ld_bt;
  p.q_per_seq = q_per_seq;
  p.C = C;
  p.B = B;
  p.mode = mode;
  p.x_off = x_off;
  const int longest = cu_q != nullptr ? max_q_len : q_per_seq;
  int nseg = (longest + 63) / 64;
  nseg = nseg < 1 ? 1 : nseg > 4096 ? 4096 : nseg;
  dim3 grid((C / 2 + 127) / 128, B, nseg);
  cudaError_t e;
  if (L == 2) e = launch_pdl(short_conv_kernel<2>, grid, dim3(128), 0, stream, p);
  else if (L == 3) e = launch_pdl(short_conv_kernel<3>, grid, dim3(128), 0, stream, p);
  else e = launch_pdl(short_conv_kernel<4>, grid, dim3(128), 0, stream, p);
  eredu_count_launches(1);
  return static_cast<int>(e);
}
